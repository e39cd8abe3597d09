"""Torch-CPU restatement of the reference's decode fallback, used as the TIMED CPU
baseline (``bench.py`` ``cpu_baseline`` / ``--impl reference``).

TEST INFRASTRUCTURE ONLY — never imported by the product package.  It issues the
same ATen operator sequence as the reference (dequantise -> fp16 -> cat -> expand to
query heads -> softmax(q K^T / sqrt(D)) V), so it uses the host cores the way the
reference's own CPU path does (intra-op threads = torch.get_num_threads()).
Checked against the golden fixtures in tests/test_oracle_golden.py.
"""

from __future__ import annotations

import torch


def unpack_int4(packed: torch.Tensor, D: int) -> torch.Tensor:
    """src/ops/decode_d_stage.py:114-123."""
    x = packed.to(torch.int32) & 0xFF
    lo = ((x & 0x0F) << 28) >> 28
    hi = (((x >> 4) & 0x0F) << 28) >> 28
    out = torch.empty(packed.shape[0], packed.shape[1], D, dtype=torch.float32)
    out[..., 0::2] = lo.float()
    out[..., 1::2] = hi.float()
    return out


def dequantize_per_token(packed, scale, D):
    """src/ops/decode_d_stage.py:80-101 (4-bit)."""
    return (unpack_int4(packed, D) * scale.float().unsqueeze(-1)).to(torch.float16)


def decode_attention_fallback(q, kq, vq, ks, vs, k_topk, v_topk, k_stag, v_stag, k_win, v_win, B, H_KV, kv_repeat):
    """src/ops/d_stage_kv_cache.py:306-354.  q [B, H_Q, 1, D] -> [B, H_Q, 1, D]."""
    D = q.shape[-1]
    dtype = q.dtype
    H_Q = H_KV * kv_repeat
    segs_k = [dequantize_per_token(kq, ks, D).to(dtype)]
    segs_v = [dequantize_per_token(vq, vs, D).to(dtype)]
    for kk, vv in ((k_topk, v_topk), (k_stag, v_stag), (k_win, v_win)):
        if kk.shape[1] > 0:
            segs_k.append(kk.to(dtype)); segs_v.append(vv.to(dtype))
    k_all = torch.cat(segs_k, dim=1)
    v_all = torch.cat(segs_v, dim=1)
    n = k_all.shape[1]
    k_all = k_all.reshape(B, H_KV, n, D).unsqueeze(2).expand(B, H_KV, kv_repeat, n, D).reshape(B, H_Q, n, D)
    v_all = v_all.reshape(B, H_KV, n, D).unsqueeze(2).expand(B, H_KV, kv_repeat, n, D).reshape(B, H_Q, n, D)
    scores = (q @ k_all.transpose(-1, -2)) * (D ** -0.5)
    return torch.softmax(scores, dim=-1) @ v_all


def from_numpy_cache(c):
    """oracle.hq_oracle.LayerCache -> tuple of torch CPU tensors for the call above."""
    import numpy as np
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a))
    S = c.staging_ptr
    return (t(c.k_quant_packed), t(c.v_quant_packed), t(c.k_scale), t(c.v_scale), t(c.k_topk), t(c.v_topk),
            t(c.staging_k[:, :S]), t(c.staging_v[:, :S]), t(c.k_window), t(c.v_window))
