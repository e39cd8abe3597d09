"""Hybrid-precision prefill attention — host-side mirror of the reference module
``src/ops/sage_unified.py`` (``sage_vertical_attention_v2``, ``sage_unified_attention``)
plus ``full_attention_fp16_triton`` (``src/ops/v_sageattention.py``) and
``sage_fp8_attention`` (``src/ops/sage_fp8_attention.py``), all served by one sm_100a
tcgen05 / tensor-memory kernel (``hq_prefill_hybrid``) after one operand-preparation pass (``hq_prefill_quant``).

By design nothing is expanded to query heads and nothing is physically reordered:
K/V stay at kv-head granularity, the vertical lines of a query head are removed from
its INT8 pass by a bit mask and served from a small gathered BF16 copy.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from ._lib import HyQuantError, PrefillArgs

_LOG2_E = 1.44269504


def _prep_inputs(q, k, v):
    for name, t in (("q", q), ("k", k), ("v", v)):
        _lib.require_cuda(t, name)
    B, H_q, N, D = q.shape
    if D != 128:
        raise HyQuantError(f"head_dim {D} is not built (128 only)")
    H_kv = k.shape[1]
    if H_q % H_kv != 0 or k.shape[2] != N or v.shape[2] != N:
        raise HyQuantError("q/k/v shapes do not agree")
    def bf(t):
        t = t if t.dtype == torch.bfloat16 else t.to(torch.bfloat16)
        ok = t.stride(3) == 1 and all(s % 8 == 0 for s in t.stride()[:3]) and t.data_ptr() % 16 == 0
        return t if ok else t.contiguous()
    return bf(q), bf(k), bf(v), B, H_q, H_kv, N


# INT8 scale granularity of the prefill: "row" = one scale per query row and per key row (the default: an outlier
# row costs its neighbours no precision), "block" = the reference's one scale per 128 query rows / 64 key rows
# (per_block_int8, quant_per_block.py:49-101).
SCALE_GRANULARITY = "row"


def per_block_int8(q: torch.Tensor, k: torch.Tensor, km: Optional[torch.Tensor] = None, BLKQ: int = 128, BLKK: int = 64,
                   sm_scale: Optional[float] = None, tensor_layout: str = "HND"):
    """The reference's block quantiser (vendor/sageattention/triton/quant_per_block.py:49-101), same signature
    and results bit for bit: returns (q_int8, q_scale [B,H_q,ceil(L/BLKQ)] fp32, k_int8, k_scale [B,H_kv,ceil(L/BLKK)]).
    q is scaled by ``sm_scale * log2(e)`` before quantising; ``km`` (the key mean, [B,H_kv,1,D]) is subtracted from k
    in the input dtype first.  bf16 inputs."""
    for name, t in (("q", q), ("k", k)):
        _lib.require_cuda(t, name)
        if t.dtype != torch.bfloat16:
            raise HyQuantError("per_block_int8 is built for bf16 inputs")
    if tensor_layout == "NHD":
        q, k = q.transpose(1, 2), k.transpose(1, 2)
        km = None if km is None else km.transpose(1, 2)
    elif tensor_layout != "HND":
        raise ValueError(f"Unknown tensor layout: {tensor_layout}")
    if q.shape[-1] != 128:
        raise HyQuantError(f"head_dim {q.shape[-1]} is not built (128 only)")
    if sm_scale is None:
        sm_scale = q.shape[-1] ** -0.5
    lib = _lib.lib()

    def one(x, blk, mul, mean):
        ok = x.stride(3) == 1 and all(s % 8 == 0 for s in x.stride()[:3]) and x.data_ptr() % 16 == 0
        x = x if ok else x.contiguous()
        B, H, L, _ = x.shape
        xi = torch.empty(B, H, L, 128, dtype=torch.int8, device=x.device)
        sc = torch.empty(B, H, (L + blk - 1) // blk, dtype=torch.float32, device=x.device)
        mp = None
        if mean is not None:
            mean = mean.to(torch.bfloat16).reshape(B * H, 128).contiguous()
            mp = mean.data_ptr()
        rc = lib.hq_per_block_int8(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2), B, H, L, blk, float(mul), mp,
                                   xi.data_ptr(), xi.stride(0), xi.stride(1), xi.stride(2), sc.data_ptr(),
                                   _lib.stream_ptr(x.device))
        _lib.check(rc, "hq_per_block_int8")
        return xi, sc

    qi, qs = one(q, BLKQ, sm_scale * _LOG2_E, None)
    ki, ks = one(k, BLKK, 1.0, km)
    if tensor_layout == "NHD":
        qi, ki = qi.transpose(1, 2), ki.transpose(1, 2)
    return qi, qs, ki, ks


def quantize_operands(qb: torch.Tensor, kb: torch.Tensor, sm_scale: float, smooth_k: bool,
                      scale_granularity: Optional[str] = None):
    """Operand preparation (``hq_prefill_quant`` / ``hq_prefill_quant_blocks``): returns q_i8, q_bf, q_scale, k_i8,
    k_bf, k_scale, k_mean; the scale arrays hold one value per row either way."""
    gran = SCALE_GRANULARITY if scale_granularity is None else scale_granularity
    if gran not in ("row", "block"):
        raise ValueError(f"scale_granularity must be 'row' or 'block', got {gran!r}")
    B, H_q, N, _ = qb.shape
    H_kv = kb.shape[1]
    dev = qb.device
    lib = _lib.lib()
    nqb, nkb = (N + 127) // 128, (N + 63) // 64
    q_i8 = torch.empty(B, H_q, N, 128, dtype=torch.int8, device=dev)
    q_bf = torch.empty(B, H_q, N, 128, dtype=torch.bfloat16, device=dev)
    q_sc = torch.zeros(B, H_q, (N + 63) // 64 * 64, dtype=torch.float32, device=dev)
    k_i8 = torch.empty(B, H_kv, N, 128, dtype=torch.int8, device=dev)
    k_bf = torch.empty(B, H_kv, N, 128, dtype=torch.bfloat16, device=dev)
    k_sc = torch.zeros(B, H_kv, (N + 63) // 64 * 64, dtype=torch.float32, device=dev)
    k_mean = torch.empty(B, H_kv, 128, dtype=torch.bfloat16, device=dev)
    nb = C.c_int64(0)
    _lib.check(lib.hq_prefill_quant_workspace_bytes(B, H_kv, C.byref(nb)), "hq_prefill_quant_workspace_bytes")
    ws = torch.empty(int(nb.value), dtype=torch.uint8, device=dev)
    fn = lib.hq_prefill_quant if gran == "row" else lib.hq_prefill_quant_blocks
    rc = fn(qb.data_ptr(), qb.stride(0), qb.stride(1), qb.stride(2),
            kb.data_ptr(), kb.stride(0), kb.stride(1), kb.stride(2),
            B, H_q, H_kv, N, float(sm_scale), 1 if smooth_k else 0,
            q_i8.data_ptr(), q_bf.data_ptr(), q_sc.data_ptr(),
            k_i8.data_ptr(), k_bf.data_ptr(), k_sc.data_ptr(), k_mean.data_ptr(),
            ws.data_ptr(), ws.numel(), _lib.stream_ptr(dev))
    _lib.check(rc, "hq_prefill_quant")
    return q_i8, q_bf, q_sc, k_i8, k_bf, k_sc, k_mean


class PrefillPlan:
    """Prepared operands of one hybrid prefill call (INT8 / BF16 copies, vertical bookkeeping)
    plus the filled ``hq_prefill_args``; ``run()`` launches only the attention kernel."""

    def __init__(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, vertical_indices: Optional[torch.Tensor],
                 window_size: int, sm_scale: Optional[float], smooth_k: bool, scale_granularity: Optional[str] = None,
                 pv_fp8: bool = False):
        """``pv_fp8``: the P V product in FP8 E4M3 with the reference's ``sage_fp8_attention`` arithmetic (V^T quantised
        per channel, P~ = 2^(s - m + 8.807) against the exact running maximum), for INT8, window and vertical tiles alike."""
        dtype = q.dtype
        qb, kb, vb, B, H_q, H_kv, N = _prep_inputs(q, k, v)
        dev = q.device
        lib = _lib.lib()
        st = _lib.stream_ptr(dev)
        if sm_scale is None:
            sm_scale = 128 ** -0.5
        nqb, nkb = (N + 127) // 128, (N + 63) // 64
        q_i8, q_bf, q_sc, k_i8, k_bf, k_sc, k_mean = quantize_operands(qb, kb, sm_scale, smooth_k, scale_granularity)
        T = 0
        vert_k = vert_vt = nvv = vasc = None
        Npad = (N + 63) // 64 * 64
        v_t = v_t8 = v_sc8 = None
        if pv_fp8:
            v_t8 = torch.empty(B, H_kv, 128, Npad, dtype=torch.uint8, device=dev)
            v_sc8 = torch.empty(B, H_kv, 128, dtype=torch.float32, device=dev)
            scratch = torch.empty(B * H_kv * 128, dtype=torch.int32, device=dev)
            _lib.check(lib.hq_prefill_quant_v_fp8(vb.data_ptr(), vb.stride(0), vb.stride(1), vb.stride(2), B, H_kv, N,
                                                  v_t8.data_ptr(), v_sc8.data_ptr(), scratch.data_ptr(), st), "hq_prefill_quant_v_fp8")
        else:
            v_t = torch.empty(B, H_kv, 128, Npad, dtype=torch.bfloat16, device=dev)
            _lib.check(lib.hq_prefill_transpose_v(vb.data_ptr(), vb.stride(0), vb.stride(1), vb.stride(2), B, H_kv, N,
                                                  v_t.data_ptr(), st), "hq_prefill_transpose_v")
        prefix_len = max(0, N - window_size)
        if vertical_indices is not None and vertical_indices.shape[-1] > 0 and prefix_len > 0:
            if tuple(vertical_indices.shape[:2]) != (B, H_q):
                raise HyQuantError("vertical_indices must be [B, H_q, T]")
            vid = vertical_indices.to(device=dev, dtype=torch.int64).clamp(0, prefix_len - 1)   # reference :510
            vasc = vid.sort(dim=-1).values.to(torch.int32).contiguous()
            T = int(vasc.shape[-1])
            Tpad = (T + 63) // 64 * 64
            vert_k = torch.empty(B, H_q, Tpad, 128, dtype=torch.bfloat16, device=dev)
            vert_vt = torch.empty(B, H_q, 128, Tpad, dtype=torch.bfloat16, device=dev)
            nvv = torch.empty(B, H_q, nqb, dtype=torch.int32, device=dev)
        # per (query head, key) term of the INT8 score conversion; -inf on the head's vertical lines
        k_bias = torch.empty(B, H_q, Npad, dtype=torch.float32, device=dev)
        ptr = lambda t: None if t is None else t.data_ptr()     # noqa: E731
        rc = lib.hq_prefill_vertical_prepare(ptr(vasc), B, H_q, H_kv, N, window_size, T, k_bf.data_ptr(),
                                             vb.data_ptr(), vb.stride(0), vb.stride(1), vb.stride(2), k_sc.data_ptr(),
                                             ptr(vert_k), ptr(vert_vt), k_bias.data_ptr(), ptr(nvv), st)
        _lib.check(rc, "hq_prefill_vertical_prepare")
        vert_vt8 = None
        if pv_fp8 and T:
            vert_vt8 = torch.empty(B, H_q, 128, (T + 63) // 64 * 64, dtype=torch.uint8, device=dev)
            rc = lib.hq_prefill_vertical_gather_v_fp8(vasc.data_ptr(), B, H_q, H_kv, N, T, vb.data_ptr(), vb.stride(0), vb.stride(1),
                                                      vb.stride(2), v_sc8.data_ptr(), vert_vt8.data_ptr(), st)
            _lib.check(rc, "hq_prefill_vertical_gather_v_fp8")
        out = torch.empty(B, H_q, N, 128, dtype=dtype, device=dev)      # contiguous: rows 16-byte aligned
        a = PrefillArgs()
        a.struct_bytes = C.sizeof(PrefillArgs)
        a.B, a.H_Q, a.H_KV, a.N, a.head_dim, a.window, a.T = B, H_q, H_kv, N, 128, int(window_size), T
        a.out_dtype = _lib.dtype_code(dtype)
        a.sm_scale = float(sm_scale)
        a.q_i8, a.q_bf, a.q_scale = q_i8.data_ptr(), q_bf.data_ptr(), q_sc.data_ptr()
        a.k_i8, a.k_bf, a.k_scale = k_i8.data_ptr(), k_bf.data_ptr(), k_sc.data_ptr()
        a.k_bias = k_bias.data_ptr()
        if pv_fp8:
            a.v_t8, a.v_scale8, a.pv_fp8 = v_t8.data_ptr(), v_sc8.data_ptr(), 1
        else:
            a.v_t = v_t.data_ptr()
        if T:
            a.vert_k, a.vert_vt, a.nv_valid = vert_k.data_ptr(), vert_vt.data_ptr(), nvv.data_ptr()
            if vert_vt8 is not None:
                a.vert_vt8 = vert_vt8.data_ptr()
        a.out, a.o_sb, a.o_sh, a.o_sn = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        a.status = self.status.data_ptr()
        self.args, self.out, self.device = a, out, dev
        self._keep = (qb, kb, vb, q_i8, q_bf, q_sc, k_i8, k_bf, k_sc, k_mean, vert_k, vert_vt, k_bias, nvv, v_t, v_t8, v_sc8, vert_vt8)
        self.v_t8, self.v_scale8 = v_t8, v_sc8
        self.flops = 4.0 * B * H_q * 128 * N * (N + 1) / 2

    def run(self) -> torch.Tensor:
        _lib.check(_lib.lib().hq_prefill_hybrid(C.byref(self.args), _lib.stream_ptr(self.device)), "hq_prefill_hybrid")
        return self.out

    def check_status(self) -> None:
        """Synchronising check of the kernel's status word (bit 1: a bounded device wait expired)."""
        st = int(self.status.item())
        if st != 0:
            raise HyQuantError(f"hq_prefill_hybrid reported device status {st} (a bounded wait expired)")


def hybrid_prefill(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, vertical_indices: Optional[torch.Tensor],
                   window_size: int, sm_scale: Optional[float], smooth_k: bool,
                   scale_granularity: Optional[str] = None, pv_fp8: bool = False) -> torch.Tensor:
    """Causal attention [B,H_q,N,D] with INT8 QK^T on the non-vertical prefix and BF16 on the
    vertical lines and the window.  ``vertical_indices`` int64 [B,H_q,T] (any order) or None."""
    return PrefillPlan(q, k, v, vertical_indices, window_size, sm_scale, smooth_k, scale_granularity, pv_fp8).run()


def sage_vertical_attention_v2(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, vertical_indices: torch.Tensor, *,
                               window_size: int = 256, sm_scale: Optional[float] = None,
                               smooth_k: bool = True, pv_fp8: bool = False) -> torch.Tensor:
    """int8 QK for the rest, 16-bit QK for vertical lines + window (reference sage_unified.py:550-622).
    q [B,H_q,N,D], k/v [B,H_kv,N,D], vertical_indices [B,H_q,T] int64; returns q's dtype.
    ``pv_fp8`` (not in the reference's signature): the P V product in FP8 E4M3 as in :func:`sage_fp8_attention`."""
    return hybrid_prefill(q, k, v, vertical_indices, window_size, sm_scale, smooth_k, pv_fp8=pv_fp8)


def sage_unified_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, window_size: int = 0,
                           sm_scale: Optional[float] = None, smooth_k: bool = True) -> torch.Tensor:
    """int8 QK prefix + 16-bit window (reference sage_unified.py:234-313); window_size=0 keeps only the
    diagonal query block in 16 bit."""
    return hybrid_prefill(q, k, v, None, window_size, sm_scale, smooth_k)


def full_attention_fp16_triton(q, k, v, tensor_layout: str = "HND", is_causal: bool = True,
                               sm_scale: Optional[float] = None, **kwargs):
    """16-bit causal attention without quantisation (reference v_sageattention.py:14-51)."""
    del kwargs
    if tensor_layout == "NHD":
        q, k, v = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    out = hybrid_prefill(q, k, v, None, int(q.shape[2]), sm_scale, False)
    return out.transpose(1, 2) if tensor_layout == "NHD" else out


def sage_fp8_attention(q, k, v, *, is_causal: bool = True, sm_scale: Optional[float] = None, smooth_k: bool = True,
                       pv_fp8: bool = True):
    """INT8 Q K^T + FP8 P V causal attention without vertical lines or window (reference sage_fp8_attention.py:15-45,
    whose kernel exists for sm_90a only).  P V follows that kernel's arithmetic on the tcgen05 ``kind::f8f6f4`` path:
    V^T in E4M3 with one scale per channel (``max|v| / 448``), ``P~ = 2^(s - m + 8.807)`` rounded to E4M3 against the
    exact running maximum, the row sum in fp32 before the rounding, ``O = acc / l * v_scale``.  Q K^T is this library's
    INT8 path (one scale per row; the diagonal 128-query block in BF16).  FP8 P V costs accuracy (about 1e-3 rel-MSE
    against exact attention on Gaussian V, where BF16 P V gives 3e-6); ``pv_fp8=False`` runs the same call with BF16
    P V."""
    if not is_causal:
        raise HyQuantError("only causal attention is built")
    return hybrid_prefill(q, k, v, None, 0, sm_scale, smooth_k, pv_fp8=pv_fp8)
