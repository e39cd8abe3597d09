"""Generate the golden fixtures in this directory by EXECUTING the reference.

Run once, in a container where the reference checkout is available:

    HYQUANT_REFERENCE=/path/to/HyQuant python tests/golden/make_golden.py

It imports the reference's own ``src.ops`` / ``src.patch`` modules, runs their
CPU-capable functions (``quantize_per_token``, ``DStageLayerCache.freeze /
append_staging / decode_attention`` with HYBRID_ATTN_DECODE_KERNEL=pytorch,
``compute_vertical_indices``, ``reorder_kv_for_vertical``) on seeded inputs and
stores inputs' SHA-256 plus the outputs (or their SHA-256 when large) as
``*.npz``.  The tests replay the fixtures against the CPU oracle and, on a
GPU, against the CUDA kernels; they never import the reference.
"""

from __future__ import annotations

import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.environ.get("HYQUANT_REFERENCE")
if not REF or not os.path.isdir(os.path.join(REF, "src", "ops")):
    sys.exit("set HYQUANT_REFERENCE to a checkout of the reference (the directory that holds src/ops)")
sys.path.insert(0, REF)
os.environ["HYBRID_ATTN_DECODE_KERNEL"] = "pytorch"

import torch  # noqa: E402

from hyquant_b200.synth import gen_numpy  # noqa: E402

from src.ops.decode_d_stage import quantize_per_token, dequantize_per_token  # noqa: E402
from src.ops.d_stage_kv_cache import DStageLayerCache  # noqa: E402
from src.ops.sage_unified import reorder_kv_for_vertical  # noqa: E402
from src.patch._common import compute_vertical_indices  # noqa: E402


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def save(name, **kw):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **kw)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def golden_quant():
    """quantize_per_token / dequantize_per_token on bf16 and fp32 inputs."""
    rng = np.random.Generator(np.random.PCG64(11))
    x = rng.standard_normal((3, 40, 128), dtype=np.float32) * 2.0
    x[0, 0] = 0.0                                  # all-zero token -> clamp(min=1e-5)
    x[0, 1] = 1e-7                                 # below the clamp
    x[0, 2] = np.linspace(-7, 7, 128) * 0.5        # exact .5 ties after division
    x[0, 3, :] = 0.0; x[0, 3, 5] = 3.0e4           # large magnitude
    x[1, 0, :] = np.arange(128) % 16 - 8           # every code value
    x[1, 1, 17] = 65504.0 * 7                      # fp16 scale near its maximum
    xb = torch.from_numpy(x).to(torch.bfloat16)
    out = {"x_bf16_bits": bf16_bits(xb), "x_f32": x}
    for tag, t in (("bf16", xb), ("f32", torch.from_numpy(x))):
        for nb in (2, 4, 8):
            p, s = quantize_per_token(t, nb)
            out[f"{tag}_packed{nb}"] = p.numpy()
            out[f"{tag}_scale{nb}"] = s.numpy()
            out[f"{tag}_deq{nb}"] = dequantize_per_token(p, s, 128, nb).numpy()
    save("quant_per_token", **out)


def run_cache_case(name, B, H_Q, H_KV, N, W, rho, seed, dtype, n_append, probe_steps,
                   n_qry=None, k_bits=4, v_bits=4):
    """freeze -> appends (with flushes) -> decode_attention through the reference."""
    case = gen_numpy(B, H_Q, H_KV, N, 128, W, rho, seed, n_qry=n_qry)
    R = H_Q // H_KV
    tt = lambda a: torch.from_numpy(a).to(dtype)
    lc = DStageLayerCache(0, k_bits=k_bits, v_bits=v_bits, window_size=W, top_ratio=rho, use_vert=True)
    lc.update_prefill(tt(case.k), tt(case.v))
    lc.save_query_tail(tt(case.q))
    # the indices freeze() will select (same calls as d_stage_kv_cache.py:131-136)
    Wc = min(W, N)
    if N - Wc > 0:
        q_kv = lc._query_tail.reshape(B, H_KV, R, -1, 128).mean(dim=2)
        vidx = compute_vertical_indices(q_kv, lc._keys[:, :, :N - Wc, :], W, rho).numpy()
    else:
        vidx = np.zeros((B, H_KV, 0), dtype=np.int64)
    lc.freeze(kv_repeat=R)
    out = {
        "meta": np.array([B, H_Q, H_KV, N, W, seed, n_append, -1 if n_qry is None else n_qry], dtype=np.int64),
        "rho": np.array([rho]), "is_bf16": np.array([dtype == torch.bfloat16]),
        "bits": np.array([k_bits, v_bits], dtype=np.int64),
        "in_sha": np.array([sha(case.q), sha(case.k), sha(case.v), sha(case.q_decode)]),
        "frozen_k_packed_sha": np.array([sha(lc.k_quant_packed.numpy())]),
        "frozen_v_packed_sha": np.array([sha(lc.v_quant_packed.numpy())]),
        "frozen_k_scale": lc.k_scale.numpy(), "frozen_v_scale": lc.v_scale.numpy(),
        "frozen_k_topk_sha": np.array([sha(lc.k_topk.float().numpy())]),
        "frozen_vidx": vidx,
        "frozen_shapes": np.array([lc.k_quant_packed.shape[1], lc.k_topk.shape[1], lc.k_window.shape[1]]),
        "probe_steps": np.array(probe_steps, dtype=np.int64),
    }
    rng = np.random.Generator(np.random.PCG64(seed + 77))
    new_k = rng.standard_normal((n_append, B, H_KV, 1, 128), dtype=np.float32)
    new_v = rng.standard_normal((n_append, B, H_KV, 1, 128), dtype=np.float32)
    new_q = rng.standard_normal((n_append, B, H_Q, 1, 128), dtype=np.float32)
    out["append_sha"] = np.array([sha(new_k), sha(new_v), sha(new_q)])
    for step in range(1, n_append + 1):
        lc.append_staging(tt(new_k[step - 1]), tt(new_v[step - 1]))
        if step in probe_steps:
            o = lc.decode_attention(tt(new_q[step - 1]), R)
            out[f"out_step{step}"] = o.float().numpy()
            out[f"state_step{step}"] = np.array([lc.k_quant_packed.shape[1], lc._staging_ptr])
    out["final_k_packed_sha"] = np.array([sha(lc.k_quant_packed.numpy())])
    out["final_v_packed_sha"] = np.array([sha(lc.v_quant_packed.numpy())])
    out["final_k_scale_sha"] = np.array([sha(lc.k_scale.numpy())])
    out["final_v_scale_sha"] = np.array([sha(lc.v_scale.numpy())])
    save(name, **out)


def golden_vertical():
    """compute_vertical_indices: plain and GQA-native branches, fp32."""
    case = gen_numpy(2, 8, 2, 640, 128, 64, 0.05, 21)
    q, k = torch.from_numpy(case.q), torch.from_numpy(case.k)
    idx_gqa = compute_vertical_indices(q, k, 64, 0.05, kv_repeat=4)
    k_exp = k.repeat_interleave(4, dim=1)
    idx_plain = compute_vertical_indices(q, k_exp, 64, 0.05)
    pooled = q[:, :, -256:, :].mean(dim=2, keepdim=True)      # pre-pooled query (tail_len = 1)
    idx_pool = compute_vertical_indices(pooled, k, 64, 0.05, kv_repeat=4)
    save("vertical_indices", meta=np.array([2, 8, 2, 640, 64, 21]), rho=np.array([0.05]),
         in_sha=np.array([sha(case.q), sha(case.k)]),
         idx_gqa=idx_gqa.numpy(), idx_plain=idx_plain.numpy(), idx_pool=idx_pool.numpy())


def golden_reorder():
    """reorder_kv_for_vertical (rest/vertical split + per-query counts)."""
    rng = np.random.Generator(np.random.PCG64(31))
    B, H, N, D, W, T = 1, 3, 700, 8, 128, 29
    k = rng.standard_normal((B * H, N, D), dtype=np.float32)
    v = rng.standard_normal((B * H, N, D), dtype=np.float32)
    vidx = np.stack([rng.permutation(N - W)[:T] for _ in range(B * H)]).reshape(B, H, T).astype(np.int64)
    kr, vr, kv, vv, nr, nv, R, V = reorder_kv_for_vertical(
        torch.from_numpy(k), torch.from_numpy(v), torch.from_numpy(vidx), W)
    save("reorder_kv", k=k, v=v, vidx=vidx, window=np.array([W]),
         k_rest=kr.numpy(), v_rest=vr.numpy(), k_vert=kv.numpy(), v_vert=vv.numpy(),
         n_rest_valid=nr.numpy(), n_vert_valid=nv.numpy(), RV=np.array([R, V]))


def golden_bit_widths():
    """The cache life cycle at the other bit widths of the reference's modes (d_k8v8, d_k4v2, d_k2v4)."""
    for kb, vb in ((8, 8), (4, 2), (2, 4)):
        run_cache_case(f"cache_k{kb}v{vb}_f32", 1, 4, 2, 400, 64, 0.05, 40 + kb + vb, torch.float32, 130, [1, 128, 130],
                       k_bits=kb, v_bits=vb)


if __name__ == "__main__":
    torch.manual_seed(0)
    torch.set_num_threads(max(1, os.cpu_count() or 1))
    if len(sys.argv) > 1 and sys.argv[1] == "--bit-widths-only":
        golden_bit_widths()
        sys.exit(0)
    golden_bit_widths()
    golden_quant()
    # BASELINE config 0: B=1, 32q/8kv, N=1024, W=128, rho=5%, staging 64, fp32
    run_cache_case("cache_cfg0_f32", 1, 32, 8, 1024, 128, 0.05, 0, torch.float32, 64, [1, 64])
    # bf16 cache, two flushes, probes either side of each flush boundary
    run_cache_case("cache_small_bf16", 2, 8, 2, 600, 64, 0.05, 5, torch.bfloat16, 300,
                   [1, 2, 127, 128, 129, 255, 256, 300])
    # short prefill: N < W (no prefix) and N - W small
    run_cache_case("cache_tiny_f32", 1, 4, 2, 48, 64, 0.05, 6, torch.float32, 130, [1, 128, 130])
    run_cache_case("cache_short_f32", 1, 4, 1, 200, 64, 0.10, 7, torch.float32, 3, [3], n_qry=20)
    golden_vertical()
    golden_reorder()
