"""Generate the GPU-side golden fixtures (``*_gpu.npz``) by EXECUTING the reference's Triton kernels.

The reference implements ``per_block_int8``, the hybrid prefill (``sage_vertical_attention_v2``,
``sage_unified_attention``, ``full_attention_fp16_triton``) and the four-segment decode
(``fused_d_stage_decode``) only as Triton kernels, so these fixtures can only be produced on a machine
with a GPU.  ``oracle/make_ref.py`` first puts a copy of the reference's ``src`` tree into the untracked
``oracle/_ref/``; this script imports it from there:

    python oracle/make_ref.py                      # where the reference checkout is
    python tests/golden/make_golden_gpu.py [out_dir]   # on the GPU machine; default out_dir = this directory

Inputs come from ``hyquant_b200.synth.gen_numpy`` (bit-reproducible from the seed), so a fixture holds
only the seed, the SHA-256 of the inputs, the vertical-line indices the reference chose and the
reference's outputs (whole for small cases, sampled rows plus a SHA-256 of the whole for large ones).
The tests replay them against the CPU oracle and the CUDA kernels and never import the reference.
"""

from __future__ import annotations

import hashlib
import json
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
REF = os.path.join(ROOT, "oracle", "_ref")
if not os.path.isdir(os.path.join(REF, "src", "ops")):
    sys.exit("oracle/_ref is missing: run oracle/make_ref.py where the reference checkout is")
sys.path.insert(0, REF)

import torch  # noqa: E402

from hyquant_b200.synth import gen_numpy  # noqa: E402
from oracle import hq_oracle as orc  # noqa: E402

from src.ops.vendor.sageattention.triton.quant_per_block import per_block_int8  # noqa: E402
from src.ops.sage_unified import sage_unified_attention, sage_vertical_attention_v2  # noqa: E402
from src.ops.v_sageattention import full_attention_fp16_triton  # noqa: E402
from src.ops.d_stage_kv_cache import DStageLayerCache  # noqa: E402
from src.patch._common import compute_vertical_indices  # noqa: E402

DEV = "cuda"
OUT = HERE
TIMES = {}


def sha(a) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 / fp16 tensor -> its 16-bit patterns."""
    return t.detach().contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def dev_bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def save(name, **kw):
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **kw)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB", flush=True)


def timed(fn, reps=3):
    fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps


def sample_rows(N: int, count: int, seed: int) -> np.ndarray:
    """Query rows to keep from a large output: the first and last rows, both sides of the 128-row block
    boundaries around the window start, and seeded random rows."""
    rng = np.random.Generator(np.random.PCG64(seed))
    fixed = [0, 1, 63, 64, 127, 128, 129, 255, 256, N // 2 - 1, N // 2, N - 129, N - 128, N - 2, N - 1]
    fixed = [r for r in fixed if 0 <= r < N]
    rest = rng.permutation(N)[: max(0, count - len(fixed))].tolist()
    return np.array(sorted(set(fixed + rest)), dtype=np.int64)


def dense_rows(q, k, v, rows):
    """fp32 dense causal attention for the given query rows of every head: q [1,H_q,N,D] bf16 on the device."""
    H_q, H_kv = q.shape[1], k.shape[1]
    g = H_q // H_kv
    r = torch.as_tensor(rows, device=DEV)
    out = torch.empty(1, H_q, len(rows), 128, device=DEV, dtype=torch.float32)
    pos = torch.arange(k.shape[2], device=DEV)
    for h in range(H_q):
        s = (q[0, h, r].float() @ k[0, h // g].float().T) * 128 ** -0.5
        s = s.masked_fill(pos[None, :] > r[:, None], float("-inf"))
        out[0, h] = torch.softmax(s, -1) @ v[0, h // g].float()
    return out


def golden_quant():
    """per_block_int8 (quant_per_block.py:49-101): codes and scales, with and without K smoothing."""
    res = {}
    for tag, (B, H_q, H_kv, N, seed, smooth) in {"a": (1, 2, 1, 200, 61, True), "b": (2, 4, 2, 321, 62, False)}.items():
        c = gen_numpy(B, H_q, H_kv, N, 128, 64, 0.05, seed)
        q, k = dev_bf16(c.q), dev_bf16(c.k)
        km = k.mean(dim=2, keepdim=True) if smooth else None
        qi, qs, ki, ks = per_block_int8(q, k, km=km, sm_scale=128 ** -0.5, tensor_layout="HND")
        res.update({f"{tag}_meta": np.array([B, H_q, H_kv, N, seed, int(smooth)]), f"{tag}_in_sha": np.array([sha(c.q), sha(c.k)]),
                    f"{tag}_km": np.zeros(0, np.uint16) if km is None else bits(km),
                    f"{tag}_q_scale": qs.cpu().numpy(), f"{tag}_k_scale": ks.cpu().numpy(),
                    f"{tag}_code_sha": np.array([sha(qi.cpu().numpy()), sha(ki.cpu().numpy())])})
        if tag == "a":       # the codes themselves for the small case, their SHA-256 for both
            res.update({f"{tag}_q_int8": qi.cpu().numpy(), f"{tag}_k_int8": ki.cpu().numpy()})
    save("prefill_quant_gpu", **res)


def run_prefill_case(name, B, H_q, H_kv, N, W, rho, seed, n_rows, pooled_tail=None):
    """One shape through the reference's three prefill entry points.  ``n_rows`` = 0 keeps whole outputs."""
    c = gen_numpy(B, H_q, H_kv, N, 128, W, rho, seed)
    q, k, v = dev_bf16(c.q), dev_bf16(c.k), dev_bf16(c.v)
    R = H_q // H_kv
    if pooled_tail:      # vertical lines from the mean of the last `pooled_tail` queries (the benchmark's rule)
        vidx = compute_vertical_indices(q[:, :, -pooled_tail:].mean(dim=2, keepdim=True), k, W, rho, kv_repeat=R)
    else:
        vidx = compute_vertical_indices(q, k, W, rho, kv_repeat=R)
    rows = np.arange(N) if n_rows == 0 else sample_rows(N, n_rows, seed)
    ridx = torch.as_tensor(rows, device=DEV)
    outs = {}
    t0 = time.perf_counter()
    outs["vertical"] = sage_vertical_attention_v2(q, k, v, vidx, window_size=W)
    torch.cuda.synchronize()
    print(f"  {name}: first reference call {time.perf_counter() - t0:.1f} s (includes Triton compilation)", flush=True)
    outs["unified_w"] = sage_unified_attention(q, k, v, window_size=W)
    outs["unified_0"] = sage_unified_attention(q, k, v, window_size=0)
    outs["full"] = full_attention_fp16_triton(q, k, v, tensor_layout="HND", is_causal=True)
    torch.cuda.synchronize()
    dense = dense_rows(q, k, v, rows) if B == 1 else None
    res = {"meta": np.array([B, H_q, H_kv, N, W, seed, pooled_tail or 0]), "rho": np.array([rho]),
           "in_sha": np.array([sha(c.q), sha(c.k), sha(c.v)]), "vidx": vidx.cpu().numpy().astype(np.int32), "rows": rows}
    # rows kept per entry point: every sampled row of the vertical-line kernel, a thinner subset of the others
    thin = {"vertical": 1, "unified_w": 3 if N >= 8192 else (8 if n_rows == 0 else 1), "unified_0": 8 if n_rows == 0 else 3,
            "full": 8 if n_rows == 0 else 3}
    for key, o in outs.items():
        assert o.dtype == torch.bfloat16 and tuple(o.shape) == (B, H_q, N, 128)
        if not (N >= 8192 and key in ("unified_0", "full")):
            res["rows_" + key] = rows[::thin[key]]
            res["out_" + key] = bits(o[:, :, ridx[::thin[key]]])
        res["sha_" + key] = np.array([sha(bits(o))])
        if dense is not None:
            d = o[:, :, ridx].float() - dense
            res["err_" + key] = np.array([float(d.abs().max()), float((d ** 2).sum() / (dense ** 2).sum())])
            print(f"  {name} {key}: reference vs fp32 dense on the kept rows: max-abs {res['err_' + key][0]:.3e} "
                  f"rel-mse {res['err_' + key][1]:.3e}", flush=True)
    save(name, **res)
    if N >= 8192:
        TIMES[f"prefill_vertical_v2_ms_N{N}"] = timed(lambda: sage_vertical_attention_v2(q, k, v, vidx, window_size=W))
        TIMES[f"prefill_unified_w_ms_N{N}"] = timed(lambda: sage_unified_attention(q, k, v, window_size=W))
        TIMES[f"prefill_full_fp16_ms_N{N}"] = timed(lambda: full_attention_fp16_triton(q, k, v, tensor_layout="HND", is_causal=True))
        print("  timings", {k_: round(v_, 3) for k_, v_ in TIMES.items()}, flush=True)


def run_decode_case(tag, B, H_q, H_kv, N, W, rho, seed, probes, res):
    """The reference's cache life cycle on the device (eager-CUDA quantiser, Triton split-K decode)."""
    c = gen_numpy(B, H_q, H_kv, N, 128, W, rho, seed, n_qry=W)
    q, k, v = dev_bf16(c.q), dev_bf16(c.k), dev_bf16(c.v)
    R = H_q // H_kv
    layer = DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=rho, use_vert=True)
    layer.update_prefill(k, v)
    layer.save_query_tail(q)
    # the selection freeze is about to make (d_stage_kv_cache.py:131-136), repeated here to record it
    q_kv = q[:, :, -W:].reshape(B, H_kv, R, -1, 128).mean(dim=2)
    vidx = compute_vertical_indices(q_kv, k[:, :, :N - W], W, rho)
    layer.freeze(kv_repeat=R)
    T = vidx.shape[-1]
    gathered = k[:, :, :N - W].gather(2, vidx.unsqueeze(-1).expand(-1, -1, -1, 128)).reshape(B * H_kv, T, 128)
    assert torch.equal(gathered, layer.k_topk), "recorded vertical indices are not the ones freeze used"
    rng = np.random.Generator(np.random.PCG64(seed + 77))
    n_app = max(probes)
    nk = rng.standard_normal((n_app, B, H_kv, 1, 128), dtype=np.float32)
    nv = rng.standard_normal((n_app, B, H_kv, 1, 128), dtype=np.float32)
    nq = rng.standard_normal((n_app, B, H_q, 1, 128), dtype=np.float32)
    res.update({f"{tag}_meta": np.array([B, H_q, H_kv, N, W, seed, n_app]), f"{tag}_rho": np.array([rho]),
                f"{tag}_in_sha": np.array([sha(c.q), sha(c.k), sha(c.v), sha(nk), sha(nv), sha(nq)]),
                f"{tag}_vidx": vidx.cpu().numpy().astype(np.int32), f"{tag}_probes": np.array(probes),
                f"{tag}_frozen_sha": np.array([sha(layer.k_quant_packed.cpu().numpy()), sha(layer.v_quant_packed.cpu().numpy()),
                                               sha(bits(layer.k_scale)), sha(bits(layer.v_scale))])})
    for s in range(n_app):
        layer.append_staging(dev_bf16(nk[s]), dev_bf16(nv[s]))
        if s + 1 in probes:
            out = layer.decode_attention(dev_bf16(nq[s]), R)
            res[f"{tag}_out_{s + 1}"] = bits(out)
            res[f"{tag}_state_{s + 1}"] = np.array([layer.k_quant_packed.shape[1], layer._staging_ptr])
    res[f"{tag}_final_sha"] = np.array([sha(layer.k_quant_packed.cpu().numpy()), sha(bits(layer.k_scale))])
    if N >= 32768:
        qd = dev_bf16(nq[0])
        TIMES[f"decode_triton_us_N{N}_B{B}_Hq{H_q}"] = timed(lambda: layer.decode_attention(qd, R), reps=50) * 1e3
        print("  timings", {k_: round(v_, 3) for k_, v_ in TIMES.items()}, flush=True)


def main():
    global OUT
    if len(sys.argv) > 1:
        OUT = sys.argv[1]
        os.makedirs(OUT, exist_ok=True)
    which = set(sys.argv[2].split(",")) if len(sys.argv) > 2 else {"quant", "small", "decode", "8k", "32k"}
    torch.manual_seed(0)
    print(torch.cuda.get_device_name(0), "torch", torch.__version__, flush=True)
    if "quant" in which:
        golden_quant()
    if "small" in which:
        run_prefill_case("prefill_s1_gpu", 1, 2, 1, 320, 64, 0.05, 71, 0)
        run_prefill_case("prefill_s2_gpu", 1, 4, 2, 1024, 128, 0.05, 72, 64)
        run_prefill_case("prefill_s3_gpu", 1, 8, 2, 2048, 256, 0.05, 73, 40)
    if "decode" in which:
        res = {}
        run_decode_case("n1k", 1, 32, 8, 1024, 128, 0.05, 81, [1, 64, 127, 128, 130], res)
        run_decode_case("n4k", 2, 8, 2, 4096, 128, 0.05, 82, [1, 129], res)
        run_decode_case("n32k", 1, 32, 8, 32768, 128, 0.05, 83, [1, 64], res)
        save("decode_triton_gpu", **res)
    if "8k" in which:
        run_prefill_case("prefill_8k_gpu", 1, 32, 8, 8192, 128, 0.05, 2013, 24, pooled_tail=256)
    if "32k" in which:
        run_prefill_case("prefill_32k_gpu", 1, 32, 8, 32768, 128, 0.05, 2015, 24, pooled_tail=256)
    with open(os.path.join(OUT, "reference_triton_times.json"), "w") as f:
        json.dump(TIMES, f, indent=1)
    print(json.dumps(TIMES), flush=True)


if __name__ == "__main__":
    main()
