"""GPU parity tests of the hybrid prefill path (operand preparation + attention kernel).

Tolerances: INT8 codes and scales bit-exact against the oracle's block quantiser (block = 1 row);
attention outputs max-abs <= 2e-2 and rel-MSE <= 1e-4 against float64 dense causal attention
on the same BF16 inputs."""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import sage_unified as su
from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc
from tests.helpers import max_abs

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, REL_MSE = 2e-2, 1e-4


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def to_np(t):
    return t.detach().float().cpu().numpy()


def make(B, H_Q, H_KV, N, W, seed, rho=0.05):
    case = gen_numpy(B, H_Q, H_KV, N, 128, W, rho, seed)
    rb = orc.bf16_round
    return rb(case.q), rb(case.k), rb(case.v)


@pytest.mark.parametrize("N", [64, 200, 1000])
@pytest.mark.parametrize("smooth", [True, False])
def test_operand_preparation_bit_exact(N, smooth):
    q, k, v = make(1, 4, 2, N, 64, N)
    sm = 128 ** -0.5
    q_i8, q_bf, q_sc, k_i8, k_bf, k_sc, k_mean = su.quantize_operands(t_bf16(q), t_bf16(k), sm, smooth)
    km = to_np(k_mean)[:, :, None, :]
    if smooth:
        assert max_abs(km, k.mean(axis=2, keepdims=True)) <= 2e-2       # bf16 rounding of the mean
    else:
        assert np.abs(km).max() == 0
    ksm = orc.bf16_round(k - km)
    assert np.array_equal(to_np(k_bf), ksm)
    ki, ks = orc.quant_per_block_int8(ksm, 1, 1.0)           # the block quantiser's arithmetic, one row per block
    assert np.array_equal(k_sc.cpu().numpy()[..., :N], ks) and not k_sc.cpu().numpy()[..., N:].any()
    assert np.array_equal(k_i8.cpu().numpy(), ki)
    qi, qs = orc.quant_per_block_int8(q, 1, sm * orc.LOG2E)
    assert np.allclose(q_sc.cpu().numpy()[..., :N], qs, rtol=1e-6)
    assert (np.abs(q_i8.cpu().numpy().astype(int) - qi.astype(int)) <= 1).all()      # fp32 product order of sm * log2e
    assert (q_i8.cpu().numpy() != qi).mean() < 1e-3
    assert np.array_equal(to_np(q_bf), q)


def check(out, ref):
    assert np.isfinite(out).all()
    assert max_abs(out, ref) <= MAX_ABS, max_abs(out, ref)
    assert orc.rel_mse(out, ref) <= REL_MSE, orc.rel_mse(out, ref)


@pytest.mark.parametrize("B,H_Q,H_KV,N,W", [(1, 4, 2, 128, 64), (1, 4, 1, 200, 64), (2, 8, 2, 512, 128), (1, 4, 4, 1000, 256),
                                            (1, 8, 2, 2048, 128), (1, 2, 1, 1500, 0), (1, 2, 2, 77, 128)])
def test_vertical_attention_vs_dense(B, H_Q, H_KV, N, W):
    q, k, v = make(B, H_Q, H_KV, N, W, N + W)
    R = H_Q // H_KV
    vidx = hq.compute_vertical_indices(t_bf16(q), t_bf16(k), W, 0.05, kv_repeat=R)
    out = hq.sage_vertical_attention_v2(t_bf16(q), t_bf16(k), t_bf16(v), vidx, window_size=W)
    assert out.dtype == torch.bfloat16 and out.shape == (B, H_Q, N, 128)
    ref = orc.dense_causal_attention(q, k, v)
    check(to_np(out), ref)
    # the reference restatement (INT8 rest / fp16 vertical + window) lands in the same place
    if N <= 512:
        rr = orc.hybrid_prefill_reference(q, k, v, vidx.cpu().numpy(), window_size=W, round_fn=orc.bf16_round)
        assert max_abs(to_np(out), rr) <= MAX_ABS


def test_plan_reuse_and_status_word():
    q, k, v = make(1, 8, 2, 900, 128, 17)
    vidx = hq.compute_vertical_indices(t_bf16(q), t_bf16(k), 128, 0.05, kv_repeat=4)
    plan = su.PrefillPlan(t_bf16(q), t_bf16(k), t_bf16(v), vidx, 128, None, True)
    a = to_np(plan.run()).copy()
    b = to_np(plan.run())
    plan.check_status()                      # no bounded wait expired on the device
    assert np.array_equal(a, b)              # deterministic
    check(a, orc.dense_causal_attention(q, k, v))


def test_window_only_full_and_int8_only_variants():
    q, k, v = make(1, 8, 2, 700, 128, 5)
    ref = orc.dense_causal_attention(q, k, v)
    tq, tk, tv = t_bf16(q), t_bf16(k), t_bf16(v)
    check(to_np(hq.sage_unified_attention(tq, tk, tv, window_size=128)), ref)
    check(to_np(hq.sage_unified_attention(tq, tk, tv, window_size=0)), ref)
    check(to_np(hq.sage_fp8_attention(tq, tk, tv, pv_fp8=False)), ref)
    # FP8 P V (the entry point's default, checked against its own oracle in test_gpu_fp8_pv.py) is an order of magnitude
    # further from exact attention: that is the format, not the kernel
    fp8 = to_np(hq.sage_fp8_attention(tq, tk, tv))
    assert np.isfinite(fp8).all() and 1e-4 < orc.rel_mse(fp8, ref) < 5e-3
    full = to_np(hq.full_attention_fp16_triton(tq, tk, tv))
    check(full, ref)
    assert orc.rel_mse(full, ref) < 2e-5          # no quantisation at all on this path
    nhd = hq.full_attention_fp16_triton(tq.transpose(1, 2), tk.transpose(1, 2), tv.transpose(1, 2), tensor_layout="NHD")
    assert max_abs(to_np(nhd.transpose(1, 2)), full) == 0
    # fp32 inputs come back as fp32
    o32 = hq.sage_unified_attention(tq.float(), tk.float(), tv.float(), window_size=128)
    assert o32.dtype == torch.float32
    check(to_np(o32), ref)


def test_vertical_lines_are_served_in_bf16():
    """A key with a huge outlier would wreck its INT8 block; as a vertical line it is exact."""
    q, k, v = make(1, 2, 1, 1024, 128, 9)
    k[0, 0, 300] *= 32.0        # a power of two keeps the row bf16-exact
    ref = orc.dense_causal_attention(q, k, v)
    vidx = torch.tensor([[[300, 5], [300, 7]]], device=DEV)
    out = hq.sage_vertical_attention_v2(t_bf16(q), t_bf16(k), t_bf16(v), vidx, window_size=128, smooth_k=False)
    check(to_np(out), ref)


def test_full_size_rows_against_fp32_reference():
    """BASELINE prefill shape (B=1, 32q/8kv, N=8192, W=128, rho=5%): sampled query blocks against an
    fp32 dense computation on the device."""
    t = __import__("hyquant_b200.synth", fromlist=["gen_torch"]).gen_torch(1, 32, 8, 8192, 128, 128, 0.05, 2013, device=DEV)
    q, k, v = t["q"], t["k"], t["v"]
    vidx = hq.compute_vertical_indices(q, k, 128, 0.05, kv_repeat=4)
    out = hq.sage_vertical_attention_v2(q, k, v, vidx, window_size=128).float()
    kf = k.float().repeat_interleave(4, dim=1); vf = v.float().repeat_interleave(4, dim=1)
    for blk in (0, 1, 31, 63):
        rows = slice(blk * 128, blk * 128 + 128)
        s = torch.einsum("bhqd,bhkd->bhqk", q[:, :, rows].float(), kf) * 128 ** -0.5
        pos = torch.arange(8192, device=DEV)
        s = s.masked_fill(pos[None, None, None, :] > pos[rows][None, None, :, None], float("-inf"))
        ref = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, -1), vf)
        o = out[:, :, rows]
        assert (o - ref).abs().max().item() <= MAX_ABS
        assert ((o - ref) ** 2).sum().item() / (ref ** 2).sum().item() <= REL_MSE
