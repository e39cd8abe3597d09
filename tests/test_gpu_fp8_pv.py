"""FP8 P V behind ``sage_fp8_attention`` (tcgen05 kind::f8f6f4, V^T in e4m3 per channel, P~ in e4m3 against the exact
running maximum) against the CPU oracle's restatement of the reference's FP8 arithmetic.

Tolerances: V codes and scales bit for bit; attention outputs within max-abs 2e-2 / rel-MSE 1e-4 of the oracle's FP8
result (two runs of the same arithmetic differ only where an fp32 rounding flips an e4m3 rounding).  The distance of
FP8 P V from exact attention is larger than that and is printed, not hidden: it is the price of the format."""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import sage_unified as su
from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def make(B, H_Q, H_KV, N, seed):
    c = gen_numpy(B, H_Q, H_KV, N, 128, 128, 0.05, seed)
    rb = orc.bf16_round
    return rb(c.q), rb(c.k), rb(c.v)


def test_v_quantiser_bit_exact():
    q, k, v = make(2, 2, 2, 300, 3)
    v[0, 1, :, 5] = 0.0                                  # an all-zero channel: scale 0, codes 0
    plan = su.PrefillPlan(t_bf16(q), t_bf16(k), t_bf16(v), None, 0, None, True, pv_fp8=True)
    codes, scale = orc.per_channel_fp8(v)
    assert np.array_equal(plan.v_scale8.cpu().numpy(), scale)
    got = plan.v_t8.view(torch.float8_e4m3fn).float().cpu().numpy()          # [B,H,128,Npad]
    assert np.array_equal(got[..., :300], codes.transpose(0, 1, 3, 2)) and not got[..., 300:].any()


@pytest.mark.parametrize("B,H_Q,H_KV,N", [(1, 2, 1, 128), (1, 4, 2, 320), (2, 4, 1, 1000), (1, 8, 2, 2048)])
def test_fp8_pv_against_oracle(B, H_Q, H_KV, N):
    q, k, v = make(B, H_Q, H_KV, N, N)
    out = hq.sage_fp8_attention(t_bf16(q), t_bf16(k), t_bf16(v)).float().cpu().numpy()
    ref8 = orc.fp8_pv_attention_reference(q, k, v, round_fn=orc.bf16_round)
    assert np.isfinite(out).all()
    err, rm = np.abs(out - ref8).max(), orc.rel_mse(out, ref8)
    dense = orc.dense_causal_attention(q, k, v)
    print(f"N={N}: kernel vs FP8 oracle max-abs {err:.2e} rel-mse {rm:.2e}; FP8 oracle vs exact attention max-abs "
          f"{np.abs(ref8 - dense).max():.2e} rel-mse {orc.rel_mse(ref8, dense):.2e}; kernel vs exact "
          f"{np.abs(out - dense).max():.2e} {orc.rel_mse(out, dense):.2e}")
    assert err <= 2e-2 and rm <= 1e-4, (err, rm)
    # the format's own error: well above the BF16 path's, and the kernel is no further from exact attention than the oracle
    assert orc.rel_mse(out, dense) <= 1.5 * orc.rel_mse(ref8, dense) + 1e-5
    bf = hq.sage_fp8_attention(t_bf16(q), t_bf16(k), t_bf16(v), pv_fp8=False).float().cpu().numpy()
    assert orc.rel_mse(bf, dense) <= 1e-4


@pytest.mark.parametrize("B,H_Q,H_KV,N,W", [(1, 4, 2, 640, 128), (1, 8, 2, 1536, 64)])
def test_fp8_pv_with_window_and_vertical_lines(B, H_Q, H_KV, N, W):
    """The hybrid structure (INT8 rest, BF16 vertical lines and window for Q K^T) with every P V tile in FP8."""
    q, k, v = make(B, H_Q, H_KV, N, N + 1)
    vidx = hq.compute_vertical_indices(t_bf16(q), t_bf16(k), W, 0.05, kv_repeat=H_Q // H_KV)
    out = hq.sage_vertical_attention_v2(t_bf16(q), t_bf16(k), t_bf16(v), vidx, window_size=W, pv_fp8=True).float().cpu().numpy()
    ref8 = orc.fp8_pv_attention_reference(q, k, v, window_size=W, round_fn=orc.bf16_round, vertical_indices=vidx.cpu().numpy())
    err, rm = np.abs(out - ref8).max(), orc.rel_mse(out, ref8)
    assert np.isfinite(out).all() and err <= 2e-2 and rm <= 1e-4, (err, rm)
    out_w = su.hybrid_prefill(t_bf16(q), t_bf16(k), t_bf16(v), None, W, None, True, pv_fp8=True).float().cpu().numpy()
    ref_w = orc.fp8_pv_attention_reference(q, k, v, window_size=W, round_fn=orc.bf16_round)
    assert np.abs(out_w - ref_w).max() <= 2e-2 and orc.rel_mse(out_w, ref_w) <= 1e-4


def test_fp8_pv_at_8k_rows_against_dense():
    """The benchmark's 8K shape: sampled blocks against fp32 dense attention at the looser bound FP8 P V can meet."""
    from hyquant_b200.synth import gen_torch
    t = gen_torch(1, 32, 8, 8192, 128, 128, 0.05, 2013, device=DEV)
    q, k, v = t["q"], t["k"], t["v"]
    out = hq.sage_fp8_attention(q, k, v).float()
    kf = k.float().repeat_interleave(4, dim=1); vf = v.float().repeat_interleave(4, dim=1)
    pos = torch.arange(8192, device=DEV)
    for blk in (0, 17, 63):
        rows = slice(blk * 128, blk * 128 + 128)
        s = torch.einsum("bhqd,bhkd->bhqk", q[:, :, rows].float(), kf) * 128 ** -0.5
        s = s.masked_fill(pos[None, None, None, :] > pos[rows][None, None, :, None], float("-inf"))
        ref = torch.einsum("bhqk,bhkd->bhqd", torch.softmax(s, -1), vf)
        o = out[:, :, rows]
        assert torch.isfinite(o).all()
        assert ((o - ref) ** 2).sum().item() / (ref ** 2).sum().item() <= 5e-3
