"""GPU parity tests: vertical-line scores, exact top-k, cache reorganisation."""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import _lib
from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc
from tests.helpers import load, max_abs, sha

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


@pytest.mark.parametrize("B,H_Q,H_KV,N,W,nq", [(2, 8, 2, 640, 64, 640), (1, 32, 8, 1024, 128, 1024), (1, 4, 4, 200, 64, 7),
                                                (1, 16, 1, 333, 32, 100), (1, 8, 8, 129, 128, 1)])
def test_vertical_scores_and_topk(B, H_Q, H_KV, N, W, nq):
    case = gen_numpy(B, H_Q, H_KV, N, 128, W, 0.05, 21, n_qry=nq)
    q, k = orc.bf16_round(case.q), orc.bf16_round(case.k)
    R = H_Q // H_KV
    s_gpu = hq.vertical_scores(t_bf16(q), t_bf16(k), W, R)
    s_ref = orc.vertical_scores(q, k, W, R)
    assert s_gpu.shape == s_ref.shape
    sg = s_gpu.cpu().numpy()
    assert max_abs(sg, s_ref) <= 1e-3 * max(1.0, np.abs(s_ref).max())
    # top-k: bit-exact given identical fp32 scores (descending, ties to the lower index)
    kk = orc.vertical_topk_count(sg.shape[-1], 0.05)
    idx, asc = hq.topk_indices(s_gpu, kk, want_ascending=True)
    assert idx.dtype == torch.int64 and asc.dtype == torch.int32
    assert np.array_equal(idx.cpu().numpy(), orc.topk_desc(sg, kk))
    assert np.array_equal(asc.cpu().numpy(), np.sort(orc.topk_desc(sg, kk), axis=-1))
    # the public entry point
    out = hq.compute_vertical_indices(t_bf16(q), t_bf16(k), W, 0.05, kv_repeat=R)
    assert np.array_equal(out.cpu().numpy(), orc.topk_desc(sg, kk))
    # K already expanded to H_Q heads gives the same scores
    if R > 1:
        s_exp = hq.vertical_scores(t_bf16(q), t_bf16(np.repeat(k, R, axis=1)), W, 1)
        assert max_abs(s_exp.cpu().numpy(), sg) <= 1e-4 * max(1.0, np.abs(sg).max())


@pytest.mark.parametrize("B,H_KV,R,N,W,nq", [(1, 8, 4, 1024, 128, 128), (2, 2, 16, 600, 64, 64), (1, 4, 7, 300, 32, 5)])
def test_vertical_scores_with_group_mean_inside(B, H_KV, R, N, W, nq):
    """The freeze-side selection: the mean over a kv-head's query heads taken inside the scoring call equals the
    eager mean in the input dtype followed by the plain call."""
    case = gen_numpy(B, H_KV * R, H_KV, N, 128, W, 0.05, 33, n_qry=nq)
    q, k = t_bf16(case.q), t_bf16(case.k)
    fused = hq.vertical_scores(q, k, W, 1, group_mean=R)
    eager = hq.vertical_scores(q.reshape(B, H_KV, R, nq, 128).mean(dim=2), k, W, 1)
    assert fused.shape == eager.shape == (B, H_KV, N - W)
    # the same numbers up to a rare last-bit difference of a 16-bit mean (fp32 summation order over the heads)
    assert max_abs(fused.cpu().numpy(), eager.cpu().numpy()) <= 2e-3 * float(eager.abs().max())
    kk = orc.vertical_topk_count(N - W, 0.05)
    a, b = hq.topk_indices(fused, kk), hq.topk_indices(eager, kk)
    same = np.mean([len(set(x.tolist()) & set(y.tolist())) / kk for x, y in zip(a.reshape(-1, kk).cpu().numpy(), b.reshape(-1, kk).cpu().numpy())])
    assert same >= 0.95


def test_vertical_reference_rounding_mode_and_empty_prefix():
    case = gen_numpy(1, 8, 2, 512, 128, 64, 0.05, 5)
    q, k = orc.bf16_round(case.q), orc.bf16_round(case.k)
    s = hq.vertical_scores(t_bf16(q), t_bf16(k), 64, 4, round_like_reference=True).cpu().numpy()
    assert np.array_equal(orc.bf16_round(s), s)            # scores are bf16-exact in this mode
    pooled = orc.bf16_round(q[:, :, -64:].mean(axis=2))
    ref = np.einsum("bhrd,bhpd->bhrp", pooled.reshape(1, 2, 4, 128), k[:, :, :448]).reshape(1, 8, 448)
    assert max_abs(s, ref) <= 2e-2 * max(1.0, np.abs(ref).max())
    out = hq.compute_vertical_indices(t_bf16(q[:, :, :5]), t_bf16(k[:, :, :60]), 64, 0.05, kv_repeat=4)
    assert out.shape == (1, 8, 0) and out.dtype == torch.int64


@pytest.mark.parametrize("n,k", [(1, 1), (7, 7), (100, 1), (1000, 50), (4097, 205), (131072 - 256, 6541), (20000, 16384)])
def test_topk_exact_with_ties(n, k):
    rng = np.random.Generator(np.random.PCG64(n + k))
    rows = 3
    s = rng.standard_normal((rows, n), dtype=np.float32)
    s[1] = np.round(s[1] * 4) / 4            # heavy ties
    s[2, : n // 2] = 1.5                      # a plateau that straddles the threshold
    s[0, 0] = -0.0
    idx, asc = hq.topk_indices(torch.from_numpy(s).to(DEV), k, want_ascending=True)
    ref = orc.topk_desc(s, k)
    assert np.array_equal(idx.cpu().numpy(), ref)
    assert np.array_equal(asc.cpu().numpy(), np.sort(ref, axis=-1))


def test_topk_limits():
    s = torch.zeros(1, 40000, device=DEV)
    with pytest.raises(hq.HyQuantError):
        hq.topk_indices(s, 16385)
    with pytest.raises(hq.HyQuantError):
        hq.topk_indices(s[:, :10], 11)


def test_vertical_indices_fixture_sets():
    """The reference's fp32 selection (golden) against the device selection on bf16-rounded
    inputs: sets agree except for near-ties moved by the bf16 rounding of the inputs."""
    g = load("vertical_indices")
    B, H_Q, H_KV, N, W, seed = [int(x) for x in g["meta"]]
    case = gen_numpy(B, H_Q, H_KV, N, 128, W, 0.05, seed)
    out = hq.compute_vertical_indices(t_bf16(case.q), t_bf16(case.k), W, 0.05, kv_repeat=H_Q // H_KV).cpu().numpy()
    ref = g["idx_gqa"]
    assert out.shape == ref.shape
    for a, b in zip(out.reshape(-1, out.shape[-1]), ref.reshape(-1, ref.shape[-1])):
        assert len(set(a.tolist()) & set(b.tolist())) >= 0.9 * len(a)


@pytest.mark.parametrize("BH,N,W,T", [(2, 1024, 128, 45), (3, 300, 64, 0), (1, 130, 128, 1), (2, 64, 64, 0), (8, 4096, 128, 199)])
def test_cache_reorganize_bit_exact(BH, N, W, T):
    rng = np.random.Generator(np.random.PCG64(N + T))
    k = orc.bf16_round(rng.standard_normal((1, BH, N, 128), dtype=np.float32) * 1.7)
    v = orc.bf16_round(rng.standard_normal((1, BH, N, 128), dtype=np.float32))
    P = N - W
    vidx = np.stack([rng.permutation(P)[:T] for _ in range(BH)]).reshape(1, BH, T).astype(np.int64) if T else None
    layer = hq.DStageLayerCache(0, window_size=W, top_ratio=0.05, use_vert=False)
    layer.update_prefill(t_bf16(k), t_bf16(v))
    layer.freeze(kv_repeat=1, vertical_indices=None if vidx is None else torch.from_numpy(vidx))
    qt = np.zeros((1, BH, 1, 128), np.float32)
    oc = orc.freeze(k, v, qt if T else None, 1, W, 0.05, vidx_override=vidx, use_vert=T > 0)
    assert np.array_equal(layer.k_quant_packed.cpu().numpy(), oc.k_quant_packed)
    assert np.array_equal(layer.v_quant_packed.cpu().numpy(), oc.v_quant_packed)
    assert np.array_equal(layer.k_scale.cpu().numpy().view(np.uint16), oc.k_scale.view(np.uint16))
    assert np.array_equal(layer.v_scale.cpu().numpy().view(np.uint16), oc.v_scale.view(np.uint16))
    assert np.array_equal(layer.k_topk.float().cpu().numpy(), oc.k_topk)
    assert np.array_equal(layer.v_topk.float().cpu().numpy(), oc.v_topk)
    assert np.array_equal(layer.k_window.float().cpu().numpy(), oc.k_window)
    assert np.array_equal(layer.v_window.float().cpu().numpy(), oc.v_window)
    assert layer._staging_buf_k.shape == (BH, 128, 128) and float(layer._staging_buf_k.abs().sum()) == 0.0
