"""The CPU oracle against fixtures produced by the reference's own Triton kernels on a B200
(``tests/golden/make_golden_gpu.py``): the block quantiser, the hybrid prefill kernels and the split-K decode.

Tolerances, each stated where it is used: the reference's results carry the rounding of Triton's approximate
fp32 division and of fp16 / bf16 tiles, so the restatement is compared to within one bf16 output step rather than
bit for bit; INT4 codes and fp16 scales of a cache frozen by the reference on the device are compared by hash."""

import numpy as np
import pytest

from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc
from tests.helpers import load, sha


def _prefill_case(name):
    g = load(name)
    B, H_q, H_kv, N, W, seed, pooled = [int(x) for x in g["meta"]]
    c = gen_numpy(B, H_q, H_kv, N, 128, W, float(g["rho"][0]), seed)
    assert [sha(c.q), sha(c.k), sha(c.v)] == list(g["in_sha"]), "seeded inputs differ from the fixture's"
    rb = orc.bf16_round
    return g, rb(c.q), rb(c.k), rb(c.v), W


def test_block_quantiser_against_triton():
    """Scales within one fp32 ulp, codes equal except a fraction < 1e-3 that is off by one step (div.full.f32)."""
    g = load("prefill_quant_gpu")
    for tag in "ab":
        B, H_q, H_kv, N, seed, smooth = [int(x) for x in g[tag + "_meta"]]
        c = gen_numpy(B, H_q, H_kv, N, 128, 64, 0.05, seed)
        assert [sha(c.q), sha(c.k)] == list(g[tag + "_in_sha"])
        q, k = orc.bf16_round(c.q), orc.bf16_round(c.k)
        km = orc.bf16_bits_to_f32(g[tag + "_km"]) if smooth else None
        if smooth:      # the mean torch forms on the device is the bf16 rounding of the fp32 mean
            assert np.array_equal(km, orc.bf16_round(k.mean(axis=2, keepdims=True)))
        qi, qs, ki, ks = orc.per_block_int8(q, k, km=km, sm_scale=128 ** -0.5, round_fn=orc.bf16_round)
        for mine, ref in ((qs, g[tag + "_q_scale"]), (ks, g[tag + "_k_scale"])):
            assert mine.shape == ref.shape
            assert np.all(np.abs(mine.view(np.int32) - ref.view(np.int32)) <= 1)
        if tag == "a":
            for mine, ref in ((qi, g["a_q_int8"]), (ki, g["a_k_int8"])):
                d = np.abs(mine.astype(int) - ref.astype(int))
                assert d.max() <= 1 and (d != 0).mean() < 1e-3
            assert np.array_equal(ki, g["a_k_int8"])          # identical scales here, hence identical codes


@pytest.mark.parametrize("name", ["prefill_s1_gpu", "prefill_s2_gpu"])
def test_hybrid_prefill_restatement_against_triton(name):
    """sage_vertical_attention_v2 and sage_unified_attention(window > 0): the numpy restatement lands within one
    bf16 step (2^-8 at outputs of magnitude < 1) of the Triton kernel's output, rel-MSE < 5e-6."""
    g, q, k, v, W = _prefill_case(name)
    B, H_q = q.shape[:2]
    out = orc.hybrid_prefill_reference(q, k, v, g["vidx"].astype(np.int64), window_size=W, round_fn=orc.bf16_round)
    ref = orc.bf16_bits_to_f32(g["out_vertical"])
    got = out[:, :, g["rows_vertical"]]
    assert np.abs(got - ref).max() <= 2 ** -7 and orc.rel_mse(got, ref) < 5e-6
    assert (got == ref).mean() > 0.7                           # most outputs agree bit for bit
    out = orc.hybrid_prefill_reference(q, k, v, np.zeros((B, H_q, 0), np.int64), window_size=W, round_fn=orc.bf16_round)
    ref = orc.bf16_bits_to_f32(g["out_unified_w"])
    got = out[:, :, g["rows_unified_w"]]
    assert np.abs(got - ref).max() <= 2 ** -7 and orc.rel_mse(got, ref) < 5e-6
    # the yardstick of the GPU tests: the reference's kernel against exact attention, as recorded on the device
    dense = orc.dense_causal_attention(q, k, v)[:, :, g["rows"]]
    ref_all = orc.bf16_bits_to_f32(g["out_vertical"])
    if len(g["rows_vertical"]) == len(g["rows"]):
        assert abs(np.abs(ref_all - dense).max() - float(g["err_vertical"][0])) < 2e-3


@pytest.mark.parametrize("tag", ["n1k", "n4k", "n32k"])
def test_decode_cache_against_reference_on_device(tag):
    """A cache frozen by the reference on the device (eager CUDA quantiser) and decoded by its Triton split-K kernel:
    codes and scales hash-equal under either scale rounding of the oracle's quantiser, outputs within 2e-4 /
    rel-MSE 2e-5 of the oracle's exact four-segment attention."""
    g = load("decode_triton_gpu")
    B, H_q, H_kv, N, W, seed, n_app = [int(x) for x in g[tag + "_meta"]]
    rho, R = float(g[tag + "_rho"][0]), H_q // H_kv
    c = gen_numpy(B, H_q, H_kv, N, 128, W, rho, seed, n_qry=W)
    rng = np.random.Generator(np.random.PCG64(seed + 77))
    nk = rng.standard_normal((n_app, B, H_kv, 1, 128), dtype=np.float32)
    nv = rng.standard_normal((n_app, B, H_kv, 1, 128), dtype=np.float32)
    nq = rng.standard_normal((n_app, B, H_q, 1, 128), dtype=np.float32)
    assert [sha(c.q), sha(c.k), sha(c.v), sha(nk), sha(nv), sha(nq)] == list(g[tag + "_in_sha"])
    rb = orc.bf16_round
    q, k, v = rb(c.q), rb(c.k), rb(c.v)
    vidx = g[tag + "_vidx"].astype(np.int64)
    for recip in ((True, False) if tag != "n32k" else (True,)):
        oc = orc.freeze(k, v, q[:, :, -W:], R, W, rho, round_fn=rb, vidx_override=vidx, reciprocal_scale=recip)
        got = [sha(oc.k_quant_packed), sha(oc.v_quant_packed), sha(oc.k_scale.view(np.uint16)), sha(oc.v_scale.view(np.uint16))]
        assert got == list(g[tag + "_frozen_sha"])
    # the reference's bf16 scores select the same SET of vertical lines as fp32 scores do on these inputs
    if tag == "n1k":
        own = orc.freeze(k, v, q[:, :, -W:], R, W, rho, round_fn=rb)
        assert all(set(own.vidx[b, h]) == set(vidx[b, h]) for b in range(B) for h in range(H_kv))
    probes = [int(s) for s in g[tag + "_probes"]]
    for s in range(n_app):
        orc.append_staging(oc, rb(nk[s]), rb(nv[s]))
        if s + 1 in probes:
            assert [oc.k_quant_packed.shape[1], oc.staging_ptr] == [int(x) for x in g[f"{tag}_state_{s + 1}"]]
            ref = orc.bf16_bits_to_f32(g[f"{tag}_out_{s + 1}"])
            out = orc.decode_attention_exact(rb(nq[s]), oc, R)
            assert np.abs(out - ref).max() <= 2e-4 + 2 ** -8 * np.abs(ref).max()
            assert orc.rel_mse(out, ref) <= 2e-5
    assert [sha(oc.k_quant_packed), sha(oc.k_scale.view(np.uint16))] == list(g[tag + "_final_sha"])
