"""The CPU oracle replayed against fixtures produced by executing the reference
(tests/golden/make_golden.py).  Integer / byte results must be bit-exact."""

import numpy as np
import pytest

from oracle import hq_oracle as orc
from tests.helpers import CacheCase, load, sha, max_abs


def test_quantize_per_token_bit_exact():
    g = load("quant_per_token")
    xb = orc.bf16_bits_to_f32(g["x_bf16_bits"])
    for tag, x in (("bf16", xb), ("f32", g["x_f32"])):
        for nb in (2, 4, 8):
            p, s = orc.quantize_per_token(x, nb)
            assert np.array_equal(s.view(np.uint16), g[f"{tag}_scale{nb}"].view(np.uint16)), (tag, nb)
            assert np.array_equal(p, g[f"{tag}_packed{nb}"]), (tag, nb)
            d = orc.dequantize_per_token(p, s, nb)
            assert np.array_equal(d.view(np.uint16), g[f"{tag}_deq{nb}"].view(np.uint16)), (tag, nb)


def test_pack_unpack_roundtrip():
    q = (np.arange(256) % 16 - 8).astype(np.int8).reshape(2, 128)
    assert np.array_equal(orc.unpack_int4(orc.pack_int4(q)), q.astype(np.float32))
    q2 = (np.arange(256) % 4 - 2).astype(np.int8).reshape(2, 128)
    assert np.array_equal(orc.unpack_int2(orc.pack_int2(q2)), q2.astype(np.float32))


@pytest.mark.parametrize("name", ["cache_cfg0_f32", "cache_small_bf16", "cache_tiny_f32", "cache_short_f32",
                                  "cache_k8v8_f32", "cache_k4v2_f32", "cache_k2v4_f32"])
def test_freeze_append_decode(name):
    cc = CacheCase(name)
    g = cc.g
    c = cc.oracle_freeze()
    assert [c.k_quant_packed.shape[1], c.k_topk.shape[1], c.k_window.shape[1]] == list(g["frozen_shapes"])
    assert sha(c.k_quant_packed) == g["frozen_k_packed_sha"][0]
    assert sha(c.v_quant_packed) == g["frozen_v_packed_sha"][0]
    assert np.array_equal(c.k_scale.view(np.uint16), g["frozen_k_scale"].view(np.uint16))
    assert np.array_equal(c.v_scale.view(np.uint16), g["frozen_v_scale"].view(np.uint16))
    assert sha(c.k_topk.astype(np.float32)) == g["frozen_k_topk_sha"][0]
    tol = 2e-2 if cc.is_bf16 else 2e-5
    for step in range(1, cc.n_append + 1):
        orc.append_staging(c, cc.new_k[step - 1], cc.new_v[step - 1])
        if step in cc.probe_steps:
            assert [c.k_quant_packed.shape[1], c.staging_ptr] == list(g[f"state_step{step}"])
            ref = g[f"out_step{step}"]
            out = orc.decode_attention_fallback(cc.new_q[step - 1], c, cc.R, round_fn=cc.round_fn)
            assert max_abs(out, ref) < tol, (step, max_abs(out, ref))
            exact = orc.decode_attention_exact(cc.new_q[step - 1], c, cc.R)
            assert max_abs(exact, ref) < 2e-2
            assert orc.rel_mse(exact, ref) < 1e-4
    assert sha(c.k_quant_packed) == g["final_k_packed_sha"][0]
    assert sha(c.v_quant_packed) == g["final_v_packed_sha"][0]
    assert sha(c.k_scale) == g["final_k_scale_sha"][0]
    assert sha(c.v_scale) == g["final_v_scale_sha"][0]


def test_vertical_indices():
    from hyquant_b200.synth import gen_numpy
    g = load("vertical_indices")
    B, H_Q, H_KV, N, W, seed = [int(x) for x in g["meta"]]
    case = gen_numpy(B, H_Q, H_KV, N, 128, W, float(g["rho"][0]), seed)
    assert [sha(case.q), sha(case.k)] == list(g["in_sha"])
    R = H_Q // H_KV
    assert np.array_equal(orc.compute_vertical_indices(case.q, case.k, W, 0.05, kv_repeat=R), g["idx_gqa"])
    assert np.array_equal(orc.compute_vertical_indices(case.q, np.repeat(case.k, R, axis=1), W, 0.05), g["idx_plain"])
    pooled = case.q[:, :, -256:, :].mean(axis=2, keepdims=True)
    assert np.array_equal(orc.compute_vertical_indices(pooled, case.k, W, 0.05, kv_repeat=R), g["idx_pool"])


def test_reorder_kv_for_vertical():
    g = load("reorder_kv")
    kr, vr, kv, vv, nr, nv, R, V = orc.reorder_kv_for_vertical(g["k"], g["v"], g["vidx"], int(g["window"][0]))
    assert [R, V] == list(g["RV"])
    for a, b in ((kr, "k_rest"), (vr, "v_rest"), (kv, "k_vert"), (vv, "v_vert"), (nr, "n_rest_valid"), (nv, "n_vert_valid")):
        assert np.array_equal(a, g[b]), b


def test_lse_merge_matches_single_pass():
    rng = np.random.Generator(np.random.PCG64(3))
    q = rng.standard_normal((4, 128)); k = rng.standard_normal((300, 128)); v = rng.standard_normal((300, 128))
    sm = 128 ** -0.5
    full = orc.decode_partials(q, k, v, sm)
    ref = full[2] / full[1][..., None]
    cuts = [0, 1, 130, 130, 300]             # includes an empty shard
    parts = [orc.decode_partials(q, k[a:b], v[a:b], sm) for a, b in zip(cuts[:-1], cuts[1:])]
    m = np.stack([p[0] for p in parts]); l = np.stack([p[1] for p in parts]); acc = np.stack([p[2] for p in parts])
    assert max_abs(orc.lse_merge(m, l, acc), ref) < 1e-12


def test_hybrid_prefill_restatement_close_to_dense():
    from hyquant_b200.synth import gen_numpy
    case = gen_numpy(1, 4, 2, 512, 128, 128, 0.05, 41)
    q, k, v = orc.bf16_round(case.q), orc.bf16_round(case.k), orc.bf16_round(case.v)
    vidx = orc.compute_vertical_indices(q, k, 128, 0.05, kv_repeat=2)
    out = orc.hybrid_prefill_reference(q, k, v, vidx, window_size=128, round_fn=orc.bf16_round)
    ref = orc.dense_causal_attention(q, k, v)
    assert max_abs(out, ref) < 2e-2
    assert orc.rel_mse(out, ref) < 1e-4


def test_torch_cpu_baseline_matches_fixture():
    """The torch-CPU restatement that bench.py times agrees with the reference's outputs."""
    import torch
    from oracle import hq_oracle_torch as ot
    cc = CacheCase("cache_cfg0_f32")
    c = cc.oracle_freeze()
    for step in range(1, cc.n_append + 1):
        orc.append_staging(c, cc.new_k[step - 1], cc.new_v[step - 1])
    out = ot.decode_attention_fallback(torch.from_numpy(cc.new_q[cc.n_append - 1]), *ot.from_numpy_cache(c), cc.B, cc.H_KV, cc.R)
    assert max_abs(out.numpy(), cc.g[f"out_step{cc.n_append}"]) < 2e-5
