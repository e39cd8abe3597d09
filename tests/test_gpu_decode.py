"""GPU parity tests of the decode path: CUDA kernels (through the C ABI) against
the CPU oracle on the same seeded inputs, against the golden fixtures produced
by executing the reference, and size-independent properties at full size.

Tolerances (stated by the build target): INT4 codes, fp16 scales and top-k
indices bit-exact; attention outputs max-abs <= 2e-2 and rel-MSE <= 1e-4.
"""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import decode_d_stage as dd
from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc
from tests.helpers import CacheCase, load, max_abs, sha

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_ABS, REL_MSE = 2e-2, 1e-4


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def to_np(t):
    return t.detach().float().cpu().numpy()


# ---------------------------------------------------------------- quantiser

@pytest.mark.parametrize("nbits", [2, 4, 8])
def test_quantize_matches_reference_fixture_bit_exact(nbits):
    g = load("quant_per_token")
    x = orc.bf16_bits_to_f32(g["x_bf16_bits"])
    p, s = hq.quantize_per_token(t_bf16(x), nbits)
    assert np.array_equal(p.cpu().numpy(), g[f"bf16_packed{nbits}"])
    assert np.array_equal(s.cpu().numpy().view(np.uint16), g[f"bf16_scale{nbits}"].view(np.uint16))
    p32, s32 = hq.quantize_per_token(torch.from_numpy(g["x_f32"]).to(DEV), nbits)
    assert np.array_equal(p32.cpu().numpy(), g[f"f32_packed{nbits}"])
    assert np.array_equal(s32.cpu().numpy().view(np.uint16), g[f"f32_scale{nbits}"].view(np.uint16))
    deq = hq.dequantize_per_token(p, s, 128, nbits)
    # a row whose scale overflows fp16 dequantises to 0 * inf = NaN on both sides (the NaN's sign bit is free)
    assert np.array_equal(deq.cpu().numpy(), g[f"bf16_deq{nbits}"], equal_nan=True)


@pytest.mark.parametrize("nbits", [2, 4, 8])
@pytest.mark.parametrize("shape", [(1, 1, 128), (8, 128, 128), (3, 1000, 128), (128, 128, 128)])
def test_quantize_matches_oracle_bit_exact(shape, nbits):
    rng = np.random.Generator(np.random.PCG64(shape[1]))
    x = orc.bf16_round(rng.standard_normal(shape, dtype=np.float32) * rng.uniform(0.01, 30, shape[:2] + (1,)).astype(np.float32))
    p, s = hq.quantize_per_token(t_bf16(x), nbits)
    po, so = orc.quantize_per_token(x, nbits)
    assert np.array_equal(p.cpu().numpy(), po)
    assert np.array_equal(s.cpu().numpy().view(np.uint16), so.view(np.uint16))
    # CUDA-eager scale rounding mode
    BH, n, _ = shape
    pk = torch.empty(BH, n, 16 * nbits, dtype=torch.int8, device=DEV); sc = torch.empty(BH, n, dtype=torch.float16, device=DEV)
    dd.quantize_per_token_into(t_bf16(x), pk, sc, 0, scale_mode=1, nbits=nbits)
    po1, so1 = orc.quantize_per_token(x, nbits, reciprocal_scale=True)
    assert np.array_equal(pk.cpu().numpy(), po1) and np.array_equal(sc.cpu().numpy().view(np.uint16), so1.view(np.uint16))


@pytest.mark.parametrize("nbits", [2, 4, 8])
def test_quantize_ties_and_near_ties_bit_exact(nbits):
    """Quotients x / scale on a half-integer, and one to three units in the last place beside it: where rounding the
    product with the reciprocal could differ from rounding the IEEE quotient, the kernel has to take the division.
    fp32 inputs, scales that are exact in fp16 (the row maximum is q_max times the scale)."""
    qmax = 2 ** (nbits - 1) - 1
    rng = np.random.Generator(np.random.PCG64(nbits))
    rows = []
    for s in [1.0, 0.5, 0.333251953125, 3.0517578125e-05, 1023.5, 0.0999755859375, 7.152557373046875e-07 * 64]:
        s = np.float32(np.float16(s))
        for rep in range(4):
            row = np.zeros(128, dtype=np.float32)
            row[0] = np.float32(qmax) * s                      # pins the scale (exactly q_max * s)
            ks = rng.integers(-qmax - 1, qmax, size=127).astype(np.float32) + np.float32(0.5)
            x = (ks * s).astype(np.float32)                    # quotient = k + 0.5 (exact for these scales where the product is exact)
            ulps = rng.integers(-3, 4, size=127)
            bits_ = x.view(np.int32) + ulps.astype(np.int32)   # a few units in the last place beside the tie
            row[1:] = bits_.view(np.float32)
            row[1:] = np.clip(row[1:], -row[0], row[0])        # keep row[0] the maximum
            rows.append(row)
    x = np.stack(rows)[None]                                   # [1, n, 128]
    for mode in (0, 1):
        pk = torch.empty(1, x.shape[1], 16 * nbits, dtype=torch.int8, device=DEV)
        sc = torch.empty(1, x.shape[1], dtype=torch.float16, device=DEV)
        dd.quantize_per_token_into(torch.from_numpy(x).to(DEV), pk, sc, 0, scale_mode=mode, nbits=nbits)
        po, so = orc.quantize_per_token(x, nbits, reciprocal_scale=bool(mode))
        assert np.array_equal(sc.cpu().numpy().view(np.uint16), so.view(np.uint16))
        assert np.array_equal(pk.cpu().numpy(), po)


def test_quantize_empty_and_append_offset():
    p, s = hq.quantize_per_token(torch.zeros(4, 0, 128, dtype=torch.bfloat16, device=DEV), 4)
    assert p.shape == (4, 0, 64) and s.shape == (4, 0)
    rng = np.random.Generator(np.random.PCG64(2))
    x = orc.bf16_round(rng.standard_normal((2, 128, 128), dtype=np.float32))
    pk = torch.full((2, 512, 64), 0x55, dtype=torch.int8, device=DEV)
    sc = torch.full((2, 512), 9.0, dtype=torch.float16, device=DEV)
    dd.quantize_per_token_into(t_bf16(x), pk, sc, 256)
    po, so = orc.quantize_per_token(x, 4)
    assert np.array_equal(pk[:, 256:384].cpu().numpy(), po)
    assert np.array_equal(sc[:, 256:384].cpu().numpy().view(np.uint16), so.view(np.uint16))
    assert (pk[:, :256] == 0x55).all() and (pk[:, 384:] == 0x55).all() and (sc[:, :256] == 9).all()
    with pytest.raises(hq.HyQuantError):
        dd.quantize_per_token_into(t_bf16(x), pk, sc, 400)


# ---------------------------------------------------------- decode attention

def build_case(BH_KV, R, n_quant, n_topk, n_staging, n_window, seed, k_bits=4, v_bits=4):
    """Random four-segment cache (numpy, bf16-exact) + query; oracle LayerCache."""
    rng = np.random.Generator(np.random.PCG64(seed))
    D = 128
    def rnd(n, scale=1.0):
        a = rng.standard_normal((BH_KV, n, D), dtype=np.float32) * scale
        a[..., 5] += 4.0
        return orc.bf16_round(a)
    kq, ks = orc.quantize_per_token(rnd(n_quant), k_bits)
    vq, vs = orc.quantize_per_token(rnd(n_quant), v_bits)
    c = orc.LayerCache(B=1, H_KV=BH_KV, D=D, k_bits=k_bits, v_bits=v_bits, k_quant_packed=kq, v_quant_packed=vq,
                       k_scale=ks, v_scale=vs, k_topk=rnd(n_topk), v_topk=rnd(n_topk),
                       k_window=rnd(n_window), v_window=rnd(n_window),
                       staging_k=rnd(128), staging_v=rnd(128), staging_ptr=n_staging)
    q = orc.bf16_round(rng.standard_normal((1, BH_KV * R, 1, D), dtype=np.float32))
    return c, q


def run_gpu(c, q, R, **kw):
    ti8 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    S = c.staging_ptr
    args = (t_bf16(q.reshape(-1, 128)), ti8(c.k_quant_packed), ti8(c.v_quant_packed), ti8(c.k_scale), ti8(c.v_scale),
            t_bf16(c.k_topk), t_bf16(c.v_topk), t_bf16(c.staging_k)[:, :S], t_bf16(c.staging_v)[:, :S],
            t_bf16(c.k_window), t_bf16(c.v_window))
    if kw:
        plan = dd.DecodePlan(*args, R, None, k_bits=c.k_bits, v_bits=c.v_bits, **kw)
        out = plan.run(args[0])
        ws = plan.ws
    else:
        out = hq.fused_d_stage_decode(*args, c.k_bits, c.v_bits, kv_repeat=R)
        ws = dd.decode_workspace(torch.device(DEV, torch.cuda.current_device()), c.H_KV, R)
    torch.cuda.synchronize()
    assert dd.decode_status(ws) == 0
    return to_np(out)


def check_close(out, ref):
    assert np.isfinite(out).all()
    assert max_abs(out, ref) <= MAX_ABS, max_abs(out, ref)
    assert orc.rel_mse(out, ref) <= REL_MSE, orc.rel_mse(out, ref)


@pytest.mark.parametrize("n_quant", [0, 1, 31, 32, 33, 127, 128, 129, 511, 512, 513, 4113])
@pytest.mark.parametrize("n_staging", [0, 1, 127])
def test_decode_edge_lengths(n_quant, n_staging):
    c, q = build_case(2, 4, n_quant, 3 if n_quant else 0, n_staging, 128, seed=n_quant * 131 + n_staging)
    ref = orc.decode_attention_exact(q, c, 4).reshape(-1, 128)
    check_close(run_gpu(c, q, 4), ref)


@pytest.mark.parametrize("bits", [(8, 8), (4, 2), (2, 4), (8, 4), (2, 2), (4, 8), (8, 2), (2, 8)])
@pytest.mark.parametrize("R,lens", [(4, (700, 37, 5, 64)), (1, (33, 0, 0, 1)), (8, (0, 9, 127, 128)), (16, (4113, 300, 1, 128)),
                                    (7, (1, 0, 0, 0))])
def test_decode_other_bit_widths(bits, R, lens):
    """Every (k_bits, v_bits) pair other than 4/4 (one instantiation of the split-K kernel each): all segment
    combinations, GQA ratios up to 16, split invariance and the un-normalised partial mode."""
    kb, vb = bits
    nq, nt, ns, nw = lens
    c, q = build_case(3, R, nq, nt, ns, nw, seed=kb * 100 + vb * 10 + R, k_bits=kb, v_bits=vb)
    ref = orc.decode_attention_exact(q, c, R).reshape(-1, 128)
    out = run_gpu(c, q, R)
    check_close(out, ref)
    one = run_gpu(c, q, R, num_splits=1)
    check_close(one, ref)
    assert np.all(np.abs(out - one) <= 2e-3 + 2.0 ** -7 * np.abs(one))      # fp32 summation order, then one bf16 rounding
    # partial mode: (m, l, acc) of the whole cache, normalised on the host
    ti8 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    S = c.staging_ptr
    plan = dd.DecodePlan(t_bf16(q.reshape(-1, 128)), ti8(c.k_quant_packed), ti8(c.v_quant_packed), ti8(c.k_scale), ti8(c.v_scale),
                         t_bf16(c.k_topk), t_bf16(c.v_topk), t_bf16(c.staging_k)[:, :S], t_bf16(c.staging_v)[:, :S],
                         t_bf16(c.k_window), t_bf16(c.v_window), R, None, k_bits=kb, v_bits=vb)
    rows = 3 * R
    m = torch.empty(rows, device=DEV); l = torch.empty(rows, device=DEV); acc = torch.empty(rows, 128, device=DEV)
    plan.run(t_bf16(q.reshape(-1, 128)), partial=(m, l, acc))
    check_close((acc / l[:, None]).cpu().numpy(), ref)


@pytest.mark.parametrize("R", [1, 2, 4, 7, 8, 16])
def test_decode_gqa_ratios(R):
    c, q = build_case(3, R, 700, 37, 5, 64, seed=R)
    ref = orc.decode_attention_exact(q, c, R).reshape(-1, 128)
    check_close(run_gpu(c, q, R), ref)


@pytest.mark.parametrize("segs", [(300, 0, 0, 128), (300, 45, 0, 0), (0, 0, 0, 1), (0, 0, 1, 0), (0, 9, 0, 0), (64, 1, 1, 1)])
def test_decode_empty_segments(segs):
    c, q = build_case(2, 4, *segs, seed=sum(segs))
    ref = orc.decode_attention_exact(q, c, 4).reshape(-1, 128)
    check_close(run_gpu(c, q, 4), ref)


@pytest.mark.parametrize("R,heads,nq", [(4, 8, 900), (4, 8, 1900), (4, 8, 3400), (8, 4, 2500), (16, 8, 1100), (16, 2, 2300),
                                        (4, 32, 20000), (1, 64, 9000)])
def test_decode_cluster_merge_against_workspace_merge(R, heads, nq):
    """Shapes whose automatic plan has 2 to 8 splits per head: the splits of a head run as one thread-block cluster
    and merge through distributed shared memory.  Same result as the workspace merge with as many explicit splits
    (fp32 summation order apart), and as the oracle."""
    c, q = build_case(heads, R, nq, 40, 17, 128, seed=heads * 1000 + nq)
    ref = orc.decode_attention_exact(q, c, R).reshape(-1, 128)
    out = run_gpu(c, q, R)
    check_close(out, ref)
    for s in (2, 3, 5, 8):
        plain = run_gpu(c, q, R, num_splits=s)
        assert np.all(np.abs(out - plain) <= 2e-3 + 2.0 ** -7 * np.abs(plain))


def test_decode_split_invariance_and_partials():
    c, q = build_case(4, 4, 5000, 250, 77, 128, seed=9)
    ref = orc.decode_attention_exact(q, c, 4).reshape(-1, 128)
    outs = [run_gpu(c, q, 4, num_splits=s) for s in (1, 2, 7, 33)]
    for o in outs:
        check_close(o, ref)
        assert max_abs(o, outs[0]) < 2e-2
    # partial mode of two "shards" (prefix | everything else) merged == single pass
    import copy
    a, b = copy.copy(c), copy.copy(c)
    a.k_topk = a.v_topk = np.zeros((4, 0, 128), np.float32); a.k_window = a.v_window = np.zeros((4, 0, 128), np.float32)
    a.staging_ptr = 0
    b.k_quant_packed = b.v_quant_packed = np.zeros((4, 0, 64), np.int8); b.k_scale = b.v_scale = np.zeros((4, 0), np.float16)
    ms, ls, accs = [], [], []
    for sh in (a, b):
        ti8 = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(DEV)
        S = sh.staging_ptr
        plan = dd.DecodePlan(t_bf16(q.reshape(-1, 128)), ti8(sh.k_quant_packed), ti8(sh.v_quant_packed), ti8(sh.k_scale),
                             ti8(sh.v_scale), t_bf16(sh.k_topk), t_bf16(sh.v_topk), t_bf16(sh.staging_k)[:, :S],
                             t_bf16(sh.staging_v)[:, :S], t_bf16(sh.k_window), t_bf16(sh.v_window), 4, None)
        m = torch.empty(16, dtype=torch.float32, device=DEV); l = torch.empty_like(m)
        acc = torch.empty(16, 128, dtype=torch.float32, device=DEV)
        plan.run(t_bf16(q.reshape(-1, 128)), partial=(m, l, acc))
        ms.append(m); ls.append(l); accs.append(acc)
    merged = hq.lse_merge(torch.stack(ms), torch.stack(ls), torch.stack(accs), out_dtype=torch.float32)
    check_close(to_np(merged), ref)
    # the merge kernel against the oracle's algebra on the same partials
    om = orc.lse_merge(to_np(torch.stack(ms)).astype(np.float64), to_np(torch.stack(ls)).astype(np.float64),
                       to_np(torch.stack(accs)).astype(np.float64))
    assert max_abs(to_np(merged), om) < 1e-5


def test_decode_strided_inputs_and_out_dtypes():
    c, q = build_case(2, 4, 300, 10, 3, 64, seed=4)
    ref = orc.decode_attention_exact(q, c, 4).reshape(-1, 128)
    ti8 = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    kq = torch.zeros(2, 600, 64, dtype=torch.int8, device=DEV); kq[:, :300] = ti8(c.k_quant_packed)
    vq = torch.zeros(2, 600, 64, dtype=torch.int8, device=DEV); vq[:, :300] = ti8(c.v_quant_packed)
    ks = torch.zeros(2, 777, dtype=torch.float16, device=DEV); ks[:, :300] = ti8(c.k_scale)
    vs = torch.zeros(2, 777, dtype=torch.float16, device=DEV); vs[:, :300] = ti8(c.v_scale)
    for qdt in (torch.bfloat16, torch.float32, torch.float16):
        qq = torch.from_numpy(q.reshape(-1, 128)).to(DEV).to(qdt)
        out = hq.fused_d_stage_decode(qq, kq[:, :300], vq[:, :300], ks[:, :300], vs[:, :300], t_bf16(c.k_topk), t_bf16(c.v_topk),
                                      t_bf16(c.staging_k)[:, :3], t_bf16(c.staging_v)[:, :3], t_bf16(c.k_window),
                                      t_bf16(c.v_window), 4, 4, kv_repeat=4)
        assert out.dtype == qdt and out.shape == (8, 128)
        check_close(to_np(out), ref)


@pytest.mark.parametrize("name", ["cache_cfg0_f32", "cache_small_bf16", "cache_tiny_f32", "cache_short_f32",
                                  "cache_k8v8_f32", "cache_k4v2_f32", "cache_k2v4_f32"])
def test_cache_lifecycle_against_reference_fixture(name):
    """prefill -> freeze -> appends with flushes -> decode through the reference-named
    cache class.  bf16 fixtures: compared with the reference's outputs directly (its
    vertical selection is taken as given, bf16 scores tie).  fp32 fixtures: the device
    path is bf16, so inputs are rounded to bf16 and compared with the pinned oracle."""
    cc = CacheCase(name)
    g = cc.g
    rb = orc.bf16_round
    k, v, qt = rb(cc.k), rb(cc.v), rb(cc.query_tail)
    cache = hq.DStageKVCache(num_layers=1, k_bits=cc.k_bits, v_bits_fn=lambda i: cc.v_bits, window_size=cc.W, top_ratio=cc.rho)
    layer = cache.get_layer(0)
    cache.update(t_bf16(k), t_bf16(v), 0)
    layer.save_query_tail(t_bf16(cc.q))
    if cc.is_bf16:
        layer.freeze(kv_repeat=cc.R, vertical_indices=torch.from_numpy(g["frozen_vidx"]))
        oc = cc.oracle_freeze()
        assert sha(layer.k_quant_packed.cpu().numpy()) == g["frozen_k_packed_sha"][0]
        assert sha(layer.v_quant_packed.cpu().numpy()) == g["frozen_v_packed_sha"][0]
        assert np.array_equal(layer.k_scale.cpu().numpy().view(np.uint16), g["frozen_k_scale"].view(np.uint16))
        assert sha(to_np(layer.k_topk)) == g["frozen_k_topk_sha"][0]
    else:
        layer.freeze(kv_repeat=cc.R)
        own = orc.freeze(k, v, qt, cc.R, cc.W, cc.rho, k_bits=cc.k_bits, v_bits=cc.v_bits, round_fn=rb)
        gv = None if layer.vertical_indices is None else layer.vertical_indices.cpu().numpy()
        if own.vidx is not None and own.vidx.shape[-1] > 0:
            # the device scores differ from the oracle's in the last bits, which may swap
            # near-ties: require the same set up to 2%, then hand the device's selection to
            # the oracle so that everything downstream is compared bit-exactly
            for a, b in zip(gv.reshape(-1, gv.shape[-1]), own.vidx.reshape(-1, gv.shape[-1])):
                assert len(set(a.tolist()) & set(b.tolist())) >= 0.98 * len(a) - 1
        oc = orc.freeze(k, v, qt, cc.R, cc.W, cc.rho, k_bits=cc.k_bits, v_bits=cc.v_bits, round_fn=rb, vidx_override=gv)
        assert np.array_equal(layer.k_quant_packed.cpu().numpy(), oc.k_quant_packed)
        assert np.array_equal(layer.v_quant_packed.cpu().numpy(), oc.v_quant_packed)
        assert np.array_equal(layer.k_scale.cpu().numpy().view(np.uint16), oc.k_scale.view(np.uint16))
        assert np.array_equal(to_np(layer.k_topk), oc.k_topk) and np.array_equal(to_np(layer.v_topk), oc.v_topk)
    assert [layer.k_quant_packed.shape[1], layer.k_topk.shape[1], layer.k_window.shape[1]] == list(g["frozen_shapes"])
    assert np.array_equal(to_np(layer.k_window), oc.k_window) and layer.phase == "decode"
    nk, nv, nq = rb(cc.new_k), rb(cc.new_v), rb(cc.new_q)
    for step in range(1, cc.n_append + 1):
        cache.update(t_bf16(nk[step - 1]), t_bf16(nv[step - 1]), 0)
        orc.append_staging(oc, nk[step - 1], nv[step - 1])
        if step in cc.probe_steps:
            assert [layer.k_quant_packed.shape[1], layer._staging_ptr] == list(g[f"state_step{step}"])
            out = to_np(layer.decode_attention(t_bf16(nq[step - 1]), cc.R))
            assert out.shape == (cc.B, cc.H_Q, 1, 128)
            check_close(out, orc.decode_attention_exact(nq[step - 1], oc, cc.R))
            check_close(out, orc.decode_attention_fallback(nq[step - 1], oc, cc.R))
            if cc.is_bf16:
                check_close(out, g[f"out_step{step}"])          # the reference's own output
    assert cache.get_seq_length() == cc.N + cc.n_append
    assert np.array_equal(layer.k_quant_packed.cpu().numpy(), oc.k_quant_packed)
    assert np.array_equal(layer.v_quant_packed.cpu().numpy(), oc.v_quant_packed)
    assert np.array_equal(layer.v_scale.cpu().numpy().view(np.uint16), oc.v_scale.view(np.uint16))
    if cc.is_bf16:
        assert sha(layer.k_quant_packed.cpu().numpy()) == g["final_k_packed_sha"][0]
        assert sha(layer.k_scale.cpu().numpy()) == g["final_k_scale_sha"][0]
    cache.reset()
    assert cache.get_seq_length() == 0 and cache.get_layer(0).phase == "prefill"


def test_cache_growth_beyond_initial_capacity():
    case = gen_numpy(1, 4, 1, 300, 128, 64, 0.05, 3)
    rb = orc.bf16_round
    k, v, q = rb(case.k), rb(case.v), rb(case.q)
    layer = hq.DStageLayerCache(0, window_size=64, top_ratio=0.05)
    layer.update_prefill(t_bf16(k), t_bf16(v)); layer.save_query_tail(t_bf16(q)); layer.freeze(kv_repeat=4)
    oc = orc.freeze(k, v, q[:, :, -64:], 4, 64, 0.05, round_fn=rb)
    rng = np.random.Generator(np.random.PCG64(8))
    n = 128 * 12 + 5    # forces at least one re-allocation of the capacity buffers
    for step in range(n):
        kk = rb(rng.standard_normal((1, 1, 1, 128), dtype=np.float32)); vv = rb(rng.standard_normal((1, 1, 1, 128), dtype=np.float32))
        layer.append_staging(t_bf16(kk), t_bf16(vv)); orc.append_staging(oc, kk, vv)
    assert np.array_equal(layer.k_quant_packed.cpu().numpy(), oc.k_quant_packed)
    qd = rb(case.q_decode)
    check_close(to_np(layer.decode_attention(t_bf16(qd), 4)), orc.decode_attention_exact(qd, oc, 4))


def test_unsupported_configurations_fail_loudly(monkeypatch):
    layer = hq.DStageLayerCache(0, k_bits=3, v_bits=8, window_size=64)       # widths are 2, 4 or 8
    layer.update_prefill(torch.zeros(1, 1, 100, 128, dtype=torch.bfloat16, device=DEV),
                         torch.zeros(1, 1, 100, 128, dtype=torch.bfloat16, device=DEV))
    with pytest.raises(hq.HyQuantError):
        layer.freeze(kv_repeat=1)
    c, q = build_case(1, 4, 64, 0, 1, 8, seed=1)
    layer = hq.DStageLayerCache(0, window_size=8, use_vert=False)
    layer.update_prefill(t_bf16(np.zeros((1, 1, 40, 128))), t_bf16(np.zeros((1, 1, 40, 128)))); layer.freeze(4)
    monkeypatch.setenv("HYBRID_ATTN_DECODE_KERNEL", "pytorch")
    with pytest.raises(hq.HyQuantError):
        layer.decode_attention(t_bf16(q), 4)


# ------------------------------------------------- full-size properties (32K)

def test_full_size_split_and_shard_invariance():
    """BASELINE decode shape (32q/8kv, 32K prefix, W=128, rho=5%): results do not
    depend on the split count, and a 4-way sequence sharding merged with the LSE
    kernel equals the single pass."""
    g = torch.Generator(device=DEV); g.manual_seed(1015)
    BH, R, N = 8, 4, 32768
    T = 1632; nq = N - 128 - T
    kv = torch.randn(2, BH, nq, 128, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    kq, ks = hq.quantize_per_token(kv[0], 4); vq, vs = hq.quantize_per_token(kv[1], 4)
    bf = lambda n: torch.randn(BH, n, 128, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    kt, vt, kw, vw, kst, vst = bf(T), bf(T), bf(128), bf(128), bf(128), bf(128)
    q = torch.randn(BH * R, 128, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    full = hq.fused_d_stage_decode(q, kq, vq, ks, vs, kt, vt, kst[:, :64], vst[:, :64], kw, vw, 4, 4, kv_repeat=R).float()
    one = dd.DecodePlan(q, kq, vq, ks, vs, kt, vt, kst[:, :64], vst[:, :64], kw, vw, R, None, num_splits=1).run(q).float()
    assert (full - one).abs().max().item() < 1e-2
    # fp32 dense reference on the dequantised cache (torch, on device) as yardstick
    kd = torch.cat([dd._unpack_int4(kq, 128) * ks.float()[..., None], kt.float(), kst[:, :64].float(), kw.float()], 1)
    vd = torch.cat([dd._unpack_int4(vq, 128) * vs.float()[..., None], vt.float(), vst[:, :64].float(), vw.float()], 1)
    sc = torch.einsum("hrd,hnd->hrn", q.float().reshape(BH, R, 128), kd) * 128 ** -0.5
    ref = torch.einsum("hrn,hnd->hrd", torch.softmax(sc, -1), vd).reshape(BH * R, 128)
    assert (full - ref).abs().max().item() <= MAX_ABS
    assert ((full - ref) ** 2).sum().item() / (ref ** 2).sum().item() <= REL_MSE
    G = 4
    ms, ls, accs = [], [], []
    qb = [(i * nq // G) // 128 * 128 for i in range(G)] + [nq]
    tb = [i * T // G for i in range(G)] + [T]
    for r in range(G):
        last = r == G - 1
        e = kw[:, :0]
        plan = dd.DecodePlan(q, kq[:, qb[r]:qb[r + 1]], vq[:, qb[r]:qb[r + 1]], ks[:, qb[r]:qb[r + 1]].contiguous(),
                             vs[:, qb[r]:qb[r + 1]].contiguous(), kt[:, tb[r]:tb[r + 1]], vt[:, tb[r]:tb[r + 1]],
                             kst[:, :64] if last else e, vst[:, :64] if last else e, kw if last else e, vw if last else e, R, None)
        m = torch.empty(BH * R, dtype=torch.float32, device=DEV); l = torch.empty_like(m)
        acc = torch.empty(BH * R, 128, dtype=torch.float32, device=DEV)
        plan.run(q, partial=(m, l, acc)); ms.append(m); ls.append(l); accs.append(acc)
    merged = hq.lse_merge(torch.stack(ms), torch.stack(ls), torch.stack(accs), out_dtype=torch.float32)
    assert (merged - ref).abs().max().item() <= MAX_ABS
    assert (merged - full).abs().max().item() < 1e-2


@pytest.mark.parametrize("world", [2, 3, 8])
def test_sequence_shards_of_a_layer_merge_to_the_full_result(world):
    """`shard_layer_sequence` splits a frozen layer cache into per-rank caches; decoding every shard in
    partial mode (all on this one GPU, one after the other) and merging equals the unsharded decode,
    before and after a staging flush on the tail rank."""
    import hyquant_b200 as hq
    from hyquant_b200 import sharded
    from hyquant_b200.decode_d_stage import lse_merge
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV, N, W = 2, 8, 2, 4096 + 77, 128
    R = H_Q // H_KV
    t = gen_torch(B, H_Q, H_KV, N, 128, W, 0.05, 321, n_qry=W, device="cuda")
    full = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=0.05, use_vert=True)
    full.update_prefill(t["k"], t["v"])
    full.save_query_tail(t["q"])
    full.freeze(kv_repeat=R)
    g = torch.Generator(device="cuda").manual_seed(5)
    new = [(torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16(),
            torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()) for _ in range(140)]
    for kn, vn in new[:9]:
        full.append_staging(kn, vn)
    shards = [sharded.shard_layer_sequence(full, world, r) for r in range(world)]
    plan = sharded.sequence_shard_plan(full._n_quant, full.k_topk.shape[1], world)
    assert sum(s._n_quant for s in shards) == full._n_quant and plan[0][0] == 0
    assert sum(s.k_topk.shape[1] for s in shards) == full.k_topk.shape[1]
    q = t["q_decode"]
    rows = B * H_Q

    def sharded_decode():
        m = torch.empty(world, rows, device="cuda"); l = torch.empty_like(m)
        acc = torch.empty(world, rows, 128, device="cuda")
        for r, s in enumerate(shards):
            s.decode_attention(q, R, partial=(m[r], l[r], acc[r]))
        return lse_merge(m, l, acc, out_dtype=q.dtype).reshape(B, H_Q, 1, 128)

    want = full.decode_attention(q, R)
    got = sharded_decode()
    assert float((got.float() - want.float()).abs().max()) <= 2e-2 * 0.25
    for kn, vn in new[9:]:                      # crosses one flush of 128 tokens
        full.append_staging(kn, vn)
        shards[-1].append_staging(kn, vn)
    assert shards[-1]._n_quant == plan[-1][1] - plan[-1][0] + 128 and shards[-1]._staging_ptr == full._staging_ptr
    want = full.decode_attention(q, R)
    got = sharded_decode()
    assert float((got.float() - want.float()).abs().max()) <= 2e-2 * 0.25


def test_overlapped_launch_equals_plain_launch():
    """HQ_DECODE_OVERLAP_PREVIOUS changes when a call's blocks start, not what they compute.  Two identical
    layer caches take the same 300 appended tokens (two staging flushes); one decodes with plain launches,
    the other with launches that may overlap the kernel before them (the staging append or the flush)."""
    import hyquant_b200 as hq
    from hyquant_b200.decode_d_stage import decode_status
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV, N, W = 1, 32, 8, 8192 + 5, 128
    R = H_Q // H_KV
    t = gen_torch(B, H_Q, H_KV, N, 128, W, 0.05, 99, n_qry=W, device="cuda")
    layers = []
    for overlap in (False, True):
        layer = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=0.05, use_vert=True)
        layer.overlap_previous = overlap
        layer.update_prefill(t["k"], t["v"])
        layer.save_query_tail(t["q"])
        layer.freeze(kv_repeat=R)
        layers.append(layer)
    g = torch.Generator(device="cuda").manual_seed(11)
    for step in range(300):
        kn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        vn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        qn = torch.randn(B, H_Q, 1, 128, generator=g, device="cuda").bfloat16()
        outs = []
        for layer in layers:
            layer.append_staging(kn, vn)
            outs.append(layer.decode_attention(qn, R).clone())
        assert torch.equal(outs[0], outs[1]), f"step {step}"
    assert layers[1]._plan.args.flags == 1 and layers[0]._plan.args.flags == 0
    assert decode_status(layers[1]._plan.ws) == 0


def test_overlapped_launches_back_to_back_in_a_graph():
    """A captured sequence of overlapped decode launches over different caches (the bench's launch pattern)
    replays to the same outputs as plain launches."""
    import hyquant_b200 as hq
    from hyquant_b200.decode_d_stage import decode_status
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV, W = 1, 32, 8, 128
    R = H_Q // H_KV
    plans, qs, want = [], [], []
    for i, n in enumerate((1024, 4096 + 33, 16384, 700, 32768)):
        t = gen_torch(B, H_Q, H_KV, n, 128, W, 0.05, 500 + i, n_qry=W, device="cuda")
        layer = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=0.05, use_vert=True)
        layer.update_prefill(t["k"], t["v"])
        layer.save_query_tail(t["q"])
        layer.freeze(kv_repeat=R)
        for j in range(3 + i):
            layer.append_staging(t["k"][:, :, j:j + 1].contiguous(), t["v"][:, :, j:j + 1].contiguous())
        q2 = t["q_decode"].reshape(-1, 128)
        plan = layer._decode_plan(q2, R)
        plan.args.flags = 0
        want.append(plan.run(q2).clone())
        plans.append((layer, plan)); qs.append(q2)
    torch.cuda.synchronize()
    outs = [torch.zeros_like(w) for w in want]
    for _, plan in plans:
        plan.args.flags = 1
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        for _ in range(2):
            for (_, plan), q2, o in zip(plans, qs, outs):
                plan.run(q2, out=o)
    s.synchronize()
    for o, w in zip(outs, want):
        assert torch.equal(o, w)
    for o in outs:
        o.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for (_, plan), q2, o in zip(plans, qs, outs):
            plan.run(q2, out=o)
    for _ in range(3):
        graph.replay()
    torch.cuda.synchronize()
    for o, w in zip(outs, want):
        assert torch.equal(o, w)
    assert decode_status(plans[0][1].ws) == 0


def _dense_yardstick(q, kq, vq, ks, vs, segs, R, heads):
    """fp32 attention over the dequantised cache of a few kv heads (torch, on the device)."""
    kd = torch.cat([dd._unpack_int4(kq[heads], 128) * ks[heads].float()[..., None]] + [s[0][heads].float() for s in segs], 1)
    vd = torch.cat([dd._unpack_int4(vq[heads], 128) * vs[heads].float()[..., None]] + [s[1][heads].float() for s in segs], 1)
    qh = q.float().reshape(-1, R, 128)[heads]
    sc = torch.einsum("hrd,hnd->hrn", qh, kd) * 128 ** -0.5
    return torch.einsum("hrn,hnd->hrd", torch.softmax(sc, -1), vd).reshape(-1, 128)


@pytest.mark.parametrize("name,B,H_Q,H_KV,N", [("batched 64q/8kv x 16, 32K", 16, 64, 8, 32768),
                                                ("long context 32q/2kv x 4, 128K", 4, 32, 2, 131072)])
def test_full_size_batched_and_long_context_shapes(name, B, H_Q, H_KV, N):
    """The other two BASELINE decode shapes at full size: the result does not depend on the split count, equals a
    four-way sequence sharding merged by the LSE kernel, and sampled heads match an fp32 dense computation on the
    dequantised cache."""
    g = torch.Generator(device=DEV); g.manual_seed(N + B)
    BH, R = B * H_KV, H_Q // H_KV
    T = int((N - 128) * 0.05); nq = N - 128 - T
    bf = lambda n: torch.randn(BH, n, 128, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    kq, ks = hq.quantize_per_token(bf(nq), 4)
    vq, vs = hq.quantize_per_token(bf(nq), 4)
    kt, vt, kw, vw, kst, vst = bf(T), bf(T), bf(128), bf(128), bf(64), bf(64)
    q = torch.randn(BH * R, 128, generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    full = hq.fused_d_stage_decode(q, kq, vq, ks, vs, kt, vt, kst, vst, kw, vw, 4, 4, kv_repeat=R).float()
    one = dd.DecodePlan(q, kq, vq, ks, vs, kt, vt, kst, vst, kw, vw, R, None, num_splits=1).run(q).float()
    assert (full - one).abs().max().item() < 1e-2
    heads = torch.tensor([0, BH // 2, BH - 1], device=DEV)
    ref = _dense_yardstick(q, kq, vq, ks, vs, [(kt, vt), (kst, vst), (kw, vw)], R, heads)
    got = full.reshape(BH, R, 128)[heads].reshape(-1, 128)
    assert (got - ref).abs().max().item() <= MAX_ABS
    assert ((got - ref) ** 2).sum().item() / (ref ** 2).sum().item() <= REL_MSE
    G = 4
    from hyquant_b200 import sharded
    ms, ls, accs = [], [], []
    for r, (q0, q1, t0, t1) in enumerate(sharded.sequence_shard_plan(nq, T, G)):
        last = r == G - 1
        e = kw[:, :0]
        plan = dd.DecodePlan(q, kq[:, q0:q1], vq[:, q0:q1], ks[:, q0:q1].contiguous(), vs[:, q0:q1].contiguous(),
                             kt[:, t0:t1], vt[:, t0:t1], kst if last else e, vst if last else e, kw if last else e,
                             vw if last else e, R, None)
        m = torch.empty(BH * R, dtype=torch.float32, device=DEV); l = torch.empty_like(m)
        acc = torch.empty(BH * R, 128, dtype=torch.float32, device=DEV)
        plan.run(q, partial=(m, l, acc)); ms.append(m); ls.append(l); accs.append(acc)
    merged = hq.lse_merge(torch.stack(ms), torch.stack(ls), torch.stack(accs), out_dtype=torch.float32)
    assert (merged - full).abs().max().item() < 1e-2


@pytest.mark.parametrize("bits", [(4, 4), (8, 8), (4, 2), (2, 8)])
def test_decode_step_equals_append_then_decode(bits):
    """`decode_step` (the new token attended to and stored by the decode kernel itself) against the reference's two
    calls, over 300 steps: same cache contents bit for bit (staging rows, flushed codes and scales), same outputs up
    to the order of the fp32 partial sums."""
    import hyquant_b200 as hq
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV, N, W = 2, 8, 2, 2048 + 9, 128
    R = H_Q // H_KV
    t = gen_torch(B, H_Q, H_KV, N, 128, W, 0.05, 77, n_qry=W, device="cuda")
    layers = []
    for _ in range(2):
        layer = hq.DStageLayerCache(0, k_bits=bits[0], v_bits=bits[1], window_size=W, top_ratio=0.05, use_vert=True)
        layer.update_prefill(t["k"], t["v"]); layer.save_query_tail(t["q"]); layer.freeze(kv_repeat=R)
        layers.append(layer)
    g = torch.Generator(device="cuda").manual_seed(3)
    worst = 0.0
    for step in range(300):
        kn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        vn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        qn = torch.randn(B, H_Q, 1, 128, generator=g, device="cuda").bfloat16()
        layers[0].append_staging(kn, vn)
        want = layers[0].decode_attention(qn, R)
        got = layers[1].decode_step(qn, kn, vn, R)
        worst = max(worst, float((got.float() - want.float()).abs().max()))
        assert layers[0]._staging_ptr == layers[1]._staging_ptr and layers[0]._n_quant == layers[1]._n_quant
    assert worst <= 4e-3, worst
    a, b = layers
    assert a.get_seq_length() == b.get_seq_length() == N + 300
    assert torch.equal(a._staging_buf_k[:, :a._staging_ptr], b._staging_buf_k[:, :b._staging_ptr])
    assert torch.equal(a._staging_buf_v[:, :a._staging_ptr], b._staging_buf_v[:, :b._staging_ptr])
    assert torch.equal(a.k_quant_packed, b.k_quant_packed) and torch.equal(a.v_scale, b.v_scale)
    assert decode_status_of(b) == 0


def decode_status_of(layer):
    from hyquant_b200.decode_d_stage import decode_status
    return decode_status(layer._plan.ws)


@pytest.mark.parametrize("bits", [(4, 4), (8, 8), (2, 2)])
@pytest.mark.parametrize("heads,N", [((1, 8, 2), 3000), ((2, 32, 8), 9000)])
def test_codes_as_planes_of_one_tensor_equal_separate_tensors(bits, heads, N):
    """The cache class keeps K and V codes of equal width as two planes of one tensor, which the decode kernel reads with
    one tensor-map request per unit; the same cache handed over as separate contiguous tensors takes two bulk copies
    per unit.  Same bytes in shared memory, so the outputs are equal bit for bit."""
    import hyquant_b200 as hq
    from hyquant_b200 import decode_d_stage as dds
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV = heads
    R, W = H_Q // H_KV, 128
    t = gen_torch(B, H_Q, H_KV, N, 128, W, 0.05, 5 + N, n_qry=W, device="cuda")
    layer = hq.DStageLayerCache(0, k_bits=bits[0], v_bits=bits[1], window_size=W, top_ratio=0.05, use_vert=True)
    layer.update_prefill(t["k"], t["v"]); layer.save_query_tail(t["q"]); layer.freeze(kv_repeat=R)
    assert layer._vq.data_ptr() - layer._kq.data_ptr() == layer._kq.shape[1] * layer._kq.shape[2]      # planes of one tensor
    g = torch.Generator(device="cuda").manual_seed(11)
    for step in range(3):
        kn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        vn = torch.randn(B, H_KV, 1, 128, generator=g, device="cuda").bfloat16()
        layer.append_staging(kn, vn)
    q = torch.randn(B, H_Q, 1, 128, generator=g, device="cuda").bfloat16()
    planes = layer.decode_attention(q, R)
    S = layer._staging_ptr
    apart = dds.fused_d_stage_decode(q.reshape(-1, 128), layer.k_quant_packed.contiguous(), layer.v_quant_packed.contiguous(),
                                     layer.k_scale.contiguous(), layer.v_scale.contiguous(), layer.k_topk, layer.v_topk,
                                     layer._staging_buf_k[:, :S], layer._staging_buf_v[:, :S], layer.k_window, layer.v_window,
                                     bits[0], bits[1], kv_repeat=R)
    assert torch.equal(planes.reshape(-1, 128), apart)
    assert decode_status_of(layer) == 0


def test_multi_token_append_equals_token_by_token():
    """append_staging with several tokens at once (a chunked prefill continuation) leaves the cache exactly as the same
    tokens appended one by one do, across two flushes of the staging buffer."""
    import hyquant_b200 as hq
    from hyquant_b200.synth import gen_torch
    B, H_Q, H_KV, N, W = 1, 8, 2, 700, 64
    t = gen_torch(B, H_Q, H_KV, N, 128, W, 0.05, 91, n_qry=W, device="cuda")
    a, b = [hq.DStageLayerCache(0, window_size=W, top_ratio=0.05) for _ in range(2)]
    for layer in (a, b):
        layer.update_prefill(t["k"], t["v"]); layer.save_query_tail(t["q"]); layer.freeze(kv_repeat=4)
    g = torch.Generator(device="cuda").manual_seed(2)
    kn = torch.randn(B, H_KV, 300, 128, generator=g, device="cuda").bfloat16()
    vn = torch.randn(B, H_KV, 300, 128, generator=g, device="cuda").bfloat16()
    for lo, hi in ((0, 7), (7, 130), (130, 131), (131, 300)):
        a.append_staging(kn[:, :, lo:hi], vn[:, :, lo:hi])
    for i in range(300):
        b.append_staging(kn[:, :, i:i + 1], vn[:, :, i:i + 1])
    assert a._staging_ptr == b._staging_ptr == 300 - 256 and a._n_quant == b._n_quant
    assert a.get_seq_length() == b.get_seq_length() == N + 300
    assert torch.equal(a.k_quant_packed, b.k_quant_packed) and torch.equal(a.v_quant_packed, b.v_quant_packed)
    assert torch.equal(a.k_scale, b.k_scale) and torch.equal(a.v_scale, b.v_scale)
    assert torch.equal(a._staging_buf_k[:, :44], b._staging_buf_k[:, :44]) and torch.equal(a._staging_buf_v[:, :44], b._staging_buf_v[:, :44])
    q = torch.randn(B, H_Q, 1, 128, generator=g, device="cuda").bfloat16()
    assert torch.equal(a.decode_attention(q, 4), b.decode_attention(q, 4))


@pytest.mark.parametrize("seed", range(24))
def test_decode_random_shapes_both_code_layouts(seed):
    """Random head counts, GQA ratios, bit widths and segment lengths: against the oracle, and with K / V codes handed over
    as planes of one tensor (one request per unit) equal bit for bit to separate tensors (two requests)."""
    rng = np.random.Generator(np.random.PCG64(1000 + seed))
    bits = [(4, 4), (4, 4), (8, 8), (2, 2), (4, 2), (8, 4)][seed % 6]
    BH = int(rng.choice([1, 2, 3, 8, 16, 40]))
    R = int(rng.choice([1, 2, 4, 5, 8, 12, 16]))
    nq = int(rng.choice([0, 17, 200, 1500, 6000])) + int(rng.integers(0, 40))
    nt, ns, nw = int(rng.integers(0, 90)), int(rng.integers(0, 128)), int(rng.choice([0, 64, 128]))
    if nq + nt + ns + nw == 0:
        nw = 64
    c, q = build_case(BH, R, nq, nt, ns, nw, seed=seed, k_bits=bits[0], v_bits=bits[1])
    ref = orc.decode_attention_exact(q, c, R).reshape(-1, 128)
    out = run_gpu(c, q, R)
    check_close(out, ref)
    if bits[0] == bits[1] and nq > 0:
        row = 16 * bits[0]
        cap = (nq + 127) // 128 * 128 + 128
        kv = torch.zeros(BH, 2, cap, row, dtype=torch.int8, device=DEV)
        kv[:, 0, :nq] = torch.from_numpy(np.ascontiguousarray(c.k_quant_packed)).to(DEV)
        kv[:, 1, :nq] = torch.from_numpy(np.ascontiguousarray(c.v_quant_packed)).to(DEV)
        ti = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
        S = c.staging_ptr
        planes = hq.fused_d_stage_decode(t_bf16(q.reshape(-1, 128)), kv[:, 0, :nq], kv[:, 1, :nq], ti(c.k_scale), ti(c.v_scale),
                                         t_bf16(c.k_topk), t_bf16(c.v_topk), t_bf16(c.staging_k)[:, :S], t_bf16(c.staging_v)[:, :S],
                                         t_bf16(c.k_window), t_bf16(c.v_window), bits[0], bits[1], kv_repeat=R)
        assert np.array_equal(to_np(planes), out)
