"""The decode entry point that brings its own scratch (``hq_decode_splitk_static``).

Some callers of this library may not allocate device memory: a serving runtime that hands
the GPU's memory to its own pool and bans ``cudaMalloc`` in operator callbacks, or a plugin
loaded into a host that owns every allocation.  For them the library keeps a fixed 4 MiB
scratch array in its own image.  This test calls that entry point through the C ABI twice in
a row and expects the results of the ordinary entry point bit for bit (same kernel, same split
plan), compares one case with the CPU oracle's exact attention, reads the status word back and
checks that an oversized shape and unknown flag bits are refused."""

import ctypes as C

import numpy as np
import pytest
import torch

from hyquant_b200 import _lib
from hyquant_b200 import decode_d_stage as dd
from oracle import hq_oracle as orc

pytestmark = pytest.mark.gpu


def _case(BH, R, nq, nt, ns, nw, seed):
    g = torch.Generator(device="cuda"); g.manual_seed(seed)
    bf = lambda n: torch.randn(BH, n, 128, generator=g, device="cuda").to(torch.bfloat16)
    kq, ks = dd.quantize_per_token(bf(nq), 4)
    vq, vs = dd.quantize_per_token(bf(nq), 4)
    q = torch.randn(BH * R, 128, generator=g, device="cuda").to(torch.bfloat16)
    return q, (kq, vq, ks, vs, bf(nt), bf(nt), bf(ns), bf(ns), bf(nw), bf(nw))


@pytest.mark.parametrize("BH,R,nq", [(8, 4, 4000), (2, 8, 700)])
def test_static_scratch_matches_workspace_entry_point(BH, R, nq):
    lib = _lib.lib()
    q, segs = _case(BH, R, nq, 60, 17, 128, seed=nq)
    plan = dd.DecodePlan(q, *segs, R, None)
    ref = plan.run(q).float().clone()
    torch.cuda.synchronize()
    stream = torch.cuda.current_stream().cuda_stream
    for attempt in range(2):                         # two calls in a row share the scratch
        out = torch.full_like(q, float("nan"))
        a = _lib.DecodeArgs.from_buffer_copy(plan.args)   # same pointers, sizes and split plan
        a.out, a.out_stride = out.data_ptr(), out.stride(0)
        a.workspace, a.workspace_bytes = None, 0      # ignored by this entry point
        rc = lib.hq_decode_splitk_static(C.byref(a), stream)
        assert rc == 0, lib.hq_last_error()
        torch.cuda.synchronize()
        got = out.float()
        assert torch.isfinite(got).all()
        assert torch.equal(got, ref)                  # same kernel, same split plan: the same bits
        st = C.c_int(-1)
        assert lib.hq_decode_static_status(C.byref(st)) == 0 and st.value == 0      # no bounded wait ran out
    # and the ordinary entry point still gives the same answer afterwards
    assert torch.equal(plan.run(q).float(), ref)
    # against the CPU oracle: exact softmax attention over the four segments (tolerance of the decode tests)
    kq, vq, ks, vs, kt, vt, kg, vg, kw, vw = segs
    f = lambda t: t.float().cpu().numpy()
    oc = orc.LayerCache(B=1, H_KV=BH, D=128, k_bits=4, v_bits=4, k_quant_packed=kq.cpu().numpy(), v_quant_packed=vq.cpu().numpy(),
                        k_scale=ks.cpu().numpy(), v_scale=vs.cpu().numpy(), k_topk=f(kt), v_topk=f(vt), k_window=f(kw),
                        v_window=f(vw), staging_k=f(kg), staging_v=f(vg), staging_ptr=kg.shape[1], seq_len=0)
    exact = orc.decode_attention_exact(f(q).reshape(1, BH * R, 1, 128), oc, R).reshape(BH * R, 128)
    assert np.abs(f(ref) - exact).max() <= 2e-2 and orc.rel_mse(f(ref), exact) <= 1e-4


def test_static_scratch_refuses_oversized_shapes():
    lib = _lib.lib()
    need = C.c_int64(0)
    assert lib.hq_decode_workspace_bytes(4096, 16, C.byref(need)) == 0 and need.value > (4 << 20)
    a = _lib.DecodeArgs()
    a.struct_bytes = C.sizeof(_lib.DecodeArgs)
    a.BH_KV, a.kv_repeat, a.head_dim = 4096, 16, 128
    assert lib.hq_decode_splitk_static(C.byref(a), None) == -4
    assert b"4194304" in lib.hq_last_error()


def test_static_scratch_refuses_unknown_flags():
    lib = _lib.lib()
    q, segs = _case(2, 4, 300, 8, 3, 16, seed=5)
    plan = dd.DecodePlan(q, *segs, 4, None)
    out = torch.empty_like(q)
    a = _lib.DecodeArgs.from_buffer_copy(plan.args)
    a.q, a.q_stride, a.out, a.out_stride = q.data_ptr(), q.stride(0), out.data_ptr(), out.stride(0)
    a.flags = 0x40
    assert lib.hq_decode_splitk_static(C.byref(a), torch.cuda.current_stream().cuda_stream) == -1
