"""The decode entry point that brings its own scratch (``hq_decode_splitk_static``).

Some callers of this library may not allocate device memory: a serving runtime that hands
the GPU's memory to its own pool and bans ``cudaMalloc`` in operator callbacks, or a plugin
loaded into a host that owns every allocation.  For them the library keeps a fixed 4 MiB
scratch array in its own image.  This test calls that entry point through the C ABI twice in
a row and expects the results of the ordinary entry point (same kernel, same split plan, so
the same bits), and checks that an oversized shape is refused."""

import ctypes as C

import numpy as np
import pytest
import torch

from hyquant_b200 import _lib
from hyquant_b200 import decode_d_stage as dd

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
        assert (got - ref).abs().max().item() <= 2e-2
        assert ((got - ref) ** 2).sum().item() <= 1e-4 * (ref ** 2).sum().item()
    # and the ordinary entry point still gives the same answer afterwards
    assert (plan.run(q).float() - ref).abs().max().item() <= 2e-2


def test_static_scratch_refuses_oversized_shapes():
    lib = _lib.lib()
    need = C.c_int64(0)
    assert lib.hq_decode_workspace_bytes(4096, 16, C.byref(need)) == 0 and need.value > (4 << 20)
    a = _lib.DecodeArgs()
    a.struct_bytes = C.sizeof(_lib.DecodeArgs)
    a.BH_KV, a.kv_repeat, a.head_dim = 4096, 16, 128
    assert lib.hq_decode_splitk_static(C.byref(a), None) == -4
    assert b"4194304" in lib.hq_last_error()
