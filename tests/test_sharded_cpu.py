"""Host-side logic of the multi-GPU decode paths on CPU: shard plans, and the
all-gather + merge plumbing with two gloo ranks (the partial states come from the
oracle here; on GPUs they come from the decode kernel in partial mode)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hyquant_b200 import sharded
from oracle import hq_oracle as orc


def test_kv_head_ranges_cover_all_heads():
    for h, w in ((8, 1), (8, 2), (8, 4), (8, 8), (2, 2)):
        got = [sharded.kv_head_range(h, w, r) for r in range(w)]
        assert got[0][0] == 0 and got[-1][1] == h and all(a[1] == b[0] for a, b in zip(got, got[1:]))
    with pytest.raises(ValueError):
        sharded.kv_head_range(2, 4, 0)


@pytest.mark.parametrize("nq,nt,w", [(124396, 6548, 8), (124396, 6548, 2), (100, 3, 4), (0, 0, 2), (31008, 1632, 4)])
def test_sequence_plan_is_a_partition(nq, nt, w):
    plan = sharded.sequence_shard_plan(nq, nt, w)
    assert plan[0][0] == 0 and plan[-1][1] == nq and plan[0][2] == 0 and plan[-1][3] == nt
    for a, b in zip(plan, plan[1:]):
        assert a[1] == b[0] and a[3] == b[2]
    assert all(p[0] % 128 == 0 and p[0] <= p[1] and p[2] <= p[3] for p in plan)


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _worker(rank, world, port, q, k, v, ref, cuts, errs):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        dist.init_process_group("gloo", rank=rank, world_size=world)
        a, b = cuts[rank], cuts[rank + 1]
        m, l, acc = orc.decode_partials(q, k[a:b], v[a:b], 128 ** -0.5)
        m = np.where(np.isinf(m), -np.inf, m)
        tm, tl, tacc = (torch.from_numpy(x.astype(np.float32)) for x in (m, l, acc))
        gm, gl, gacc = sharded.gather_partials(tm, tl, tacc)
        assert gm.shape == (world, q.shape[0]) and gacc.shape == (world, q.shape[0], 128)
        out = orc.lse_merge(gm.numpy().astype(np.float64), gl.numpy().astype(np.float64), gacc.numpy().astype(np.float64))
        errs[rank] = float(np.abs(out - ref).max())
        dist.destroy_process_group()
    except Exception as e:  # pragma: no cover
        errs[rank] = repr(e)


def test_two_rank_gather_and_merge_equals_single_pass():
    rng = np.random.Generator(np.random.PCG64(12))
    q = rng.standard_normal((8, 128)); k = rng.standard_normal((777, 128)); v = rng.standard_normal((777, 128))
    m, l, acc = orc.decode_partials(q, k, v, 128 ** -0.5)
    ref = acc / l[:, None]
    world = 2
    mgr = mp.Manager()
    errs = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), q, k, v, ref, [0, 384, 777], errs), nprocs=world, join=True)
    assert all(isinstance(errs[r], float) and errs[r] < 1e-5 for r in range(world)), dict(errs)
