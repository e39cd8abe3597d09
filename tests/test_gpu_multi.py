"""Two-GPU checks (skipped on a single GPU): sequence-sharded decode with an NCCL all-gather of the
softmax partials equals the single-GPU decode; KV-head sharding equals slicing the full result."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def _build(dev, BH, nq, nt, ns, nw, seed):
    from hyquant_b200 import decode_d_stage as dd
    g = torch.Generator(device=dev); g.manual_seed(seed)
    bf = lambda n: torch.randn(BH, n, 128, generator=g, device=dev).to(torch.bfloat16)
    kq, ks = dd.quantize_per_token(bf(nq), 4)
    vq, vs = dd.quantize_per_token(bf(nq), 4)
    return dict(kq=kq, vq=vq, ks=ks, vs=vs, kt=bf(nt), vt=bf(nt), kst=bf(ns), vst=bf(ns), kw=bf(nw), vw=bf(nw))


def _worker(rank, world, port, errs):
    try:
        os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
        import torch.distributed as dist
        import hyquant_b200 as hq
        from hyquant_b200 import decode_d_stage as dd, sharded
        dev = torch.device("cuda", rank)
        torch.cuda.set_device(dev)
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
        BH, R, nq, nt, ns, nw = 4, 4, 9000, 300, 37, 128
        c = _build(dev, BH, nq, nt, ns, nw, seed=5)                     # same seed on every rank
        g = torch.Generator(device=dev); g.manual_seed(6)
        q = torch.randn(BH * R, 128, generator=g, device=dev).to(torch.bfloat16)
        full = hq.fused_d_stage_decode(q, c["kq"], c["vq"], c["ks"], c["vs"], c["kt"], c["vt"], c["kst"], c["vst"],
                                       c["kw"], c["vw"], 4, 4, kv_repeat=R).float()
        # --- sequence sharding
        q0, q1, t0, t1 = sharded.sequence_shard_plan(nq, nt, world)[rank]
        last = rank == world - 1
        e = c["kw"][:, :0]
        plan = dd.DecodePlan(q, c["kq"][:, q0:q1], c["vq"][:, q0:q1], c["ks"][:, q0:q1].contiguous(), c["vs"][:, q0:q1].contiguous(),
                             c["kt"][:, t0:t1], c["vt"][:, t0:t1], c["kst"] if last else e, c["vst"] if last else e,
                             c["kw"] if last else e, c["vw"] if last else e, R, None)
        m = torch.empty(BH * R, dtype=torch.float32, device=dev); l = torch.empty_like(m)
        acc = torch.empty(BH * R, 128, dtype=torch.float32, device=dev)
        plan.run(q, partial=(m, l, acc))
        gm, gl, gacc = sharded.gather_partials(m, l, acc)
        merged = hq.lse_merge(gm, gl, gacc, out_dtype=torch.float32)
        e1 = (merged - full).abs().max().item()
        # --- kv-head sharding: this rank's heads only, no collective
        h0, h1 = sharded.kv_head_range(BH, world, rank)
        sl = slice(h0, h1)
        part = hq.fused_d_stage_decode(q[h0 * R:h1 * R], c["kq"][sl], c["vq"][sl], c["ks"][sl], c["vs"][sl], c["kt"][sl],
                                       c["vt"][sl], c["kst"][sl], c["vst"][sl], c["kw"][sl], c["vw"][sl], 4, 4, kv_repeat=R).float()
        e2 = (part - full[h0 * R:h1 * R]).abs().max().item()
        # --- the layer-level path: a frozen cache split by shard_layer_sequence, decoded through
        # SequenceShardedLayer (kernel writes the per-rank message, one all-gather, strided merge),
        # across a staging flush on the tail rank
        from hyquant_b200.synth import gen_torch
        t = gen_torch(2, 8, 2, 4096 + 77, 128, 128, 0.05, 321, n_qry=128, device=dev)     # same seed on every rank
        lay = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=128, top_ratio=0.05, use_vert=True)
        lay.update_prefill(t["k"], t["v"]); lay.save_query_tail(t["q"]); lay.freeze(kv_repeat=4)
        sh = sharded.SequenceShardedLayer(sharded.shard_layer_sequence(lay, world, rank))
        g2 = torch.Generator(device=dev); g2.manual_seed(11)
        e3 = 0.0
        for step in range(140):
            kn = torch.randn(2, 2, 1, 128, generator=g2, device=dev).to(torch.bfloat16)
            vn = torch.randn(2, 2, 1, 128, generator=g2, device=dev).to(torch.bfloat16)
            lay.append_staging(kn, vn)
            sh.append_staging(kn, vn, last)
            if step % 23 == 0 or step >= 126:
                want = lay.decode_attention(t["q_decode"], 4).float()
                got = sh.decode_attention(t["q_decode"], 4).float()
                e3 = max(e3, (got - want).abs().max().item())
        torch.cuda.synchronize()
        errs[rank] = (e1, e2, e3)
        dist.destroy_process_group()
    except Exception as ex:  # pragma: no cover
        import traceback
        errs[rank] = traceback.format_exc()


def test_two_gpu_sequence_and_head_sharding():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    errs = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), errs), nprocs=world, join=True)
    for r in range(world):
        assert isinstance(errs[r], tuple), errs[r]
        assert errs[r][0] < 1e-2 and errs[r][1] < 1e-2 and errs[r][2] < 1e-2, dict(errs)
