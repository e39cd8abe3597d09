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
        # --- the same layer-level path with the exchange and the merge in one kernel over peer memory
        px = sharded.PeerExchange(rows=2 * 8)
        shp = sharded.SequenceShardedLayer(sh.layer, exchange=px)
        e4 = 0.0
        for step in range(150):                                  # crosses a staging flush on the tail rank
            shp.fused = step % 3 == 0                            # second kernel exchanges / decode kernel does it itself
            q_s = torch.randn(2, 8, 1, 128, generator=g2, device=dev).to(torch.bfloat16)
            kn = torch.randn(2, 2, 1, 128, generator=g2, device=dev).to(torch.bfloat16)
            vn = torch.randn(2, 2, 1, 128, generator=g2, device=dev).to(torch.bfloat16)
            want = lay.decode_step(q_s, kn, vn, 4).float()
            got = shp.decode_step(q_s, kn, vn, 4, last).float()
            e4 = max(e4, (got - want).abs().max().item())
        e4 = e4 if px.status() == 0 else 1e9
        px.close()
        torch.cuda.synchronize()
        errs[rank] = (e1, e2, e3, e4)
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
        assert max(errs[r]) < 1e-2, dict(errs)


def _peer_buffers(world, rows):
    import ctypes as C
    from hyquant_b200 import _lib
    n = C.c_int64()
    _lib.check(_lib.lib().hq_peer_exchange_bytes(world, rows, C.byref(n)), "hq_peer_exchange_bytes")
    return [torch.zeros(n.value, dtype=torch.uint8, device="cuda") for _ in range(world)]


def _local_views(buf, world, rows, seq):
    """Torch views of a rank's own (m, l, acc) of call ``seq`` inside its exchange buffer."""
    import ctypes as C
    from hyquant_b200 import _lib
    m, l, acc = C.c_void_p(), C.c_void_p(), C.c_void_p()
    _lib.check(_lib.lib().hq_peer_slot(buf.data_ptr(), world, rows, seq, C.byref(m), C.byref(l), C.byref(acc)), "hq_peer_slot")
    f32 = buf.view(torch.float32)
    o = (m.value - buf.data_ptr()) // 4
    return f32[o:o + rows], f32[o + rows:o + 2 * rows], f32[o + 2 * rows:o + 130 * rows].view(rows, 128)


def _recv_view(buf, world, rows, seq, src):
    """Torch view [rows * 130, 2] (int32: value bits, sequence number) of what rank ``src`` stores for call ``seq``."""
    import ctypes as C
    from hyquant_b200 import _lib
    w = C.c_void_p()
    _lib.check(_lib.lib().hq_peer_recv_slot(buf.data_ptr(), world, rows, seq, src, C.byref(w)), "hq_peer_recv_slot")
    o = (w.value - buf.data_ptr()) // 4
    return buf.view(torch.int32)[o:o + 2 * 130 * rows].view(130 * rows, 2)


def _message(m, l, acc):
    return torch.cat([m, l, acc.reshape(-1)]).contiguous().view(torch.int32)


def _run_exchange(bufs, world, rank, rows, seq, out, timeout_ns=0):
    import ctypes as C
    from hyquant_b200 import _lib
    a = _lib.PeerExchangeArgs()
    a.struct_bytes, a.world, a.rank, a.rows, a.seq = C.sizeof(_lib.PeerExchangeArgs), world, rank, rows, seq
    a.out, a.out_stride, a.out_dtype, a.timeout_ns = out.data_ptr(), out.stride(0), _lib.dtype_code(out.dtype), timeout_ns
    for j, b in enumerate(bufs):
        a.bufs[j] = b.data_ptr()
    _lib.check(_lib.lib().hq_peer_exchange_merge(C.byref(a), _lib.stream_ptr(out.device)), "hq_peer_exchange_merge")


@pytest.mark.parametrize("rows,world", [(16, 2), (128, 4), (1500, 3)])
def test_peer_exchange_kernel_one_gpu(rows, world):
    """The exchange + merge kernel of rank 0 with the peers' buffers in this GPU's own memory and their words
    already in place (no second kernel to wait for): it must deliver rank 0's words to every peer buffer
    and write the log-sum-exp merge of all ranks' partials."""
    import hyquant_b200 as hq
    g = torch.Generator(device="cuda").manual_seed(rows + world)
    m = torch.randn(world, rows, generator=g, device="cuda") * 4
    m[1, ::7] = float("-inf")                                   # an empty shard for some rows
    l = torch.rand(world, rows, generator=g, device="cuda") + 0.1
    l[1, ::7] = 0
    acc = torch.randn(world, rows, 128, generator=g, device="cuda")
    acc[1, ::7] = 0
    want = hq.lse_merge(m, l, acc, out_dtype=torch.float32)
    bufs = _peer_buffers(world, rows)
    for seq in (1, 2, 3):
        lm, ll, la = _local_views(bufs[0], world, rows, seq)
        lm.copy_(m[0]); ll.copy_(l[0]); la.copy_(acc[0])
        for src in range(1, world):
            rv = _recv_view(bufs[0], world, rows, seq, src)
            rv[:, 0] = _message(m[src], l[src], acc[src])
            rv[:, 1] = seq
        out = torch.empty(rows, 128, dtype=torch.float32, device="cuda")
        _run_exchange(bufs, world, 0, rows, seq, out)
        torch.cuda.synchronize()
        assert torch.allclose(out, want, rtol=1e-5, atol=1e-6)
        for j in range(1, world):
            rv = _recv_view(bufs[j], world, rows, seq, 0)
            assert torch.equal(rv[:, 0], _message(m[0], l[0], acc[0])) and bool((rv[:, 1] == seq).all())
        assert int(bufs[0].view(torch.int32)[0]) == 0


def test_peer_exchange_wait_runs_out():
    """A peer that never stores its words: the wait ends at its time limit, bit 1 of the status word is set and
    the device stays usable."""
    world, rows = 2, 8
    bufs = _peer_buffers(world, rows)
    out = torch.empty(rows, 128, dtype=torch.float32, device="cuda")
    _run_exchange(bufs, world, 0, rows, 1, out, timeout_ns=20_000_000)        # 20 ms
    torch.cuda.synchronize()
    assert int(bufs[0].view(torch.int32)[0]) == 2
    assert float((torch.ones(4, device="cuda") * 2).sum()) == 8.0


class _FakeExchange:
    """What DecodePlan.run needs from a PeerExchange, over buffers in this GPU's own memory."""

    def __init__(self, bufs, world, rank, timeout_ns=0):
        import ctypes as C
        self._arr = (C.c_void_p * 16)(*[b.data_ptr() for b in bufs])
        self.bufs_addr, self.world, self.rank, self.timeout_ns = C.addressof(self._arr), world, rank, timeout_ns


@pytest.mark.parametrize("R,BH", [(4, 4), (16, 2)])
def test_decode_with_in_kernel_exchange_one_gpu(R, BH):
    """Rank 0 of a two-way sequence split, with rank 1's state already in rank 0's exchange buffer: the decode
    kernel must store rank 0's state into rank 1's buffer and write the merge, which equals the unsplit decode."""
    import hyquant_b200 as hq
    from hyquant_b200 import decode_d_stage as dd, sharded
    nq, nt, ns, nw = 5000, 200, 37, 128
    c = _build("cuda", BH, nq, nt, ns, nw, seed=9)
    g = torch.Generator(device="cuda").manual_seed(10)
    q = torch.randn(BH * R, 128, generator=g, device="cuda").to(torch.bfloat16)
    full = hq.fused_d_stage_decode(q, c["kq"], c["vq"], c["ks"], c["vs"], c["kt"], c["vt"], c["kst"], c["vst"],
                                   c["kw"], c["vw"], 4, 4, kv_repeat=R).float()
    world, rows = 2, BH * R
    plans = []
    e = c["kw"][:, :0]
    for rank in range(world):
        q0, q1, t0, t1 = sharded.sequence_shard_plan(nq, nt, world)[rank]
        last = rank == world - 1
        plans.append(dd.DecodePlan(q, c["kq"][:, q0:q1], c["vq"][:, q0:q1], c["ks"][:, q0:q1].contiguous(), c["vs"][:, q0:q1].contiguous(),
                                   c["kt"][:, t0:t1], c["vt"][:, t0:t1], c["kst"] if last else e, c["vst"] if last else e,
                                   c["kw"] if last else e, c["vw"] if last else e, R, None))
    m1 = torch.empty(rows, device="cuda"); l1 = torch.empty_like(m1); a1 = torch.empty(rows, 128, device="cuda")
    plans[1].run(q, partial=(m1, l1, a1))
    m0 = torch.empty(rows, device="cuda"); l0 = torch.empty_like(m0); a0 = torch.empty(rows, 128, device="cuda")
    plans[0].run(q, partial=(m0, l0, a0))
    bufs = _peer_buffers(world, rows)
    for seq in (1, 2):
        rv = _recv_view(bufs[0], world, rows, seq, 1)
        rv[:, 0] = _message(m1, l1, a1)
        rv[:, 1] = seq
        out = torch.empty(rows, 128, dtype=torch.float32, device="cuda")
        plans[0].run(q, out=out, peer=(_FakeExchange(bufs, world, 0), seq))
        torch.cuda.synchronize()
        assert (out - full).abs().max().item() < 1e-2
        sent = _recv_view(bufs[1], world, rows, seq, 0)
        assert bool((sent[:, 1] == seq).all())
        assert torch.equal(sent[:, 0], _message(m0, l0, a0))           # the same state as the partial-mode call
        assert int(bufs[0].view(torch.int32)[0]) == 0
    # and a call without a peer afterwards is the plain one again
    assert torch.equal(plans[0].run(q, out=torch.empty(rows, 128, dtype=torch.float32, device="cuda")),
                       plans[0].run(q, out=torch.empty(rows, 128, dtype=torch.float32, device="cuda")))
