"""Multi-GPU decode: one process per GPU, ``torch.distributed`` for the plumbing.

Two ways the path shards (the reference itself has neither; results equal the
single-GPU result):

* KV-head groups — every (batch, kv-head) is independent in decode, flush, freeze and
  prefill, so rank r owns kv-heads ``kv_head_range(H_KV, world, r)`` and their query
  heads.  No collective on the data path; outputs stay per rank.
* Sequence shards (very long prefixes) — contiguous 128-token-aligned ranges of the INT4
  prefix and contiguous ranges of the BF16 vertical-line segment per rank; window and
  staging live on the last rank, which also receives the staging flushes.  Each rank runs
  the decode kernel in partial mode; the un-normalised softmax states ``(m, l, acc)``
  (66.5 KB per rank at B=4, 32 query heads) are exchanged and merged on every rank by one
  kernel that stores them into the peers' buffers over NVLink and waits for theirs
  (:class:`PeerExchange`, ``hq_peer_exchange_merge``).  ``exchange="nccl"`` keeps the plain
  form for comparison: one ``all_gather_into_tensor`` followed by ``hq_lse_merge``.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

import ctypes as C

import torch


def kv_head_range(h_kv: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous kv-head range of ``rank``; requires ``h_kv % world == 0``."""
    if h_kv % world != 0:
        raise ValueError(f"{h_kv} kv heads do not divide over {world} ranks")
    per = h_kv // world
    return rank * per, (rank + 1) * per


def sequence_shard_plan(n_quant: int, n_topk: int, world: int, align: int = 128) -> List[Tuple[int, int, int, int]]:
    """Per rank ``(q0, q1, t0, t1)``: INT4 prefix tokens [q0, q1) (starts aligned to ``align``)
    and vertical-line tokens [t0, t1).  Ranges are contiguous, disjoint and cover everything;
    a rank may get an empty range."""
    plan = []
    for r in range(world):
        q0 = (r * n_quant // world) // align * align
        q1 = n_quant if r == world - 1 else ((r + 1) * n_quant // world) // align * align
        t0, t1 = r * n_topk // world, (r + 1) * n_topk // world
        plan.append((q0, max(q0, q1), t0, t1))
    return plan


def gather_partials(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, group=None):
    """All-gather one rank's ``(m [rows], l [rows], acc [rows, D])`` into ``[G, rows]``,
    ``[G, rows]``, ``[G, rows, D]``.  One collective: the three are packed into a single
    ``[rows, D + 2]`` message."""
    import torch.distributed as dist
    world = dist.get_world_size(group)
    rows, d = acc.shape
    msg = torch.empty(rows, d + 2, dtype=torch.float32, device=acc.device)
    msg[:, :d] = acc
    msg[:, d] = m
    msg[:, d + 1] = l
    out = torch.empty(world, rows, d + 2, dtype=torch.float32, device=acc.device)
    dist.all_gather_into_tensor(out.view(world * rows, d + 2), msg, group=group)
    return out[:, :, d].contiguous(), out[:, :, d + 1].contiguous(), out[:, :, :d].contiguous()


def shard_layer_sequence(layer, world: int, rank: int):
    """This rank's sequence shard of a frozen ``DStageLayerCache`` that holds the whole cache:
    a new layer cache owning copies of its INT4-prefix and vertical-line ranges; window and live
    staging tokens go to the last rank only, which is also the rank whose prefix grows at a flush."""
    from .d_stage_kv_cache import GROUP_SIZE, DStageLayerCache
    if layer.phase != "decode":
        raise ValueError("shard_layer_sequence needs a frozen cache")
    q0, q1, t0, t1 = sequence_shard_plan(layer._n_quant, layer.k_topk.shape[1], world)[rank]
    tail = rank == world - 1
    s = DStageLayerCache(layer.layer_idx, layer.k_bits, layer.v_bits, layer.window_size, layer.top_ratio, layer.use_vert)
    s._B, s._H_KV, s._D = layer._B, layer._H_KV, layer._D
    BH, dev = layer._kq.shape[0], layer._kq.device
    n = q1 - q0
    s._alloc_prefix(BH, n, dev)
    for dst, src in ((s._kq, layer._kq), (s._vq, layer._vq), (s._ks, layer._ks), (s._vs, layer._vs)):
        dst[:, :n].copy_(src[:, q0:q1])
    s._n_quant = n
    s.k_topk, s.v_topk = layer.k_topk[:, t0:t1].contiguous(), layer.v_topk[:, t0:t1].contiguous()
    w = layer.k_window.shape[1] if tail else 0
    s.k_window, s.v_window = layer.k_window[:, :w].contiguous(), layer.v_window[:, :w].contiguous()
    s._staging_buf_k = layer._staging_buf_k.clone() if tail else torch.zeros_like(layer._staging_buf_k)
    s._staging_buf_v = layer._staging_buf_v.clone() if tail else torch.zeros_like(layer._staging_buf_v)
    s._staging_ptr = layer._staging_ptr if tail else 0
    assert s._staging_buf_k.shape[1] == GROUP_SIZE
    s._seq_len = n + (t1 - t0) + w + s._staging_ptr
    s._lib = layer._lib
    s.phase = "decode"
    return s


def shard_layer_heads(layer, world: int, rank: int):
    """This rank's KV-head group of a frozen ``DStageLayerCache`` that holds the whole cache: a new layer cache
    owning copies of kv-heads ``kv_head_range(H_KV, world, rank)`` of every batch entry (all four segments).  Its
    decode output equals rows ``[h0 * R, h1 * R)`` of every batch entry of the full cache's output; nothing is
    exchanged between ranks."""
    from .d_stage_kv_cache import DStageLayerCache
    if layer.phase != "decode":
        raise ValueError("shard_layer_heads needs a frozen cache")
    B, H_KV = layer._B, layer._H_KV
    h0, h1 = kv_head_range(H_KV, world, rank)
    dev = layer._kq.device
    idx = (torch.arange(B, device=dev)[:, None] * H_KV + torch.arange(h0, h1, device=dev)[None, :]).reshape(-1)
    s = DStageLayerCache(layer.layer_idx, layer.k_bits, layer.v_bits, layer.window_size, layer.top_ratio, layer.use_vert)
    s._B, s._H_KV, s._D = B, h1 - h0, layer._D
    n = layer._n_quant
    s._alloc_prefix(idx.numel(), n, dev)
    for dst, src in ((s._kq, layer._kq), (s._vq, layer._vq), (s._ks, layer._ks), (s._vs, layer._vs)):
        dst[:, :n].copy_(src[idx, :n])
    s._n_quant = n
    s.k_topk, s.v_topk = layer.k_topk[idx].contiguous(), layer.v_topk[idx].contiguous()
    s.k_window, s.v_window = layer.k_window[idx].contiguous(), layer.v_window[idx].contiguous()
    s._staging_buf_k, s._staging_buf_v = layer._staging_buf_k[idx].contiguous(), layer._staging_buf_v[idx].contiguous()
    s._staging_ptr = layer._staging_ptr
    s._seq_len = layer._seq_len
    if layer.vertical_indices is not None:
        s.vertical_indices = layer.vertical_indices[:, h0:h1].contiguous()
    s._lib = layer._lib
    s.phase = "decode"
    return s


class PeerExchange:
    """Exchange buffers of a process group on one node, for ``hq_peer_exchange_merge``.

    Every rank allocates one buffer (``cudaMalloc`` inside the library), the 64-byte CUDA IPC handles are
    all-gathered through ``torch.distributed`` and each rank maps its peers' buffers.  ``rows`` = batch x query
    heads of the calls that will use it.  One instance serves any number of layers: calls are numbered by
    ``next_seq()``, and every rank must make the same calls in the same order on one stream."""

    def __init__(self, rows: int, group=None, timeout_s: float = 2.0):
        import torch.distributed as dist
        from . import _lib
        self._lib = _lib.lib()
        self.group, self.rows = group, rows
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.timeout_ns = int(timeout_s * 1e9)
        nbytes = C.c_int64()
        _lib.check(self._lib.hq_peer_exchange_bytes(self.world, rows, C.byref(nbytes)), "hq_peer_exchange_bytes")
        self.nbytes = nbytes.value
        self._local = C.c_void_p()
        handle = C.create_string_buffer(64)
        _lib.check(self._lib.hq_peer_buffer_create(self.nbytes, C.byref(self._local), handle), "hq_peer_buffer_create")
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        for j, h in enumerate(handles):
            if j == self.rank:
                self.ptrs.append(self._local.value)
                continue
            p = C.c_void_p()
            _lib.check(self._lib.hq_peer_buffer_open(h, C.byref(p)), "hq_peer_buffer_open")
            self.ptrs.append(p.value)
            self._opened.append(p.value)
        dist.barrier(group=group)          # every buffer exists, is zero-filled and mapped before the first call
        self.seq = 0
        self._slots = {}
        self._args = _lib.PeerExchangeArgs()
        a = self._args
        a.struct_bytes, a.world, a.rank, a.rows, a.timeout_ns = C.sizeof(_lib.PeerExchangeArgs), self.world, self.rank, rows, self.timeout_ns
        for j, ptr in enumerate(self.ptrs):
            a.bufs[j] = ptr
        self._bufs_arr = (C.c_void_p * 16)(*self.ptrs)
        self.bufs_addr = C.addressof(self._bufs_arr)     # for hq_decode_args.peer_bufs

    def next_seq(self) -> int:
        self.seq += 1
        return self.seq

    def slot(self, seq: int) -> Tuple[int, int, int]:
        """Device addresses of this rank's ``m``, ``l``, ``acc`` for call ``seq`` (where the decode kernel writes)."""
        from . import _lib
        got = self._slots.get(seq & 1)
        if got is None:
            m, l, acc = C.c_void_p(), C.c_void_p(), C.c_void_p()
            _lib.check(self._lib.hq_peer_slot(self._local, self.world, self.rows, seq, C.byref(m), C.byref(l),
                                              C.byref(acc)), "hq_peer_slot")
            got = self._slots[seq & 1] = (m.value, l.value, acc.value)
        return got

    def exchange_merge(self, seq: int, out: torch.Tensor):
        from . import _lib
        a = self._args
        a.seq, a.out, a.out_stride, a.out_dtype = seq, out.data_ptr(), out.stride(0), _lib.dtype_code(out.dtype)
        rc = self._lib.hq_peer_exchange_merge(C.byref(a), _lib.stream_ptr(out.device))
        if rc != 0:
            _lib.check(rc, "hq_peer_exchange_merge")

    def status(self) -> int:
        """The buffer's status word (bit 1: a wait for a peer ran out); synchronises the device."""
        from . import _lib
        word = C.c_int(0)
        _lib.check(self._lib.hq_peer_status(self._local, C.byref(word)), "hq_peer_status")
        return word.value

    def close(self):
        """Unmap the peers' buffers and free the local one; every rank calls it (it synchronises the group first)."""
        import torch.distributed as dist
        if self._local.value is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        for ptr in self._opened:
            self._lib.hq_peer_buffer_close(ptr)
        dist.barrier(group=self.group)
        self._lib.hq_peer_buffer_destroy(self._local)
        self._local = C.c_void_p()
        self._opened = []


class SequenceShardedLayer:
    """One rank's shard of a frozen layer cache plus the merge step.

    ``layer`` is a ``DStageLayerCache`` in decode phase that holds only this rank's
    ranges (empty window/staging on every rank but the last).  ``decode_attention``
    returns the full result on every rank."""

    def __init__(self, layer, group=None, exchange="nccl", fused=False):
        """``exchange``: a :class:`PeerExchange` (exchange and merge over peer memory), or ``"nccl"``
        (all-gather, then merge).  With a PeerExchange, ``fused`` picks between a second small kernel doing the
        exchange and the merge with one block per query row (``hq_peer_exchange_merge``, the default: measured
        faster at 2 and 8 GPUs) and the decode kernel doing them itself in the block that finishes a kv-head (one
        launch per call; few blocks do all the waiting, which costs more than the launch it saves when there are
        few kv-heads with many query heads each)."""
        self.layer = layer
        self.group = group
        self.exchange = exchange
        self.fused = fused
        self._bufs = None

    def append_staging(self, key_states, value_states, is_tail_rank: bool):
        if is_tail_rank:
            self.layer.append_staging(key_states, value_states)

    def decode_step(self, query_states, key_states, value_states, kv_repeat: int, is_tail_rank: bool,
                    out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``append_staging`` + ``decode_attention``; on the tail rank the decode kernel takes the new token
        itself (``DStageLayerCache.decode_step``), the other ranks have nothing to append."""
        return self.decode_attention(query_states, kv_repeat, out=out, new_kv=(key_states, value_states) if is_tail_rank else None)

    def decode_attention(self, query_states: torch.Tensor, kv_repeat: int, out: Optional[torch.Tensor] = None,
                         new_kv=None) -> torch.Tensor:
        """Partial decode over this rank's shard, exchange of the per-rank message
        ``m [rows] | l [rows] | acc [rows, D]`` (the kernel writes straight into it), merge on every rank.
        ``out``: an optional [B, H_Q, 1, D] tensor with contiguous rows to write into."""
        import torch.distributed as dist
        from . import _lib
        B, H_Q, _, D = query_states.shape
        rows = B * H_Q

        def partial_decode(partial, out=None, peer=None):
            if new_kv is not None:
                self.layer.decode_step(query_states, new_kv[0], new_kv[1], kv_repeat, partial=partial, out=out, peer=peer)
            else:
                self.layer.decode_attention(query_states, kv_repeat, partial=partial, out=out, peer=peer)

        if out is None:
            out = torch.empty(B, H_Q, 1, D, dtype=query_states.dtype, device=query_states.device)
        out2 = out.view(rows, D)
        if isinstance(self.exchange, PeerExchange):
            px = self.exchange
            if px.rows != rows:
                raise ValueError(f"the exchange buffers were made for {px.rows} query rows, this call has {rows}")
            seq = px.next_seq()
            if self.fused:
                partial_decode(None, out=out, peer=(px, seq))
            else:
                partial_decode(px.slot(seq))
                px.exchange_merge(seq, out2)
            return out
        world = dist.get_world_size(self.group)
        if self._bufs is None or self._bufs[0].numel() != rows * (D + 2):
            dev = query_states.device
            msg = torch.empty(rows * (D + 2), dtype=torch.float32, device=dev)
            self._bufs = (msg, torch.empty(world, rows * (D + 2), dtype=torch.float32, device=dev))
        msg, gathered = self._bufs
        m, l, acc = msg[:rows], msg[rows:2 * rows], msg[2 * rows:].view(rows, D)
        partial_decode((m, l, acc))
        dist.all_gather_into_tensor(gathered, msg, group=self.group)
        base, fl, stride = gathered.data_ptr(), 4, gathered.stride(0)
        rc = _lib.lib().hq_lse_merge_strided(base, base + fl * rows, base + fl * 2 * rows, stride, stride, stride, world, rows,
                                             out2.data_ptr(), _lib.dtype_code(out2.dtype), out2.stride(0),
                                             _lib.stream_ptr(out2.device))
        _lib.check(rc, "hq_lse_merge_strided")
        return out
