"""Multi-GPU decode: one process per GPU, ``torch.distributed`` for the plumbing.

Two ways the path shards (the reference itself has neither; results equal the
single-GPU result):

* KV-head groups — every (batch, kv-head) is independent in decode, flush, freeze and
  prefill, so rank r owns kv-heads ``kv_head_range(H_KV, world, r)`` and their query
  heads.  No collective on the data path; outputs stay per rank.
* Sequence shards (very long prefixes) — contiguous 128-token-aligned ranges of the INT4
  prefix and contiguous ranges of the BF16 vertical-line segment per rank; window and
  staging live on the last rank, which also receives the staging flushes.  Each rank runs
  the decode kernel in partial mode, the un-normalised softmax states ``(m, l, acc)`` are
  all-gathered (NCCL over NVLink; 66.5 KB per rank at B=4, 32 query heads) and merged by
  ``hq_lse_merge`` on every rank.
"""

from __future__ import annotations

from typing import List, Optional, Tuple

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


class SequenceShardedLayer:
    """One rank's shard of a frozen layer cache plus the merge step.

    ``layer`` is a ``DStageLayerCache`` in decode phase that holds only this rank's
    ranges (empty window/staging on every rank but the last).  ``decode_attention``
    returns the full result on every rank."""

    def __init__(self, layer, group=None):
        self.layer = layer
        self.group = group
        self._bufs = None

    def append_staging(self, key_states, value_states, is_tail_rank: bool):
        if is_tail_rank:
            self.layer.append_staging(key_states, value_states)

    def decode_attention(self, query_states: torch.Tensor, kv_repeat: int) -> torch.Tensor:
        """Partial decode over this rank's shard, one all-gather of the per-rank message
        ``m [rows] | l [rows] | acc [rows, D]`` (the kernel writes straight into it), merge on every rank."""
        import torch.distributed as dist
        from . import _lib
        B, H_Q, _, D = query_states.shape
        rows = B * H_Q
        world = dist.get_world_size(self.group)
        if self._bufs is None or self._bufs[0].numel() != rows * (D + 2):
            dev = query_states.device
            msg = torch.empty(rows * (D + 2), dtype=torch.float32, device=dev)
            self._bufs = (msg, torch.empty(world, rows * (D + 2), dtype=torch.float32, device=dev))
        msg, gathered = self._bufs
        m, l, acc = msg[:rows], msg[rows:2 * rows], msg[2 * rows:].view(rows, D)
        self.layer.decode_attention(query_states, kv_repeat, partial=(m, l, acc))
        dist.all_gather_into_tensor(gathered, msg, group=self.group)
        out = torch.empty(rows, D, dtype=query_states.dtype, device=query_states.device)
        base, fl, stride = gathered.data_ptr(), 4, gathered.stride(0)
        rc = _lib.lib().hq_lse_merge_strided(base, base + fl * rows, base + fl * 2 * rows, stride, stride, stride, world, rows,
                                             out.data_ptr(), _lib.dtype_code(out.dtype), out.stride(0),
                                             _lib.stream_ptr(out.device))
        _lib.check(rc, "hq_lse_merge_strided")
        return out.reshape(B, H_Q, 1, D)
