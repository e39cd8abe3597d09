"""One generated token's decode attention for every layer as ONE CUDA-graph replay.

The reference appends and attends layer by layer from Python, with the cache lengths as host integers
(``src/ops/d_stage_kv_cache.py:195-303``); here the lengths travel with the step's inputs: the caller fills one pinned
host message (every layer's new q / k / v rows), :class:`DecodeStepGraph` adds every layer's ``(n_quant, n_staging)``,
and the replayed graph is copy in -> one fused append + attention launch per layer -> copy out.  The decode kernels
read the lengths from the message (``hq_decode_args.lengths``), so the same graph serves every step; only the step on
which a staging buffer fills (one in 128) runs eagerly, because it quantises 128 tokens first.
"""

from __future__ import annotations

from typing import List

import torch

from ._lib import HyQuantError


class DecodeStepGraph:
    def __init__(self, layers: List, batch: int, h_q: int, h_kv: int, device=None):
        if not layers or any(l.phase != "decode" for l in layers):
            raise HyQuantError("DecodeStepGraph needs frozen layer caches")
        self.layers, self.B, self.H_Q, self.H_KV = layers, batch, h_q, h_kv
        self.R = h_q // h_kv
        dev = layers[0].k_window.device if device is None else device
        n, D = len(layers), 128
        rows = batch * (h_q + 2 * h_kv)
        self._row_bytes = rows * D * 2
        msg = n * self._row_bytes + n * 8                       # q | k | v rows of every layer, then (n_quant, n_staging) per layer
        self.host_in = torch.zeros(msg, dtype=torch.uint8).pin_memory()
        self.dev_in = torch.zeros(msg, dtype=torch.uint8, device=dev)
        self.host_out = torch.empty(n, batch, h_q, 1, D, dtype=torch.bfloat16).pin_memory()
        self.dev_out = torch.empty(n, batch, h_q, 1, D, dtype=torch.bfloat16, device=dev)

        def views(buf):
            x = buf[:n * self._row_bytes].view(torch.bfloat16).view(n, rows, D)
            q = [x[i, :batch * h_q].view(batch, h_q, 1, D) for i in range(n)]
            k = [x[i, batch * h_q:batch * (h_q + h_kv)].view(batch, h_kv, 1, D) for i in range(n)]
            v = [x[i, batch * (h_q + h_kv):].view(batch, h_kv, 1, D) for i in range(n)]
            return q, k, v, buf[n * self._row_bytes:].view(torch.int32).view(n, 2)

        self.host_q, self.host_k, self.host_v, self._host_len = views(self.host_in)     # the caller fills host_q/k/v
        self._host_len_np = self._host_len.numpy()        # same memory; element-wise tensor writes would cost microseconds each
        self._q, self._k, self._v, self._len = views(self.dev_in)
        for i, layer in enumerate(layers):
            layer.bind_lengths(self._len[i])
        self._graph = None
        self._warm = False

    def _eager(self):
        self.dev_in.copy_(self.host_in, non_blocking=True)
        for i, layer in enumerate(self.layers):
            layer.decode_step(self._q[i], self._k[i], self._v[i], self.R, out=self.dev_out[i])
        self.host_out.copy_(self.dev_out, non_blocking=True)

    def _capture(self):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.dev_in.copy_(self.host_in, non_blocking=True)
            for i, layer in enumerate(self.layers):
                # the first launch follows the copy, the others the previous layer's launch, which writes none of
                # this layer's cache: they may overlap its end
                layer.capture_decode_step(self._q[i], self._k[i], self._v[i], self.R, self.dev_out[i], overlap=i > 0)
            self.host_out.copy_(self.dev_out, non_blocking=True)
        self._graph = g
        self._ptrs = [l._kq.data_ptr() for l in self.layers]

    def step(self, synchronize: bool = True) -> torch.Tensor:
        """Run one token: ``host_q / host_k / host_v`` hold the new rows of every layer; returns ``host_out``
        ([layers, B, H_Q, 1, D], valid after the stream has been synchronised)."""
        from .d_stage_kv_cache import GROUP_SIZE
        flush = False
        lens = []
        for layer in self.layers:
            nq, ns = layer._n_quant, layer._staging_ptr
            if ns >= GROUP_SIZE - 1:           # that layer appends, quantises its 128 staged tokens, then attends
                nq, ns, flush = nq + GROUP_SIZE, 0, True
            lens.append((nq, ns))
        self._host_len_np[:] = lens
        if flush or not self._warm:
            self._eager()
            self._warm = True
            if flush and self._graph is not None and self._ptrs != [l._kq.data_ptr() for l in self.layers]:
                self._graph = None             # a prefix buffer was re-allocated to grow: capture again
        else:
            if self._graph is None:
                self._capture()
            self._graph.replay()
            for layer in self.layers:
                layer.count_replayed_step()
        if synchronize:
            torch.cuda.current_stream().synchronize()
        return self.host_out

    def close(self):
        for layer in self.layers:
            layer.bind_lengths(None)
        self._graph = None
