"""Four-segment KV cache for decode — host-side mirror of the reference module
``src/ops/d_stage_kv_cache.py`` (``DStageLayerCache`` / ``DStageKVCache``: same
constructor, methods, attributes and Hugging Face ``Cache`` surface).

Layout in HBM, all at KV-head granularity (BH = B * H_KV):
  k/v_quant_packed  int8 [BH, cap, 64]   INT4 prefix, 2 codes per byte, pre-allocated capacity
  k/v_scale         fp16 [BH, cap]       per-token scales
  k/v_topk          bf16 [BH, T, 128]    frozen vertical-line tokens (descending score)
  k/v_window        bf16 [BH, W, 128]    last-W prefill tokens
  _staging_buf_k/v  bf16 [BH, 128, 128]  decode tokens waiting to be quantised

Differences from the reference by design: the prefix lives in capacity buffers
that the staging flush appends to in place (no O(N) ``torch.cat`` per flush), the
prefill->decode transition runs as three kernels (scores, top-k, fused
gather/compact/quantise) and decode attention is one kernel launch.  The public
attributes (``k_quant_packed`` ...) are views of the live part of those buffers.
"""

from __future__ import annotations

import os
from typing import Any, Callable, Optional, Tuple

import torch

from . import _lib
from ._lib import HyQuantError
from . import decode_d_stage as _dd
from .decode_d_stage import GROUP_SIZE, DecodePlan, quantize_per_token_into
from .patch._common import topk_indices, vertical_scores, vertical_topk_count

try:
    from transformers.cache_utils import Cache as _HF_Cache
except Exception:  # transformers not available
    _HF_Cache = object


def _check_decode_kernel_env():
    choice = os.environ.get("HYBRID_ATTN_DECODE_KERNEL", "sm100").lower()
    if choice not in ("sm100", "splitk_mma"):
        raise HyQuantError(
            f"HYBRID_ATTN_DECODE_KERNEL={choice!r}: this build has one decode kernel (sm100) and no "
            "PyTorch/Triton fallback")


class DStageLayerCache:
    """Per-layer KV cache with the prefill -> decode phase transition."""

    def __init__(self, layer_idx: int, k_bits: int = 4, v_bits: int = 4, window_size: int = 256,
                 top_ratio: float = 0.05, use_vert: bool = True):
        self.layer_idx = layer_idx
        self.k_bits = k_bits
        self.v_bits = v_bits
        self.window_size = window_size
        self.top_ratio = top_ratio
        self.use_vert = use_vert
        self.phase: str = "prefill"
        self._seq_len: int = 0
        self._keys: Optional[torch.Tensor] = None        # [B, H_KV, N, D]
        self._values: Optional[torch.Tensor] = None
        self._query_tail: Optional[torch.Tensor] = None   # [B, H_Q, W, D]
        self._kq: Optional[torch.Tensor] = None           # capacity buffers
        self._vq: Optional[torch.Tensor] = None
        self._ks: Optional[torch.Tensor] = None
        self._vs: Optional[torch.Tensor] = None
        self._n_quant: int = 0
        self.k_topk: Optional[torch.Tensor] = None
        self.v_topk: Optional[torch.Tensor] = None
        self._staging_buf_k: Optional[torch.Tensor] = None
        self._staging_buf_v: Optional[torch.Tensor] = None
        self._staging_ptr: int = 0
        self.k_window: Optional[torch.Tensor] = None
        self.v_window: Optional[torch.Tensor] = None
        self._B = self._H_KV = self._D = 0
        self._plan: Optional[DecodePlan] = None
        self._lib = None
        self.vertical_indices: Optional[torch.Tensor] = None   # [B, H_KV, T] chosen at freeze
        self.overlap_previous: bool = True     # decode launches may overlap the end of the previous kernel
        self._plan_fresh: bool = False
        self._lengths: Optional[torch.Tensor] = None   # device int32 [2] = (n_quant, n_staging) the kernel reads, if bound

    # ---- views of the live prefix (reference attribute names) -----------------
    @property
    def k_quant_packed(self):
        return None if self._kq is None else self._kq[:, :self._n_quant]

    @property
    def v_quant_packed(self):
        return None if self._vq is None else self._vq[:, :self._n_quant]

    @property
    def k_scale(self):
        return None if self._ks is None else self._ks[:, :self._n_quant]

    @property
    def v_scale(self):
        return None if self._vs is None else self._vs[:, :self._n_quant]

    # ---- prefill --------------------------------------------------------------
    def update_prefill(self, key_states: torch.Tensor, value_states: torch.Tensor):
        """Accumulate BF16 K/V during prefill (reference :82-95)."""
        if self._keys is None:
            self._keys, self._values = key_states, value_states
        else:
            self._keys = torch.cat([self._keys, key_states], dim=2)
            self._values = torch.cat([self._values, value_states], dim=2)
        self._seq_len = self._keys.shape[2]
        return self._keys, self._values

    def save_query_tail(self, query_states: torch.Tensor):
        """Keep the last W queries of the prefill for freeze (reference :97-100)."""
        W = min(self.window_size, query_states.shape[2])
        self._query_tail = query_states[:, :, -W:, :].detach()

    # ---- prefill -> decode ----------------------------------------------------
    def _alloc_prefix(self, BH: int, n: int, device):
        cap = n + max(8 * GROUP_SIZE, n // 8)
        cap = (cap + GROUP_SIZE - 1) // GROUP_SIZE * GROUP_SIZE
        if self.k_bits == self.v_bits:
            # K and V codes of a head as two planes of one tensor [BH, 2, cap, row]: the decode kernel then fetches a
            # unit's K rows and V rows with one tensor-map request instead of two copies (hq_decode_splitk looks for
            # this layout through the pointers and strides it is given)
            kv = torch.empty(BH, 2, cap, self._D * self.k_bits // 8, dtype=torch.int8, device=device)
            self._kq, self._vq = kv[:, 0], kv[:, 1]
        else:
            self._kq = torch.empty(BH, cap, self._D * self.k_bits // 8, dtype=torch.int8, device=device)
            self._vq = torch.empty(BH, cap, self._D * self.v_bits // 8, dtype=torch.int8, device=device)
        self._ks = torch.empty(BH, cap, dtype=torch.float16, device=device)
        self._vs = torch.empty(BH, cap, dtype=torch.float16, device=device)

    def _grow_prefix(self, need: int):
        BH, cap = self._kq.shape[0], self._kq.shape[1]
        if need <= cap:
            return
        old = (self._kq, self._vq, self._ks, self._vs)
        self._alloc_prefix(BH, max(need, cap + cap // 2), self._kq.device)
        n = self._n_quant
        self._kq[:, :n].copy_(old[0][:, :n]); self._vq[:, :n].copy_(old[1][:, :n])
        self._ks[:, :n].copy_(old[2][:, :n]); self._vs[:, :n].copy_(old[3][:, :n])

    def freeze(self, kv_repeat: int = 1, *, vertical_indices: Optional[torch.Tensor] = None):
        """Quantise the prefix, keep window + vertical-line tokens in BF16, release
        the BF16 K/V (reference :106-189, including its candidate range: the
        selection helper subtracts the window from the already-sliced prefix, so
        vertical lines are chosen among positions [0, N - 2W)).

        ``vertical_indices`` (int64 [B, H_KV, T], distinct prefix positions per
        head, an extension of the reference signature) skips the selection and
        freezes exactly those rows in BF16, in the given order."""
        assert self.phase == "prefill" and self._keys is not None
        if self.k_bits not in (2, 4, 8) or self.v_bits not in (2, 4, 8):
            raise HyQuantError(f"bit widths must be 2, 4 or 8, got K{self.k_bits}/V{self.v_bits}")
        _lib.require_cuda(self._keys, "keys")
        B, H_KV, N, D = self._keys.shape
        if D != 128:
            raise HyQuantError(f"head_dim {D} is not built (128 only)")
        self._B, self._H_KV, self._D = B, H_KV, D
        BH = B * H_KV
        W = min(self.window_size, N)
        prefix_len = N - W
        device = self._keys.device
        dtype = self._keys.dtype
        keys = self._keys if self._keys.dtype == torch.bfloat16 else self._keys.to(torch.bfloat16)
        values = self._values if self._values.dtype == torch.bfloat16 else self._values.to(torch.bfloat16)
        keys = keys.reshape(BH, N, D) if keys.is_contiguous() else keys.contiguous().reshape(BH, N, D)
        values = values.reshape(BH, N, D) if values.is_contiguous() else values.contiguous().reshape(BH, N, D)

        T = 0
        vidx = vasc = None
        if vertical_indices is not None and prefix_len > 0 and vertical_indices.shape[-1] > 0:
            vidx = vertical_indices.to(device=device, dtype=torch.int64).reshape(B, H_KV, -1).contiguous()
            T = int(vidx.shape[-1])
            vasc = vidx.sort(dim=-1).values.to(torch.int32).contiguous()
        elif vertical_indices is None and prefix_len > 0 and self.use_vert and self._query_tail is not None \
                and kv_repeat >= 1:
            cand = max(0, prefix_len - self.window_size)
            if cand > 0:
                # group mean of the saved queries, in the input dtype like the reference (:131-133): inside the
                # scoring call when the queries already have the keys' 16-bit dtype
                kpre = keys.reshape(B, H_KV, N, D)[:, :, :prefix_len]
                if kv_repeat > 1 and self._query_tail.dtype == keys.dtype:
                    scores = vertical_scores(self._query_tail, kpre, self.window_size, 1, group_mean=kv_repeat)
                else:
                    q_kv = self._query_tail.reshape(B, H_KV, kv_repeat, -1, D).mean(dim=2)
                    scores = vertical_scores(q_kv.to(keys.dtype), kpre, self.window_size, 1)
                T = vertical_topk_count(cand, self.top_ratio)
                vidx, vasc = topk_indices(scores, T, want_ascending=True)       # [B, H_KV, T]
        self.vertical_indices = vidx
        n_quant = prefix_len - T
        self._alloc_prefix(BH, n_quant, device)
        self.k_topk = torch.empty(BH, T, D, dtype=torch.bfloat16, device=device)
        self.v_topk = torch.empty(BH, T, D, dtype=torch.bfloat16, device=device)
        self.k_window = torch.empty(BH, W, D, dtype=torch.bfloat16, device=device)
        self.v_window = torch.empty(BH, W, D, dtype=torch.bfloat16, device=device)
        rc = _lib.lib().hq_cache_reorganize_bits(
            keys.data_ptr(), values.data_ptr(), keys.stride(0), BH, N, W, T,
            vidx.data_ptr() if T else None, vasc.data_ptr() if T else None,
            self.k_topk.data_ptr(), self.v_topk.data_ptr(), self.k_window.data_ptr(), self.v_window.data_ptr(),
            self._kq.data_ptr(), self._vq.data_ptr(), self._kq.stride(0), self._vq.stride(0),
            self._ks.data_ptr(), self._vs.data_ptr(), self._ks.stride(0),
            self.k_bits, self.v_bits, _dd.SCALE_MODE, _lib.stream_ptr(device))
        _lib.check(rc, "hq_cache_reorganize_bits")
        self._n_quant = n_quant
        if dtype != torch.bfloat16:   # keep the reference's attribute dtype for non-bf16 models
            self.k_topk, self.v_topk = self.k_topk.to(dtype), self.v_topk.to(dtype)
            self.k_window, self.v_window = self.k_window.to(dtype), self.v_window.to(dtype)
        self._staging_buf_k = torch.zeros(BH, GROUP_SIZE, D, device=device, dtype=dtype)
        self._staging_buf_v = torch.zeros(BH, GROUP_SIZE, D, device=device, dtype=dtype)
        self._staging_ptr = 0
        self._keys = self._values = self._query_tail = None
        self._plan = None
        self._lib = _lib.lib()
        self.phase = "decode"

    # ---- decode ---------------------------------------------------------------
    def append_staging(self, key_states: torch.Tensor, value_states: torch.Tensor):
        """Append new decode token(s) to the staging ring (reference :195-207)."""
        B, H_KV, S, D = key_states.shape
        BH = B * H_KV
        if (S == 1 and key_states.dtype == torch.bfloat16 and self._staging_buf_k.dtype == torch.bfloat16
                and key_states.stride(3) == 1 and value_states.stride(3) == 1):
            # one token: a single small kernel instead of two strided tensor copies
            k2, v2 = key_states.reshape(BH, D), value_states.reshape(BH, D)
            rc = self._lib.hq_staging_append(k2.data_ptr(), v2.data_ptr(), k2.stride(0), v2.stride(0),
                                             self._staging_buf_k.data_ptr(), self._staging_buf_v.data_ptr(), BH,
                                             self._staging_ptr, _lib.stream_ptr(k2.device))
            if rc != 0:
                _lib.check(rc, "hq_staging_append")
            self._staging_ptr += 1
            if self._staging_ptr >= GROUP_SIZE:
                self._flush_staging_buffer()
            self._seq_len += 1
            return
        k = key_states.reshape(BH, S, D)
        v = value_states.reshape(BH, S, D)
        # several tokens (or another dtype): one copy per run of tokens up to the next flush, not one per token
        i = 0
        while i < S:
            r = min(GROUP_SIZE - self._staging_ptr, S - i)
            self._staging_buf_k[:, self._staging_ptr:self._staging_ptr + r].copy_(k[:, i:i + r])
            self._staging_buf_v[:, self._staging_ptr:self._staging_ptr + r].copy_(v[:, i:i + r])
            self._staging_ptr += r
            i += r
            if self._staging_ptr >= GROUP_SIZE:
                self._flush_staging_buffer()
        self._seq_len += S

    def _flush_staging_buffer(self):
        """Quantise the full staging buffer and append it to the prefix in place
        (reference :209-217)."""
        n = self._n_quant
        if n + GROUP_SIZE > self._kq.shape[1]:
            self._grow_prefix(n + GROUP_SIZE)
            self._plan = None
        quantize_per_token_into(self._staging_buf_k, self._kq, self._ks, n, nbits=self.k_bits)
        quantize_per_token_into(self._staging_buf_v, self._vq, self._vs, n, nbits=self.v_bits)
        self._n_quant = n + GROUP_SIZE
        self._staging_ptr = 0

    def _decode_plan(self, q2d: torch.Tensor, kv_repeat: int) -> DecodePlan:
        if self._staging_buf_k.dtype != torch.bfloat16:
            _check_decode_kernel_env()
            # non-bf16 models: segments are cast on the way in (as the reference kernel
            # does on load), so nothing can be cached across steps
            return DecodePlan(q2d, self.k_quant_packed, self.v_quant_packed, self.k_scale, self.v_scale,
                              self.k_topk, self.v_topk, self._staging_buf_k[:, :self._staging_ptr],
                              self._staging_buf_v[:, :self._staging_ptr], self.k_window, self.v_window,
                              kv_repeat, None, k_bits=self.k_bits, v_bits=self.v_bits)
        p = self._plan
        if p is None or p.kv_repeat != kv_repeat:
            _check_decode_kernel_env()
            # After freeze this cache's segments are written only by its own staging append and
            # flush kernels (staging buffer, newest 128 prefix tokens), so the decode kernel may
            # start fetching older units while whatever runs just before it finishes.  The
            # first decode after a freeze or a prefix growth is launched plainly: the kernel
            # before it may be the one that wrote the whole prefix.
            p = DecodePlan(q2d, self._kq, self._vq, self._ks, self._vs, self.k_topk, self.v_topk,
                           self._staging_buf_k, self._staging_buf_v, self.k_window, self.v_window,
                           kv_repeat, None, overlap_previous=self.overlap_previous, k_bits=self.k_bits, v_bits=self.v_bits)
            p.args.flags = 0
            self._plan = p
            self._plan_fresh = True
        elif self.overlap_previous and self._plan_fresh:
            self._plan_fresh = False
            p.args.flags = _lib.HQ_DECODE_OVERLAP_PREVIOUS
        p.args.n_quant = self._n_quant
        p.args.n_staging = self._staging_ptr
        p.args.lengths = None if self._lengths is None else self._lengths.data_ptr()
        return p

    def decode_attention(self, query_states: torch.Tensor, kv_repeat: int, *, partial=None,
                         out: Optional[torch.Tensor] = None, peer=None) -> torch.Tensor:
        """Attention of one new token over the four segments (reference :219-303).

        query_states [B, H_Q, 1, D] -> [B, H_Q, 1, D] in the query dtype.
        ``partial=(m, l, acc)`` requests the un-normalised softmax state instead
        (sequence-sharded decode).  ``out`` (not in the reference): a [B, H_Q, 1, D] tensor with
        contiguous rows to write into instead of a new one."""
        B_, H_Q_, _, D_ = query_states.shape
        q2d = query_states.reshape(B_ * H_Q_, D_)
        plan = self._decode_plan(q2d, kv_repeat)
        res = plan.run(q2d, out=None if out is None else out.view(B_ * H_Q_, D_), partial=partial, peer=peer)
        if partial is not None:
            return None
        return out if out is not None else res.reshape(B_, H_Q_, 1, D_)

    @staticmethod
    def _rope_eager(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
        """x cos + rotate_half(x) sin in x's dtype, as Hugging Face's apply_rotary_pos_emb does ([B, H, 1, D] with [B, D])."""
        half = x.shape[-1] // 2
        rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
        return (x * cos[:, None, None, :]) + (rot * sin[:, None, None, :])

    def decode_step(self, query_states: torch.Tensor, key_states: torch.Tensor, value_states: torch.Tensor,
                    kv_repeat: int, *, out: Optional[torch.Tensor] = None, partial=None, peer=None, rope=None) -> torch.Tensor:
        """``append_staging(key_states, value_states)`` followed by ``decode_attention(query_states, kv_repeat)``
        (reference :195-303) as one kernel launch: the decode kernel attends to the new token from where it
        is and stores it into its staging slot on the way.  Same result as the two calls up to the order of
        the fp32 partial sums.  The step that fills the staging buffer takes the two-call route, because the
        reference flushes (quantises the 128 staged tokens) before that step's attention.

        ``rope=(cos, sin)`` (not in the reference, whose patched forwards rotate q and k with separate eager kernels before
        the cache, src/patch/patch_llama.py:58-65): bf16 ``[B, D]`` or ``[B, 1, D]`` rotary factors of this step's position;
        ``query_states`` and ``key_states`` are then given UNROTATED and the kernel rotates them itself."""
        B, H_KV, S, D = key_states.shape
        cos = sin = None
        if rope is not None:
            cos, sin = (t.reshape(B, D) for t in rope)
        fused = (S == 1 and self._staging_ptr < GROUP_SIZE - 1
                 and key_states.dtype == torch.bfloat16 and value_states.dtype == torch.bfloat16
                 and self._staging_buf_k.dtype == torch.bfloat16 and key_states.stride(3) == 1 and value_states.stride(3) == 1)
        if fused:
            k2, v2 = key_states.reshape(B * H_KV, D), value_states.reshape(B * H_KV, D)
            fused = (k2.data_ptr() % 16 == 0 and v2.data_ptr() % 16 == 0 and k2.stride(0) % 8 == 0 and v2.stride(0) % 8 == 0)
            if fused and cos is not None:
                fused = (cos.dtype == torch.bfloat16 and sin.dtype == torch.bfloat16 and cos.stride(1) == 1 and sin.stride(1) == 1
                         and cos.stride(0) == sin.stride(0) and cos.stride(0) % 8 == 0 and cos.data_ptr() % 16 == 0
                         and sin.data_ptr() % 16 == 0 and query_states.dtype == torch.bfloat16)
        if not fused:
            if cos is not None:
                query_states, key_states = self._rope_eager(query_states, cos, sin), self._rope_eager(key_states, cos, sin)
            self.append_staging(key_states, value_states)
            return self.decode_attention(query_states, kv_repeat, out=out, partial=partial, peer=peer)
        B_, H_Q_, _, D_ = query_states.shape
        q2d = query_states.reshape(B_ * H_Q_, D_)
        plan = self._decode_plan(q2d, kv_repeat)
        a = plan.args
        a.k_new, a.v_new, a.kn_stride, a.vn_stride = k2.data_ptr(), v2.data_ptr(), k2.stride(0), v2.stride(0)
        if cos is not None:
            a.rope_cos, a.rope_sin, a.rope_stride, a.rope_heads_per_batch = cos.data_ptr(), sin.data_ptr(), cos.stride(0), H_KV
        try:
            res = plan.run(q2d, out=None if out is None else out.view(B_ * H_Q_, D_), partial=partial, peer=peer)
        finally:
            a.k_new = a.v_new = None
            a.rope_cos = a.rope_sin = None
        self._staging_ptr += 1
        self._seq_len += 1
        if partial is not None:
            return None
        return out if out is not None else res.reshape(B_, H_Q_, 1, D_)

    # ---- decode launches that stay valid in a CUDA graph --------------------------------------------
    def bind_lengths(self, record: Optional[torch.Tensor]):
        """Make the decode kernel take ``(n_quant, n_staging)`` from ``record`` (device int32 [2], e.g. a slice of the buffer
        the step's inputs are copied into) instead of from the launch arguments, so that a captured launch stays valid
        while the cache grows.  The caller writes :meth:`step_lengths` into it before each step; ``None`` unbinds."""
        if record is not None and (record.dtype != torch.int32 or record.numel() != 2 or not record.is_cuda):
            raise HyQuantError("the length record must be a CUDA int32 tensor of two elements")
        self._lengths = record
        self._plan = None

    def step_lengths(self) -> Tuple[int, int]:
        """``(n_quant, n_staging)`` as the next :meth:`decode_step` has to see them (before its token is counted)."""
        return self._n_quant, self._staging_ptr

    def next_step_flushes(self) -> bool:
        """True when the next appended token fills the staging buffer (that step quantises 128 tokens first)."""
        return self._staging_ptr >= GROUP_SIZE - 1

    def capture_decode_step(self, query_states, key_states, value_states, kv_repeat: int, out: torch.Tensor,
                            overlap: bool = True):
        """Issue the fused ``decode_step`` launch WITHOUT counting the token: for use inside a CUDA-graph capture
        (lengths bound with :meth:`bind_lengths`; every tensor argument must keep its address across replays).
        After each replay call :meth:`count_replayed_step`."""
        if self._lengths is None:
            raise HyQuantError("bind_lengths first: a captured launch must not carry the lengths in its arguments")
        B, H_KV, S, D = key_states.shape
        B_, H_Q_, _, D_ = query_states.shape
        q2d = query_states.reshape(B_ * H_Q_, D_)
        k2, v2 = key_states.reshape(B * H_KV, D), value_states.reshape(B * H_KV, D)
        plan = self._decode_plan(q2d, kv_repeat)
        a = plan.args
        a.flags = _lib.HQ_DECODE_OVERLAP_PREVIOUS if (overlap and self.k_bits == 4 and self.v_bits == 4) else 0
        a.k_new, a.v_new, a.kn_stride, a.vn_stride = k2.data_ptr(), v2.data_ptr(), k2.stride(0), v2.stride(0)
        try:
            plan.run(q2d, out=out.view(B_ * H_Q_, D_))
        finally:
            a.k_new = a.v_new = None

    def count_replayed_step(self):
        """Account for one replay of a launch captured by :meth:`capture_decode_step` (one token appended)."""
        if self._staging_ptr >= GROUP_SIZE - 1:
            raise HyQuantError("this step fills the staging buffer: it has to go through decode_step (flush), not a replay")
        self._staging_ptr += 1
        self._seq_len += 1

    def get_seq_length(self) -> int:
        return self._seq_len


class DStageKVCache(_HF_Cache):
    """The Hugging Face ``Cache`` surface of the reference's ``DStageKVCache`` (src/ops/d_stage_kv_cache.py:360-494),
    taken over method by method because generation code and the patched forwards call it by these names (``update``,
    ``get_seq_length``, ``get_mask_sizes``, ``get_layer``, ``crop`` ...).  It holds no algorithm: every layer is a
    :class:`DStageLayerCache`, whose freeze / append / attention run on this library's kernels."""

    is_compileable = False

    def __init__(self, num_layers: int = 32, k_bits: int | Callable[[int], int] = 4,
                 v_bits_fn: Callable[[int], int] = lambda i: 4 if i == 0 else 2,
                 window_size: int = 256, top_ratio: float = 0.05, use_vert: bool = True):
        try:
            super().__init__()
        except (TypeError, ValueError):
            # newer transformers require layer arguments this cache does not use;
            # provide the attributes their Cache helpers look at
            self.layers = []
            self.layer_class_to_replicate = None
            self.offloading = False
        self.num_layers = num_layers
        self.window_size = window_size
        self.top_ratio = top_ratio
        self.use_vert = use_vert
        k_bits_fn = k_bits if callable(k_bits) else (lambda i, _kb=k_bits: _kb)
        self._layers = [
            DStageLayerCache(layer_idx=i, k_bits=k_bits_fn(i), v_bits=v_bits_fn(i), window_size=window_size,
                             top_ratio=top_ratio, use_vert=use_vert)
            for i in range(num_layers)
        ]
        self._seen_tokens: int = 0

    def update(self, key_states: torch.Tensor, value_states: torch.Tensor, layer_idx: int,
               cache_kwargs: Optional[dict[str, Any]] = None) -> Tuple[torch.Tensor, torch.Tensor]:
        layer = self._layers[layer_idx]
        if layer.phase == "prefill":
            result = layer.update_prefill(key_states, value_states)
            if layer_idx == 0:
                self._seen_tokens = layer.get_seq_length()
            return result
        layer.append_staging(key_states, value_states)
        if layer_idx == 0:
            self._seen_tokens = layer.get_seq_length()
        return key_states, value_states

    def get_seq_length(self, layer_idx: int = 0) -> int:
        if layer_idx < len(self._layers):
            return self._layers[layer_idx].get_seq_length()
        return 0

    def get_max_cache_shape(self) -> int:
        return -1

    def reset(self):
        for layer in self._layers:
            layer.__init__(layer.layer_idx, layer.k_bits, layer.v_bits, layer.window_size, layer.top_ratio,
                           layer.use_vert)
        self._seen_tokens = 0

    def get_mask_sizes(self, query_length: int, layer_idx: int = 0) -> Tuple[int, int]:
        kv_length = self.get_seq_length(layer_idx)
        if kv_length == 0:
            return query_length, 0
        return kv_length, max(0, kv_length - query_length)

    def get_layer(self, layer_idx: int) -> DStageLayerCache:
        return self._layers[layer_idx]

    @property
    def seen_tokens(self) -> int:
        return self._seen_tokens

    def batch_repeat_interleave(self, repeats: int):
        raise NotImplementedError("DStageKVCache does not support beam search yet.")

    def batch_select_indices(self, indices: torch.Tensor):
        raise NotImplementedError("DStageKVCache does not support beam search yet.")

    def crop(self, max_length: int):
        pass

    def __len__(self) -> int:
        return self.num_layers

    def __getitem__(self, idx: int):
        layer = self._layers[idx]
        if layer.phase == "prefill" and layer._keys is not None:
            return (layer._keys, layer._values)
        return (None, None)

    def __iter__(self):
        for i in range(len(self._layers)):
            yield self[i]

    def __bool__(self) -> bool:
        return True


QuantizedKVCache = DStageKVCache
