"""Decode-side operators: per-token INT4 quantiser and the fused four-segment
decode attention.  Host-side mirror of the reference module
``src/ops/decode_d_stage.py`` (same names, argument meaning and return
conventions); the device work is done by the sm_100a kernels behind the C ABI
(``hq_quant_pack_int4``, ``hq_decode_splitk``).

What differs from the reference by design:
  * one kernel launch per decode call (split-K partials and their log-sum-exp
    merge are fused), no ``torch.cat`` of the BF16 segments;
  * K and V prefixes in 8, 4 or 2 bits, every pair by the same kernel;
  * CUDA tensors only — there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple

import torch

from . import _lib
from ._lib import DecodeArgs, HyQuantError

_LOG2_E = 1.44269504
GROUP_SIZE = 128  # staging flush threshold (tokens); reference decode_d_stage.py:19

# Scale rounding of the quantiser.  1 (default) = max|x| * fp32(1 / q_max): what eager PyTorch computes on a CUDA
# device, i.e. the reference's production path (its quantiser always runs on the GPU; pinned by the fixtures the
# reference produced on a B200).  0 = IEEE max|x| / q_max: eager PyTorch on the CPU, what the fixtures produced by
# running the reference on the CPU pin.  The two differ in the last bit of an fp16 scale in rare cases.
SCALE_MODE = 1


# ----------------------------------------------------------------------------
# quantise / dequantise (reference decode_d_stage.py:50-149)
# ----------------------------------------------------------------------------

def quantize_per_token_into(x: torch.Tensor, packed: torch.Tensor, scale: torch.Tensor,
                            dst_token_offset: int = 0, scale_mode: Optional[int] = None, nbits: int = 4) -> None:
    """Quantise ``x`` [BH, n, 128] and write codes/scales at token
    ``dst_token_offset`` of the capacity buffers ``packed`` [BH, cap, 16 * nbits] int8 and
    ``scale`` [BH, cap] fp16 (in-place append; replaces the ``torch.cat`` growth of
    ``_flush_staging_buffer``, reference d_stage_kv_cache.py:209-217)."""
    _lib.require_cuda(x, "x")
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8, got {nbits}")
    BH, n, D = x.shape
    if D != 128:
        raise HyQuantError(f"head_dim {D} is not built (128 only)")
    if x.stride(2) != 1 or x.stride(1) % 8 or x.stride(0) % 8 or x.data_ptr() % 16:
        x = x.contiguous()               # the kernel reads a row as 16-byte pieces
    if packed.dtype != torch.int8 or scale.dtype != torch.float16:
        raise HyQuantError("packed must be int8 and scale fp16")
    if packed.stride(2) != 1 or packed.stride(1) != 16 * nbits or scale.stride(1) != 1:
        raise HyQuantError(f"capacity buffers must be row-contiguous ([BH, cap, {16 * nbits}] / [BH, cap])")
    if dst_token_offset + n > packed.shape[1] or dst_token_offset + n > scale.shape[1]:
        raise HyQuantError("append exceeds the capacity of the quantised prefix buffers")
    rc = _lib.lib().hq_quant_pack(
        x.data_ptr(), _lib.dtype_code(x.dtype), x.stride(0), x.stride(1), BH, n, nbits,
        packed.data_ptr(), packed.stride(0), scale.data_ptr(), scale.stride(0),
        dst_token_offset, SCALE_MODE if scale_mode is None else scale_mode, _lib.stream_ptr(x.device))
    _lib.check(rc, "hq_quant_pack")


def quantize_per_token(x: torch.Tensor, nbits: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Per-token symmetric quantisation (reference decode_d_stage.py:50-77).

    x [BH, N, D] bf16/fp16/fp32 -> (packed [BH, N, D * nbits // 8] int8, scale [BH, N] fp16),
    bit-exact with the reference for nbits 2, 4 and 8.
    """
    if nbits not in (2, 4, 8):
        raise ValueError(f"nbits must be 2, 4, or 8, got {nbits}")
    _lib.require_cuda(x, "x")
    BH, N, D = x.shape
    packed = torch.empty(BH, N, D * nbits // 8, dtype=torch.int8, device=x.device)
    scale = torch.empty(BH, N, dtype=torch.float16, device=x.device)
    quantize_per_token_into(x, packed, scale, 0, nbits=nbits)
    return packed, scale


def _unpack_int4(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[BH, N, D//2] int8 -> [BH, N, D] float32, sign-extended (reference :114-123)."""
    x = packed.to(torch.int32) & 0xFF
    lo = ((x & 0x0F) << 28) >> 28
    hi = (((x >> 4) & 0x0F) << 28) >> 28
    out = torch.empty(packed.shape[0], packed.shape[1], D, device=packed.device, dtype=torch.float32)
    out[..., 0::2] = lo.float()
    out[..., 1::2] = hi.float()
    return out


def _unpack_int2(packed: torch.Tensor, D: int) -> torch.Tensor:
    """[BH, N, D//4] int8 -> [BH, N, D] float32, sign-extended (reference :138-150)."""
    x = packed.to(torch.int32) & 0xFF
    out = torch.empty(packed.shape[0], packed.shape[1], D, device=packed.device, dtype=torch.float32)
    for i in range(4):
        out[..., i::4] = ((((x >> (2 * i)) & 0x03) << 30) >> 30).float()
    return out


def dequantize_per_token(packed: torch.Tensor, scale: torch.Tensor, D: int, nbits: int) -> torch.Tensor:
    """Inverse of :func:`quantize_per_token` -> fp16 (reference :80-101).  A debugging
    utility built from torch ops; the decode kernels never materialise this."""
    if nbits == 8:
        q = packed.float()
    elif nbits == 4:
        q = _unpack_int4(packed, D)
    elif nbits == 2:
        q = _unpack_int2(packed, D)
    else:
        raise ValueError(f"nbits must be 2, 4, or 8, got {nbits}")
    return (q * scale.float().unsqueeze(-1)).to(torch.float16)


def _quantize_by_bits(x: torch.Tensor, bits: int):
    return quantize_per_token(x, bits)


def _dequantize_by_bits(packed, scale, D, bits):
    return dequantize_per_token(packed, scale, D, bits)


# ----------------------------------------------------------------------------
# decode attention (reference decode_d_stage.py:823-1005)
# ----------------------------------------------------------------------------

_ws_cache: dict = {}


def decode_workspace(device: torch.device, BH_KV: int, kv_repeat: int) -> torch.Tensor:
    """Scratch for the split-K partials and tickets, zero-filled once, cached per
    (device, stream, shape) — calls on different streams never share one."""
    stream = _lib.stream_ptr(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream, BH_KV, kv_repeat)
    ws = _ws_cache.get(key)
    if ws is None:
        nbytes = C.c_int64(0)
        _lib.check(_lib.lib().hq_decode_workspace_bytes(BH_KV, kv_repeat, C.byref(nbytes)), "hq_decode_workspace_bytes")
        ws = torch.zeros(int(nbytes.value), dtype=torch.uint8, device=device)
        _ws_cache[key] = ws
    return ws


def decode_status(ws: torch.Tensor) -> int:
    """Status word of a workspace (0 = ok, bit 0 = a bounded device wait expired)."""
    return int(ws[:4].view(torch.int32).item())


def _rows_ok(t: torch.Tensor, row_elems: int) -> bool:
    return t.stride(2) == 1 and t.stride(1) == row_elems and (t.stride(0) * t.element_size()) % 16 == 0 \
        and t.data_ptr() % 16 == 0


def _seg(t: Optional[torch.Tensor], row_elems: int) -> Optional[torch.Tensor]:
    if t is None or t.shape[1] == 0:
        return None
    return t if _rows_ok(t, row_elems) else t.contiguous()


class DecodePlan:
    """A filled ``hq_decode_args`` that can be re-launched with new q/out
    pointers and a new staging length — keeps per-step host work to a few
    attribute writes.  Holds references to every tensor it points at."""

    def __init__(self, q, k_quant_packed, v_quant_packed, k_scale, v_scale,
                 k_topk, v_topk, k_staging, v_staging, k_window, v_window,
                 kv_repeat: int, sm_scale: Optional[float], num_splits: int = 0, overlap_previous: bool = False,
                 k_bits: int = 4, v_bits: int = 4):
        """``overlap_previous``: launch with ``HQ_DECODE_OVERLAP_PREVIOUS`` — the kernel's blocks may
        start, and fetch cache units that are older than the newest 128 prefix tokens or lie in the
        vertical-line / window segments, while the kernel launched just before it on the stream is
        finishing.  Only for callers that know that kernel writes none of those."""
        _lib.require_cuda(q, "q")
        BH_Q, D = q.shape
        if D != 128:
            raise HyQuantError(f"head_dim {D} is not built (128 only)")
        if BH_Q % kv_repeat != 0:
            raise HyQuantError("q rows must be a multiple of kv_repeat")
        if not 1 <= kv_repeat <= 16:
            raise HyQuantError(f"kv_repeat {kv_repeat} outside 1..16")
        self.device = q.device
        self.BH_KV = BH_Q // kv_repeat
        self.kv_repeat = kv_repeat
        a = DecodeArgs()
        a.struct_bytes = C.sizeof(DecodeArgs)
        a.BH_KV, a.kv_repeat, a.head_dim = self.BH_KV, kv_repeat, D
        a.sm_scale = float(D ** -0.5 if sm_scale is None else sm_scale)
        a.num_splits = num_splits
        if k_bits not in (2, 4, 8) or v_bits not in (2, 4, 8):
            raise ValueError(f"bit widths must be 2, 4 or 8, got K{k_bits} V{v_bits}")
        a.k_bits, a.v_bits = k_bits, v_bits
        # the launch-overlap prologue belongs to the K4/V4 kernel
        a.flags = _lib.HQ_DECODE_OVERLAP_PREVIOUS if (overlap_previous and k_bits == 4 and v_bits == 4) else 0
        keep = []
        n_quant = 0 if k_quant_packed is None else int(k_quant_packed.shape[1])
        a.n_quant = n_quant
        if n_quant > 0:
            kp, vp = _seg(k_quant_packed, 16 * k_bits), _seg(v_quant_packed, 16 * v_bits)
            ks = k_scale if k_scale.stride(1) == 1 else k_scale.contiguous()
            vs = v_scale if v_scale.stride(1) == 1 else v_scale.contiguous()
            if ks.dtype != torch.float16 or vs.dtype != torch.float16 or kp.dtype != torch.int8:
                raise HyQuantError("packed K/V must be int8 and scales fp16")
            a.k_packed, a.v_packed = kp.data_ptr(), vp.data_ptr()
            a.kp_stride_bh, a.vp_stride_bh = kp.stride(0), vp.stride(0)
            a.k_scale, a.v_scale = ks.data_ptr(), vs.data_ptr()
            a.ks_stride_bh, a.vs_stride_bh = ks.stride(0), vs.stride(0)
            keep += [kp, vp, ks, vs]
        for name, kt, vt in (("topk", k_topk, v_topk), ("staging", k_staging, v_staging), ("window", k_window, v_window)):
            ks_, vs_ = _seg(kt, 128), _seg(vt, 128)
            n = 0 if ks_ is None else int(ks_.shape[1])
            if n > 0:
                if ks_.dtype != torch.bfloat16:
                    ks_, vs_ = ks_.to(torch.bfloat16), vs_.to(torch.bfloat16)   # the reference casts on load
                kptr, vptr, kst, vst = ks_.data_ptr(), vs_.data_ptr(), ks_.stride(0), vs_.stride(0)
                keep += [ks_, vs_]
            else:
                kptr = vptr = None
                kst = vst = 0
            if name == "topk":
                a.n_topk, a.k_topk, a.v_topk, a.kt_stride_bh, a.vt_stride_bh = n, kptr, vptr, kst, vst
            elif name == "staging":
                a.n_staging, a.k_staging, a.v_staging, a.kg_stride_bh, a.vg_stride_bh = n, kptr, vptr, kst, vst
            else:
                a.n_window, a.k_window, a.v_window, a.kw_stride_bh, a.vw_stride_bh = n, kptr, vptr, kst, vst
        self.ws = decode_workspace(q.device, self.BH_KV, kv_repeat)
        a.workspace, a.workspace_bytes = self.ws.data_ptr(), self.ws.numel()
        self.args = a
        self._keep = keep
        self._fn = _lib.lib().hq_decode_splitk

    def run(self, q: torch.Tensor, out: Optional[torch.Tensor] = None, partial=None, peer=None) -> torch.Tensor:
        """Launch on the current stream.  ``partial=(m, l, acc)`` fp32 tensors
        selects the un-normalised (sequence-sharded) output.  ``peer=(exchange, seq)``
        (a ``sharded.PeerExchange`` and the call's sequence number): this call covers one
        sequence shard; the kernel exchanges its state with the other ranks and ``out`` is
        the merged result."""
        a = self.args
        if peer is not None:
            px, seq = peer
            a.peer_bufs, a.peer_world, a.peer_rank, a.peer_seq, a.peer_timeout_ns = px.bufs_addr, px.world, px.rank, seq, px.timeout_ns
        else:
            a.peer_world = 0
        qb = q if (q.dtype == torch.bfloat16 and q.stride(1) == 1) else q.to(torch.bfloat16).contiguous()
        a.q, a.q_stride = qb.data_ptr(), qb.stride(0)
        if partial is not None:
            # fp32 tensors, or raw device addresses (slots of a peer-exchange buffer)
            a.partial_m, a.partial_l, a.partial_acc = [x if isinstance(x, int) else x.data_ptr() for x in partial]
            a.out, a.out_stride, a.out_dtype = None, 0, _lib.HQ_F32
        else:
            if out is None:
                out = torch.empty(q.shape[0], 128, dtype=q.dtype, device=q.device)
            a.partial_m = a.partial_l = a.partial_acc = None
            a.out, a.out_stride, a.out_dtype = out.data_ptr(), out.stride(0), _lib.dtype_code(out.dtype)
        rc = self._fn(C.byref(a), _lib.stream_ptr(self.device))
        if rc != 0:
            _lib.check(rc, "hq_decode_splitk")
        return out


def fused_d_stage_decode(
    q: torch.Tensor,                        # [BH_Q, D]
    k_quant_packed: torch.Tensor,           # [BH_KV, N_quant, D//2] int8
    v_quant_packed: torch.Tensor,
    k_scale: torch.Tensor,                  # [BH_KV, N_quant] fp16 per-token
    v_scale: torch.Tensor,
    k_topk: torch.Tensor,                   # [BH_KV, N_topk, D]
    v_topk: torch.Tensor,
    k_staging: torch.Tensor,                # [BH_KV, N_staging, D]
    v_staging: torch.Tensor,
    k_window: torch.Tensor,                 # [BH_KV, N_window, D]
    v_window: torch.Tensor,
    k_bits: int,
    v_bits: int,
    kv_repeat: int = 1,
    sm_scale: Optional[float] = None,
) -> torch.Tensor:
    """Fused 4-segment decode: quantised prefix + topk + staging + window
    (reference decode_d_stage.py:916-1005).  Returns [BH_Q, D] in q's dtype.
    Inputs are borrowed and never mutated; zero-length segments are allowed."""
    plan = DecodePlan(q, k_quant_packed, v_quant_packed, k_scale, v_scale,
                      k_topk, v_topk, k_staging, v_staging, k_window, v_window, kv_repeat, sm_scale,
                      k_bits=k_bits, v_bits=v_bits)
    return plan.run(q)


def lse_merge(m: torch.Tensor, l: torch.Tensor, acc: torch.Tensor, out_dtype=torch.bfloat16) -> torch.Tensor:
    """Merge G shards' softmax partials: m, l [G, rows] fp32, acc [G, rows, 128] fp32
    -> [rows, 128] (algebra of the reference's _splitk_reduce_kernel,
    decode_d_stage.py:764-781)."""
    _lib.require_cuda(acc, "acc")
    G, rows, D = acc.shape
    m, l, acc = m.contiguous(), l.contiguous(), acc.contiguous()
    out = torch.empty(rows, D, dtype=out_dtype, device=acc.device)
    rc = _lib.lib().hq_lse_merge(m.data_ptr(), l.data_ptr(), acc.data_ptr(), G, rows, out.data_ptr(),
                                 _lib.dtype_code(out_dtype), out.stride(0), _lib.stream_ptr(acc.device))
    _lib.check(rc, "hq_lse_merge")
    return out
