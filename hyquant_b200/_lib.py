"""ctypes binding of the C ABI declared in ``include/hyquant_b200.h``.

The library is the product: when it is missing (and cannot be built) or a call
fails, the Python entry points raise — there is no CPU or PyTorch fallback.
"""

from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libhyquant_b200.so")

HQ_BF16, HQ_F16, HQ_F32 = 0, 1, 2
HQ_DECODE_OVERLAP_PREVIOUS = 1
HQ_OK = 0
ERR_NAMES = {-1: "HQ_ERR_INVALID", -2: "HQ_ERR_UNSUPPORTED", -3: "HQ_ERR_ALIGNMENT",
             -4: "HQ_ERR_WORKSPACE", -5: "HQ_ERR_CUDA", -6: "HQ_ERR_TIMEOUT"}

# every symbol include/hyquant_b200.h declares
EXPORTS = [
    "hq_version", "hq_last_error",
    "hq_quant_pack", "hq_quant_pack_int4", "hq_staging_append",
    "hq_decode_workspace_bytes", "hq_decode_splitk", "hq_decode_splitk_static", "hq_decode_static_status",
    "hq_lse_merge", "hq_lse_merge_strided",
    "hq_vertical_scores", "hq_vertical_scores_grouped",
    "hq_topk",
    "hq_cache_reorganize", "hq_cache_reorganize_bits", "hq_lse_merge_partial",
    "hq_prefill_quant_workspace_bytes", "hq_prefill_quant", "hq_prefill_quant_blocks", "hq_per_block_int8",
    "hq_prefill_vertical_prepare", "hq_prefill_transpose_v", "hq_prefill_quant_v_fp8", "hq_prefill_vertical_gather_v_fp8",
    "hq_prefill_hybrid", "hq_tc_peak",
    "hq_peer_exchange_bytes", "hq_peer_slot", "hq_peer_recv_slot", "hq_peer_exchange_merge", "hq_peer_status",
    "hq_peer_buffer_create", "hq_peer_buffer_open", "hq_peer_buffer_close", "hq_peer_buffer_destroy",
]


class HyQuantError(RuntimeError):
    pass


class DecodeArgs(C.Structure):
    """Mirror of ``hq_decode_args``."""
    _fields_ = [
        ("struct_bytes", C.c_int32), ("BH_KV", C.c_int32), ("kv_repeat", C.c_int32), ("head_dim", C.c_int32),
        ("n_quant", C.c_int32), ("n_topk", C.c_int32), ("n_staging", C.c_int32), ("n_window", C.c_int32),
        ("out_dtype", C.c_int32), ("num_splits", C.c_int32), ("sm_scale", C.c_float), ("flags", C.c_int32),
        ("k_bits", C.c_int32), ("v_bits", C.c_int32),
        ("q", C.c_void_p), ("q_stride", C.c_int64),
        ("k_packed", C.c_void_p), ("v_packed", C.c_void_p), ("kp_stride_bh", C.c_int64), ("vp_stride_bh", C.c_int64),
        ("k_scale", C.c_void_p), ("v_scale", C.c_void_p), ("ks_stride_bh", C.c_int64), ("vs_stride_bh", C.c_int64),
        ("k_topk", C.c_void_p), ("v_topk", C.c_void_p), ("kt_stride_bh", C.c_int64), ("vt_stride_bh", C.c_int64),
        ("k_staging", C.c_void_p), ("v_staging", C.c_void_p), ("kg_stride_bh", C.c_int64), ("vg_stride_bh", C.c_int64),
        ("k_window", C.c_void_p), ("v_window", C.c_void_p), ("kw_stride_bh", C.c_int64), ("vw_stride_bh", C.c_int64),
        ("out", C.c_void_p), ("out_stride", C.c_int64),
        ("partial_m", C.c_void_p), ("partial_l", C.c_void_p), ("partial_acc", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64),
        ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("kn_stride", C.c_int64), ("vn_stride", C.c_int64),
        ("peer_bufs", C.c_void_p), ("peer_world", C.c_int32), ("peer_rank", C.c_int32), ("peer_seq", C.c_uint32),
        ("peer_reserved", C.c_int32), ("peer_timeout_ns", C.c_int64),
        ("lengths", C.c_void_p),
        ("rope_cos", C.c_void_p), ("rope_sin", C.c_void_p), ("rope_stride", C.c_int64),
        ("rope_heads_per_batch", C.c_int32), ("rope_reserved", C.c_int32),
    ]


class PrefillArgs(C.Structure):
    """Mirror of ``hq_prefill_args``."""
    _fields_ = [
        ("struct_bytes", C.c_int32), ("B", C.c_int32), ("H_Q", C.c_int32), ("H_KV", C.c_int32), ("N", C.c_int32),
        ("head_dim", C.c_int32), ("window", C.c_int32), ("T", C.c_int32), ("out_dtype", C.c_int32),
        ("sm_scale", C.c_float),
        ("q_i8", C.c_void_p), ("q_bf", C.c_void_p), ("q_scale", C.c_void_p),
        ("k_i8", C.c_void_p), ("k_bf", C.c_void_p), ("k_scale", C.c_void_p), ("k_bias", C.c_void_p),
        ("v_t", C.c_void_p), ("vert_k", C.c_void_p), ("vert_vt", C.c_void_p),
        ("nv_valid", C.c_void_p),
        ("out", C.c_void_p), ("o_sb", C.c_int64), ("o_sh", C.c_int64), ("o_sn", C.c_int64),
        ("status", C.c_void_p),
        ("v_t8", C.c_void_p), ("v_scale8", C.c_void_p), ("pv_fp8", C.c_int32), ("reserved0", C.c_int32),
        ("vert_vt8", C.c_void_p),
    ]


class PeerExchangeArgs(C.Structure):
    """Mirror of ``hq_peer_exchange_args``."""
    _fields_ = [
        ("struct_bytes", C.c_int32), ("world", C.c_int32), ("rank", C.c_int32), ("rows", C.c_int32),
        ("seq", C.c_uint32), ("out_dtype", C.c_int32), ("out_stride", C.c_int64), ("out", C.c_void_p),
        ("timeout_ns", C.c_int64), ("bufs", C.c_void_p * 16),
    ]


_lib = None
_lock = threading.Lock()


def _declare(lib):
    vp, i32, i64 = C.c_void_p, C.c_int, C.c_int64
    lib.hq_version.restype = C.c_char_p
    lib.hq_last_error.restype = C.c_char_p
    lib.hq_quant_pack_int4.argtypes = [vp, i32, i64, i64, i32, i32, vp, i64, vp, i64, i64, i32, vp]
    lib.hq_quant_pack.argtypes = [vp, i32, i64, i64, i32, i32, i32, vp, i64, vp, i64, i64, i32, vp]
    lib.hq_lse_merge_partial.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, vp, vp, vp, vp]
    lib.hq_staging_append.argtypes = [vp, vp, i64, i64, vp, vp, i32, i32, vp]
    lib.hq_decode_workspace_bytes.argtypes = [i32, i32, C.POINTER(i64)]
    lib.hq_decode_splitk.argtypes = [C.POINTER(DecodeArgs), vp]
    lib.hq_decode_splitk_static.argtypes = [C.POINTER(DecodeArgs), vp]
    lib.hq_decode_static_status.argtypes = [C.POINTER(C.c_int)]
    lib.hq_lse_merge.argtypes = [vp, vp, vp, i32, i32, vp, i32, i64, vp]
    lib.hq_lse_merge_strided.argtypes = [vp, vp, vp, i64, i64, i64, i32, i32, vp, i32, i64, vp]
    lib.hq_vertical_scores.argtypes = [vp, i32, i64, i64, i64, i32, i32, i32, i32,
                                       vp, i64, i64, i64, i32, i32, i32, i32, vp, vp, vp]
    lib.hq_vertical_scores_grouped.argtypes = [vp, i32, i64, i64, i64, i32, i32, i32, i32, i32,
                                               vp, i64, i64, i64, i32, i32, i32, vp, vp, vp]
    lib.hq_topk.argtypes = [vp, i64, i32, i32, i32, vp, vp, vp]
    lib.hq_cache_reorganize.argtypes = [vp, vp, i64, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp,
                                        vp, vp, i64, vp, vp, i64, i32, vp]
    lib.hq_cache_reorganize_bits.argtypes = [vp, vp, i64, i32, i32, i32, i32, vp, vp, vp, vp, vp, vp,
                                             vp, vp, i64, i64, vp, vp, i64, i32, i32, i32, vp]
    lib.hq_prefill_quant_workspace_bytes.argtypes = [i32, i32, C.POINTER(i64)]
    lib.hq_prefill_quant.argtypes = [vp, i64, i64, i64, vp, i64, i64, i64, i32, i32, i32, i32, C.c_float, i32,
                                     vp, vp, vp, vp, vp, vp, vp, vp, i64, vp]
    lib.hq_prefill_quant_blocks.argtypes = lib.hq_prefill_quant.argtypes
    lib.hq_per_block_int8.argtypes = [vp, i64, i64, i64, i32, i32, i32, i32, C.c_float, vp, vp, i64, i64, i64, vp, vp]
    lib.hq_prefill_vertical_prepare.argtypes = [vp, i32, i32, i32, i32, i32, i32, vp, vp, i64, i64, i64,
                                                vp, vp, vp, vp, vp, vp]
    lib.hq_prefill_transpose_v.argtypes = [vp, i64, i64, i64, i32, i32, i32, vp, vp]
    lib.hq_prefill_quant_v_fp8.argtypes = [vp, i64, i64, i64, i32, i32, i32, vp, vp, vp, vp]
    lib.hq_prefill_vertical_gather_v_fp8.argtypes = [vp, i32, i32, i32, i32, i32, vp, i64, i64, i64, vp, vp, vp]
    lib.hq_prefill_hybrid.argtypes = [C.POINTER(PrefillArgs), vp]
    lib.hq_tc_peak.argtypes = [i32, i32, vp, C.POINTER(C.c_int), vp]
    lib.hq_peer_exchange_bytes.argtypes = [i32, i32, C.POINTER(i64)]
    lib.hq_peer_slot.argtypes = [vp, i32, i32, C.c_uint32, C.POINTER(vp), C.POINTER(vp), C.POINTER(vp)]
    lib.hq_peer_recv_slot.argtypes = [vp, i32, i32, C.c_uint32, i32, C.POINTER(vp)]
    lib.hq_peer_exchange_merge.argtypes = [C.POINTER(PeerExchangeArgs), vp]
    lib.hq_peer_status.argtypes = [vp, C.POINTER(C.c_int)]
    lib.hq_peer_buffer_create.argtypes = [i64, C.POINTER(vp), C.c_char_p]
    lib.hq_peer_buffer_open.argtypes = [C.c_char_p, C.POINTER(vp)]
    lib.hq_peer_buffer_close.argtypes = [vp]
    lib.hq_peer_buffer_destroy.argtypes = [vp]
    for name in EXPORTS:
        if name not in ("hq_version", "hq_last_error"):
            getattr(lib, name).restype = C.c_int


def lib():
    """Load (building first if the sources are newer) and return the library."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            from . import build as _b
            try:
                _b.build()
            except Exception as e:  # no compiler on this machine
                raise HyQuantError(
                    f"{LIB_PATH} is missing and could not be built ({e}); "
                    "hyquant_b200 has no fallback path") from e
        try:
            l = C.CDLL(LIB_PATH)
        except OSError as e:
            raise HyQuantError(f"cannot load {LIB_PATH}: {e}") from e
        missing = [s for s in EXPORTS if not hasattr(l, s)]
        if missing:
            raise HyQuantError(f"{LIB_PATH} lacks symbols {missing}; rebuild with python -m hyquant_b200.build --force")
        _declare(l)
        _lib = l
    return _lib


def check(rc: int, what: str):
    if rc != HQ_OK:
        msg = lib().hq_last_error().decode(errors="replace")
        raise HyQuantError(f"{what} failed: {ERR_NAMES.get(rc, rc)}: {msg}")


def dtype_code(dt) -> int:
    import torch
    if dt == torch.bfloat16:
        return HQ_BF16
    if dt == torch.float16:
        return HQ_F16
    if dt == torch.float32:
        return HQ_F32
    raise HyQuantError(f"unsupported dtype {dt}")


_raw_stream = None


def stream_ptr(device=None) -> int:
    """cudaStream_t of torch's current stream on ``device`` (an int handle).  Uses torch's raw-stream
    query, a fraction of the cost of building a ``torch.cuda.Stream`` object per call."""
    global _raw_stream
    import torch
    if _raw_stream is None:
        _raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", False)
    if _raw_stream:
        idx = None if device is None else getattr(device, "index", device)
        return _raw_stream(torch.cuda.current_device() if idx is None else idx)
    return torch.cuda.current_stream(device).cuda_stream


def require_cuda(t, name: str):
    if not t.is_cuda:
        raise HyQuantError(f"{name} must be a CUDA tensor: hyquant_b200 runs on sm_100a only and has no CPU path")
