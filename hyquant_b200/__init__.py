"""hyquant_b200 — the hybrid-precision attention hot path of HyQuant, built for
NVIDIA B200 (sm_100a): hand-written CUDA kernels behind a C ABI
(``include/hyquant_b200.h``), with the reference's Python operator interface on
top.

Public entry points carry the reference's names (``src.ops`` / ``src.patch``):

    from hyquant_b200 import (fused_d_stage_decode, DStageKVCache, create_cache_for_mode,
                              compute_vertical_indices, quantize_per_token)

``install_as_src()`` registers the package under the reference's module names
(``src.ops``, ``src.ops.decode_d_stage``, ``src.patch._common`` ...), so code
written against the reference imports this implementation unchanged.
"""

from __future__ import annotations

import sys
import types

from ._lib import HyQuantError, lib  # noqa: F401
from .decode_d_stage import (  # noqa: F401
    GROUP_SIZE, DecodePlan, dequantize_per_token, fused_d_stage_decode, lse_merge,
    quantize_per_token, quantize_per_token_into,
)
from .d_stage_kv_cache import DStageKVCache, DStageLayerCache, QuantizedKVCache  # noqa: F401
from .sage_unified import (  # noqa: F401
    full_attention_fp16_triton, hybrid_prefill, sage_fp8_attention, sage_unified_attention, sage_vertical_attention_v2,
)
from .patch._common import (  # noqa: F401
    D_STAGE_MODES, compute_vertical_indices, handle_d_stage_cache, is_d_stage_mode, topk_indices,
    validate_patch_args, vertical_scores,
)

__all__ = [
    "fused_d_stage_decode", "DStageKVCache", "DStageLayerCache", "create_cache_for_mode",
    "compute_vertical_indices", "quantize_per_token", "dequantize_per_token", "lse_merge",
    "sage_vertical_attention_v2", "sage_unified_attention", "sage_fp8_attention", "full_attention_fp16_triton",
    "install_as_src", "HyQuantError",
]


def create_cache_for_mode(mode: str, num_layers: int, head_dim: int = 128, k_bits: int = 4, v_bits: int = 4,
                          **kwargs):
    """Cache for a patch mode, or None for non-D-stage modes (reference src/ops/__init__.py:28-67)."""
    if not is_d_stage_mode(mode):
        return None
    if mode == "d_stage":
        return DStageKVCache(num_layers=num_layers, k_bits=k_bits, v_bits_fn=lambda i, _vb=v_bits: _vb,
                             window_size=kwargs.get("window_size", 256), top_ratio=kwargs.get("top_ratio", 0.05),
                             use_vert=True)
    cfg = D_STAGE_MODES[mode]
    return DStageKVCache(num_layers=num_layers, k_bits=cfg["k_bits"], v_bits_fn=lambda i, _vb=cfg["v_bits"]: _vb,
                         window_size=kwargs.get("window_size", 256), top_ratio=kwargs.get("top_ratio", 0.05),
                         use_vert=cfg["vert"])


def install_as_src() -> None:
    """Alias this package as the reference's ``src`` tree in ``sys.modules``."""
    from . import d_stage_kv_cache, decode_d_stage
    from . import patch as patch_pkg
    from .patch import _common
    src = types.ModuleType("src")
    ops = types.ModuleType("src.ops")
    names = ["sage_unified_attention", "sage_vertical_attention_v2", "sage_fp8_attention",
             "full_attention_fp16_triton", "fused_d_stage_decode", "DStageKVCache", "create_cache_for_mode"]
    for name in names:
        setattr(ops, name, globals()[name])
    ops.__all__ = names
    from . import sage_unified
    ops.sage_unified = sage_unified
    ops.decode_d_stage = decode_d_stage
    ops.d_stage_kv_cache = d_stage_kv_cache
    src.ops, src.patch = ops, patch_pkg
    sys.modules.update({
        "src": src, "src.ops": ops, "src.ops.decode_d_stage": decode_d_stage,
        "src.ops.d_stage_kv_cache": d_stage_kv_cache, "src.ops.sage_unified": sage_unified,
        "src.patch": patch_pkg, "src.patch._common": _common,
    })
    # the reference keeps one module per model family; here they are views of one builder
    from .patch import forwards
    for mod, fn in (("patch_llama", "patch_llama3_attention_forward_model"),
                    ("patch_qwen", "patch_qwen3_attention_forward_model"),
                    ("patch_glm", "patch_glm4_attention_forward_model")):
        m = types.ModuleType(f"src.patch.{mod}")
        setattr(m, fn, getattr(forwards, fn))
        setattr(patch_pkg, mod, m)
        sys.modules[f"src.patch.{mod}"] = m
