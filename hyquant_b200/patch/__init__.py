"""Attention-forward patches — host-side mirror of the reference ``src/patch``."""

from ._common import (  # noqa: F401
    D_STAGE_MODES, compute_vertical_indices, handle_d_stage_cache, infer_kv_repeat, is_d_stage_cache,
    is_d_stage_mode, validate_patch_args,
)
from .forwards import (  # noqa: F401
    _infer_patch_target, build_attention_forward, patch_attention_forward_model, patch_glm4_attention_forward_model,
    patch_llama3_attention_forward_model, patch_qwen3_attention_forward_model,
)

__all__ = [
    "patch_attention_forward_model", "patch_glm4_attention_forward_model", "patch_llama3_attention_forward_model",
    "patch_qwen3_attention_forward_model",
]
