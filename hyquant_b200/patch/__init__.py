"""Attention-forward patches — host-side mirror of the reference ``src/patch``."""

from ._common import (  # noqa: F401
    D_STAGE_MODES, compute_vertical_indices, handle_d_stage_cache, infer_kv_repeat, is_d_stage_cache,
    is_d_stage_mode, validate_patch_args,
)
