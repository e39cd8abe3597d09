"""In-place attention-forward patches for Hugging Face Llama-3 / Qwen3 / GLM-4 models —
host-side mirror of the reference modules ``src/patch/patch_llama.py``, ``patch_qwen.py``,
``patch_glm.py`` and ``src/patch/__init__.py`` (same entry-point names, keyword arguments,
mode names and errors).  One builder serves the three families; they differ only in the
projection step (Qwen3 normalises q/k per head) and in whether the D-stage decode branch
exists (the reference's GLM patch has none, ``patch_glm.py:79-164``).

Mode dispatch (reference ``patch_llama.py:97-255``):
  dense, or any non-D-stage mode at q_len == 1   -> the model's own attention interface
  D-stage mode, q_len == 1, DStageKVCache        -> four-segment decode kernel
  D-stage mode, q_len  > 1                        -> hybrid prefill ("vquant_vert") or 16-bit causal
  full_attention / sage_w / sage_w0 / vquant_vert -> the corresponding prefill operator
Modes that exist in the reference only as CPU-side ablation baselines (sparse_only,
minference_sparse) and the cache-less quantise/dequantise emulation of decode are not built
and raise ``HyQuantError``.
"""

from __future__ import annotations

import importlib
from types import MethodType
from typing import Optional

import torch

from .._lib import HyQuantError
from ._common import (
    D_STAGE_MODES, compute_vertical_indices, handle_d_stage_cache, infer_kv_repeat, is_d_stage_cache,
    pop_past_key_value_aliases, resolve_attention_interface, trim_4d_attention_mask, validate_patch_args,
)

_FAMILIES = {
    # family: (modeling module, attention class, q/k head norm, D-stage decode branch)
    "llama": ("transformers.models.llama.modeling_llama", "LlamaAttention", False, True),
    "qwen": ("transformers.models.qwen3.modeling_qwen3", "Qwen3Attention", True, True),
    "glm4": ("transformers.models.glm4.modeling_glm4", "Glm4Attention", False, False),
}


def build_attention_forward(family: str, *, mode: str, window_size: int, top_ratio: float,
                            use_vertical_indices: bool = True):
    """Patched ``forward`` for the attention modules of ``family``."""
    mod_name, _, qk_norm, d_stage_decode = _FAMILIES[family]
    modeling = importlib.import_module(mod_name)
    apply_rotary_pos_emb = modeling.apply_rotary_pos_emb
    eager_attention_forward = modeling.eager_attention_forward
    del use_vertical_indices
    # Llama and Qwen3 rotate with the half-split rotate_half over the whole head, which the decode kernel can apply itself;
    # GLM-4's interleaved partial rotation stays on the eager path
    fuse_rope = family in ("llama", "qwen")

    def patched_attention_forward(self, hidden_states: torch.Tensor, position_embeddings=None,
                                  attention_mask: Optional[torch.Tensor] = None, past_key_values: Optional[object] = None,
                                  cache_position: Optional[torch.LongTensor] = None, **kwargs):
        from .. import sage_unified as su
        output_attentions = bool(kwargs.pop("output_attentions", False))
        kwargs.pop("use_cache", None)
        kwargs.pop("position_ids", None)
        past_key_values = pop_past_key_value_aliases(past_key_values, kwargs)
        if position_embeddings is None:
            raise ValueError("position_embeddings are required for patched attention.")

        input_shape = hidden_states.shape[:-1]
        hidden_shape = (*input_shape, -1, self.head_dim)
        q = self.q_proj(hidden_states).view(hidden_shape)
        k = self.k_proj(hidden_states).view(hidden_shape)
        if qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        query_states, key_states = q.transpose(1, 2), k.transpose(1, 2)
        value_states = self.v_proj(hidden_states).view(hidden_shape).transpose(1, 2)
        cos, sin = position_embeddings
        q_len = int(query_states.shape[2])
        has_d_cache = (d_stage_decode and mode in D_STAGE_MODES and past_key_values is not None
                       and is_d_stage_cache(past_key_values))
        fused_step = None
        rope_in_kernel = False
        if has_d_cache and q_len == 1 and past_key_values.get_layer(self.layer_idx).phase == "decode":
            # decode step on a frozen cache: rotary embedding (where the family's form allows), append and attention in one
            # launch (DStageLayerCache.decode_step with rope=); q and k then stay unrotated here
            fused_step = past_key_values.get_layer(self.layer_idx)
            rope_in_kernel = fuse_rope and query_states.dtype == torch.bfloat16 and cos.shape[-1] == 128
        if not rope_in_kernel:
            query_states, key_states = apply_rotary_pos_emb(query_states, key_states, cos, sin)
        if fused_step is not None:
            pass
        elif has_d_cache:
            key_states, value_states = handle_d_stage_cache(self.layer_idx, past_key_values, query_states, key_states,
                                                            value_states, self, sin, cos, cache_position)
        elif past_key_values is not None:
            key_states, value_states = past_key_values.update(
                key_states, value_states, self.layer_idx, {"sin": sin, "cos": cos, "cache_position": cache_position})
        if not (has_d_cache and q_len == 1):
            attention_mask = trim_4d_attention_mask(attention_mask, key_states)
        kv_repeat = infer_kv_repeat(self)
        attn_weights = None

        def finish(o):      # [B, H, N, D] -> [B, N, H, D] in the model dtype
            return o.transpose(1, 2).to(hidden_states.dtype).contiguous()

        if mode == "dense" or (q_len == 1 and not (mode in D_STAGE_MODES and d_stage_decode)):
            interface = resolve_attention_interface(self.config, eager_attention_forward, output_attentions=output_attentions)
            attn_output, attn_weights = interface(
                self, query_states, key_states, value_states, attention_mask,
                dropout=0.0 if not self.training else float(getattr(self, "attention_dropout", 0.0)),
                scaling=getattr(self, "scaling", None), sliding_window=getattr(self, "sliding_window", None), **kwargs)
        elif q_len == 1:
            if not has_d_cache:
                raise HyQuantError(f"mode '{mode}' decodes against a DStageKVCache; pass one as past_key_values "
                                   "(the cache-less quantise/dequantise emulation is not built)")
            if fused_step is not None:
                attn_output = finish(fused_step.decode_step(query_states, key_states, value_states, kv_repeat,
                                                            rope=(cos, sin) if rope_in_kernel else None))
            else:
                layer_cache = past_key_values.get_layer(self.layer_idx)
                attn_output = finish(layer_cache.decode_attention(query_states, kv_repeat))
        elif mode in D_STAGE_MODES:
            if D_STAGE_MODES[mode]["prefill_kernel"] == "vquant_vert":
                vidx = compute_vertical_indices(query_states, key_states, window_size, top_ratio, kv_repeat=kv_repeat)
                attn_output = finish(su.sage_vertical_attention_v2(query_states, key_states, value_states, vidx,
                                                                   window_size=window_size, smooth_k=True))
            else:
                attn_output = finish(su.full_attention_fp16_triton(query_states, key_states, value_states,
                                                                   tensor_layout="HND", is_causal=True))
        elif mode == "full_attention":
            attn_output = finish(su.full_attention_fp16_triton(query_states, key_states, value_states,
                                                               tensor_layout="HND", is_causal=True))
        elif mode in ("sage_w", "sage_w0"):
            attn_output = finish(su.sage_unified_attention(query_states, key_states, value_states,
                                                           window_size=window_size if mode == "sage_w" else 0, smooth_k=True))
        elif mode == "vquant_vert":
            vidx = compute_vertical_indices(query_states, key_states, window_size, top_ratio, kv_repeat=kv_repeat)
            attn_output = finish(su.sage_vertical_attention_v2(query_states, key_states, value_states, vidx,
                                                               window_size=window_size, smooth_k=True))
        elif mode in ("sparse_only", "minference_sparse"):
            raise HyQuantError(f"mode '{mode}' is a CPU-side ablation baseline of the reference and is not built")
        else:
            raise ValueError(f"Unsupported mode '{mode}' in patched attention forward.")

        attn_output = attn_output.reshape(*input_shape, -1).contiguous()
        attn_output = self.o_proj(attn_output)
        return attn_output, (attn_weights if output_attentions else None)

    return patched_attention_forward


def _patch_family(model: torch.nn.Module, family: str, *, mode: str, window_size: int, top_ratio: float,
                  k_bits: Optional[int] = None, v_bits: Optional[int] = None, report_stats: bool = False,
                  use_vertical_indices: bool = True) -> torch.nn.Module:
    mode = validate_patch_args(mode=mode, window_size=window_size, top_ratio=top_ratio, k_bits=k_bits, v_bits=v_bits)
    del report_stats
    mod_name, cls_name, _, _ = _FAMILIES[family]
    attn_cls = getattr(importlib.import_module(mod_name), cls_name)
    fwd = build_attention_forward(family, mode=mode, window_size=window_size, top_ratio=top_ratio,
                                  use_vertical_indices=use_vertical_indices)
    patched = 0
    for module in model.modules():
        if isinstance(module, attn_cls):
            if not hasattr(module, "_original_forward"):
                module._original_forward = module.forward
            module.forward = MethodType(fwd, module)
            patched += 1
    if patched == 0:
        raise RuntimeError(f"No {cls_name} modules were found to patch.")
    return model


def patch_llama3_attention_forward_model(model, *, mode: str = "sage_w", window_size: int = 256, top_ratio: float = 0.05,
                                         k_bits=None, v_bits=None, report_stats: bool = False,
                                         use_vertical_indices: bool = True):
    """Patch all LlamaAttention modules in place (reference patch_llama.py:266-298)."""
    return _patch_family(model, "llama", mode=mode, window_size=window_size, top_ratio=top_ratio, k_bits=k_bits,
                         v_bits=v_bits, report_stats=report_stats, use_vertical_indices=use_vertical_indices)


def patch_qwen3_attention_forward_model(model, *, mode: str = "sage_w", window_size: int = 256, top_ratio: float = 0.05,
                                        k_bits=None, v_bits=None, report_stats: bool = False,
                                        use_vertical_indices: bool = True):
    """Patch all Qwen3Attention modules in place (reference patch_qwen.py)."""
    return _patch_family(model, "qwen", mode=mode, window_size=window_size, top_ratio=top_ratio, k_bits=k_bits,
                         v_bits=v_bits, report_stats=report_stats, use_vertical_indices=use_vertical_indices)


def patch_glm4_attention_forward_model(model, *, mode: str = "sage_w", window_size: int = 256, top_ratio: float = 0.05,
                                       k_bits=None, v_bits=None, report_stats: bool = False,
                                       use_vertical_indices: bool = True):
    """Patch all Glm4Attention modules in place (reference patch_glm.py)."""
    return _patch_family(model, "glm4", mode=mode, window_size=window_size, top_ratio=top_ratio, k_bits=k_bits,
                         v_bits=v_bits, report_stats=report_stats, use_vertical_indices=use_vertical_indices)


def _infer_patch_target(model) -> str:
    """Reference src/patch/__init__.py:8-24."""
    model_type = str(getattr(getattr(model, "config", None), "model_type", "")).lower()
    combined = f"{model_type} {model.__class__.__name__.lower()}"
    if "glm4" in combined or "chatglm" in combined or "glm" in combined:
        return "glm4"
    if "qwen3" in combined or "qwen" in combined:
        return "qwen"
    if "llama" in combined:
        return "llama"
    raise ValueError(f"Unable to infer patch target from model_type='{model_type}', class='{model.__class__.__name__}'. "
                     "Please set patch_target explicitly to one of: qwen, llama, glm4.")


def patch_attention_forward_model(model, *, mode: str = "sage_w", window_size: int = 256, top_ratio: float = 0.05,
                                  report_stats: bool = False, use_vertical_indices: bool = True,
                                  patch_target: str = "auto"):
    """Patch attention forward for qwen/llama/glm4 with optional auto detection
    (reference src/patch/__init__.py:27-69)."""
    if patch_target == "auto":
        patch_target = _infer_patch_target(model)
    if patch_target not in _FAMILIES:
        raise ValueError("Unsupported patch_target. Expected one of: auto, qwen, llama, glm4.")
    return _patch_family(model, patch_target, mode=mode, window_size=window_size, top_ratio=top_ratio,
                         report_stats=report_stats, use_vertical_indices=use_vertical_indices)
