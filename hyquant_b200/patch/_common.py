"""Shared helpers of the attention patches — host-side mirror of the reference
module ``src/patch/_common.py`` (mode table, argument validation,
``compute_vertical_indices``, the prefill/decode cache hook).  Vertical-line
scoring and top-k run on the sm_100a kernels (``hq_vertical_scores``,
``hq_topk``)."""

from __future__ import annotations

import math
from typing import Any, Callable, Optional, Tuple

import torch

from .. import _lib
from .._lib import HyQuantError

_VALID_MODES = {
    "dense", "full_attention",
    "sage_w", "sage_w0", "vquant_vert", "minference_sparse", "sparse_only",
    "d_k4v4", "d_k4v4_vert", "d_k8v8",
    "d_k4v2", "d_k4v2_vert",
    "d_k2v4", "d_k2v4_vert",
    "hybrid_full", "hybrid_k4v2", "hybrid_k2v4",
}
_VALID_K_BITS = {2, 4, 8}
_VALID_V_BITS = {2, 4, 8}

# reference _common.py:38-49
D_STAGE_MODES = {
    "d_k4v4":       {"k_bits": 4, "v_bits": 4, "vert": False, "prefill_kernel": "full"},
    "d_k4v4_vert":  {"k_bits": 4, "v_bits": 4, "vert": True,  "prefill_kernel": "full"},
    "d_k8v8":       {"k_bits": 8, "v_bits": 8, "vert": False, "prefill_kernel": "full"},
    "d_k4v2":       {"k_bits": 4, "v_bits": 2, "vert": False, "prefill_kernel": "full"},
    "d_k4v2_vert":  {"k_bits": 4, "v_bits": 2, "vert": True,  "prefill_kernel": "full"},
    "d_k2v4":       {"k_bits": 2, "v_bits": 4, "vert": False, "prefill_kernel": "full"},
    "d_k2v4_vert":  {"k_bits": 2, "v_bits": 4, "vert": True,  "prefill_kernel": "full"},
    "hybrid_full":  {"k_bits": 4, "v_bits": 4, "vert": True,  "prefill_kernel": "vquant_vert"},
    "hybrid_k4v2":  {"k_bits": 4, "v_bits": 2, "vert": True,  "prefill_kernel": "vquant_vert"},
    "hybrid_k2v4":  {"k_bits": 2, "v_bits": 4, "vert": True,  "prefill_kernel": "vquant_vert"},
}


def is_d_stage_mode(mode: str) -> bool:
    return mode == "d_stage" or mode in D_STAGE_MODES


def validate_patch_args(mode: str, window_size: int, top_ratio: float,
                        k_bits: Optional[int] = None, v_bits: Optional[int] = None) -> str:
    """Reference _common.py:57-78 (same errors)."""
    if mode not in _VALID_MODES:
        raise ValueError(f"Unsupported mode '{mode}'. Expected one of: {sorted(_VALID_MODES)}.")
    if window_size < 0:
        raise ValueError(f"window_size must be >= 0, got {window_size}.")
    if not (0.0 < top_ratio <= 1.0):
        raise ValueError(f"top_ratio must be in (0, 1], got {top_ratio}.")
    if mode == "d_stage":
        if k_bits not in _VALID_K_BITS:
            raise ValueError(f"k_bits must be in {sorted(_VALID_K_BITS)}, got {k_bits}.")
        if v_bits not in _VALID_V_BITS:
            raise ValueError(f"v_bits must be in {sorted(_VALID_V_BITS)}, got {v_bits}.")
    return mode


# Small Hugging Face glue the patched forwards need; names, arguments and results follow the reference's helpers
# (src/patch/_common.py:80-141) so that code written against them keeps working.

def repeat_interleave_manual(x: torch.Tensor, repeats: int, dim: int) -> torch.Tensor:
    """Each slice along ``dim`` ``repeats`` times in a row (GQA expansion of K / V heads), as a contiguous tensor."""
    if repeats == 1:
        return x
    shape = list(x.shape)
    expanded = x.unsqueeze(dim + 1).expand(*shape[:dim + 1], repeats, *shape[dim + 1:])
    shape[dim] *= repeats
    return expanded.reshape(shape).contiguous()


def infer_kv_repeat(attn_module: torch.nn.Module) -> int:
    """Query heads per KV head of an attention module: its ``num_key_value_groups`` if it has one, else the ratio of
    its head counts, else 1."""
    groups = getattr(attn_module, "num_key_value_groups", None)
    if groups is not None:
        return max(1, int(groups))
    heads, kv_heads = getattr(attn_module, "num_heads", None), getattr(attn_module, "num_key_value_heads", None)
    if heads is not None and kv_heads is not None:
        return max(1, int(heads) // max(1, int(kv_heads)))
    return 1


def resolve_attention_interface(config: Any, eager_attention_forward: Callable[..., Any], *,
                                output_attentions: bool = False) -> Callable[..., Any]:
    """The attention function transformers would use for ``config``; eager when it is asked for, when attention weights
    are wanted from sdpa, or when the registry is not available."""
    name = getattr(config, "_attn_implementation", "eager")
    if name == "eager" or (name == "sdpa" and output_attentions):
        return eager_attention_forward
    try:
        from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS as registry
    except Exception:
        return eager_attention_forward
    return registry.get(name, eager_attention_forward)


def pop_past_key_value_aliases(past_key_value: Any, kwargs: dict) -> Any:
    """The cache object, whichever keyword the transformers version passes it under (the alias is removed from kwargs)."""
    for alias in ("past_key_values", "past_key_value"):
        if past_key_value is None and alias in kwargs:
            past_key_value = kwargs.pop(alias)
    return past_key_value


def trim_4d_attention_mask(attention_mask: Any, key_states: Any) -> Any:
    """A 4-D mask cut to the key length; anything else is passed through."""
    if attention_mask is None or getattr(attention_mask, "ndim", None) != 4:
        return attention_mask
    return attention_mask[..., : key_states.shape[-2]]


# ----------------------------------------------------------------------------
# vertical-line selection
# ----------------------------------------------------------------------------

def vertical_scores(query_states: torch.Tensor, key_states: torch.Tensor, window_size: int,
                    kv_repeat: int = 1, *, round_like_reference: bool = False,
                    group_mean: int = 1) -> Optional[torch.Tensor]:
    """fp32 scores [B, H_Q, P] of the pooled last-``window_size`` queries against
    the prefix keys (reference _common.py:161-185).  ``round_like_reference``
    rounds the pooled query and the scores to the input dtype as the reference's
    in-dtype mean / matmul do; by default both stay fp32.

    ``group_mean`` = G > 1 is the selection of the cache's freeze: ``query_states`` holds
    G query heads per kv-head, which are averaged first (per token, in the input dtype,
    reference d_stage_kv_cache.py:131-133); the scores are then [B, H_KV, P]."""
    _lib.require_cuda(query_states, "query_states")
    B, H_Q, n_q, D = query_states.shape
    if D != 128:
        raise HyQuantError(f"head_dim {D} is not built (128 only)")
    key_len = int(key_states.shape[2])
    P = max(0, key_len - window_size)
    if P == 0:
        return None
    H = int(key_states.shape[1])
    if group_mean > 1:
        if H * group_mean != H_Q:
            raise AssertionError(f"H_Q ({H_Q}) != H_KV ({H}) * group_mean ({group_mean})")
        H_Q = H
    if not (H == H_Q or H * kv_repeat == H_Q):
        raise AssertionError(f"H_Q ({H_Q}) != H_KV ({H}) * kv_repeat ({kv_repeat})")
    if key_states.dtype not in (torch.bfloat16, torch.float16):
        raise HyQuantError("vertical scoring on the device takes bf16/fp16 keys")
    q = query_states if query_states.dtype == key_states.dtype else query_states.to(key_states.dtype)
    if q.stride(3) != 1:
        q = q.contiguous()
    k = key_states
    if k.stride(3) != 1 or (k.stride(2) % 8) or (k.stride(1) % 8) or (k.stride(0) % 8) or k.data_ptr() % 16:
        k = k.contiguous()
    tail_len = min(window_size, n_q)
    if tail_len == 0:          # the reference's slice [-0:] keeps every query
        tail_len = n_q
    pooled = torch.empty(B, H_Q, D, dtype=torch.float32, device=q.device)
    scores = torch.empty(B, H_Q, P, dtype=torch.float32, device=q.device)
    rl = 1 if round_like_reference else 0
    if group_mean > 1:
        rc = _lib.lib().hq_vertical_scores_grouped(
            q.data_ptr(), _lib.dtype_code(k.dtype), q.stride(0), q.stride(1), q.stride(2), B, H, group_mean, n_q, tail_len,
            k.data_ptr(), k.stride(0), k.stride(1), k.stride(2), P, rl, rl,
            pooled.data_ptr(), scores.data_ptr(), _lib.stream_ptr(q.device))
        _lib.check(rc, "hq_vertical_scores_grouped")
        return scores
    rc = _lib.lib().hq_vertical_scores(
        q.data_ptr(), _lib.dtype_code(k.dtype), q.stride(0), q.stride(1), q.stride(2), B, H_Q, n_q, tail_len,
        k.data_ptr(), k.stride(0), k.stride(1), k.stride(2), H, P, rl, rl,
        pooled.data_ptr(), scores.data_ptr(), _lib.stream_ptr(q.device))
    _lib.check(rc, "hq_vertical_scores")
    return scores


def topk_indices(scores: torch.Tensor, k: int, want_ascending: bool = False):
    """Exact top-k of fp32 ``scores`` [..., n] -> int64 [..., k], descending score,
    ties towards the lower index (replaces torch.topk(sorted=True),
    reference _common.py:189).  With ``want_ascending`` also returns the same set
    as int32 in ascending position."""
    _lib.require_cuda(scores, "scores")
    n = scores.shape[-1]
    s2 = scores.reshape(-1, n)
    if s2.dtype != torch.float32:
        s2 = s2.float()
    if s2.stride(1) != 1:
        s2 = s2.contiguous()
    rows = s2.shape[0]
    idx = torch.empty(rows, k, dtype=torch.int64, device=scores.device)
    asc = torch.empty(rows, k, dtype=torch.int32, device=scores.device) if want_ascending else None
    rc = _lib.lib().hq_topk(s2.data_ptr(), s2.stride(0), rows, n, k, idx.data_ptr(),
                            asc.data_ptr() if asc is not None else None, _lib.stream_ptr(scores.device))
    _lib.check(rc, "hq_topk")
    idx = idx.reshape(*scores.shape[:-1], k)
    if want_ascending:
        return idx, asc.reshape(*scores.shape[:-1], k)
    return idx


def vertical_topk_count(prefix_len: int, top_ratio: float) -> int:
    return min(max(1, int(math.ceil(prefix_len * top_ratio))), prefix_len)


def compute_vertical_indices(query_states: torch.Tensor, key_states: torch.Tensor, window_size: int,
                             top_ratio: float, kv_repeat: int = 1) -> torch.Tensor:
    """Per-head important key indices (reference _common.py:144-190).

    query_states [B, H_Q, Q, D]; key_states [B, H, K, D] with H == H_Q or
    H == H_Q // kv_repeat (GQA-native).  Returns int64 [B, H_Q, top_k], positions
    in [0, K - window_size), descending score.
    """
    batch, num_heads = query_states.shape[:2]
    scores = vertical_scores(query_states, key_states, window_size, kv_repeat)
    if scores is None:
        return torch.empty((batch, num_heads, 0), device=query_states.device, dtype=torch.int64)
    return topk_indices(scores, vertical_topk_count(scores.shape[-1], top_ratio))


def is_d_stage_cache(past_key_values: Any) -> bool:
    return hasattr(past_key_values, "get_layer") and hasattr(past_key_values, "_layers")


def handle_d_stage_cache(layer_idx: int, past_key_values: Any, query_states: torch.Tensor,
                         key_states: torch.Tensor, value_states: torch.Tensor,
                         attn_module: torch.nn.Module, sin: torch.Tensor, cos: torch.Tensor,
                         cache_position: Optional[torch.LongTensor]) -> Tuple[torch.Tensor, torch.Tensor]:
    """Prefill: keep the query tail and accumulate K/V.  Decode: freeze once,
    then append the new token to staging (reference _common.py:198-228)."""
    layer_cache = past_key_values.get_layer(layer_idx)
    q_len = query_states.shape[2]
    if q_len > 1:
        layer_cache.save_query_tail(query_states)
        return past_key_values.update(key_states, value_states, layer_idx,
                                      {"sin": sin, "cos": cos, "cache_position": cache_position})
    kv_repeat = infer_kv_repeat(attn_module)
    if layer_cache.phase == "prefill":
        layer_cache.freeze(kv_repeat=kv_repeat)
    layer_cache.append_staging(key_states, value_states)
    return key_states, value_states
