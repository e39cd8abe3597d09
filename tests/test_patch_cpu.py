"""Host logic of the model patches (reference src/patch/__init__.py, patch_llama.py, patch_qwen.py,
patch_glm.py): target detection, argument errors, and that `dense` mode leaves a model's output unchanged."""

import pytest
import torch

import hyquant_b200
from hyquant_b200 import HyQuantError
from hyquant_b200.patch import (
    _infer_patch_target, patch_attention_forward_model, patch_glm4_attention_forward_model,
    patch_llama3_attention_forward_model, patch_qwen3_attention_forward_model,
)

transformers = pytest.importorskip("transformers")


def tiny(family, layers=2, dtype=torch.float32):
    from transformers import (Glm4Config, Glm4ForCausalLM, LlamaConfig, LlamaForCausalLM, Qwen3Config,
                              Qwen3ForCausalLM)
    cfg_cls, model_cls = {"llama": (LlamaConfig, LlamaForCausalLM), "qwen": (Qwen3Config, Qwen3ForCausalLM),
                          "glm4": (Glm4Config, Glm4ForCausalLM)}[family]
    cfg = cfg_cls(hidden_size=256, intermediate_size=512, num_hidden_layers=layers, num_attention_heads=2,
                  num_key_value_heads=1, head_dim=128, vocab_size=128, max_position_embeddings=8192, pad_token_id=0)
    torch.manual_seed(0)
    return model_cls(cfg).eval().to(dtype)


@pytest.mark.parametrize("family", ["llama", "qwen", "glm4"])
def test_dense_mode_is_identity(family):
    m = tiny(family)
    ids = torch.randint(1, 128, (2, 33))
    with torch.no_grad():
        want = m(ids).logits
    assert patch_attention_forward_model(m, mode="dense") is m
    with torch.no_grad():
        got = m(ids).logits
    assert torch.equal(want, got)
    for mod in m.modules():
        if mod.__class__.__name__.endswith("Attention"):
            assert hasattr(mod, "_original_forward")


@pytest.mark.parametrize("family", ["llama", "qwen", "glm4"])
def test_infer_patch_target(family):
    assert _infer_patch_target(tiny(family, layers=1)) == family

    class Other(torch.nn.Module):
        pass
    with pytest.raises(ValueError, match="Unable to infer patch target"):
        _infer_patch_target(Other())


def test_argument_errors():
    m = tiny("llama", layers=1)
    with pytest.raises(ValueError, match="Unsupported patch_target"):
        patch_attention_forward_model(m, patch_target="mistral")
    with pytest.raises(ValueError, match="Unsupported mode"):
        patch_llama3_attention_forward_model(m, mode="nope")
    with pytest.raises(ValueError, match="window_size"):
        patch_llama3_attention_forward_model(m, mode="sage_w", window_size=-1)
    with pytest.raises(ValueError, match="top_ratio"):
        patch_llama3_attention_forward_model(m, mode="sage_w", top_ratio=0.0)
    with pytest.raises(RuntimeError, match="No Qwen3Attention modules"):
        patch_qwen3_attention_forward_model(m, mode="dense")
    with pytest.raises(RuntimeError, match="No Glm4Attention modules"):
        patch_glm4_attention_forward_model(m, mode="dense")


def test_unbuilt_modes_fail_loudly():
    """No CPU path: a quantised mode on CPU tensors, and the reference's CPU-side ablation modes, raise."""
    ids = torch.randint(1, 128, (1, 64))
    for mode in ("sparse_only", "minference_sparse", "hybrid_full", "sage_w"):
        m = patch_attention_forward_model(tiny("llama", layers=1), mode=mode, window_size=16, top_ratio=0.1)
        with pytest.raises(HyQuantError), torch.no_grad():
            m(ids)


def test_decode_in_d_stage_mode_needs_the_cache():
    m = patch_attention_forward_model(tiny("llama", layers=1), mode="d_k4v4", window_size=16, top_ratio=0.1)
    from transformers import DynamicCache
    cache = DynamicCache(config=m.config)
    k = torch.zeros(1, 1, 8, 128)
    cache.update(k, k, 0)
    with pytest.raises(HyQuantError, match="DStageKVCache"), torch.no_grad():
        m(torch.randint(1, 128, (1, 1)), past_key_values=cache)


def test_install_as_src_exposes_patch_modules():
    hyquant_b200.install_as_src()
    from src.patch import patch_attention_forward_model as f0
    from src.patch.patch_glm import patch_glm4_attention_forward_model as f3
    from src.patch.patch_llama import patch_llama3_attention_forward_model as f1
    from src.patch.patch_qwen import patch_qwen3_attention_forward_model as f2
    assert f0 is patch_attention_forward_model and f1 is patch_llama3_attention_forward_model
    assert f2 is patch_qwen3_attention_forward_model and f3 is patch_glm4_attention_forward_model
