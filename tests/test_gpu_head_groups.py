"""KV-head groups are independent in decode and in prefill: a rank that holds kv-heads [h0, h1) of every batch entry
computes exactly the rows of those heads' query heads.  One GPU plays each rank in turn; nothing is exchanged.

Tolerances: prefill bit for bit (a head's tiles never meet another head's); decode max-abs <= 5e-3 (the split plan,
and with it the order of the fp32 partial sums, depends on how many heads a call has)."""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import sharded
from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


@pytest.mark.parametrize("world", [2, 4])
def test_decode_head_groups_equal_slices_of_the_full_result(world):
    B, H_Q, H_KV, N, W = 2, 16, 4, 3000, 128
    R = H_Q // H_KV
    c = gen_numpy(B, H_Q, H_KV, N, 128, W, 0.05, 41, n_qry=W)
    layer = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=0.05)
    layer.update_prefill(t_bf16(c.k), t_bf16(c.v))
    layer.save_query_tail(t_bf16(c.q))
    layer.freeze(kv_repeat=R)
    g = torch.Generator(device=DEV); g.manual_seed(3)
    for _ in range(5):
        layer.append_staging(torch.randn(B, H_KV, 1, 128, generator=g, device=DEV).to(torch.bfloat16),
                             torch.randn(B, H_KV, 1, 128, generator=g, device=DEV).to(torch.bfloat16))
    qd = t_bf16(c.q_decode)
    full = layer.decode_attention(qd, R).float()
    exact = orc.decode_attention_exact(orc.bf16_round(c.q_decode), _as_oracle(layer), R)
    assert np.abs(full.cpu().numpy() - exact).max() <= 2e-2
    for rank in range(world):
        h0, h1 = sharded.kv_head_range(H_KV, world, rank)
        part = sharded.shard_layer_heads(layer, world, rank)
        assert part.k_quant_packed.shape[0] == B * (h1 - h0) and part._n_quant == layer._n_quant
        out = part.decode_attention(qd[:, h0 * R:h1 * R].contiguous(), R).float()
        assert (out - full[:, h0 * R:h1 * R]).abs().max().item() <= 5e-3
        # the group keeps working as a cache of its own: a token appended to it only
        kn = torch.randn(B, h1 - h0, 1, 128, generator=g, device=DEV).to(torch.bfloat16)
        part.append_staging(kn, kn)
        assert part._staging_ptr == layer._staging_ptr + 1


def _as_oracle(layer):
    f = lambda t: t.float().cpu().numpy()
    return orc.LayerCache(B=layer._B, H_KV=layer._H_KV, D=128, k_bits=4, v_bits=4,
                          k_quant_packed=layer.k_quant_packed.cpu().numpy(), v_quant_packed=layer.v_quant_packed.cpu().numpy(),
                          k_scale=layer.k_scale.cpu().numpy(), v_scale=layer.v_scale.cpu().numpy(),
                          k_topk=f(layer.k_topk), v_topk=f(layer.v_topk), k_window=f(layer.k_window), v_window=f(layer.v_window),
                          staging_k=f(layer._staging_buf_k), staging_v=f(layer._staging_buf_v),
                          staging_ptr=layer._staging_ptr, seq_len=0)


@pytest.mark.parametrize("world", [2, 4])
def test_prefill_head_groups_equal_slices_of_the_full_result(world):
    B, H_Q, H_KV, N, W = 1, 16, 4, 1536, 128
    R = H_Q // H_KV
    c = gen_numpy(B, H_Q, H_KV, N, 128, W, 0.05, 43)
    q, k, v = t_bf16(c.q), t_bf16(c.k), t_bf16(c.v)
    vidx = hq.compute_vertical_indices(q, k, W, 0.05, kv_repeat=R)
    full = hq.sage_vertical_attention_v2(q, k, v, vidx, window_size=W)
    for rank in range(world):
        h0, h1 = sharded.kv_head_range(H_KV, world, rank)
        qs = slice(h0 * R, h1 * R)
        vi = hq.compute_vertical_indices(q[:, qs], k[:, h0:h1], W, 0.05, kv_repeat=R)
        assert torch.equal(vi, vidx[:, qs])
        out = hq.sage_vertical_attention_v2(q[:, qs], k[:, h0:h1], v[:, h0:h1], vi, window_size=W)
        assert torch.equal(out, full[:, qs])
