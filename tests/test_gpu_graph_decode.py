"""One token of every layer as one CUDA-graph replay (``DecodeStepGraph``): the decode kernels take the cache lengths
from a device record that travels with the step's inputs, so one captured graph serves every step; the step that fills
the staging buffers runs eagerly.  Results must equal the layer-by-layer path across two staging flushes: cache
contents bit for bit, outputs within 2e-3 (the captured launch keeps the split count of the step it was captured at,
the layer-by-layer path re-chooses it as the cache grows, so the order of the fp32 partial sums can differ)."""

import numpy as np
import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200.graph_decode import DecodeStepGraph
from hyquant_b200.synth import gen_numpy

pytestmark = pytest.mark.gpu
DEV = "cuda"


def t_bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV).to(torch.bfloat16)


def _layers(n, B, H_Q, H_KV, N, W):
    out = []
    for i in range(n):
        c = gen_numpy(B, H_Q, H_KV, N, 128, W, 0.05, 50 + i, n_qry=W)
        layer = hq.DStageLayerCache(i, k_bits=4, v_bits=4, window_size=W, top_ratio=0.05)
        layer.update_prefill(t_bf16(c.k), t_bf16(c.v))
        layer.save_query_tail(t_bf16(c.q))
        layer.freeze(kv_repeat=H_Q // H_KV)
        out.append(layer)
    return out


def test_graph_replay_equals_layer_by_layer_across_flushes():
    n, B, H_Q, H_KV, N, W, steps = 3, 2, 8, 2, 1500, 128, 270
    R = H_Q // H_KV
    ref_layers, layers = _layers(n, B, H_Q, H_KV, N, W), _layers(n, B, H_Q, H_KV, N, W)
    g = DecodeStepGraph(layers, B, H_Q, H_KV)
    gen = torch.Generator(); gen.manual_seed(9)
    replays = 0
    for s in range(steps):
        q = torch.randn(n, B, H_Q, 1, 128, generator=gen).to(torch.bfloat16)
        k = torch.randn(n, B, H_KV, 1, 128, generator=gen).to(torch.bfloat16)
        v = torch.randn(n, B, H_KV, 1, 128, generator=gen).to(torch.bfloat16)
        for i in range(n):
            g.host_q[i].copy_(q[i]); g.host_k[i].copy_(k[i]); g.host_v[i].copy_(v[i])
        had_graph = g._graph is not None
        out = g.step().clone()
        replays += int(had_graph and g._graph is not None and not any(l._staging_ptr == 0 for l in layers))
        for i in range(n):
            ref = ref_layers[i].decode_step(q[i].to(DEV), k[i].to(DEV), v[i].to(DEV), R)
            assert (out[i].to(DEV).float() - ref.float()).abs().max().item() <= 2e-3, (s, i)
            assert (layers[i]._n_quant, layers[i]._staging_ptr) == (ref_layers[i]._n_quant, ref_layers[i]._staging_ptr)
    assert replays > 250                        # all but the warm-up, the capture and the two flush steps were replays
    for i in range(n):
        assert torch.equal(layers[i].k_quant_packed, ref_layers[i].k_quant_packed)
        assert torch.equal(layers[i]._staging_buf_k, ref_layers[i]._staging_buf_k)
    g.close()
    # unbound again, the layers work as before
    q = torch.randn(B, H_Q, 1, 128, generator=gen).to(torch.bfloat16).to(DEV)
    assert torch.equal(layers[0].decode_attention(q, R), ref_layers[0].decode_attention(q, R))


def test_lengths_record_overrides_the_arguments():
    """The kernel must follow the device record, not the launch arguments."""
    (layer,) = _layers(1, 1, 8, 2, 900, 64)
    gen = torch.Generator(device=DEV); gen.manual_seed(2)
    for _ in range(20):
        kv = torch.randn(1, 2, 1, 128, generator=gen, device=DEV).to(torch.bfloat16)
        layer.append_staging(kv, kv)
    q = torch.randn(1, 8, 1, 128, generator=gen, device=DEV).to(torch.bfloat16)
    want = layer.decode_attention(q, 4).clone()                    # 20 staged tokens
    rec = torch.tensor([layer._n_quant, 20], dtype=torch.int32, device=DEV)
    layer.bind_lengths(rec)
    plan = layer._decode_plan(q.reshape(8, 128), 4)
    plan.args.n_staging = 3                                        # a stale host value
    out = torch.empty_like(want)
    plan.run(q.reshape(8, 128), out=out.view(8, 128))
    assert torch.equal(out, want)
    rec[1] = 3
    out3 = torch.empty_like(want)
    plan.run(q.reshape(8, 128), out=out3.view(8, 128))
    assert not torch.equal(out3, want)
    layer.bind_lengths(None)


def test_rope_inside_the_decode_step_equals_eager_rope():
    """decode_step(rope=(cos, sin)) on unrotated q / k against Hugging Face's eager rotation followed by the plain
    decode_step: outputs and the stored K rows bit for bit (the kernel rounds every product and the sum to bf16 as the
    eager bf16 arithmetic does), across a staging flush."""
    B, H_Q, H_KV, N, W = 2, 8, 2, 700, 64
    R = H_Q // H_KV
    a, b = _layers(1, B, H_Q, H_KV, N, W)[0], _layers(1, B, H_Q, H_KV, N, W)[0]
    gen = torch.Generator(device=DEV); gen.manual_seed(4)
    inv = 1.0 / (10000 ** (torch.arange(0, 128, 2, device=DEV).float() / 128))
    for step in range(140):
        q = torch.randn(B, H_Q, 1, 128, generator=gen, device=DEV).to(torch.bfloat16)
        k = torch.randn(B, H_KV, 1, 128, generator=gen, device=DEV).to(torch.bfloat16)
        v = torch.randn(B, H_KV, 1, 128, generator=gen, device=DEV).to(torch.bfloat16)
        pos = torch.tensor([N + step, N + step + 3], device=DEV).float()            # a position per batch entry
        ang = pos[:, None] * inv[None, :]
        cos = torch.cat((ang.cos(), ang.cos()), -1).to(torch.bfloat16)               # [B, 128] as HF's rotary module gives it
        sin = torch.cat((ang.sin(), ang.sin()), -1).to(torch.bfloat16)

        def eager(x):
            rot = torch.cat((-x[..., 64:], x[..., :64]), dim=-1)
            return (x * cos[:, None, None, :]) + (rot * sin[:, None, None, :])

        want = a.decode_step(eager(q), eager(k), v, R)
        got = b.decode_step(q, k, v, R, rope=(cos[:, None, :], sin[:, None, :]))
        assert torch.equal(got, want), step
    assert torch.equal(a._staging_buf_k, b._staging_buf_k) and torch.equal(a.k_quant_packed, b.k_quant_packed)
