"""CPU checks of the boundary: the shared library builds, loads and exports every
symbol the public header declares; host-side argument checks fail loudly."""

import ctypes as C
import os
import re

import pytest
import torch

import hyquant_b200 as hq
from hyquant_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def header_symbols():
    text = open(os.path.join(ROOT, "include", "hyquant_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(hq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.lib()
    syms = header_symbols()
    assert syms, "no declarations found in the header"
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/hyquant_b200.h but not exported"
    assert sorted(_lib.EXPORTS) == syms
    assert b"sm_100a" in lib.hq_version()


def test_decode_args_struct_matches_header_size():
    # the C side checks struct_bytes; a mismatch must come back as HQ_ERR_INVALID, not a crash
    a = _lib.DecodeArgs()
    a.struct_bytes = C.sizeof(_lib.DecodeArgs) - 8
    rc = _lib.lib().hq_decode_splitk(C.byref(a), None)
    assert rc == -1
    assert b"struct_bytes" in _lib.lib().hq_last_error()


def test_argument_validation_without_gpu():
    lib = _lib.lib()
    n = C.c_int64(0)
    assert lib.hq_decode_workspace_bytes(8, 4, C.byref(n)) == 0 and n.value > 0
    assert lib.hq_decode_workspace_bytes(8, 17, C.byref(n)) == -1
    assert lib.hq_topk(None, 0, 1, 10, 20, None, None, None) == -1          # k > n
    assert lib.hq_quant_pack_int4(None, 0, 0, 0, 2, 2, None, 0, None, 0, 0, 0, None) == -1
    assert lib.hq_lse_merge(None, None, None, 0, 4, None, 0, 0, None) == -1


def test_peer_exchange_layout_and_validation_without_gpu():
    """The address arithmetic of the exchange buffer (no memory is touched): the local state and every
    (parity, source rank) receive slot lie inside the buffer and do not overlap; bad arguments are refused."""
    lib = _lib.lib()
    world, rows = 8, 128
    n = C.c_int64(0)
    assert lib.hq_peer_exchange_bytes(world, rows, C.byref(n)) == 0
    assert lib.hq_peer_exchange_bytes(17, rows, C.byref(n)) == -1 and lib.hq_peer_exchange_bytes(0, rows, C.byref(n)) == -1
    assert lib.hq_peer_exchange_bytes(world, rows, C.byref(n)) == 0
    base = 1 << 20                                            # a made-up, 256-byte aligned device address
    spans = [(base, base + 256)]                              # the header
    for seq in (1, 2):
        m, l, acc = C.c_void_p(), C.c_void_p(), C.c_void_p()
        assert lib.hq_peer_slot(base, world, rows, seq, C.byref(m), C.byref(l), C.byref(acc)) == 0
        assert l.value == m.value + 4 * rows and acc.value == m.value + 8 * rows and acc.value % 16 == 0
        spans.append((m.value, m.value + 4 * 130 * rows))
        for src in range(world):
            w = C.c_void_p()
            assert lib.hq_peer_recv_slot(base, world, rows, seq, src, C.byref(w)) == 0
            assert w.value % 8 == 0
            spans.append((w.value, w.value + 8 * 130 * rows))
    w = C.c_void_p()
    assert lib.hq_peer_recv_slot(base, world, rows, 1, world, C.byref(w)) == -1
    # same parity, same slot: calls seq and seq + 2 reuse it
    w2 = C.c_void_p()
    lib.hq_peer_recv_slot(base, world, rows, 1, 3, C.byref(w)); lib.hq_peer_recv_slot(base, world, rows, 3, 3, C.byref(w2))
    assert w.value == w2.value
    spans.sort()
    assert spans[0][0] == base and spans[-1][1] <= base + n.value
    assert all(a1 <= b0 for (_, a1), (b0, _) in zip(spans, spans[1:]))
    a = _lib.PeerExchangeArgs()
    a.struct_bytes = C.sizeof(_lib.PeerExchangeArgs) - 8
    assert lib.hq_peer_exchange_merge(C.byref(a), None) == -1
    a.struct_bytes, a.world, a.rank, a.rows, a.seq = C.sizeof(_lib.PeerExchangeArgs), 2, 0, 4, 0
    assert lib.hq_peer_exchange_merge(C.byref(a), None) == -1                  # seq starts at 1


def test_product_path_has_no_cpu_fallback():
    x = torch.zeros(1, 4, 128)
    with pytest.raises(hq.HyQuantError):
        hq.quantize_per_token(x, 4)
    with pytest.raises(hq.HyQuantError):
        hq.compute_vertical_indices(torch.zeros(1, 2, 8, 128), torch.zeros(1, 2, 300, 128), 64, 0.05)
    with pytest.raises(hq.HyQuantError):
        hq.fused_d_stage_decode(torch.zeros(4, 128), *[torch.zeros(1, 0, 64)] * 10, 4, 4, kv_repeat=4)
    with pytest.raises(hq.HyQuantError):
        hq.fused_d_stage_decode(torch.zeros(4, 128), *[torch.zeros(1, 0, 64)] * 10, 8, 8, kv_repeat=4)
    with pytest.raises(ValueError):
        hq.quantize_per_token(x, 3)


def test_reference_interface_names():
    hq.install_as_src()
    import src.ops as ops
    from src.ops.d_stage_kv_cache import DStageKVCache, DStageLayerCache
    from src.ops.decode_d_stage import GROUP_SIZE, fused_d_stage_decode, quantize_per_token
    from src.patch._common import D_STAGE_MODES, compute_vertical_indices, handle_d_stage_cache, validate_patch_args
    assert GROUP_SIZE == 128 and "hybrid_full" in D_STAGE_MODES
    cache = ops.create_cache_for_mode("hybrid_full", num_layers=2, window_size=128, top_ratio=0.05)
    assert isinstance(cache, DStageKVCache) and len(cache) == 2 and cache.get_seq_length() == 0
    assert cache.get_layer(1).k_bits == 4 and cache.get_layer(1).use_vert
    assert ops.create_cache_for_mode("dense", 2) is None
    assert cache.get_mask_sizes(5) == (5, 0) and cache.get_max_cache_shape() == -1 and bool(cache)
    with pytest.raises(NotImplementedError):
        cache.batch_repeat_interleave(2)
    with pytest.raises(ValueError):
        validate_patch_args("nope", 128, 0.05)
    with pytest.raises(ValueError):
        validate_patch_args("d_k4v4", -1, 0.05)
    with pytest.raises(ValueError):
        validate_patch_args("d_k4v4", 1, 0.0)


def test_integration_doc_struct_matches_the_binding():
    """The ctypes mirror of hq_decode_args printed in INTEGRATION.md must be the one the package binds: a reader who
    pastes it gets the size the library checks (struct_bytes)."""
    import ctypes as C
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    text = open(os.path.join(root, "INTEGRATION.md")).read()
    m = re.search(r"class hq_decode_args\(C\.Structure\):.*?_fields_ = (\[.*?\])\n\ndef ", text, re.S)
    assert m, "the struct listing is missing from INTEGRATION.md"
    fields = eval(m.group(1), {"C": C})
    Doc = type("Doc", (C.Structure,), {"_fields_": fields})
    assert [f[0] for f in fields] == [f[0] for f in _lib.DecodeArgs._fields_]
    assert C.sizeof(Doc) == C.sizeof(_lib.DecodeArgs)
