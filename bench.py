#!/usr/bin/env python
"""Benchmark of the hybrid-precision decode attention path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (per GPU): decode attention at Llama-3.1-8B shapes — batch 1, 32 query /
8 KV heads, head_dim 128, prefix 32768, window 128, rho 5 % (1632 BF16
vertical-line tokens, 31008 INT4 tokens), 64 live staging tokens, K4V4 with
per-token scales.  One *step* is one generated token: 32 decode-attention calls,
one per layer, each over its own cache (32 x 40 MB = 1.3 GB > L2, so no call
re-reads a cache that is still in L2).  Inputs are seeded synthetic tensors with
the outlier / vertical-line structure of ``hyquant_b200.synth``.

Reported metric: achieved HBM throughput in GB/s = algorithmic bytes per call x
calls / device time (whole job, summed over GPUs), with the per-call and
per-token latencies beside it.  ``value`` times the kernels with every input
resident in HBM; ``e2e`` drives the reference-named cache API per layer with the
new token's q/k/v coming from pinned host memory and the attention output read
back to the host inside the timed region.

``--impl reference`` times the reference's own CPU path (its PyTorch fallback of
``DStageLayerCache.decode_attention``, fp32, all host threads) on one layer call per step of
the same workload, from the untracked copy of the reference under ``oracle/_ref`` when it is
there (``oracle/make_ref.py``), else the torch-CPU restatement in ``oracle/``.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

B, H_Q, H_KV, D = 1, 32, 8, 128
N_PREFIX, W, RHO, STAGING = 32768, 128, 0.05, 64
LAYERS = 32
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(bh_kv, bh_q, n_quant, n_bf16, k_bits=4, v_bits=4):
    """Bytes one decode call must move: a quantised token = 16 bytes per bit of width for K and for V
    (64+64 B at 4 bits) + 2+2 B scales, a BF16 token = 256+256 B, plus q read and out written
    (2 x 256 B per query head)."""
    return bh_kv * ((16 * k_bits + 16 * v_bits + 4) * n_quant + 512 * n_bf16) + 512 * bh_q


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s: no measured peak file beside bench.py)"


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.002)

    def start(self):
        if self.nv is not None:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t is not None:
            self._t.join()
        med = float(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------
# workload construction (device)
# ---------------------------------------------------------------------------

def build_layer(hq, torch, seed, n_prefix, device, b=B, h_q=H_Q, h_kv=H_KV, staging=STAGING, k_bits=4, v_bits=4):
    """Seeded K/V/Q -> vertical selection over [0, N-W) -> frozen four-segment cache."""
    from hyquant_b200.synth import gen_torch
    t = gen_torch(b, h_q, h_kv, n_prefix, D, W, RHO, seed, n_qry=256, device=device)
    layer = hq.DStageLayerCache(0, k_bits=k_bits, v_bits=v_bits, window_size=W, top_ratio=RHO, use_vert=True)
    layer.update_prefill(t["k"], t["v"])
    layer.save_query_tail(t["q"])
    r = h_q // h_kv
    # vertical lines from the 256 pooled queries, KV-group mean, candidates [0, N-W)
    pooled = t["q"].float().mean(dim=2, keepdim=True).reshape(b, h_kv, r, 1, D).mean(dim=2).to(t["k"].dtype)
    vidx = hq.compute_vertical_indices(pooled, t["k"], W, RHO, kv_repeat=1)
    layer.freeze(kv_repeat=r, vertical_indices=vidx)
    g = torch.Generator(device=device); g.manual_seed(seed + 7)
    for _ in range(staging):
        kn = torch.randn(b, h_kv, 1, D, generator=g, device=device).to(torch.bfloat16)
        vn = torch.randn(b, h_kv, 1, D, generator=g, device=device).to(torch.bfloat16)
        layer.append_staging(kn, vn)
    return layer, t["q_decode"]


def layer_bytes(layer, h_q_total):
    n_bf16 = layer.k_topk.shape[1] + layer._staging_ptr + layer.k_window.shape[1]
    return algorithmic_bytes(layer.k_window.shape[0], h_q_total, layer._n_quant, n_bf16, layer.k_bits, layer.v_bits)


def time_kernel_steps(torch, layers, qs, steps, warmup, dist=None, flush=None, graph=True, kv_repeat=None, overlap=True,
                      repeats=1):
    """K steps of (one decode launch per layer), device-timed; returns ms for the K steps, launches in them.
    ``repeats`` > 1 times the K-step block that many times back to back (each bracketed by its own events) and
    returns the median, so that a short block is not judged from one sample.
    ``flush``: a buffer larger than L2 that is rewritten before every step (outside the
    timed events) when the step's own caches do not exceed L2."""
    r = H_Q // H_KV if kv_repeat is None else kv_repeat
    plans = []
    outs = []
    for layer, q in zip(layers, qs):
        q2 = q.reshape(-1, D)
        plan = layer._decode_plan(q2, r)
        # consecutive calls work on different caches and only write their own output and the shared
        # workspace, so each may be launched to overlap the end of the call before it
        plan.args.flags = 1 if overlap else 0
        layer._plan_fresh = not overlap
        plans.append((plan, q2))
        outs.append(torch.empty_like(q2))
    for _ in range(warmup):
        for (p, q2), o in zip(plans, outs):
            p.run(q2, out=o)
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    def launch_all():
        for (p, q2), o in zip(plans, outs):
            p.run(q2, out=o)

    step_fn = launch_all
    if graph:
        # one token's launches captured once and replayed: the host cost of 32 Python
        # calls per step is not part of the kernel-side number
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            launch_all()
        step_fn = g.replay
        step_fn()
        torch.cuda.synchronize()
    totals = []
    for _ in range(max(1, repeats)):
        if flush is None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(steps):
                step_fn()
            e1.record()
            torch.cuda.synchronize()
            totals.append(e0.elapsed_time(e1))
        else:
            evs = []
            for _ in range(steps):
                flush.zero_()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                step_fn()
                e1.record()
                evs.append((e0, e1))
            torch.cuda.synchronize()
            totals.append(sum(a.elapsed_time(b) for a, b in evs))
    total = float(np.median(totals))
    if dist is not None:
        dist.barrier()
    return total, steps * len(plans)


def time_e2e_steps(torch, hq, layers, steps, warmup, seed, dist=None, graph=True):
    """Per step: q/k/v of the new token for every layer from pinned host memory -> device; per layer append
    to staging (flush when full) and decode attention; every layer's output back to the host.
    ``graph``: the step runs as one CUDA-graph replay (``DecodeStepGraph``: copy in, one fused append + attention launch
    per layer with the cache lengths read from the copied message, copy out); else layer by layer from Python."""
    r = H_Q // H_KV
    n = len(layers)
    g = torch.Generator(); g.manual_seed(seed)
    tot = steps + warmup
    rows = B * (H_Q + 2 * H_KV)
    # one pinned message per step: the new token's q | k | v rows of every layer; one pinned result per step
    hin = torch.randn(tot, n, rows, D, generator=g).to(torch.bfloat16).pin_memory()
    h2d = n * (B * H_Q * D + 2 * B * H_KV * D) * 2
    d2h = n * B * H_Q * D * 2
    if graph:
        from hyquant_b200.graph_decode import DecodeStepGraph
        dg = DecodeStepGraph(layers, B, H_Q, H_KV)
        msg = dg.host_in[:n * rows * D * 2].view(torch.bfloat16).view(n, rows, D)
        h2d += n * 8                          # + (n_quant, n_staging) of every layer

        def one_step(s):
            msg.copy_(hin[s])                 # the host produces the step's inputs into the message
            dg.step(synchronize=True)         # the step's result is on the host
    else:
        hout = torch.empty(n, B, H_Q, 1, D, dtype=torch.bfloat16).pin_memory()
        dev = layers[0].k_window.device
        xdev = torch.empty(n, rows, D, dtype=torch.bfloat16, device=dev)
        odev = torch.empty(n, B, H_Q, 1, D, dtype=torch.bfloat16, device=dev)
        qv = [xdev[li, :B * H_Q].view(B, H_Q, 1, D) for li in range(n)]
        kv = [xdev[li, B * H_Q:B * (H_Q + H_KV)].view(B, H_KV, 1, D) for li in range(n)]
        vv = [xdev[li, B * (H_Q + H_KV):].view(B, H_KV, 1, D) for li in range(n)]
        ov = [odev[li] for li in range(n)]

        def one_step(s):
            xdev.copy_(hin[s], non_blocking=True)
            for li, layer in enumerate(layers):
                layer.decode_step(qv[li], kv[li], vv[li], r, out=ov[li])      # append + attention, one launch
            hout.copy_(odev, non_blocking=True)
            torch.cuda.synchronize()      # the step's result is on the host

    for s in range(warmup):
        one_step(s)
    if dist is not None:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for s in range(warmup, tot):
        one_step(s)
    e1.record()
    torch.cuda.synchronize()
    wall_ms = (time.perf_counter() - t0) * 1e3
    if graph:
        dg.close()
    return max(e0.elapsed_time(e1), wall_ms), h2d, d2h


# ---------------------------------------------------------------------------
# CPU baseline (oracle port of the reference's PyTorch fallback)
# ---------------------------------------------------------------------------

def bench_bit_widths(torch, hq, dev, graph):
    """The decode call at the reference's other cache modes (d_k8v8, d_k4v2, d_k2v4), same shapes as the headline
    workload and the same launch pattern (graph replay, each launch overlapping the end of the one before), on four
    caches with an L2 flush between steps."""
    out = []
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for kb, vb in ((8, 8), (4, 2), (2, 4), (4, 4)):      # 4/4 again: this leg's launch pattern for comparison
        ls, qq = zip(*[build_layer(hq, torch, 6000 + 16 * kb + vb + i, N_PREFIX, dev, k_bits=kb, v_bits=vb) for i in range(4)])
        ms, cnt = time_kernel_steps(torch, list(ls), list(qq), 10, 3, flush=flush, graph=graph)
        us = ms * 1e3 / cnt
        bts = layer_bytes(ls[0], B * H_Q)
        out.append({"k_bits": kb, "v_bits": vb, "prefix": N_PREFIX, "us_per_call": round(us, 2), "bytes_per_call": bts,
                    "gbps": round(bts / us / 1e3, 1), "kernel": "hq::decode_splitk_kernel<1, true, %d, %d>" % (kb, vb)})
        del ls, qq
    return out


SHARD_TOL = 5e-3      # a sharded result may differ from the single-GPU one by the order of fp32 partial sums only


def bench_batched_decode(torch, hq, dev, rank, world, dist, graph):
    """Batched decode at Qwen3-32B attention shapes (batch 16, 64 query / 8 KV heads, prefix 32K): the KV heads
    are split over the ranks, each rank decodes its heads, nothing is exchanged.  Total work is fixed.
    Before the timing, one full cache (same seed on every rank) is decoded whole and as this rank's head group
    (``sharded.shard_layer_heads``); the two must agree."""
    from hyquant_b200 import sharded
    b, h_q, h_kv, n = 16, 64, 8, 32768
    if h_kv % world:
        return None
    hq_l, hkv_l = h_q // world, h_kv // world
    r = h_q // h_kv
    err = None
    if world > 1:
        full, qd = build_layer(hq, torch, 7700, n, dev, b=b, h_q=h_q, h_kv=h_kv)
        ref = full.decode_attention(qd, r).float()
        mine = sharded.shard_layer_heads(full, world, rank)
        del full
        h0, h1 = sharded.kv_head_range(h_kv, world, rank)
        got = mine.decode_attention(qd[:, h0 * r:h1 * r].contiguous(), r).float()
        t = (got - ref[:, h0 * r:h1 * r]).abs().max().reshape(1).double()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        err = float(t[0])
        del mine, ref, got
        torch.cuda.empty_cache()
    caches = 4
    ls, qq = zip(*[build_layer(hq, torch, 7000 + 10 * i + rank, n, dev, b=b, h_q=hq_l, h_kv=hkv_l) for i in range(caches)])
    bts = layer_bytes(ls[0], b * hq_l)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if caches * bts < (256 << 20) else None
    ms, cnt = time_kernel_steps(torch, list(ls), list(qq), 10, 3, dist, flush=flush, graph=graph, kv_repeat=r, repeats=5)
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    us = ms * 1e3 / cnt
    return {"workload": "batch 16, 64q/8kv, d=128, prefix 32768, W=128, rho=5%, K4V4, 64 staging tokens",
            "sharding": f"kv heads over {world} rank(s), {hkv_l} per rank, no collective", "scaling": "strong",
            "us_per_call": round(us, 2), "bytes_per_call_per_rank": bts,
            "gbps_all_ranks": round(bts * world / us / 1e3, 1), "caches_per_rank": caches,
            "frac_of_hbm_peak_per_gpu": round(bts / us / 1e3 / measured_peak()[0], 3),
            "sharded_max_abs_err": err, "sharded_ok": err is None or err <= SHARD_TOL,
            "l2": "caches exceed L2" if flush is None else "flushed before each pass"}


def bench_long_context_decode(torch, hq, dev, rank, world, dist):
    """Long-context decode at GLM-4-9B attention shapes (batch 4, 32 query / 2 KV heads, prefix 128K): each step
    appends one token per layer (a staging flush every 128 tokens) and decodes.  With more than one rank the prefix
    is sequence-sharded; the partial softmax states are exchanged over peer memory and merged by one small kernel
    after the decode kernel (``hq_peer_exchange_merge``).  The form in which the decode kernel does the exchange
    itself and the NCCL all-gather + merge form are timed after it for comparison.  Before the timing every rank
    decodes the full cache once and each of the three sharded forms once; the results must agree."""
    from hyquant_b200 import sharded
    b, h_q, h_kv, n = 4, 32, 2, 131072
    nl, steps, warm = 4, 2048, 8                 # 2048 generated tokens: 16 staging flushes per layer
    r = h_q // h_kv
    layers, qs, refs = [], [], []
    px = sharded.PeerExchange(rows=b * h_q) if world > 1 else None
    for i in range(nl):
        full, qd = build_layer(hq, torch, 9000 + i, n, dev, b=b, h_q=h_q, h_kv=h_kv)     # same seed on every rank
        if world > 1:
            refs.append(full.decode_attention(qd, r).float())
            shard = sharded.shard_layer_sequence(full, world, rank)
            del full
            layers.append(sharded.SequenceShardedLayer(shard, exchange=px))
        else:
            layers.append(full)
        qs.append(qd)
    torch.cuda.empty_cache()
    errs = {}
    if world > 1:
        for form in ("peer_exchange_kernel", "exchange_inside_decode_kernel", "nccl_allgather"):
            worst = 0.0
            for layer, q, ref in zip(layers, qs, refs):
                layer.exchange = "nccl" if form == "nccl_allgather" else px
                layer.fused = form == "exchange_inside_decode_kernel"
                worst = max(worst, float((layer.decode_attention(q, r).float() - ref).abs().max()))
            t = torch.tensor([worst], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            errs[form] = float(t[0])
        for layer in layers:
            layer.exchange, layer.fused = px, False
        del refs
    g = torch.Generator(device=dev); g.manual_seed(4242)
    n_nccl = 256 if world > 1 else 0
    kn = torch.randn(steps + 2 * n_nccl + 3 * warm, b, h_kv, 1, D, generator=g, device=dev).to(torch.bfloat16)
    vn = torch.randn(steps + 2 * n_nccl + 3 * warm, b, h_kv, 1, D, generator=g, device=dev).to(torch.bfloat16)
    tail = rank == world - 1

    outs = [torch.empty_like(q) for q in qs]

    def one(s):
        for layer, q, o in zip(layers, qs, outs):
            if world > 1:
                layer.decode_step(q, kn[s], vn[s], r, tail, out=o)
            else:
                layer.decode_step(q, kn[s], vn[s], r, out=o)

    def timed(s0, count):
        for s in range(s0, s0 + warm):
            one(s)
        torch.cuda.synchronize()
        if dist is not None:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for s in range(s0 + warm, s0 + warm + count):
            one(s)
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t[0])
        return ms * 1e3 / (count * nl)

    us = timed(0, steps)
    res_extra = {}
    if world > 1:
        for layer in layers:
            layer.fused = True
        us_two = timed(steps + warm, n_nccl)
        status = px.status()
        for layer in layers:
            layer.exchange = "nccl"
        res_extra = {"us_per_layer_token_exchange_inside_decode_kernel": round(us_two, 2),
                     "us_per_layer_token_nccl_allgather": round(timed(steps + n_nccl + 2 * warm, n_nccl), 2),
                     "peer_exchange_status": status, "sharded_max_abs_err": errs,
                     "sharded_ok": status == 0 and all(e <= SHARD_TOL for e in errs.values())}
        px.close()
    full_bytes = algorithmic_bytes(b * h_kv, b * h_q, n - W - int((n - W) * RHO), int((n - W) * RHO) + W + 64)
    out = {"workload": "batch 4, 32q/2kv, d=128, prefix 131072, W=128, rho=5%, K4V4; per step and layer: append one "
                       "token (flush at 128) + decode", "layers": nl, "steps": steps,
           "sharding": "single GPU" if world == 1 else f"sequence-sharded over {world} ranks; one kernel stores (m, l, acc) into the peers' "
                       "buffers over NVLink, waits for theirs and merges",
           "scaling": "strong", "us_per_layer_token": round(us, 2), "cache_bytes_per_layer": full_bytes,
           "gbps_all_ranks": round(full_bytes / us / 1e3, 1),
           "frac_of_hbm_peak_per_gpu": round(full_bytes / world / us / 1e3 / measured_peak()[0], 3),
           "launch_mode": "python, host-driven: " + ("two launches per layer and token (decode of the shard, taking the new token on the tail rank; exchange + merge)" if world > 1 else "decode_step (append + decode in one launch)"),
           "l2": "4 layer caches of 138 MB in turn; a layer's shard is re-read only after the other three"}
    out.update(res_extra)
    return out


def bench_prefill_heads(torch, hq, dev, rank, world, dist, n=32768):
    """The 32K hybrid prefill with its KV-head groups over the ranks (8 KV heads -> 8 / world per rank with their
    query heads; every (batch, kv-head) is independent, so nothing is exchanged).  Total work is fixed.  Times the
    attention kernel and, separately, the whole call including operand preparation, max over ranks."""
    from hyquant_b200.sage_unified import PrefillPlan
    from hyquant_b200.synth import gen_torch
    from hyquant_b200 import sharded
    if H_KV % world:
        return None
    r = H_Q // H_KV
    t = gen_torch(1, H_Q, H_KV, n, D, W, RHO, 2000 + n.bit_length(), n_qry=n, device=dev)     # same seed on every rank
    h0, h1 = sharded.kv_head_range(H_KV, world, rank)
    q, k, v = t["q"][:, h0 * r:h1 * r], t["k"][:, h0:h1], t["v"][:, h0:h1]
    vidx = hq.compute_vertical_indices(q[:, :, -256:].mean(dim=2, keepdim=True), k, W, RHO, kv_repeat=r)

    def whole():
        return PrefillPlan(q, k, v, vidx, W, None, True)

    plan = whole()
    for _ in range(2):
        plan.run()
    torch.cuda.synchronize()
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    reps = 3
    e[0].record()
    for _ in range(reps):
        plan.run()
    e[1].record()
    e[2].record()
    for _ in range(reps):
        whole().run()
    e[3].record()
    torch.cuda.synchronize()
    plan.check_status()
    ms = torch.tensor([e[0].elapsed_time(e[1]) / reps, e[2].elapsed_time(e[3]) / reps], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    flops = 4.0 * H_Q * D * n * (n + 1) / 2
    return {"workload": f"hybrid prefill, B=1, 32q/8kv, d=128, seq {n}, W=128, rho=5%", "scaling": "strong",
            "sharding": f"kv heads over {world} rank(s), {H_KV // world} per rank with their query heads, no collective",
            "ms_kernel": round(float(ms[0]), 3), "ms_with_preparation": round(float(ms[1]), 3),
            "tflops_all_ranks": round(flops / float(ms[0]) / 1e9, 1)}


def measure_tensor_peaks(torch, dev):
    """TFLOP/s (TOP/s) of this GPU's tcgen05 pipe for kind::i8, kind::f8f6f4 (e4m3) and kind::f16 (bf16), from the
    library's probe kernel: products issued back to back on every SM with the operands resident in shared memory (no
    loads, no epilogue) - an upper bound measured here rather than a nominal figure.  Median of 5 launches of ~1 ms."""
    import ctypes as C
    from hyquant_b200 import _lib
    lib = _lib.lib()
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    sms = C.c_int(0)
    out = {}
    for kind, name, kdim in ((0, "i8", 128), (1, "f8f6f4_e4m3", 128), (2, "f16_bf16", 64)):
        steps = 4096
        st = _lib.stream_ptr(dev)
        _lib.check(lib.hq_tc_peak(kind, 256, status.data_ptr(), C.byref(sms), st), "hq_tc_peak")
        times = []
        for _ in range(5):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            _lib.check(lib.hq_tc_peak(kind, steps, status.data_ptr(), C.byref(sms), st), "hq_tc_peak")
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        ms = float(np.median(times))
        out[name] = round(sms.value * steps * 2.0 * 128 * 256 * kdim / ms / 1e9, 1)
    out["status"] = int(status.item())
    out["how"] = "tcgen05.mma 128x256 products back to back on every SM, operands in shared memory, accumulators in tensor memory"
    return out


# ---------------------------------------------------------------------------
# the reference's own kernels on this GPU (Triton, compiled for sm_100 by the installed Triton)
# ---------------------------------------------------------------------------

def reference_dir():
    p = os.path.join(ROOT, "oracle", "_ref")
    return p if os.path.isdir(os.path.join(p, "src", "ops")) else None


def bench_reference_triton(torch, hq, dev, layer, q_decode, prefill_seqs):
    """The reference's Triton kernels on the same inputs, as the kernel to beat: its split-K decode on the headline
    cache (the reference's ``DStageLayerCache`` filled with this library's segments) and its
    ``sage_vertical_attention_v2`` (the whole call, as the reference has no separate preparation) at the prefill
    sizes.  Needs the untracked copy of the reference under ``oracle/_ref``."""
    ref = reference_dir()
    if ref is None:
        return {"unavailable": "oracle/_ref is absent (oracle/make_ref.py makes it where the reference checkout is)"}
    sys.path.insert(0, ref)
    os.environ.pop("HYBRID_ATTN_DECODE_KERNEL", None)
    try:
        from src.ops.d_stage_kv_cache import DStageLayerCache as RefLayer
        from src.ops.sage_unified import sage_vertical_attention_v2 as ref_prefill
    except Exception as e:      # e.g. no Triton on this machine
        return {"unavailable": f"the reference does not import here: {type(e).__name__}: {e}"}
    from hyquant_b200.synth import gen_torch
    out = {}
    r = H_Q // H_KV
    rl = RefLayer(0, k_bits=4, v_bits=4, window_size=W, top_ratio=RHO, use_vert=True)
    rl._B, rl._H_KV, rl._D, rl.phase = B, H_KV, D, "decode"
    rl.k_quant_packed, rl.v_quant_packed, rl.k_scale, rl.v_scale = layer.k_quant_packed, layer.v_quant_packed, layer.k_scale, layer.v_scale
    rl.k_topk, rl.v_topk, rl.k_window, rl.v_window = layer.k_topk, layer.v_topk, layer.k_window, layer.v_window
    rl._staging_buf_k, rl._staging_buf_v, rl._staging_ptr = layer._staging_buf_k, layer._staging_buf_v, layer._staging_ptr

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps

    theirs = rl.decode_attention(q_decode, r)
    ours = layer.decode_attention(q_decode, r)
    out["decode_us_per_call_32k"] = round(timed(lambda: rl.decode_attention(q_decode, r), 100) * 1e3, 2)
    out["decode_ours_us_per_call_same_loop"] = round(timed(lambda: layer.decode_attention(q_decode, r), 100) * 1e3, 2)
    out["decode_max_abs_diff_ours_vs_reference"] = float((ours.float() - theirs.float()).abs().max())
    out["decode_note"] = ("python-driven back-to-back calls on one cache (L2-warm); the reference's call is two torch.cat + two Triton "
                          "launches (_splitk_partial_kernel, _splitk_reduce_kernel)")
    for n in prefill_seqs:
        t = gen_torch(1, H_Q, H_KV, n, D, W, RHO, 2000 + n.bit_length(), n_qry=n, device=dev)
        vidx = hq.compute_vertical_indices(t["q"][:, :, -256:].mean(dim=2, keepdim=True), t["k"], W, RHO, kv_repeat=r)
        theirs = ref_prefill(t["q"], t["k"], t["v"], vidx, window_size=W)
        ours = hq.sage_vertical_attention_v2(t["q"], t["k"], t["v"], vidx, window_size=W)
        d = ours.float() - theirs.float()
        out[f"prefill_ms_{n}"] = round(timed(lambda: ref_prefill(t["q"], t["k"], t["v"], vidx, window_size=W), 3), 3)
        out[f"prefill_ours_ms_{n}_whole_call"] = round(timed(lambda: hq.sage_vertical_attention_v2(t["q"], t["k"], t["v"], vidx, window_size=W), 3), 3)
        out[f"prefill_max_abs_diff_{n}"] = float(d.abs().max())
        out[f"prefill_rel_mse_{n}"] = float((d ** 2).sum() / (theirs.float() ** 2).sum())
        del t, theirs, ours, d
        torch.cuda.empty_cache()
    return out


def bench_cache_ops(torch, hq, dev, hbm_peak):
    """The cache-side rows of the path at the headline shape (B = 1, 8 KV heads, 32K prefix): the prefill -> decode
    reorganisation (``freeze``: vertical-line selection + gather + compaction + quantisation), the selection alone,
    the per-token quantiser alone on the whole prefix, and one staging flush.  Each with its algorithmic bytes, and the
    reference's own ``freeze`` (eager PyTorch on the same GPU) beside it when ``oracle/_ref`` is there."""
    from hyquant_b200.synth import gen_torch, n_vertical
    from hyquant_b200 import decode_d_stage as dd
    r = H_Q // H_KV
    t = gen_torch(B, H_Q, H_KV, N_PREFIX, D, W, RHO, 1015, n_qry=W, device=dev)
    k, v, q = t["k"], t["v"], t["q"]

    def timed(fn, reps, setup=None):
        (setup or (lambda: None))()
        fn()
        torch.cuda.synchronize()
        total = 0.0
        for _ in range(reps):
            if setup is not None:
                setup()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            total += e0.elapsed_time(e1)
        return total / reps

    out = {"workload": f"B={B}, {H_KV} kv heads, d={D}, prefix {N_PREFIX}, W={W}, rho={RHO:.0%}; one layer"}
    state = {}

    def new_layer():
        layer = hq.DStageLayerCache(0, k_bits=4, v_bits=4, window_size=W, top_ratio=RHO, use_vert=True)
        layer.update_prefill(k, v)
        layer.save_query_tail(q)
        state["layer"] = layer

    ms = timed(lambda: state["layer"].freeze(kv_repeat=r), 5, setup=new_layer)
    layer = state["layer"]
    nq, nt = layer._n_quant, layer.k_topk.shape[1]
    heads = B * H_KV
    # K prefix read for the scores, K and V read once for the reorganisation, codes + scales and BF16 rows written
    fr_bytes = heads * (256 * (N_PREFIX - W) + 512 * N_PREFIX + 132 * nq + 512 * (nt + W))
    out["freeze"] = {"ms": round(ms, 4), "bytes": fr_bytes, "gbps": round(fr_bytes / ms / 1e6, 1),
                     "frac_of_measured_hbm": None if not hbm_peak else round(fr_bytes / ms / 1e6 / hbm_peak, 3),
                     "what": "DStageLayerCache.freeze: hq_vertical_scores_grouped + hq_topk + hq_cache_reorganize_bits, allocations included"}
    ms = timed(lambda: hq.compute_vertical_indices(q, k, W, RHO, kv_repeat=r), 10)
    sel_bytes = heads * 256 * (N_PREFIX - W)
    out["vertical_selection"] = {"ms": round(ms, 4), "bytes": sel_bytes, "gbps": round(sel_bytes / ms / 1e6, 1),
                                 "what": "compute_vertical_indices per query head: pooled scores over the prefix keys + exact top-k"}
    # the quantiser alone, on eight layers' worth of rows and back to back so that the launch is not what is timed
    x = k.reshape(heads, N_PREFIX, D).repeat(8, 1, 1)
    pk = torch.empty(x.shape[0], N_PREFIX, 64, dtype=torch.int8, device=dev)
    sc = torch.empty(x.shape[0], N_PREFIX, dtype=torch.float16, device=dev)
    dd.quantize_per_token_into(x, pk, sc, 0, nbits=4)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(5):
        dd.quantize_per_token_into(x, pk, sc, 0, nbits=4)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / 5
    qb = x.shape[0] * N_PREFIX * (256 + 66)
    out["quantize_per_token"] = {"ms": round(ms, 4), "bytes": qb, "gbps": round(qb / ms / 1e6, 1),
                                 "frac_of_measured_hbm": None if not hbm_peak else round(qb / ms / 1e6 / hbm_peak, 3),
                                 "what": "hq_quant_pack (4 bits) over 64 heads x 32768 rows, five launches back to back"}
    del x, pk, sc
    g = torch.Generator(device=dev).manual_seed(5)
    kn = torch.randn(B, H_KV, 127, D, generator=g, device=dev).bfloat16()
    layer.append_staging(kn, kn)

    def refill():
        layer._staging_ptr = 128

    ms = timed(lambda: layer._flush_staging_buffer(), 10, setup=refill)
    out["staging_flush"] = {"us": round(ms * 1e3, 2), "what": "128 staged tokens of every head quantised and appended in place (two launches)"}
    ref = reference_dir()
    if ref is not None:
        try:
            sys.path.insert(0, ref)
            from src.ops.d_stage_kv_cache import DStageLayerCache as RefLayer

            def new_ref():
                rl = RefLayer(0, k_bits=4, v_bits=4, window_size=W, top_ratio=RHO, use_vert=True)
                rl.update_prefill(k, v)
                rl.save_query_tail(q)
                state["ref"] = rl

            out["reference_freeze_ms_same_gpu"] = round(timed(lambda: state["ref"].freeze(kv_repeat=r), 3, setup=new_ref), 3)
            state.pop("ref", None)
        except Exception as e:
            out["reference_freeze_ms_same_gpu"] = f"unavailable: {type(e).__name__}: {e}"
    del t, layer, state
    torch.cuda.empty_cache()
    return out


def build_cpu_layer(seed=1015, n_prefix=N_PREFIX):
    from hyquant_b200.synth import gen_numpy, n_vertical
    from oracle import hq_oracle as orc
    case = gen_numpy(B, H_Q, H_KV, n_prefix, D, W, RHO, seed, n_qry=256)
    k, v, q = orc.bf16_round(case.k), orc.bf16_round(case.v), orc.bf16_round(case.q)
    r = H_Q // H_KV
    pooled = q.mean(axis=2, keepdims=True).reshape(B, H_KV, r, 1, D).mean(axis=2)
    vidx = orc.compute_vertical_indices(pooled, k, W, RHO)
    c = orc.freeze(k, v, q, r, W, RHO, round_fn=orc.bf16_round, vidx_override=vidx)
    rng = np.random.Generator(np.random.PCG64(seed + 7))
    for _ in range(STAGING):
        orc.append_staging(c, orc.bf16_round(rng.standard_normal((B, H_KV, 1, D), dtype=np.float32)),
                           orc.bf16_round(rng.standard_normal((B, H_KV, 1, D), dtype=np.float32)))
    return c, orc.bf16_round(case.q_decode)


def time_cpu_calls(calls, warmup):
    """Seconds per decode-attention call of the reference's CPU path on the host cores (fp32, all intra-op
    threads), the call's algorithmic bytes, the threads used and what ran: "reference" = the reference's own
    ``DStageLayerCache`` (PyTorch fallback, HYBRID_ATTN_DECODE_KERNEL=pytorch) from ``oracle/_ref``, built by its own
    ``freeze`` from the same seeded K/V; "port" = the torch-CPU restatement in ``oracle/`` when that copy is absent."""
    import torch
    torch.set_num_threads(os.cpu_count() or 1)
    r = H_Q // H_KV
    ref = reference_dir()
    if ref is not None:
        try:
            sys.path.insert(0, ref)
            os.environ["HYBRID_ATTN_DECODE_KERNEL"] = "pytorch"
            from src.ops.d_stage_kv_cache import DStageLayerCache as RefLayer
        except Exception:
            ref = None
    if ref is not None:
        from hyquant_b200.synth import gen_numpy
        case = gen_numpy(B, H_Q, H_KV, N_PREFIX, D, W, RHO, 1015, n_qry=256)
        layer = RefLayer(0, k_bits=4, v_bits=4, window_size=W, top_ratio=RHO, use_vert=True)
        layer.update_prefill(torch.from_numpy(case.k), torch.from_numpy(case.v))
        layer.save_query_tail(torch.from_numpy(case.q))
        layer.freeze(kv_repeat=r)
        g = torch.Generator(); g.manual_seed(1022)
        for _ in range(STAGING):
            layer.append_staging(torch.randn(B, H_KV, 1, D, generator=g), torch.randn(B, H_KV, 1, D, generator=g))
        q = torch.from_numpy(case.q_decode)
        fn = lambda: layer.decode_attention(q, r)      # noqa: E731
        nbytes = algorithmic_bytes(B * H_KV, B * H_Q, layer.k_quant_packed.shape[1],
                                   layer.k_topk.shape[1] + layer._staging_ptr + layer.k_window.shape[1])
        kind = "reference"
    else:
        from oracle import hq_oracle_torch as ot
        c, qd = build_cpu_layer()
        segs = ot.from_numpy_cache(c)
        q = torch.from_numpy(qd)
        fn = lambda: ot.decode_attention_fallback(q, *segs, B, H_KV, r)      # noqa: E731
        nbytes = algorithmic_bytes(B * H_KV, B * H_Q, c.k_quant_packed.shape[1],
                                   c.k_topk.shape[1] + c.staging_ptr + c.k_window.shape[1])
        kind = "port"
    for _ in range(warmup):
        fn()
    t0 = time.perf_counter()
    for _ in range(calls):
        fn()
    dt = (time.perf_counter() - t0) / calls
    return dt, nbytes, torch.get_num_threads(), kind


CPU_SAMPLE = {"reference": "decode-attention calls of one layer (1/32 of a token) of the same 32K workload through the reference's own "
                           "DStageLayerCache (PyTorch fallback path, fp32, cache frozen by the reference from the same seeded K/V), "
                           "intra-op threads = cores",
              "port": "decode-attention calls of one layer (1/32 of a token) of the same 32K workload, torch-CPU restatement of the "
                      "reference's PyTorch fallback in fp32, intra-op threads = cores"}


CONFIG = {"workload": "decode attention, Llama-3.1-8B shapes (B=1, 32q/8kv, d=128), prefix 32768, W=128, rho=5%, "
                      "staging 64, K4V4 per-token scales, 32 layer caches per token",
          "l2_policy": "inputs larger than L2 (32 distinct 40 MB caches per step = 1.3 GB)",
          "parallelism": "one replica of the workload per GPU (KV-head groups are independent; no collective)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    calls = max(1, args.steps)
    dt, nbytes, cores, kind = time_cpu_calls(calls, max(1, min(args.warmup, 2)))
    gbs = nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": calls, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
        "us_per_call": dt * 1e6,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": kind,
                         "sample": f"{calls} step(s), each one of the " + CPU_SAMPLE[kind]},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def run_ours(args):
    import torch
    import hyquant_b200 as hq
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback "
                         "(use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist_.init_process_group("nccl", device_id=dev)
        dist = dist_
    layers, qs = [], []
    if args.no_decode:
        args.layers, args.no_e2e, args.no_sweep, args.no_cpu_baseline, args.no_extra = 1, True, True, True, True
    for li in range(args.layers):
        layer, qd = build_layer(hq, torch, 1015 + 100 * rank + li, N_PREFIX, dev)
        layers.append(layer); qs.append(qd)
    call_bytes = layer_bytes(layers[0], B * H_Q)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()      # a profiler started with its collection off (e.g. ncu --profile-from-start off) begins here, after the set-up

    sampler = ClockSampler(local)
    sampler.start()
    # the K-step block is timed `repeats` times back to back and the median is reported, so that the
    # headline does not rest on one 10 ms sample
    ms, launches = time_kernel_steps(torch, layers, qs, args.steps, args.warmup, dist, graph=not args.no_graph,
                                     overlap=not args.no_overlap, repeats=args.repeats)
    ms_plain = None
    if not args.no_overlap and not args.no_decode:
        ms_plain, _ = time_kernel_steps(torch, layers, qs, args.steps, args.warmup, dist, graph=not args.no_graph, overlap=False,
                                        repeats=min(3, args.repeats))
    if args.no_e2e:
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = time_e2e_steps(torch, hq, layers, args.steps, max(args.warmup, 3), 99 + rank, dist, graph=not args.no_graph)
    clocks = sampler.stop()      # sampled every 2 ms over the three decode loops (graph, plain launches, e2e)
    e2e_bytes = sum(layer_bytes(l, B * H_Q) for l in layers)     # staging has grown by then; close enough per step

    if dist is not None:
        t = torch.tensor([ms, e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms = float(t[0]), float(t[1])
    ms_per_step = ms / args.steps
    us_per_call = ms_per_step * 1e3 / args.layers
    gbs_one = call_bytes / (us_per_call * 1e-6) / 1e9
    value = gbs_one * world
    e2e_val = e2e_bytes / (e2e_ms / args.steps * 1e-3) / 1e9 * world
    peak, peak_src = measured_peak()

    sweep = []
    if rank == 0 and not args.no_sweep:
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)     # 2 x L2
        for n in (1024, 2048, 4096, 8192, 16384, 32768):
            ncache = 16
            ls, qq = zip(*[build_layer(hq, torch, 5000 + n + i, n, dev) for i in range(ncache)])
            m, cnt = time_kernel_steps(torch, list(ls), list(qq), 10, 3, flush=flush, graph=not args.no_graph)
            us = m * 1e3 / cnt
            bts = layer_bytes(ls[0], B * H_Q)
            sweep.append({"prefix": n, "staging": STAGING, "us_per_call": round(us, 3), "gbps": round(bts / us / 1e3, 1),
                          "bytes": bts, "caches": len(ls), "l2": "flushed before each pass over the caches"})
            del ls, qq
        # the same call at 32K with the staging buffer empty (right after a flush), one token, full
        for st_ in (0, 1, 127):
            ls, qq = zip(*[build_layer(hq, torch, 5500 + st_ + i, N_PREFIX, dev, staging=st_) for i in range(8)])
            m, cnt = time_kernel_steps(torch, list(ls), list(qq), 10, 3, flush=flush, graph=not args.no_graph)
            us = m * 1e3 / cnt
            bts = layer_bytes(ls[0], B * H_Q)
            sweep.append({"prefix": N_PREFIX, "staging": st_, "us_per_call": round(us, 3), "gbps": round(bts / us / 1e3, 1),
                          "bytes": bts, "caches": len(ls), "l2": "flushed before each pass over the caches"})
            del ls, qq
        del flush
    prefill = []
    tensor_peaks = None
    if rank == 0 and not args.no_prefill:
        tensor_peaks = measure_tensor_peaks(torch, dev)
        from hyquant_b200.synth import gen_torch
        from hyquant_b200.sage_unified import PrefillPlan
        bf16_peak = None
        try:
            bf16_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        except Exception:
            pass
        for n in [int(x) for x in args.prefill_seq.split(",")]:
            t = gen_torch(1, H_Q, H_KV, n, D, W, RHO, 2000 + n.bit_length(), n_qry=n, device=dev)
            vidx = hq.compute_vertical_indices(t["q"][:, :, -256:].mean(dim=2, keepdim=True), t["k"], W, RHO, kv_repeat=H_Q // H_KV)
            plan = PrefillPlan(t["q"], t["k"], t["v"], vidx, W, None, True)
            for _ in range(2):
                plan.run()
            torch.cuda.synchronize()
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
            reps = 5 if n <= 8192 else 3
            ev[0].record()
            for _ in range(reps):
                plan.run()
            ev[1].record()
            # the whole call as the reference's entry point makes it: vertical-line selection, quantisation, V transpose,
            # vertical gather and the attention kernel (device time; the allocator serves the buffers from its cache)
            ev[2].record()
            for _ in range(reps):
                vi = hq.compute_vertical_indices(t["q"][:, :, -256:].mean(dim=2, keepdim=True), t["k"], W, RHO, kv_repeat=H_Q // H_KV)
                PrefillPlan(t["q"], t["k"], t["v"], vi, W, None, True).run()
            ev[3].record()
            torch.cuda.synchronize()
            plan.check_status()
            ms_, ms_all = ev[0].elapsed_time(ev[1]) / reps, ev[2].elapsed_time(ev[3]) / reps
            # the reference's sage_fp8_attention entry point (INT8 Q K^T, no vertical lines or window): FP8 P V on
            # kind::f8f6f4 with the exact running maximum its arithmetic needs, and the same call with BF16 P V
            pv = {}
            for tag, fp8 in (("fp8_pv", True), ("bf16_pv", False)):
                pl = PrefillPlan(t["q"], t["k"], t["v"], None, 0, None, True, pv_fp8=fp8)
                pl.run()
                torch.cuda.synchronize()
                f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                f0.record()
                for _ in range(reps):
                    pl.run()
                f1.record()
                torch.cuda.synchronize()
                pl.check_status()
                pv[tag] = round(f0.elapsed_time(f1) / reps, 3)
                del pl
            prefill.append({"seq": n, "ms": round(ms_, 3), "tflops": round(plan.flops / ms_ / 1e9, 1),
                            "sage_fp8_attention_ms": pv,
                            "frac_of_measured_bf16_sustained": None if not bf16_peak else round(plan.flops / ms_ / 1e9 / bf16_peak, 3),
                            # INT8 Q K^T and BF16 P V are half of the flops each: the time the two pipes would need at their
                            # measured probe rates is the bound this fraction is taken against
                            "frac_of_measured_i8_qk_bf16_pv_bound": round(
                                (0.5 * plan.flops / tensor_peaks["i8"] + 0.5 * plan.flops / tensor_peaks["f16_bf16"]) / 1e9 / ms_, 3),
                            "ms_with_selection_and_preparation": round(ms_all, 3),
                            "tflops_with_selection_and_preparation": round(plan.flops / ms_all / 1e9, 1),
                            "kernel": "hq::prefill_tc_kernel (tcgen05 kind::i8 QK^T + kind::f16 BF16 tiles and PV, TMEM accumulators)"})
            del plan, t
    batched = long_ctx = bit_widths = prefill_heads = ref_triton = cache_ops = None
    legs = set() if args.no_extra else set(args.extra_legs.split(","))
    if "cache" in legs and rank == 0:
        cache_ops = bench_cache_ops(torch, hq, dev, peak if peak_src.startswith("measured") else None)
        torch.cuda.empty_cache()
    if "reference" in legs and rank == 0:
        ref_triton = bench_reference_triton(torch, hq, dev, layers[0], qs[0], [int(x) for x in args.prefill_seq.split(",")])
        torch.cuda.empty_cache()
    if "prefill_heads" in legs and (world > 1 or args.prefill_heads_single):
        prefill_heads = bench_prefill_heads(torch, hq, dev, rank, world, dist)
        torch.cuda.empty_cache()
    if "bits" in legs and rank == 0:
        bit_widths = bench_bit_widths(torch, hq, dev, not args.no_graph)
        torch.cuda.empty_cache()
    if "batched" in legs:
        batched = bench_batched_decode(torch, hq, dev, rank, world, dist, not args.no_graph)
        torch.cuda.empty_cache()
    if "long" in legs:
        long_ctx = bench_long_context_decode(torch, hq, dev, rank, world, dist)
        torch.cuda.empty_cache()
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline:
            dt, nb, cores, kind = time_cpu_calls(5, 1)
            cpu = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": kind,
                   "sample": "5 " + CPU_SAMPLE[kind], "ms_per_call": dt * 1e3}
        line = {
            "metric": "decode_attn_hbm_gbps", "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": CONFIG,
            "us_per_call": us_per_call, "us_per_token_32_layers": ms_per_step * 1e3,
            "us_per_call_without_overlap": None if ms_plain is None else ms_plain / args.steps * 1e3 / args.layers,
            "bytes_per_call": call_bytes, "frac_of_8TBps": gbs_one / 8000.0,
            "clocks": clocks,
            "e2e": {"value": e2e_val, "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms / args.steps,
                    "path": "per step one pinned host message (q/k/v of every layer and every layer's cache lengths) to the device, one fused append_staging + decode_attention launch per layer (DStageLayerCache.decode_step), one message with every layer's output back to the host" +
                            ("; the whole step is one CUDA-graph replay (DecodeStepGraph): the kernels read the lengths from the message" if not args.no_graph else "; launched layer by layer from Python")},
            "gpu_launches": launches,
            "launch_mode": ("python" if args.no_graph else "cuda graph replay of one token (32 launches)") +
                           ("" if args.no_overlap else "; programmatic dependent launch: a call's blocks start and fetch their first "
                            "cache units while the call before it merges its splits; q, staging, output and workspace wait for it"),
            "roofline": {"bound": "hbm", "achieved": gbs_one, "peak": peak, "unit": "GB/s", "frac": gbs_one / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                         "kernel": "hq::decode_splitk_kernel<1, true, 4, 4, 0>", "algorithmic_bytes_per_launch": call_bytes},
            "cpu_baseline": cpu,
            "sweep": sweep,
            "prefill": prefill,
            "tensor_pipe_peaks_measured": tensor_peaks,
            "bit_width_decode": bit_widths,
            "batched_decode": batched,
            "long_context_decode": long_ctx,
            "prefill_kv_head_groups": prefill_heads,
            "reference_triton_sm100": ref_triton,
            "cache_ops": cache_ops,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()
    bad = [name for name, leg in (("batched_decode", batched), ("long_context_decode", long_ctx))
           if leg is not None and leg.get("sharded_ok") is False]
    if bad:
        raise SystemExit(f"sharded result differs from the single-GPU result (or a peer wait ran out) in: {bad}")


# DRAM bytes per launch of the decode kernel from an ncu capture of this workload (dram__bytes_read.sum +
# dram__bytes_write.sum of hq::decode_splitk_kernel<1, true, 4, 4, 0>, mean of two launches); to be taken again
# whenever the kernel's loads change
TRAFFIC_BYTES_PER_LAUNCH = 40302592


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-sweep", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-prefill", action="store_true")
    ap.add_argument("--no-decode", action="store_true", help="profiling: minimal decode leg, prefill only")
    ap.add_argument("--prefill-seq", default="8192,32768", help="comma-separated prefill sequence lengths")
    ap.add_argument("--no-graph", action="store_true", help="launch from Python instead of replaying a CUDA graph")
    ap.add_argument("--layers", type=int, default=LAYERS, help="layer caches per step (32 = the workload; fewer for profiling)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-overlap", action="store_true", help="launch every decode call plainly (no programmatic dependent launch)")
    ap.add_argument("--no-extra", action="store_true", help="skip the bit-width, batched (64q/8kv x 16) and 128K long-context decode legs")
    ap.add_argument("--extra-legs", default="bits,batched,long,prefill_heads,reference,cache",
                    help="which of those legs to run (comma-separated); prefill_heads = the 32K prefill with its KV-head groups "
                         "over the ranks (N > 1), reference = the reference's Triton kernels on the same inputs (needs oracle/_ref)")
    ap.add_argument("--prefill-heads-single", action="store_true", help="run the prefill_heads leg on one GPU too")
    ap.add_argument("--repeats", type=int, default=10, help="times the K-step block is timed; the median is reported")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
