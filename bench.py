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

``--impl reference`` times the CPU restatement of the reference's own PyTorch
fallback path (oracle/hq_oracle.py) on the host cores, on one layer call per
step of the same workload.
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
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


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


def time_kernel_steps(torch, layers, qs, steps, warmup, dist=None, flush=None, graph=True, kv_repeat=None, overlap=True):
    """K steps of (one decode launch per layer), device-timed; returns ms total, launches.
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
    if flush is None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            step_fn()
        e1.record()
        torch.cuda.synchronize()
        total = e0.elapsed_time(e1)
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
        total = sum(a.elapsed_time(b) for a, b in evs)
    if dist is not None:
        dist.barrier()
    return total, steps * len(plans)


def time_e2e_steps(torch, hq, layers, steps, warmup, seed, dist=None):
    """Per step: q/k/v of the new token for every layer from pinned host memory -> device; per layer append
    to staging (flush when full) and decode attention; every layer's output back to the host."""
    r = H_Q // H_KV
    n = len(layers)
    g = torch.Generator(); g.manual_seed(seed)
    tot = steps + warmup
    rows = B * (H_Q + 2 * H_KV)
    # one pinned message per step: the new token's q | k | v rows of every layer; one pinned result per step
    hin = torch.randn(tot, n, rows, D, generator=g).to(torch.bfloat16).pin_memory()
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
    h2d = n * (B * H_Q * D + 2 * B * H_KV * D) * 2
    d2h = n * B * H_Q * D * 2
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


def bench_batched_decode(torch, hq, dev, rank, world, dist, graph):
    """Batched decode at Qwen3-32B attention shapes (batch 16, 64 query / 8 KV heads, prefix 32K): the KV heads
    are split over the ranks, each rank decodes its heads, nothing is exchanged.  Total work is fixed."""
    b, h_q, h_kv, n = 16, 64, 8, 32768
    if h_kv % world:
        return None
    hq_l, hkv_l = h_q // world, h_kv // world
    caches = 4
    ls, qq = zip(*[build_layer(hq, torch, 7000 + 10 * i + rank, n, dev, b=b, h_q=hq_l, h_kv=hkv_l) for i in range(caches)])
    bts = layer_bytes(ls[0], b * hq_l)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev) if caches * bts < (256 << 20) else None
    ms, cnt = time_kernel_steps(torch, list(ls), list(qq), 10, 3, dist, flush=flush, graph=graph, kv_repeat=h_q // h_kv)
    if dist is not None:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
    us = ms * 1e3 / cnt
    return {"workload": "batch 16, 64q/8kv, d=128, prefix 32768, W=128, rho=5%, K4V4, 64 staging tokens",
            "sharding": f"kv heads over {world} rank(s), {hkv_l} per rank, no collective", "scaling": "strong",
            "us_per_call": round(us, 2), "bytes_per_call_per_rank": bts,
            "gbps_all_ranks": round(bts * world / us / 1e3, 1), "caches_per_rank": caches,
            "l2": "caches exceed L2" if flush is None else "flushed before each pass"}


def bench_long_context_decode(torch, hq, dev, rank, world, dist):
    """Long-context decode at GLM-4-9B attention shapes (batch 4, 32 query / 2 KV heads, prefix 128K): each step
    appends one token per layer (a staging flush every 128 tokens) and decodes.  With more than one rank the prefix
    is sequence-sharded; the partial softmax states are exchanged over peer memory and merged by one small kernel
    after the decode kernel (``hq_peer_exchange_merge``).  The form in which the decode kernel does the exchange
    itself and the NCCL all-gather + merge form are timed after it for comparison."""
    from hyquant_b200 import sharded
    b, h_q, h_kv, n = 4, 32, 2, 131072
    nl, steps, warm = 4, 2048, 8                 # 2048 generated tokens: 16 staging flushes per layer
    r = h_q // h_kv
    layers, qs = [], []
    px = sharded.PeerExchange(rows=b * h_q) if world > 1 else None
    for i in range(nl):
        full, qd = build_layer(hq, torch, 9000 + i, n, dev, b=b, h_q=h_q, h_kv=h_kv)     # same seed on every rank
        if world > 1:
            shard = sharded.shard_layer_sequence(full, world, rank)
            del full
            layers.append(sharded.SequenceShardedLayer(shard, exchange=px))
        else:
            layers.append(full)
        qs.append(qd)
    torch.cuda.empty_cache()
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
                     "peer_exchange_status": status}
        px.close()
    full_bytes = algorithmic_bytes(b * h_kv, b * h_q, n - W - int((n - W) * RHO), int((n - W) * RHO) + W + 64)
    out = {"workload": "batch 4, 32q/2kv, d=128, prefix 131072, W=128, rho=5%, K4V4; per step and layer: append one "
                       "token (flush at 128) + decode", "layers": nl, "steps": steps,
           "sharding": "single GPU" if world == 1 else f"sequence-sharded over {world} ranks; one kernel stores (m, l, acc) into the peers' "
                       "buffers over NVLink, waits for theirs and merges",
           "scaling": "strong", "us_per_layer_token": round(us, 2), "cache_bytes_per_layer": full_bytes,
           "gbps_all_ranks": round(full_bytes / us / 1e3, 1),
           "launch_mode": "python, host-driven: " + ("two launches per layer and token (decode of the shard, taking the new token on the tail rank; exchange + merge)" if world > 1 else "decode_step (append + decode in one launch)"),
           "l2": "4 layer caches of 138 MB in turn; a layer's shard is re-read only after the other three"}
    out.update(res_extra)
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
    """Seconds per decode-attention call of the reference's CPU path (torch-CPU
    restatement, fp32, all intra-op threads), and the call's algorithmic bytes."""
    import torch
    from oracle import hq_oracle_torch as ot
    torch.set_num_threads(os.cpu_count() or 1)
    c, qd = build_cpu_layer()
    r = H_Q // H_KV
    segs = ot.from_numpy_cache(c)
    q = torch.from_numpy(qd)
    for _ in range(warmup):
        ot.decode_attention_fallback(q, *segs, B, H_KV, r)
    t0 = time.perf_counter()
    for _ in range(calls):
        ot.decode_attention_fallback(q, *segs, B, H_KV, r)
    dt = (time.perf_counter() - t0) / calls
    nbytes = algorithmic_bytes(B * H_KV, B * H_Q, c.k_quant_packed.shape[1],
                               c.k_topk.shape[1] + c.staging_ptr + c.k_window.shape[1])
    return dt, nbytes, torch.get_num_threads()


CONFIG = {"workload": "decode attention, Llama-3.1-8B shapes (B=1, 32q/8kv, d=128), prefix 32768, W=128, rho=5%, "
                      "staging 64, K4V4 per-token scales, 32 layer caches per token",
          "l2_policy": "inputs larger than L2 (32 distinct 40 MB caches per step = 1.3 GB)",
          "parallelism": "one replica of the workload per GPU (KV-head groups are independent; no collective)"}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    calls = max(1, args.steps)
    dt, nbytes, cores = time_cpu_calls(calls, max(1, min(args.warmup, 2)))
    gbs = nbytes / dt / 1e9
    line = {
        "impl": "reference", "metric": "decode_attn_hbm_gbps", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": calls, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": CONFIG,
        "us_per_call": dt * 1e6,
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                         "sample": "one layer's decode-attention call per step (1/32 of a token) of the same 32K workload, "
                                   "torch-CPU restatement of the reference's PyTorch fallback in fp32, intra-op threads = cores"},
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

    sampler = ClockSampler(local)
    sampler.start()
    ms, launches = time_kernel_steps(torch, layers, qs, args.steps, args.warmup, dist, graph=not args.no_graph,
                                     overlap=not args.no_overlap)
    ms_plain = None
    if not args.no_overlap and not args.no_decode:
        ms_plain, _ = time_kernel_steps(torch, layers, qs, args.steps, args.warmup, dist, graph=not args.no_graph, overlap=False)
    if args.no_e2e:
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = time_e2e_steps(torch, hq, layers, args.steps, args.warmup, 99 + rank, dist)
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
    if rank == 0 and not args.no_prefill:
        from hyquant_b200.synth import gen_torch
        from hyquant_b200.sage_unified import PrefillPlan
        bf16_peak = None
        try:
            bf16_peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops_sustained"])
        except Exception:
            pass
        for n in [int(x) for x in args.prefill_seq.split(",")]:
            t = gen_torch(1, H_Q, H_KV, n, D, W, RHO, 2000 + n.bit_length(), n_qry=n, device=dev)
            t0 = time.perf_counter()
            vidx = hq.compute_vertical_indices(t["q"][:, :, -256:].mean(dim=2, keepdim=True), t["k"], W, RHO, kv_repeat=H_Q // H_KV)
            plan = PrefillPlan(t["q"], t["k"], t["v"], vidx, W, None, True)
            torch.cuda.synchronize()
            prep_ms = (time.perf_counter() - t0) * 1e3
            for _ in range(2):
                plan.run()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 5 if n <= 8192 else 3
            e0.record()
            for _ in range(reps):
                plan.run()
            e1.record()
            torch.cuda.synchronize()
            ms_ = e0.elapsed_time(e1) / reps
            prefill.append({"seq": n, "ms": round(ms_, 3), "tflops": round(plan.flops / ms_ / 1e9, 1),
                            "frac_of_measured_bf16_sustained": None if not bf16_peak else round(plan.flops / ms_ / 1e9 / bf16_peak, 3),
                            "prepare_ms_first_call": round(prep_ms, 2),
                            "kernel": "hq::prefill_tc_kernel (tcgen05 kind::i8 QK^T + kind::f16 BF16 tiles and PV, TMEM accumulators)"})
            del plan, t
    batched = long_ctx = bit_widths = None
    legs = set() if args.no_extra else set(args.extra_legs.split(","))
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
            dt, nb, cores = time_cpu_calls(5, 1)
            cpu = {"value": nb / dt / 1e9, "unit": "GB/s", "cores": cores, "kind": "port",
                   "sample": "5 decode-attention calls of one layer of the same 32K workload (torch-CPU restatement of "
                             "the reference's PyTorch fallback in fp32, intra-op threads = cores)", "ms_per_call": dt * 1e3}
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
                    "path": "per step one pinned host message (q/k/v of every layer) to the device, DStageLayerCache.decode_step per layer (append_staging + decode_attention as one launch; the patched models' decode path), one message with every layer's output back to the host"},
            "gpu_launches": launches,
            "launch_mode": ("python" if args.no_graph else "cuda graph replay of one token (32 launches)") +
                           ("" if args.no_overlap else "; programmatic dependent launch: a call's blocks start and fetch their first "
                            "cache units while the call before it merges its splits; q, staging, output and workspace wait for it"),
            "roofline": {"bound": "hbm", "achieved": gbs_one, "peak": peak, "unit": "GB/s", "frac": gbs_one / peak,
                         "traffic": TRAFFIC_BYTES_PER_LAUNCH, "peak_source": peak_src,
                         "kernel": "hq::decode_splitk_kernel<1>", "algorithmic_bytes_per_launch": call_bytes},
            "cpu_baseline": cpu,
            "sweep": sweep,
            "prefill": prefill,
            "bit_width_decode": bit_widths,
            "batched_decode": batched,
            "long_context_decode": long_ctx,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


# DRAM bytes per launch of the decode kernel from an ncu capture of this workload
# (dram__bytes_read.sum + dram__bytes_write.sum, profiles/decode_splitk_cfg1_32k.md)
TRAFFIC_BYTES_PER_LAUNCH = 40289792


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
    ap.add_argument("--extra-legs", default="bits,batched,long", help="which of those legs to run (comma-separated)")
    args = ap.parse_args()
    args.warmup = max(3, args.warmup) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
