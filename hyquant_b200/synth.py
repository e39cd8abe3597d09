"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no datasets or checkpoints are needed by the path).

Q/K/V ~ N(0,1); four K channels carry a +4 sigma bias (channel outliers); a
``rho`` fraction of prefix key rows per (batch, kv-head) gets +3 along the unit
mean-query direction of the KV group, so they become "vertical lines" — keys
that every recent query attends to.

Two back-ends produce the same *distribution*: :func:`gen_numpy` (CPU, used by
parity tests — bit-reproducible from the seed) and :func:`gen_torch` (device
side, used by the benchmark where tensors are too large to ship from the host).
"""

from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class SynthCase:
    q: np.ndarray            # [B, H_Q, N_qry, D]  prefill queries
    k: np.ndarray            # [B, H_KV, N, D]
    v: np.ndarray            # [B, H_KV, N, D]
    q_decode: np.ndarray     # [B, H_Q, 1, D]
    outlier_channels: np.ndarray
    vertical_pos: np.ndarray  # [B, H_KV, T]


def n_vertical(n: int, window: int, rho: float) -> int:
    p = max(0, n - window)
    return min(max(1, int(math.ceil(p * rho))), p) if p > 0 else 0


def gen_numpy(B: int, H_Q: int, H_KV: int, N: int, D: int = 128, W: int = 128,
              rho: float = 0.05, seed: int = 0, n_qry: int | None = None,
              delta: float = 3.0, w_q: int | None = None) -> SynthCase:
    """float32 tensors; cast/round to bf16 at the call site when needed."""
    rng = np.random.Generator(np.random.PCG64(seed))
    n_qry = N if n_qry is None else n_qry
    w_q = W if w_q is None else w_q
    q = rng.standard_normal((B, H_Q, n_qry, D), dtype=np.float32)
    k = rng.standard_normal((B, H_KV, N, D), dtype=np.float32)
    v = rng.standard_normal((B, H_KV, N, D), dtype=np.float32)
    qd = rng.standard_normal((B, H_Q, 1, D), dtype=np.float32)
    ch = rng.permutation(D)[:4]
    k[..., ch] += 4.0
    R = H_Q // H_KV
    P = max(0, N - W)
    T = n_vertical(N, W, rho)
    vpos = np.zeros((B, H_KV, T), dtype=np.int64)
    if T > 0:
        tail = q[:, :, -min(w_q, n_qry):, :].mean(axis=2)               # [B,H_Q,D]
        g = tail.reshape(B, H_KV, R, D).mean(axis=2)                     # [B,H_KV,D]
        g = g / np.maximum(np.linalg.norm(g, axis=-1, keepdims=True), 1e-6)
        for b in range(B):
            for h in range(H_KV):
                pos = rng.permutation(P)[:T]
                vpos[b, h] = pos
                k[b, h, pos, :] += delta * g[b, h][None, :] * math.sqrt(D) / 4.0
    return SynthCase(q=q, k=k, v=v, q_decode=qd, outlier_channels=ch, vertical_pos=vpos)


def gen_torch(B: int, H_Q: int, H_KV: int, N: int, D: int = 128, W: int = 128,
              rho: float = 0.05, seed: int = 0, n_qry: int | None = None,
              delta: float = 3.0, device="cuda", dtype=None):
    """Device-side generator (torch).  Returns dict of tensors in ``dtype``."""
    import torch
    dtype = torch.bfloat16 if dtype is None else dtype
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    n_qry = N if n_qry is None else n_qry
    R = H_Q // H_KV
    q = torch.randn((B, H_Q, n_qry, D), generator=g, device=device, dtype=torch.float32)
    k = torch.randn((B, H_KV, N, D), generator=g, device=device, dtype=torch.float32)
    v = torch.randn((B, H_KV, N, D), generator=g, device=device, dtype=torch.float32)
    qd = torch.randn((B, H_Q, 1, D), generator=g, device=device, dtype=torch.float32)
    ch = torch.randperm(D, generator=g, device=device)[:4]
    k[..., ch] += 4.0
    P = max(0, N - W)
    T = n_vertical(N, W, rho)
    if T > 0:
        tail = q[:, :, -min(W, n_qry):, :].mean(dim=2)
        gm = tail.reshape(B, H_KV, R, D).mean(dim=2)
        gm = gm / gm.norm(dim=-1, keepdim=True).clamp_min(1e-6)
        pos = torch.rand((B, H_KV, P), generator=g, device=device).argsort(dim=-1)[..., :T]
        add = (delta * math.sqrt(D) / 4.0) * gm[:, :, None, :].expand(B, H_KV, T, D)
        k.scatter_add_(2, pos[..., None].expand(B, H_KV, T, D), add)
    return {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "q_decode": qd.to(dtype)}
