"""Shared helpers: fixture loading, seeded input regeneration, error metrics."""

from __future__ import annotations

import hashlib
import os

import numpy as np

from hyquant_b200.synth import gen_numpy
from oracle import hq_oracle as orc

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def load(name):
    return np.load(os.path.join(GOLDEN, name + ".npz"), allow_pickle=False)


class CacheCase:
    """Inputs of one ``make_golden.run_cache_case`` fixture, regenerated from the seed."""

    def __init__(self, name):
        g = load(name)
        self.g = g
        B, H_Q, H_KV, N, W, seed, n_append, n_qry = [int(x) for x in g["meta"]]
        self.B, self.H_Q, self.H_KV, self.N, self.W, self.seed, self.n_append = B, H_Q, H_KV, N, W, seed, n_append
        self.R = H_Q // H_KV
        self.rho = float(g["rho"][0])
        self.is_bf16 = bool(g["is_bf16"][0])
        self.k_bits, self.v_bits = ([int(x) for x in g["bits"]] if "bits" in g.files else [4, 4])
        case = gen_numpy(B, H_Q, H_KV, N, 128, W, self.rho, seed, n_qry=None if n_qry < 0 else n_qry)
        assert [sha(case.q), sha(case.k), sha(case.v), sha(case.q_decode)] == list(g["in_sha"]), \
            "seeded inputs differ from the ones the fixture was generated with"
        rf = orc.bf16_round if self.is_bf16 else (lambda a: a)
        self.round_fn = orc.bf16_round if self.is_bf16 else None
        self.q, self.k, self.v = rf(case.q), rf(case.k), rf(case.v)
        rng = np.random.Generator(np.random.PCG64(seed + 77))
        nk = rng.standard_normal((n_append, B, H_KV, 1, 128), dtype=np.float32)
        nv = rng.standard_normal((n_append, B, H_KV, 1, 128), dtype=np.float32)
        nq = rng.standard_normal((n_append, B, H_Q, 1, 128), dtype=np.float32)
        assert [sha(nk), sha(nv), sha(nq)] == list(g["append_sha"])
        self.new_k, self.new_v, self.new_q = rf(nk), rf(nv), rf(nq)
        self.probe_steps = [int(s) for s in g["probe_steps"]]
        self.query_tail = self.q[:, :, -min(W, self.q.shape[2]):, :]

    def oracle_freeze(self, own_selection=None):
        """bf16 fixtures take the reference's selection as given (bf16 scores tie)."""
        own = (not self.is_bf16) if own_selection is None else own_selection
        return orc.freeze(self.k, self.v, self.query_tail, self.R, self.W, self.rho,
                          k_bits=self.k_bits, v_bits=self.v_bits, round_fn=self.round_fn,
                          vidx_override=None if own else self.g["frozen_vidx"])


def max_abs(a, b):
    return float(np.abs(np.asarray(a, dtype=np.float64) - np.asarray(b, dtype=np.float64)).max())
