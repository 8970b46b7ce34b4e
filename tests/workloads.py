"""Seeded synthetic batches shared by the tests, the smoke check and the fixture generator (numpy only)."""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np


@dataclass
class BatchCase:
    kind: str                      # "DISTMULT" | "COMPLEX"
    edges: np.ndarray              # [B, 2|3] int64, node ids in [0, U)
    emb: np.ndarray                # [U, D] f32
    state: np.ndarray              # [U, D] f32 Adagrad state
    rel: Optional[np.ndarray]      # [R, D]
    inv_rel: Optional[np.ndarray]  # [R, D]
    dst_negs: np.ndarray           # [C, N] int64
    src_negs: Optional[np.ndarray]
    deg_rows: Optional[np.ndarray]  # [C, n_deg] batch rows the degree negatives were drawn from
    filt: np.ndarray               # [F, 2] (row, col) shared by both sides
    lr: float = 0.1

    @property
    def dims(self):
        B = self.edges.shape[0]
        C, N = self.dst_negs.shape
        return B, C, N, self.emb.shape[1], (0 if self.rel is None else self.rel.shape[0]), self.emb.shape[0]


def zipf_ids(rng, n, domain, alpha):
    """ids in [0, domain) with P(rank k) ~ 1/k^alpha, ranks scattered by a fixed permutation."""
    w = 1.0 / np.power(np.arange(1, domain + 1, dtype=np.float64), alpha)
    cdf = np.cumsum(w)
    cdf /= cdf[-1]
    ranks = np.searchsorted(cdf, rng.random(n), side="left").astype(np.int64)
    perm = np.random.default_rng(domain * 7919 + 13).permutation(domain)
    return perm[np.minimum(ranks, domain - 1)]


def deg_filter(deg_rows: Optional[np.ndarray], B: int) -> np.ndarray:
    if deg_rows is None or deg_rows.size == 0:
        return np.empty((0, 2), np.int64)
    C, nd = deg_rows.shape
    cs = int(math.ceil(float(B) / C))
    c_idx, col = np.nonzero((deg_rows // cs) == np.arange(C)[:, None])
    return np.stack([deg_rows[c_idx, col], col], axis=1).astype(np.int64)


def make_case(kind, B, C, N, D, R, U, n_deg, seed, relations=True, inverse=True, alpha=1.0, emb_scale=0.3) -> BatchCase:
    rng = np.random.default_rng(seed)
    src = zipf_ids(rng, B, U, alpha)
    dst = zipf_ids(rng, B, U, alpha)
    cols = [src]
    rel = inv_rel = None
    if relations:
        cols.append(zipf_ids(rng, B, R, 1.2))
        rel = (1.0 + 0.25 * rng.standard_normal((R, D))).astype(np.float32)
        if inverse:
            inv_rel = (1.0 + 0.25 * rng.standard_normal((R, D))).astype(np.float32)
    cols.append(dst)
    edges = np.stack(cols, axis=1).astype(np.int64)
    emb = (emb_scale * rng.standard_normal((U, D))).astype(np.float32)
    state = (0.05 * rng.random((U, D))).astype(np.float32)
    uni = rng.integers(0, U, (C, N - n_deg)).astype(np.int64)
    deg_rows = rng.integers(0, B, (C, n_deg)).astype(np.int64) if n_deg > 0 else None
    parts_d, parts_s = [], []
    if deg_rows is not None:
        parts_d.append(edges[:, -1][deg_rows])
        parts_s.append(edges[:, 0][deg_rows])
    parts_d.append(uni)
    parts_s.append(uni)
    dst_negs = np.concatenate(parts_d, axis=1)
    src_negs = np.concatenate(parts_s, axis=1) if (relations and inverse) else None
    return BatchCase(kind, edges, emb, state, rel, inv_rel, dst_negs, src_negs, deg_rows, deg_filter(deg_rows, B))


GOLDEN_CASES = {
    # name: (kind, B, C, N, D, R, U, n_deg, seed, relations, inverse)
    "distmult_d50_uniform": ("DISTMULT", 300, 3, 40, 50, 11, 157, 0, 101, True, True),
    "complex_d100_deg_padded": ("COMPLEX", 250, 4, 48, 100, 7, 180, 24, 102, True, True),
    "dot_d100_deg": ("DISTMULT", 200, 2, 64, 100, 0, 190, 32, 103, False, False),
    "distmult_d128_onechunk": ("DISTMULT", 128, 1, 100, 128, 5, 140, 10, 104, True, True),
    "complex_d50_noinverse": ("COMPLEX", 96, 3, 33, 50, 4, 90, 11, 105, True, False),
}


def golden_case(name) -> BatchCase:
    return make_case(*GOLDEN_CASES[name])
