"""End-to-end quality check: a few epochs of training on a synthetic knowledge graph with the shape of configuration 1
(14,951 entities, 1,345 relations, DistMult d=50, batch 1,000, 10 x 1,000 uniform negatives, Adagrad 0.1), once through the
GPU pipeline and once through the oracle's restatement of the reference trainer fed with the same negatives; the link-
prediction MRR of the two embedding tables must agree within 0.005 (the north-star bound) for both precision modes."""
from importlib import import_module

import numpy as np
import pytest
import torch

import ge2_oracle as O
import workloads

pytestmark = pytest.mark.gpu


def mrr_of(table, rel, test):
    """unfiltered destination-corruption MRR over all nodes (ranks as in reporting.cpp:52-54 of the reference)"""
    q = table[test[:, 0]] * rel[test[:, 1]]
    scores = q @ table.T
    pos = scores[np.arange(len(test)), test[:, 2]]
    ranks = (scores >= pos[:, None]).sum(1)  # includes the positive itself: rank >= 1
    return float((1.0 / ranks.astype(np.float32)).mean())


@pytest.mark.parametrize("precision", ["fp32", "f16"])
def test_mrr_delta_after_training(ge2, cuda_device, precision):
    pipeline = import_module("ge-2_b200.pipeline")
    rng = np.random.default_rng(2026)
    nodes, R, D, B, C, N, epochs, n_train = 14951, 1345, 50, 1000, 10, 1000, 2, 40_000
    # a learnable graph: the destination is a fixed function of (source, relation) most of the time
    src = workloads.zipf_ids(rng, n_train + 2000, nodes, 1.0)
    rels = workloads.zipf_ids(rng, n_train + 2000, R, 1.2)
    dst = np.where(rng.random(n_train + 2000) < 0.8, (src * 31 + rels * 17 + 5) % nodes, workloads.zipf_ids(rng, n_train + 2000, nodes, 1.0))
    edges = np.stack([src, rels, dst], 1).astype(np.int64)
    train, test = edges[:n_train], edges[n_train:]
    table0 = (rng.standard_normal((nodes, D)) * 0.1).astype(np.float32)
    # --- GPU ---
    cfg = pipeline.PipelineConfig("DISTMULT", B, C, N, 0.0, D, R, nodes, lr=0.1, precision=precision)
    t = lambda a: torch.from_numpy(a.copy()).to(cuda_device)
    d_table, d_state = t(table0), torch.zeros((nodes, D), device=cuda_device)
    d_rel, d_inv = torch.ones((R, D), device=cuda_device), torch.ones((R, D), device=cuda_device)
    pipe = pipeline.BatchPipeline(cfg, d_table, d_state, d_rel, torch.zeros_like(d_rel), d_inv, torch.zeros_like(d_inv))
    # --- oracle (reference trainer loop on CPU), fed with the negatives the device sampler drew ---
    table, state = table0.copy(), np.zeros((nodes, D), np.float32)
    rel, inv = np.ones((R, D), np.float32), np.ones((R, D), np.float32)
    rel_s, inv_s = np.zeros_like(rel), np.zeros_like(rel)
    nb = n_train // B
    step = 0
    for ep in range(epochs):
        perm = np.random.default_rng(ep).permutation(n_train)
        d_edges = torch.from_numpy(train[perm]).to(cuda_device)
        for b in range(nb):
            batch = d_edges[b * B:(b + 1) * B]
            pipe.step(batch, step)
            packed = pipe.packed.cpu().numpy()
            src_negs = packed[2 * B:2 * B + C * N].reshape(C, N)
            dst_negs = packed[2 * B + C * N:].reshape(C, N)
            O.train_step("DISTMULT", table, state, rel, rel_s, inv, inv_s, train[perm][b * B:(b + 1) * B], dst_negs, src_negs, None, None, 0.1, nodes)
            step += 1
    pipe.check_status()
    m_gpu = mrr_of(d_table.cpu().numpy(), d_rel.cpu().numpy(), test)
    m_ref = mrr_of(table, rel, test)
    m_init = mrr_of(table0, np.ones((R, D), np.float32), test)
    print(f"MRR[{precision}] gpu {m_gpu:.4f} oracle {m_ref:.4f} untrained {m_init:.4f}")
    assert m_ref > 2 * m_init  # training did something measurable
    assert abs(m_gpu - m_ref) <= 0.005


def test_filtered_mrr_delta_at_the_benchmarked_decoder(ge2, capi, cuda_device):
    """The decoder and sampler of the benchmark's configuration (ComplEx d=100, both corruption sides, half of the negatives
    drawn by degree with their local filter, fp16 tensor tiles) trained through the pipeline, against the oracle's restatement
    of the reference trainer fed with the same draws; both tables are then evaluated as the reference evaluates
    (filtered: every node is a candidate, true edges are masked; both sides; MRR over all ranks) by ge2_eval_ranks.
    Bound: 0.005."""
    pipeline = import_module("ge-2_b200.pipeline")
    rng = np.random.default_rng(77)
    nodes, R, D, B, C, N, epochs, n_train, n_test = 6000, 200, 100, 1000, 10, 1000, 2, 20_000, 1000
    n_all = n_train + n_test
    src = workloads.zipf_ids(rng, n_all, nodes, 1.0)
    rels = workloads.zipf_ids(rng, n_all, R, 1.2)
    dst = np.where(rng.random(n_all) < 0.8, (src * 31 + rels * 17 + 5) % nodes, workloads.zipf_ids(rng, n_all, nodes, 1.0))
    edges = np.stack([src, rels, dst], 1).astype(np.int64)
    train, test = edges[:n_train], edges[n_train:]
    table0 = (rng.standard_normal((nodes, D)) * 0.1).astype(np.float32)
    rel0 = np.zeros((R, D), np.float32)
    rel0[:, :D // 2] = 1  # complex.cpp:18-20 of the reference: (1, 0)
    cfg = pipeline.PipelineConfig("COMPLEX", B, C, N, 0.5, D, R, nodes, lr=0.1, precision="f16")
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    d_table, d_state = t(table0), torch.zeros((nodes, D), device=cuda_device)
    d_rel, d_inv = t(rel0), t(rel0)
    pipe = pipeline.BatchPipeline(cfg, d_table, d_state, d_rel, torch.zeros_like(d_rel), d_inv, torch.zeros_like(d_inv))
    table, state = table0.copy(), np.zeros((nodes, D), np.float32)
    rel, inv = rel0.copy(), rel0.copy()
    rel_s, inv_s = np.zeros_like(rel), np.zeros_like(rel)
    step = 0
    for ep in range(epochs):
        perm = np.random.default_rng(100 + ep).permutation(n_train)
        d_edges = t(train[perm])
        for b in range(n_train // B):
            pipe.step(d_edges[b * B:(b + 1) * B], step)
            packed = pipe.packed.cpu().numpy()
            src_negs = packed[2 * B:2 * B + C * N].reshape(C, N)
            dst_negs = packed[2 * B + C * N:].reshape(C, N)
            filt = O.deg_negative_local_filter(pipe.deg_rows.cpu().numpy(), B)
            O.train_step("COMPLEX", table, state, rel, rel_s, inv, inv_s, train[perm][b * B:(b + 1) * B], dst_negs, src_negs, filt, filt, 0.1, nodes)
            step += 1
    pipe.check_status()
    fd, fs = t(O.global_filter(edges, test, False)), t(O.global_filter(edges, test, True))

    def mrr_of(tab, r, ri):
        dr, sr = capi.eval_ranks("COMPLEX", tab, t(test), r, ri, dst_filter=fd, src_filter=fs)
        return O.mrr(torch.cat([dr, sr]).cpu().numpy())

    m_gpu = mrr_of(d_table, d_rel, d_inv)
    m_ref = mrr_of(t(table), t(rel), t(inv))
    m_init = mrr_of(t(table0), t(rel0), t(rel0))
    print(f"filtered MRR ComplEx d=100 f16: gpu {m_gpu:.4f} oracle {m_ref:.4f} untrained {m_init:.4f}")
    assert m_ref > 2 * m_init
    assert abs(m_gpu - m_ref) <= 0.005
