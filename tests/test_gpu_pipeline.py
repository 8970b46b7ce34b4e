"""Whole training steps on the GPU (sampler -> unique-map -> fused decoder -> Adagrad scatter) against the oracle's
restatement of the reference trainer loop, fed with the negatives the device sampler drew."""
import numpy as np
import pytest
import torch

import ge2_oracle as O
import workloads

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("decoder,D,R,deg", [("DISTMULT", 50, 40, 0.0), ("COMPLEX", 100, 25, 0.5), ("DISTMULT", 100, 1, 0.5)])
def test_three_steps_match_oracle(ge2, cuda_device, decoder, D, R, deg):
    from importlib import import_module

    pipeline = import_module("ge-2_b200.pipeline")
    rng = np.random.default_rng(11)
    nodes, B, C, N = 5000, 600, 3, 200
    table = (0.3 * rng.standard_normal((nodes, D))).astype(np.float32)
    # non-zero starting state: with state = 0 the first Adagrad step is -lr * sign(g), which turns rounding noise in a
    # near-zero gradient into a 0.2-wide difference and says nothing about parity
    state = (0.01 + 0.05 * rng.random((nodes, D))).astype(np.float32)
    has_rel = R > 1
    rel = (1 + 0.2 * rng.standard_normal((R, D))).astype(np.float32) if has_rel else None
    inv_rel = (1 + 0.2 * rng.standard_normal((R, D))).astype(np.float32) if has_rel else None
    cfg = pipeline.PipelineConfig(decoder=decoder, B=B, C=C, N=N, degree_fraction=deg, D=D, R=R, domain=nodes, lr=0.1, precision="fp32")
    t = lambda a: None if a is None else torch.from_numpy(a.copy()).to(cuda_device)
    d_table, d_state, d_rel, d_inv = t(table), t(state), t(rel), t(inv_rel)
    d_rel_state = torch.zeros_like(d_rel) if has_rel else None
    d_inv_state = torch.zeros_like(d_inv) if has_rel else None
    pipe = pipeline.BatchPipeline(cfg, d_table, d_state, d_rel, d_rel_state, d_inv, d_inv_state)
    rel_state = np.zeros_like(rel) if has_rel else None
    inv_state = np.zeros_like(inv_rel) if has_rel else None
    for step in range(3):
        cols = [workloads.zipf_ids(rng, B, nodes, 1.0)] + ([workloads.zipf_ids(rng, B, R, 1.2)] if has_rel else []) + [workloads.zipf_ids(rng, B, nodes, 1.0)]
        edges = np.stack(cols, axis=1).astype(np.int64)
        pipe.step(torch.from_numpy(edges).to(cuda_device), step)
        torch.cuda.synchronize()
        # replay the device sampler's draws through the oracle
        packed = pipe.packed.cpu().numpy()
        CN = C * N
        S = cfg.sides
        src_negs = packed[2 * B:2 * B + CN].reshape(C, N) if S == 2 else None
        dst_negs = packed[2 * B + (S - 1) * CN:].reshape(C, N)
        filt = O.deg_negative_local_filter(pipe.deg_rows.cpu().numpy(), B) if cfg.n_deg > 0 else None
        loss, U = O.train_step(decoder, table, state, rel, rel_state, inv_rel, inv_state, edges, dst_negs, src_negs, filt, filt, 0.1, nodes)
        assert int(pipe.count[0]) == U and int(pipe.count[1]) == 0 and int(pipe.status) == 0
        assert abs(float(pipe.loss) - loss) <= 1e-4 * abs(loss)
        assert np.abs(d_table.cpu().numpy() - table).max() <= 1e-4 * np.abs(table).max()
        assert np.abs(d_state.cpu().numpy() - state).max() <= 1e-4 * max(np.abs(state).max(), 1e-12)
        if has_rel:
            assert np.abs(d_rel.cpu().numpy() - rel).max() <= 1e-4 * np.abs(rel).max()
            assert np.abs(d_inv.cpu().numpy() - inv_rel).max() <= 1e-4 * np.abs(inv_rel).max()


def test_graph_replay_equals_host_issued_steps(ge2, cuda_device):
    """The resident form reads its batch index from device memory; a captured CUDA graph replayed three times must leave
    the tables where three host-issued steps leave them (up to the order of the gradient atomics)."""
    from importlib import import_module

    pipeline = import_module("ge-2_b200.pipeline")
    rng = np.random.default_rng(21)
    nodes, B, C, N, D, R, nb = 6000, 512, 2, 256, 100, 17, 5
    table = (0.3 * rng.standard_normal((nodes, D))).astype(np.float32)
    state = (0.01 + 0.05 * rng.random((nodes, D))).astype(np.float32)
    rel = (1 + 0.2 * rng.standard_normal((R, D))).astype(np.float32)
    edges = np.stack([workloads.zipf_ids(rng, nb * B, nodes, 1.0), workloads.zipf_ids(rng, nb * B, R, 1.2),
                      workloads.zipf_ids(rng, nb * B, nodes, 1.0)], axis=1).astype(np.int64)
    d_edges = torch.from_numpy(edges).to(cuda_device)
    results = []
    for mode in ("host", "graph", "pipelined"):
        cfg = pipeline.PipelineConfig("COMPLEX", B, C, N, 0.5, D, R, nodes, lr=0.1, precision="fp32")
        t = lambda a: torch.from_numpy(a.copy()).to(cuda_device)
        d_table, d_state, d_rel, d_inv = t(table), t(state), t(rel), t(rel)
        pipe = pipeline.BatchPipeline(cfg, d_table, d_state, d_rel, torch.zeros_like(d_rel), d_inv, torch.zeros_like(d_inv))
        if mode == "host":
            for _ in range(3):
                pipe.enqueue_resident(d_edges, nb)
        else:
            # one host-issued step, then the capture; the pipelined form draws batch t+1 on a side stream during step t
            g = pipe.capture_resident(d_edges, nb) if mode == "graph" else pipe.capture_pipelined(d_edges, nb)
            g.replay()
            g.replay()
        pipe.check_status()
        assert pipe.step_dev.tolist() == [3, 4]
        results.append((d_table.cpu().numpy(), d_state.cpu().numpy(), d_rel.cpu().numpy(), float(g.loss if mode == "pipelined" else pipe.loss)))
    for other in results[1:]:
        for a, b in zip(results[0][:3], other[:3]):
            assert np.abs(a - b).max() <= 1e-5 * np.abs(a).max()
        assert abs(results[0][3] - other[3]) <= 1e-5 * abs(results[0][3])
    assert np.abs(results[0][0] - table).max() > 0  # and the steps did train


@pytest.mark.gpu
def test_host_feed_trains_the_same_batches_as_the_resident_form(cuda_device):
    """Batches fed from pinned host memory through the pipelined graphs (copies on side streams) give the tables and the
    per-step losses of the resident form stepping over the same batches in the same order."""
    from importlib import import_module

    pipeline = import_module("ge-2_b200.pipeline")
    rng = np.random.default_rng(33)
    nodes, B, C, N, D, R, nb = 5000, 384, 2, 128, 64, 11, 6
    table = (0.3 * rng.standard_normal((nodes, D))).astype(np.float32)
    state = (0.01 + 0.05 * rng.random((nodes, D))).astype(np.float32)
    rel = (1 + 0.2 * rng.standard_normal((R, D))).astype(np.float32)
    edges = np.stack([workloads.zipf_ids(rng, nb * B, nodes, 1.0), workloads.zipf_ids(rng, nb * B, R, 1.2),
                      workloads.zipf_ids(rng, nb * B, nodes, 1.0)], axis=1).astype(np.int64)
    host = torch.from_numpy(edges).reshape(nb, B, 3).pin_memory()
    d_edges = torch.from_numpy(edges).to(cuda_device)
    out = []
    for mode in ("resident", "host_feed"):
        cfg = pipeline.PipelineConfig("DISTMULT", B, C, N, 0.5, D, R, nodes, lr=0.1, precision="fp32")
        t = lambda a: torch.from_numpy(a.copy()).to(cuda_device)
        d_table, d_state, d_rel, d_inv = t(table), t(state), t(rel), t(rel)
        pipe = pipeline.BatchPipeline(cfg, d_table, d_state, d_rel, torch.zeros_like(d_rel), d_inv, torch.zeros_like(d_inv))
        losses = torch.zeros(nb, dtype=torch.float32).pin_memory()
        if mode == "resident":
            for i in range(nb - 1):
                pipe.enqueue_resident(d_edges, nb)
                losses[i:i + 1].copy_(pipe.loss)
        else:
            feed = pipeline.HostFeed(pipe, 3)
            feed.start(host[0], host[1])  # trains batch 0
            losses[0:1].copy_(pipe.loss)
            for i in range(1, nb - 1):
                feed.step(host[i + 1], losses[i:i + 1])  # trains batch i, draws batch i+1
            feed.drain()
        pipe.check_status()
        out.append((d_table.cpu().numpy(), d_state.cpu().numpy(), d_rel.cpu().numpy(), losses.numpy().copy()))
    for a, b in zip(out[0], out[1]):
        assert np.abs(a - b).max() <= 1e-5 * np.abs(a).max()
    assert (out[0][3][: nb - 1] > 0).all()
