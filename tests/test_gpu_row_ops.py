"""GPU parity of the row-wise kernels (gather, scatter-add, sparse/dense Adagrad, slot remap, slab copies, sampler)."""
import numpy as np
import pytest
import torch

import ge2_oracle as O

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("D", [50, 100, 128, 7])
def test_sparse_adagrad_bit_exact(capi, cuda_device, D):
    rng = np.random.default_rng(D)
    U = 1237
    g = (rng.standard_normal((U, D)) * 0.1).astype(np.float32)
    g[::7] = 0.0
    st = (rng.random((U, D)) * 0.1).astype(np.float32)
    st[::7] = 0.0  # g = 0, state = 0: 0 / (0 + 1e-10)
    tg, ts = torch.from_numpy(g).to(cuda_device), torch.from_numpy(st.copy()).to(cuda_device)
    delta, upd = capi.sparse_adagrad(tg, ts, 0.1)
    torch.cuda.synchronize()
    od, ou = O.sparse_adagrad(g, st, 0.1)
    assert np.array_equal(delta.cpu().numpy(), od) and np.array_equal(upd.cpu().numpy(), ou)
    assert np.array_equal(ts.cpu().numpy(), st + ou)  # state updated in place, as node_embeddings_state_.add_ does


@pytest.mark.parametrize("D", [50, 100, 128])
def test_index_read_add_and_fused_scatter(capi, cuda_device, D):
    rng = np.random.default_rng(100 + D)
    rows, U = 5000, 1500
    table = rng.standard_normal((rows, D)).astype(np.float32)
    state = rng.random((rows, D)).astype(np.float32)
    ids = np.sort(rng.permutation(rows)[:U]).astype(np.int64)
    g = (rng.standard_normal((U + 100, D)) * 0.05).astype(np.float32)  # rows past the live count must be ignored
    t_table, t_state = torch.from_numpy(table.copy()).to(cuda_device), torch.from_numpy(state.copy()).to(cuda_device)
    t_ids = torch.from_numpy(np.concatenate([ids, np.zeros(100, np.int64)])).to(cuda_device)
    t_g = torch.from_numpy(g.copy()).to(cuda_device)
    count = torch.tensor([U, 0], dtype=torch.int32, device=cuda_device)
    got = capi.index_read(t_table, t_ids, n_dev=count)
    torch.cuda.synchronize()
    assert np.array_equal(got.cpu().numpy()[:U], table[ids])
    # reference sequence: gather state, accumulateGradients, indexAdd(delta), indexAdd(state update)
    delta, upd = O.sparse_adagrad(g[:U], state[ids], 0.1)
    exp_table, exp_state = table.copy(), state.copy()
    O.index_add(exp_table, ids, delta)
    O.index_add(exp_state, ids, upd)
    capi.adagrad_scatter(t_table, t_state, t_ids, t_g, 0.1, U=U + 100, U_dev=count, clear_grad=True)
    torch.cuda.synchronize()
    assert np.array_equal(t_table.cpu().numpy(), exp_table) and np.array_equal(t_state.cpu().numpy(), exp_state)
    assert float(t_g[:U].abs().max()) == 0.0 and np.array_equal(t_g[U:].cpu().numpy(), g[U:])
    # index_add on its own
    t2 = torch.from_numpy(table.copy()).to(cuda_device)
    capi.index_add(t2, t_ids[:U], torch.from_numpy(delta).to(cuda_device))
    torch.cuda.synchronize()
    assert np.array_equal(t2.cpu().numpy(), exp_table)


def test_index_out_of_bounds_sets_status(capi, cuda_device):
    table = torch.zeros((10, 8), device=cuda_device)
    ids = torch.tensor([1, 11, -1], dtype=torch.int64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    out = capi.index_read(table, ids, status=status)
    torch.cuda.synchronize()
    assert int(status) & 8


def test_dense_adagrad(capi, cuda_device):
    rng = np.random.default_rng(0)
    p = rng.standard_normal((1000, 100)).astype(np.float32)
    s = rng.random((1000, 100)).astype(np.float32)
    g = (rng.standard_normal((1000, 100)) * 0.01).astype(np.float32)
    tp, ts, tg = (torch.from_numpy(x.copy()).to(cuda_device) for x in (p, s, g))
    capi.dense_adagrad(tp, ts, tg, 0.1, clear_grad=True)
    torch.cuda.synchronize()
    O.dense_adagrad(p, g, s, 0.1)
    assert np.array_equal(tp.cpu().numpy(), p) and np.array_equal(ts.cpu().numpy(), s) and float(tg.abs().max()) == 0.0
    # pre-divided gradients of the multi-GPU all-reduce
    tp2, ts2, tg2 = (torch.from_numpy(x.copy()).to(cuda_device) for x in (p, s, g))
    capi.dense_adagrad(tp2, ts2, tg2, 0.1, grad_scale=0.25)
    torch.cuda.synchronize()
    p2, s2 = p.copy(), s.copy()
    O.dense_adagrad(p2, g * np.float32(0.25), s2, 0.1)
    assert np.array_equal(tp2.cpu().numpy(), p2) and np.array_equal(ts2.cpu().numpy(), s2)


def test_remap_edges_to_slots(capi, cuda_device):
    rng = np.random.default_rng(2)
    P, psize = 16, 1000
    resident = [3, 9, 0, 12]
    slot = np.full(P, -1, np.int64)
    slot[resident] = np.arange(4)
    for cols in (2, 3):
        parts = rng.choice(resident, (5000, 2))
        e = parts * psize + rng.integers(0, psize, (5000, 2))
        edges = np.stack([e[:, 0]] + ([rng.integers(0, 50, 5000)] if cols == 3 else []) + [e[:, 1]], axis=1).astype(np.int64)
        status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
        out = capi.remap_edges_to_slots(torch.from_numpy(edges).to(cuda_device), torch.from_numpy(slot).to(cuda_device), psize, status=status)
        torch.cuda.synchronize()
        assert int(status) == 0 and np.array_equal(out.cpu().numpy(), O.map_edges_with_partition_slots(edges, slot, psize))
    bad = np.array([[5 * psize + 1, 3 * psize]], np.int64)  # partition 5 is not resident: the reference throws
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    capi.remap_edges_to_slots(torch.from_numpy(bad).to(cuda_device), torch.from_numpy(slot).to(cuda_device), psize, status=status)
    torch.cuda.synchronize()
    assert int(status) & 8


def test_copy_slabs_matches_relay_plan(capi, cuda_device):
    rows, D = 300, 100
    src = torch.arange(4 * rows * D, dtype=torch.float32, device=cuda_device).reshape(4 * rows, D)
    dst = torch.zeros_like(src)
    capi.copy_slabs(src, dst, [(0, 2), (3, 0), (1, 1)], rows * D)
    torch.cuda.synchronize()
    s, d = src.cpu().numpy(), dst.cpu().numpy()
    assert np.array_equal(d[2 * rows:3 * rows], s[0:rows]) and np.array_equal(d[0:rows], s[3 * rows:]) and np.array_equal(d[rows:2 * rows], s[rows:2 * rows])
    assert float(np.abs(d[3 * rows:]).max()) == 0.0


@pytest.mark.parametrize("want_src", [True, False])
def test_sample_negatives_structure(capi, cuda_device, want_src):
    rng = np.random.default_rng(6)
    B, C, N, n_deg, domain = 1000, 10, 100, 50, 50_000
    edges = np.stack([rng.integers(0, domain, B), rng.integers(0, 30, B), rng.integers(0, domain, B)], axis=1).astype(np.int64)
    te = torch.from_numpy(edges).to(cuda_device)
    S = 2 if want_src else 1
    packed = torch.full((2 * B + S * C * N,), -1, dtype=torch.int64, device=cuda_device)
    deg_rows = torch.full((C, n_deg), -1, dtype=torch.int64, device=cuda_device)
    capi.sample_negatives(te, te[:, 2], 3, B, C, N, n_deg, domain, want_src, 7, 3, packed, deg_rows)
    packed2 = torch.empty_like(packed)
    capi.sample_negatives(te, te[:, 2], 3, B, C, N, n_deg, domain, want_src, 7, 4, packed2, deg_rows.clone())
    torch.cuda.synchronize()
    p, rows = packed.cpu().numpy(), deg_rows.cpu().numpy()
    assert np.array_equal(p[:B], edges[:, 0]) and np.array_equal(p[B:2 * B], edges[:, 2])
    dst_negs = p[2 * B + (S - 1) * C * N:].reshape(C, N)
    assert rows.min() >= 0 and rows.max() < B
    # materialize_negative_output of the reference: degree negatives are the dst (src) ids of the sampled rows, then uniform ids
    assert np.array_equal(dst_negs, O.materialize_negatives(edges, dst_negs[:, n_deg:], rows, False))
    assert dst_negs.min() >= 0 and dst_negs.max() < domain
    if want_src:
        src_negs = p[2 * B:2 * B + C * N].reshape(C, N)
        assert np.array_equal(src_negs, O.materialize_negatives(edges, dst_negs[:, n_deg:], rows, True))  # shared picks
    uni = dst_negs[:, n_deg:].reshape(-1)
    assert abs(uni.mean() / domain - 0.5) < 0.05 and np.unique(uni).size > 0.9 * uni.size * (1 - uni.size / domain)
    assert not np.array_equal(p, packed2.cpu().numpy())  # another batch index, other draws


def _peer_buffers(world, numel, device, rng):
    """`world` gradient buffers on ONE device laid out as ge2_dense_adagrad_peers expects (two halves, `world` 8-byte arrival
    flags, one 8-byte verdict word, one 8-byte wait-time counter); half 0 holds random gradients, half 1 a sentinel the step has to clear."""
    bufs, grads = [], []
    for _ in range(world):
        g = (0.1 * rng.standard_normal(numel)).astype(np.float32)
        b = torch.zeros(2 * numel + 2 * world + 4, dtype=torch.float32, device=device)
        b[:numel] = torch.from_numpy(g).to(device)
        b[numel:2 * numel] = 7.0
        bufs.append(b)
        grads.append(g)
    return bufs, grads


def _set_arrival(buf, numel, world, slot, epoch):
    """what a peer's announcement writes: `epoch` into arrival flag `slot` of this rank's buffer"""
    flags = buf[2 * numel:2 * numel + 2 * world].view(torch.int64)
    flags[slot] = epoch


@pytest.mark.parametrize("world", [2, 4])
def test_peer_reduced_dense_adagrad_matches_oracle(capi, cuda_device, world):
    """Model::all_reduce + the dense step against the oracle (gradients divided by the device count, summed in device
    order, then Adagrad), with the ranks' buffers emulated on one GPU: the peers' announcements are written by the host, so
    no kernel waits for another launch."""
    rng = np.random.default_rng(world)
    numel = 2 * 37 * 100
    bufs, grads = _peer_buffers(world, numel, cuda_device, rng)
    p = rng.standard_normal(numel).astype(np.float32)
    s = rng.random(numel).astype(np.float32)
    t_p, t_s = torch.from_numpy(p.copy()).to(cuda_device), torch.from_numpy(s.copy()).to(cuda_device)
    step = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    for peer in range(1, world):
        _set_arrival(bufs[0], numel, world, peer, 1)
    capi.dense_adagrad_peers(t_p, t_s, [b.data_ptr() for b in bufs], 0, numel, step, 0.1, status, grad_scale=1.0 / world, wait_budget_us=2000)
    torch.cuda.synchronize()
    assert int(status) == 0
    g = O.allreduce_relation_grads(grads)
    ep, es = O.dense_adagrad(p.copy(), g, s.copy(), 0.1)
    assert np.array_equal(t_p.cpu().numpy(), ep) and np.array_equal(t_s.cpu().numpy(), es)
    assert float(bufs[0][numel:2 * numel].abs().max()) == 0.0           # the other half is cleared for the step after next
    assert np.array_equal(bufs[0][:numel].cpu().numpy(), grads[0])      # this step's half is left for the peers to read
    flags = bufs[0][2 * numel:].view(torch.int64).cpu().tolist()
    assert flags[0] == 1 and flags[world] == 1                          # own announcement, and the verdict of step 0


def test_peer_wait_runs_out_and_leaves_everything_untouched(capi, cuda_device):
    """A peer that never announces: the bounded wait (5 ms here) ends, GE2_STATUS_PEER_TIMEOUT is set, and neither the
    tables nor the gradient buffer change by a single bit -- every block acts on the one verdict of the launch."""
    rng = np.random.default_rng(9)
    world, numel = 2, 2 * 1000 * 100
    bufs, _ = _peer_buffers(world, numel, cuda_device, rng)
    p = rng.standard_normal(numel).astype(np.float32)
    s = rng.random(numel).astype(np.float32)
    t_p, t_s = torch.from_numpy(p.copy()).to(cuda_device), torch.from_numpy(s.copy()).to(cuda_device)
    before = bufs[0][:2 * numel].clone()
    step = torch.zeros(2, dtype=torch.int64, device=cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    capi.dense_adagrad_peers(t_p, t_s, [b.data_ptr() for b in bufs], 0, numel, step, 0.1, status, grad_scale=0.5, wait_budget_us=5000)
    torch.cuda.synchronize()
    assert int(status) & 32
    assert np.array_equal(t_p.cpu().numpy(), p) and np.array_equal(t_s.cpu().numpy(), s)
    assert torch.equal(bufs[0][:2 * numel], before)
    words = bufs[0][2 * numel:].view(torch.int64).cpu().tolist()
    assert words[world] == 0              # verdict: no go
    assert words[world + 1] >= 5_000_000  # the wait-time counter saw the whole budget go by
    # the context is still usable and a later, complete step goes through
    status.zero_()
    _set_arrival(bufs[0], numel, world, 1, 1)
    capi.dense_adagrad_peers(t_p, t_s, [b.data_ptr() for b in bufs], 0, numel, step, 0.1, status, grad_scale=0.5, wait_budget_us=5000)
    torch.cuda.synchronize()
    assert int(status) == 0 and not np.array_equal(t_p.cpu().numpy(), p)
