"""The numpy restatement (oracle/ge2_oracle.py) against fixtures produced by the reference's own CPU code."""
from pathlib import Path

import numpy as np
import pytest

import ge2_oracle as O
import workloads

GOLDEN = Path(__file__).resolve().parent / "golden"


def rel_err(a, b):
    return float(np.abs(a.astype(np.float64) - b.astype(np.float64)).max() / (np.abs(b).max() + 1e-30))


@pytest.mark.parametrize("name", sorted(workloads.GOLDEN_CASES))
def test_fixture_inputs_regenerate(name):
    """The seeded generator reproduces the inputs stored in the fixture (so GPU tests can rebuild them)."""
    g = np.load(GOLDEN / f"{name}.npz")
    c = workloads.golden_case(name)
    assert np.array_equal(g["edges"], c.edges) and np.array_equal(g["emb"], c.emb) and np.array_equal(g["dst_negs"], c.dst_negs)
    assert np.array_equal(g["filt"], c.filt)


@pytest.mark.parametrize("name", sorted(workloads.GOLDEN_CASES))
def test_decoder_loss_backward_matches_reference(name):
    g = np.load(GOLDEN / f"{name}.npz")
    kind = str(g["kind"])
    rel = g["rel"] if "rel" in g else None
    inv_rel = g["inv_rel"] if "inv_rel" in g else None
    src_negs = g["src_negs"] if "src_negs" in g else None
    filt = g["filt"]
    r = O.lp_train_forward_backward(kind, g["edges"], g["emb"], rel, inv_rel, g["dst_negs"], src_negs, filt, filt if src_negs is not None else None)
    assert abs(r.loss - float(g["ref_loss"])) <= 2e-6 * abs(float(g["ref_loss"]))
    # masked entries are exactly -1e9 on both sides; compare the rest relatively
    assert np.array_equal(r.neg_scores == O.MASK_VALUE, g["ref_neg_scores"] == O.MASK_VALUE)
    keep = g["ref_neg_scores"] != O.MASK_VALUE
    assert rel_err(r.neg_scores[keep], g["ref_neg_scores"][keep]) < 1e-5
    assert rel_err(r.pos_scores, g["ref_pos_scores"]) < 1e-5
    assert rel_err(r.node_grad, g["ref_node_grad"]) < 1e-5
    if rel is not None:
        assert rel_err(r.rel_grad, g["ref_rel_grad"]) < 1e-5
    if inv_rel is not None:
        assert rel_err(r.inv_rel_grad, g["ref_inv_rel_grad"]) < 1e-5
        assert rel_err(r.inv_neg_scores[keep], g["ref_inv_neg_scores"][keep]) < 1e-5


@pytest.mark.parametrize("name", sorted(workloads.GOLDEN_CASES))
def test_sparse_adagrad_matches_reference(name):
    """accumulateGradients: the state update is bit-exact; the step differs from the reference's CPU build by at most
    a few ulp because that build's vectorised sqrt is not correctly rounded (the oracle and the CUDA kernels are)."""
    g = np.load(GOLDEN / f"{name}.npz")
    delta, upd = O.sparse_adagrad(g["ref_node_grad"], g["state"], float(g["lr"]))
    assert np.array_equal(upd, g["ref_node_state_update"])
    assert np.allclose(delta, g["ref_node_update"], rtol=1e-6, atol=1e-12)


@pytest.mark.parametrize("name", [n for n in sorted(workloads.GOLDEN_CASES) if workloads.GOLDEN_CASES[n][9]])
def test_dense_adagrad_matches_reference(name):
    g = np.load(GOLDEN / f"{name}.npz")
    p, s = g["rel"].copy(), np.zeros_like(g["rel"])
    O.dense_adagrad(p, g["ref_rel_grad"], s, float(g["lr"]))
    assert np.array_equal(s, g["ref_rel_state_after"])
    assert np.allclose(p, g["ref_rel_after"], rtol=1e-6, atol=1e-7)


def test_deg_filter_restatement():
    rng = np.random.default_rng(5)
    for B, C, nd in [(1000, 10, 50), (250, 4, 24), (7, 3, 5)]:
        rows = rng.integers(0, B, (C, nd))
        assert np.array_equal(O.deg_negative_local_filter(rows, B), workloads.deg_filter(rows, B))
    assert O.deg_negative_local_filter(np.empty((3, 0), np.int64), 10).shape == (0, 2)


def test_unique_bitmap_equals_sort_unique():
    """Contract of the reference's replay harness (gege_unique_replay_bench.cpp:142-172): same count, unique[inverse] == input,
    and the bitmap result equals the sort-based one."""
    rng = np.random.default_rng(9)
    for n, domain in [(1, 1), (10, 64), (1000, 65), (22000, 14951), (5000, 1 << 20), (300, 128)]:
        ids = rng.integers(0, domain, n)
        u, inv, invalid = O.unique_map_bitmap(ids, domain)
        su, sinv = O.unique_map_sort(ids)
        assert not invalid and np.array_equal(u, su) and np.array_equal(inv, sinv)
        assert np.array_equal(u[inv], ids) and np.all(np.diff(u) > 0)
    u, inv, invalid = O.unique_map_bitmap(np.array([3, 70, -1]), 64)
    assert invalid
    u, inv, invalid = O.unique_map_bitmap(np.empty(0, np.int64), 64)
    assert u.size == 0 and inv.size == 0 and not invalid


def test_map_tensors_split_order():
    a, b, c = np.array([5, 3, 5]), np.array([9]), np.array([3, 3, 0, 9])
    u, mapped = O.map_tensors([a, b, c], 16)
    assert u.tolist() == [0, 3, 5, 9]
    assert [m.tolist() for m in mapped] == [[2, 1, 2], [3], [1, 1, 0, 3]]


def test_partition_remap_and_relay_plan():
    slot = np.array([2, -1, 0, 1])  # partitions 0, 2, 3 resident in slots 2, 0, 1; partition size 4
    with pytest.raises(RuntimeError):  # id 4 lives in partition 1, which is not resident
        O.map_edges_with_partition_slots(np.array([[4, 0, 1]]), slot, 4)
    ok = O.map_edges_with_partition_slots(np.array([[0, 7, 13], [12, 2, 3]]), slot, 4)
    assert ok.tolist() == [[8, 7, 5], [4, 2, 11]]
    plan = O.relay_swap_plan([[0, 1], [2, 3]], [[2, 0], [1, 3]])
    assert plan == [[(0, 2, 1, 0), (1, 0, 0, 0)], [(0, 1, 0, 1), (1, 3, 1, 1)]]
    with pytest.raises(RuntimeError):
        O.relay_swap_plan([[0, 1], [2, 3]], [[4, 0], [1, 3]])
    bufs = [np.arange(8, dtype=np.float32).reshape(4, 2), 100 + np.arange(8, dtype=np.float32).reshape(4, 2)]
    new = O.relay_swap_apply(bufs, [[0, 1], [2, 3]], [[2, 0], [1, 3]], 2)
    assert new[0].tolist() == [[100, 101], [102, 103], [0, 1], [2, 3]]
    assert new[1].tolist() == [[4, 5], [6, 7], [104, 105], [106, 107]]


def test_ranks_and_mrr():
    pos = np.array([1.0, 0.0], np.float32)
    neg = np.array([[0.5, 1.0, 2.0], [-1.0, -2.0, -3.0]], np.float32)
    r = O.ranks_from_scores(pos, neg)
    assert r.tolist() == [3, 1]
    assert abs(O.mrr(r) - (1 / 3 + 1) / 2) < 1e-6


def test_tournament_selection_restatement():
    """Tournament selection of negatives (distmult_selected_neg_cuda.cpp:46-121) against the same steps in torch on CPU:
    batched products, a view into groups of consecutive negatives, the maximum of each group and its column."""
    import torch

    rng = np.random.default_rng(5)
    C, R, N, D, sel = 2, 17, 48, 16, 6
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    k = rng.standard_normal((C, N, D)).astype(np.float32)
    scores, idx = O.tournament_selected_scores(q, k, sel)
    T = N // sel
    view = torch.from_numpy(q).bmm(torch.from_numpy(k).transpose(1, 2)).view(C, R, sel, T)
    best, local = view.max(3)
    assert np.allclose(scores, best.reshape(C * R, sel).numpy(), atol=1e-5)
    assert np.array_equal(idx, (local + torch.arange(sel) * T).reshape(C, R * sel).numpy())
    with pytest.raises(ValueError):
        O.tournament_selected_scores(q, k, 5)


@pytest.mark.parametrize("kind", [O.SELECTED_DOT, O.SELECTED_L2])
def test_selected_neg_scores_restatement_against_autograd(kind):
    """Scores of chosen pairs and their gradients (distmult_selected_neg_cuda.cu:15-202) against torch autograd in float64
    on the same gather: dot product, or sqrt(max(|q - n|^2, 1e-8)) whose floor passes no gradient."""
    import torch

    rng = np.random.default_rng(kind)
    C, R, N, D, K = 2, 7, 11, 10, 3
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    n = rng.standard_normal((C, N, D)).astype(np.float32)
    sel = rng.integers(0, N, (C, R * K))
    sel[0, :2] = 4               # a negative chosen twice by one row
    n[1, 5], sel[1, 2 * K] = q[1, 2], 5   # a pair at distance 0
    tq = torch.tensor(q, dtype=torch.float64, requires_grad=True)
    tn = torch.tensor(n, dtype=torch.float64, requires_grad=True)
    picked = tn[torch.arange(C)[:, None, None], torch.tensor(sel).view(C, R, K)]
    if kind == O.SELECTED_DOT:
        out = (tq[:, :, None, :] * picked).sum(-1)
    else:
        out = torch.sqrt(torch.clamp(((tq[:, :, None, :] - picked) ** 2).sum(-1), min=1e-8))
    grad = rng.standard_normal((C * R, K)).astype(np.float32)
    out.backward(torch.tensor(grad, dtype=torch.float64).view(C, R, K))
    assert np.abs(O.selected_neg_scores(q, n, sel, kind) - out.detach().numpy().reshape(C * R, K)).max() < 1e-5
    dq, dn = O.selected_neg_scores_backward(grad, q, n, sel, kind)
    assert np.abs(dq - tq.grad.numpy()).max() < 1e-5 and np.abs(dn - tn.grad.numpy()).max() < 1e-5
