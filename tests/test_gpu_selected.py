"""The selected-negative operators (scores of chosen pairs forward and backward, tournament selection) against the oracle's
restatement of the reference's kernels for them (distmult_selected_neg_cuda.cu / .cpp).  fp32 sums in another order than the
oracle's float64: 1e-5 of the largest magnitude; selected columns must agree except on float ties."""
import numpy as np
import pytest
import torch

import ge2_oracle as O

pytestmark = pytest.mark.gpu
TOL = 1e-5

# (chunks, rows per chunk, negatives, D, selected per row)
PAIR_SHAPES = [(3, 50, 120, 32, 12), (2, 130, 1000, 100, 100), (1, 5, 7, 128, 1), (4, 9, 3, 1, 2), (2, 300, 64, 50, 7)]


def _pairs(rng, C, R, N, D, K):
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    n = rng.standard_normal((C, N, D)).astype(np.float32)
    sel = rng.integers(0, N, (C, R * K)).astype(np.int64)
    if K >= 2:
        sel[0, 1] = sel[0, 0]  # one negative chosen twice by a row: its gradient adds up
    n[C - 1, sel[C - 1, 0]] = q[C - 1, 0]  # a pair at distance 0: the L2 score is the floor and passes no gradient
    return q, n, sel


def _close(got, want):
    got = got.cpu().numpy()
    assert got.shape == want.shape
    assert np.abs(got - want).max() <= TOL * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("C,R,N,D,K", PAIR_SHAPES)
@pytest.mark.parametrize("kind,code", [("DOT", O.SELECTED_DOT), ("L2", O.SELECTED_L2)])
def test_selected_scores_forward_and_backward(capi, cuda_device, C, R, N, D, K, kind, code):
    rng = np.random.default_rng(C * 1000 + D)
    q, n, sel = _pairs(rng, C, R, N, D, K)
    grad = rng.standard_normal((C * R, K)).astype(np.float32)
    t = lambda a: torch.from_numpy(a).to(cuda_device)  # noqa: E731
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    _close(capi.selected_neg_scores(kind, t(q), t(n), t(sel), status), O.selected_neg_scores(q, n, sel, code))
    dq, dn = capi.selected_neg_scores_backward(kind, t(grad), t(q), t(n), t(sel), status)
    exp_dq, exp_dn = O.selected_neg_scores_backward(grad, q, n, sel, code)
    _close(dq, exp_dq)
    _close(dn, exp_dn)
    assert int(status.item()) == 0


def test_selected_column_out_of_range_is_reported_and_skipped(capi, cuda_device):
    rng = np.random.default_rng(3)
    C, R, N, D, K = 2, 20, 30, 40, 4
    q, n, sel = _pairs(rng, C, R, N, D, K)
    bad = sel.copy()
    bad[0, 5], bad[1, 7] = N, -1
    grad = rng.standard_normal((C * R, K)).astype(np.float32)
    t = lambda a: torch.from_numpy(a).to(cuda_device)  # noqa: E731
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    scores = capi.selected_neg_scores("DOT", t(q), t(n), t(bad), status).cpu().numpy()
    assert int(status.item()) == 8  # GE2_STATUS_BAD_INDEX
    exp = O.selected_neg_scores(q, n, sel, O.SELECTED_DOT)
    exp[5 // K, 5 % K] = 0.0
    exp[R + 7 // K, 7 % K] = 0.0
    assert np.abs(scores - exp).max() <= TOL * np.abs(exp).max()
    status.zero_()
    dq, dn = capi.selected_neg_scores_backward("DOT", t(grad), t(q), t(n), t(bad), status)
    assert int(status.item()) == 8
    masked = grad.copy()  # a zero upstream gradient on the valid stand-in columns gives the same sums
    masked[5 // K, 5 % K] = 0.0
    masked[R + 7 // K, 7 % K] = 0.0
    exp_dq, exp_dn = O.selected_neg_scores_backward(masked, q, n, sel, O.SELECTED_DOT)
    _close(dq, exp_dq)
    _close(dn, exp_dn)


def _check_tournament(scores, idx, q, n, K, score_q=None, score_n=None):
    C, R, _ = q.shape
    N = n.shape[1]
    T = N // K
    exp_scores, exp_idx = O.tournament_selected_scores(q, n, K)
    scores, idx = scores.cpu().numpy(), idx.cpu().numpy()
    assert scores.shape == (C * R, K) and idx.shape == (C, R * K)
    sel_all = np.einsum("crd,cnd->crn", q.astype(np.float64), n.astype(np.float64))
    got = np.take_along_axis(sel_all, idx.reshape(C, R, K), axis=2)
    want = np.take_along_axis(sel_all, exp_idx.reshape(C, R, K), axis=2)
    scale = max(1.0, np.abs(sel_all).max())
    assert np.abs(got - want).max() <= TOL * scale  # another winner only on a float tie
    assert (idx != exp_idx).mean() <= 0.01
    assert np.array_equal(idx.reshape(C, R, K) // T, np.broadcast_to(np.arange(K), (C, R, K)))  # one winner from every group
    if score_q is None:
        assert np.abs(scores - exp_scores).max() <= TOL * scale
    else:
        exp = O.selected_neg_scores(score_q, score_n, idx, O.SELECTED_DOT)  # the winners scored by the scorer's rows
        assert np.abs(scores - exp).max() <= TOL * max(1.0, np.abs(exp).max())


@pytest.mark.parametrize("C,R,N,D,K", [
    (3, 50, 120, 32, 12),     # groups of 10: six whole groups a tile
    (2, 130, 128, 100, 64),   # groups of 2
    (1, 64, 256, 16, 4),      # groups of exactly one tile
    (2, 70, 96, 100, 96),     # groups of 1: every negative is kept
    (2, 130, 1000, 100, 4),   # groups of 250: a running winner over four tiles, the last one ragged
    (3, 17, 130, 128, 2),     # groups of 65: one column into the second tile
    (1, 200, 1000, 50, 1),    # one group: the best negative of the chunk
    (5, 3, 33, 7, 11),        # fewer rows than a tile, groups of 3, odd D
    (2, 100, 1000, 100, 100), # the benchmarked step's chunk shape, a tenth kept
])
def test_tournament_selection_matches_oracle(capi, cuda_device, C, R, N, D, K):
    rng = np.random.default_rng(N + K)
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    n = rng.standard_normal((C, N, D)).astype(np.float32)
    scores, idx = capi.tournament_select(torch.from_numpy(q).to(cuda_device), torch.from_numpy(n).to(cuda_device), K)
    _check_tournament(scores, idx, q, n, K)


def test_tournament_with_a_separate_scorer(capi, cuda_device):
    rng = np.random.default_rng(9)
    C, R, N, D, K = 2, 90, 200, 64, 20
    q, n, sq, sn = (rng.standard_normal(s).astype(np.float32) for s in ((C, R, D), (C, N, D), (C, R, D), (C, N, D)))
    t = lambda a: torch.from_numpy(a).to(cuda_device)  # noqa: E731
    scores, idx = capi.tournament_select(t(q), t(n), K, score_chunked=t(sq), score_negatives=t(sn))
    _check_tournament(scores, idx, q, n, K, sq, sn)


def test_tournament_rejects_uneven_groups_and_accepts_empty_input(capi, cuda_device):
    q = torch.zeros((2, 5, 8), device=cuda_device)
    n = torch.zeros((2, 10, 8), device=cuda_device)
    with pytest.raises(capi.Ge2Error):
        capi.tournament_select(q, n, 3)
    scores, idx = capi.tournament_select(q[:, :0].contiguous(), n, 5)
    assert scores.shape == (0, 5) and idx.shape == (2, 0)
    # all scores equal: the first negative of every group wins
    scores, idx = capi.tournament_select(q, n, 5)
    torch.cuda.synchronize()
    assert torch.equal(idx.cpu().view(2, 5, 5), (torch.arange(5) * 2).expand(2, 5, 5)) and float(scores.abs().max()) == 0.0
