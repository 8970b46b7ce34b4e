"""ge2_eval_ranks against the oracle's restatement of the reference's evaluation (node_corrupt_forward scores, the global
filter of compute_filter_corruption, ranks as LinkPredictionReporter::computeRanks): integer ranks, bit-exact."""
import numpy as np
import pytest
import torch

import ge2_oracle as O
import workloads

pytestmark = pytest.mark.gpu


def _case(rng, nodes, R, D, n_all, B, scale=0.5):
    table = (rng.standard_normal((nodes, D)) * scale).astype(np.float32)
    rel = (rng.standard_normal((max(R, 1), D)) * scale + 1).astype(np.float32)
    inv = (rng.standard_normal((max(R, 1), D)) * scale + 1).astype(np.float32)
    src = workloads.zipf_ids(rng, n_all, nodes, 1.0)
    dst = workloads.zipf_ids(rng, n_all, nodes, 1.0)
    if R > 0:
        all_edges = np.stack([src, workloads.zipf_ids(rng, n_all, R, 1.2), dst], 1).astype(np.int64)
    else:
        all_edges = np.stack([src, dst], 1).astype(np.int64)
    return table, rel, inv, all_edges, all_edges[:B].copy()


@pytest.mark.parametrize("kind,nodes,R,D,B,inverse", [
    ("DISTMULT", 5000, 40, 50, 200, True),     # two sides, tiles cut ragged on both axes
    ("COMPLEX", 3001, 11, 100, 130, True),
    ("COMPLEX", 4096, 7, 100, 64, False),      # one side although the edges carry relations
    ("DISTMULT", 2500, 0, 100, 257, False),    # Dot: two-column edges
    ("DISTMULT", 900, 5, 128, 70, True),
    ("DISTMULT", 700, 3, 6, 10, True),
])
def test_filtered_ranks_match_oracle(capi, cuda_device, kind, nodes, R, D, B, inverse):
    rng = np.random.default_rng(nodes + D)
    table, rel, inv, all_edges, edges = _case(rng, nodes, R, D, 20 * B, B)
    fd = O.global_filter(all_edges, edges, False)
    fs = O.global_filter(all_edges, edges, True) if (R > 0 and inverse) else None
    exp_d, exp_s = O.eval_ranks(kind, table, rel if R > 0 else None, inv if (R > 0 and inverse) else None, edges, fd, fs)
    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    got_d, got_s = capi.eval_ranks(kind, t(table), t(edges), t(rel) if R > 0 else None, t(inv) if (R > 0 and inverse) else None,
                                   dst_filter=t(fd), src_filter=t(fs), status=status)
    torch.cuda.synchronize()
    assert int(status) == 0
    assert np.array_equal(got_d.cpu().numpy(), exp_d)
    if exp_s is None:
        assert got_s is None
    else:
        assert np.array_equal(got_s.cpu().numpy(), exp_s)
    # filtered evaluation removes the positive's own node: no rank can exceed the number of nodes
    assert int(got_d.max()) <= nodes and int(got_d.min()) >= 1


def test_unfiltered_counts_the_positive_itself_and_duplicate_pairs_change_nothing(capi, cuda_device):
    rng = np.random.default_rng(5)
    table, rel, inv, all_edges, edges = _case(rng, 1500, 9, 50, 2000, 100)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    exp_d, exp_s = O.eval_ranks("DISTMULT", table, rel, inv, edges)
    got_d, got_s = capi.eval_ranks("DISTMULT", t(table), t(edges), t(rel), t(inv))
    assert np.array_equal(got_d.cpu().numpy(), exp_d) and np.array_equal(got_s.cpu().numpy(), exp_s)
    assert int(got_d.min()) >= 2  # the candidate equal to the positive's destination scores exactly the positive score
    fd = O.global_filter(all_edges, edges, False)
    twice = np.concatenate([fd, fd[::-1], fd[:7]])
    once, _ = capi.eval_ranks("DISTMULT", t(table), t(edges), t(rel), t(inv), dst_filter=t(fd))
    dup, _ = capi.eval_ranks("DISTMULT", t(table), t(edges), t(rel), t(inv), dst_filter=t(twice))
    assert torch.equal(once, dup)


def test_candidate_list_and_bad_ids(capi, cuda_device):
    rng = np.random.default_rng(6)
    table, rel, inv, all_edges, edges = _case(rng, 2000, 4, 100, 1000, 50)
    neg_ids = rng.choice(2000, 333, replace=False).astype(np.int64)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    filt = np.stack([rng.integers(0, 50, 40), rng.integers(0, 333, 40)], 1).astype(np.int64)
    exp_d, exp_s = O.eval_ranks("COMPLEX", table, rel, inv, edges, filt, None, neg_ids=neg_ids)
    got_d, got_s = capi.eval_ranks("COMPLEX", t(table), t(edges), t(rel), t(inv), dst_filter=t(filt), neg_ids=t(neg_ids))
    assert np.array_equal(got_d.cpu().numpy(), exp_d) and np.array_equal(got_s.cpu().numpy(), exp_s)
    bad = edges.copy()
    bad[3, 0] = 2000      # source out of range
    bad[7, 1] = -1        # relation out of range
    status = torch.zeros(1, dtype=torch.int32, device=cuda_device)
    got_d, got_s = capi.eval_ranks("COMPLEX", t(table), t(bad), t(rel), t(inv), status=status)
    torch.cuda.synchronize()
    assert int(status) & 8
    assert int(got_d[3]) == 0 and int(got_d[7]) == 0 and int(got_s[3]) == 0
    ok = np.ones(50, bool)
    ok[[3, 7]] = False
    exp_d, _ = O.eval_ranks("COMPLEX", table, rel, inv, edges)
    assert np.array_equal(got_d.cpu().numpy()[ok], exp_d[ok])
