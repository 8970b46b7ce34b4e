"""GPU parity against the reference project's OWN GPU code.

oracle/_ref/gege_ref_cuda.so is the reference's sources compiled with -DGEGE_CUDA for sm_100 by `make -C oracle cuda`
(its unique_map_cuda.cu, and its decoder / loss / autograd / Adagrad translation units, which run on CUDA tensors).
Here the library's kernels, called through the C ABI, are compared with what that code returns for the same device
inputs: the unique-map bit for bit against map_tensors_unique_inverse_cuda under GEGE_UNIQUE_BACKEND=bitmap, the fused
link-prediction step against Model::train_batch's sequence within the stated float tolerances.

The file name sorts late on purpose: the reference's CUDA code runs in this process, after the library's own tests.
"""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

import workloads
from gpu_helpers import rel_err, run_lp_step

pytestmark = pytest.mark.gpu
REF_DIR = Path(__file__).resolve().parents[1] / "oracle" / "_ref"

# north-star tolerances: 1e-4 relative for the fp32 path, 1e-2 for 16-bit tensor tiles
TOL = {"fp32": 1e-4, "f16": 1e-2}

# (n_ids, domain) of the five stated configurations
CONFIG_PAIRS = [(22_000, 14_951), (40_000, 1_000_000), (150_000, 1_211_896), (150_000, 10_413_060), (600_000, 12_500_000)]


@pytest.fixture(scope="module")
def ref_cuda(cuda_device):
    os.environ["GEGE_UNIQUE_BACKEND"] = "bitmap"  # read once, on the reference's first call
    os.environ.setdefault("GEGE_CSR_GATHER", "0")
    os.environ.setdefault("GEGE_CSR_DEBUG", "0")
    os.environ.setdefault("GEGE_STAGE_DEBUG", "0")
    so = REF_DIR / "gege_ref_cuda.so"
    if not so.exists():
        pytest.fail(f"{so} is missing: build it with `make -C oracle cuda` where the reference checkout is available")
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import torch  # noqa: F401  (libtorch must be loaded first)
    import gege_ref_cuda

    return gege_ref_cuda


def ours_unique(capi, ids, domain):
    import torch

    u, inv, cnt = capi.unique_bitmap(ids, domain)
    torch.cuda.synchronize()
    count, status = (int(x) for x in cnt.cpu())
    return u[:count], inv, count, status


def compare_unique(capi, ref_cuda, ids_np, domain, device):
    import torch

    ids = torch.from_numpy(np.ascontiguousarray(ids_np, dtype=np.int64)).to(device)
    # sorted=False is how the bitmap backend is reached (map_tensors_unique_inverse_cuda sends sorted=True to its sort
    # backend before it looks at GEGE_UNIQUE_BACKEND, unique_map_cuda.cu:1002-1007); both must agree with the library
    ru, rinv, backend = ref_cuda.unique_inverse_cuda(ids, False, domain)
    assert backend == "bitmap", backend  # the reference silently falls back to sort on bad input; then nothing was pinned
    su, sinv, sort_backend = ref_cuda.unique_inverse_cuda(ids, True, domain)
    assert sort_backend == "sort", sort_backend
    u, inv, count, status = ours_unique(capi, ids, domain)
    assert status == 0
    assert count == ru.numel() == su.numel()
    assert torch.equal(u, ru) and torch.equal(u, su)
    assert torch.equal(inv, rinv) and torch.equal(inv, sinv)
    return count


@pytest.mark.parametrize("n,domain", CONFIG_PAIRS)
@pytest.mark.parametrize("dist", ["uniform", "zipf"])
def test_unique_map_bit_exact_against_reference_bitmap(capi, cuda_device, ref_cuda, n, domain, dist):
    rng = np.random.default_rng(n + domain)
    ids = rng.integers(0, domain, n) if dist == "uniform" else workloads.zipf_ids(rng, n, domain, 1.1)
    count = compare_unique(capi, ref_cuda, ids, domain, cuda_device)
    assert 0 < count <= min(n, domain)


def test_unique_map_degenerate_inputs_against_reference(capi, cuda_device, ref_cuda):
    domain = 1_000_000
    for ids in (np.full(5000, 777_777), np.arange(domain - 3000, domain), np.array([0, domain - 1, 0, domain - 1, 63, 64, 65]),
                np.array([5]), np.arange(64), np.arange(65)[::-1].copy()):
        compare_unique(capi, ref_cuda, ids, domain, cuda_device)
    for n, small_domain in ((1, 1), (10, 64), (1000, 65), (4096, 63), (70_000, 65_537)):
        compare_unique(capi, ref_cuda, np.random.default_rng(n).integers(0, small_domain, n), small_domain, cuda_device)


def run_reference_step(ref_cuda, case, device):
    import torch

    t = lambda a: None if a is None else torch.from_numpy(np.ascontiguousarray(a)).to(device)  # noqa: E731
    B, C, N, D, R, U = case.dims
    has_rel = case.rel is not None
    model = ref_cuda.RefModel(case.kind, max(R, 1), D, case.inv_rel is not None, case.lr, case.lr, str(device))
    if has_rel:
        model.set_relations(t(case.rel), t(case.inv_rel) if case.inv_rel is not None else torch.Tensor())
    filt = t(case.filt) if len(case.filt) else None
    out = model.train_batch(t(case.edges), t(case.emb), t(case.state), t(case.dst_negs), t(case.src_negs), filt,
                            filt if case.src_negs is not None else None, True, True)
    torch.cuda.synchronize()
    ref = {k: v.cpu().numpy() for k, v in out.items()}
    ref["loss"] = float(ref["loss"])
    return ref


def check_step(res, ref, tol, S):
    assert res["status"] == 0
    assert abs(res["loss"] - ref["loss"]) <= tol * abs(ref["loss"])
    assert rel_err(res["node_grad"], ref["node_grad"]) < tol
    if "rel_grad" in ref:
        assert rel_err(res["rel_grad"], ref["rel_grad"]) < tol
    if S == 2:
        assert rel_err(res["inv_rel_grad"], ref["inv_rel_grad"]) < tol
    masked = ref["neg_scores"] == -1e9
    assert np.array_equal(res["neg_scores"] == -1e9, masked)
    for key in (("neg_scores", "pos_scores") if S == 1 else ("neg_scores", "pos_scores", "inv_neg_scores", "inv_pos_scores")):
        a, b = res[key], ref[key]
        if key.endswith("neg_scores"):
            a, b = a[~masked], b[~masked]
        assert np.abs(a - b).max() < tol * np.abs(b).max(), key


@pytest.mark.parametrize("precision", ["fp32", "f16"])
@pytest.mark.parametrize("name", sorted(workloads.GOLDEN_CASES))
def test_fused_step_against_reference_gpu_on_fixture_cases(capi, cuda_device, ref_cuda, name, precision):
    case = workloads.golden_case(name)
    S = 2 if case.src_negs is not None else 1
    ref = run_reference_step(ref_cuda, case, cuda_device)
    res = run_lp_step(capi, case, cuda_device, precision=precision, filter_mode="pairs")
    check_step(res, ref, TOL[precision], S)


@pytest.mark.parametrize("precision", ["fp32", "f16"])
@pytest.mark.parametrize("kind,B,C,N,D,R,U,n_deg,relations,inverse", [
    ("COMPLEX", 10_000, 10, 1000, 100, 1000, 38_000, 500, True, True),    # configuration 2: the benchmark's batch
    ("DISTMULT", 12_800, 10, 2000, 128, 300, 90_000, 1000, True, True),   # configuration 5's tile shapes (d=128, 2 000 negatives)
    ("DISTMULT", 10_000, 10, 1000, 100, 0, 20_000, 0, False, False),      # configurations 3/4: Dot decoder, one side
])
def test_fused_step_against_reference_gpu_at_benchmark_shapes(capi, cuda_device, ref_cuda, precision, kind, B, C, N, D, R, U, n_deg,
                                                             relations, inverse):
    """The launch shape the headline number runs (a full round of row blocks plus split leftovers) against the
    reference's own GPU arithmetic on the same tensors."""
    case = workloads.make_case(kind, B, C, N, D, max(R, 1), U, n_deg, seed=B + N, relations=relations, inverse=inverse, alpha=1.1)
    S = 2 if case.src_negs is not None else 1
    ref = run_reference_step(ref_cuda, case, cuda_device)
    res = run_lp_step(capi, case, cuda_device, precision=precision, filter_mode="deg_rows" if n_deg else "none")
    check_step(res, ref, TOL[precision], S)


def test_adagrad_scatter_against_reference_gpu(capi, cuda_device, ref_cuda):
    """accumulateGradients + indexAdd of the reference on the GPU against ge2_adagrad_scatter on the same gradients."""
    import torch

    case = workloads.golden_case("complex_d100_deg_padded")
    B, C, N, D, R, U = case.dims
    ref = run_reference_step(ref_cuda, case, cuda_device)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)  # noqa: E731
    rng = np.random.default_rng(5)
    rows = np.sort(rng.permutation(3 * U)[:U]).astype(np.int64)
    table_np = (0.3 * rng.standard_normal((3 * U, D))).astype(np.float32)
    table_np[rows] = case.emb
    state_np = np.zeros((3 * U, D), np.float32)
    state_np[rows] = case.state
    table, state = t(table_np), t(state_np)
    capi.adagrad_scatter(table, state, t(rows), t(ref["node_grad"]), case.lr)
    torch.cuda.synchronize()
    exp_table, exp_state = t(table_np), t(state_np)
    ref_cuda.index_add(exp_table, t(rows), t(ref["node_update"]))
    ref_cuda.index_add(exp_state, t(rows), t(ref["node_state_update"]))
    torch.cuda.synchronize()
    # the state update is one fp32 add of the same square on both sides: exact; the table update differs by the
    # rounding of table + (-lr*g/(sqrt+eps)) computed fused here and as a separate delta there (same value, same add)
    assert torch.equal(state, exp_state)
    assert rel_err(table.cpu().numpy(), exp_table.cpu().numpy()) < 1e-6


def test_tournament_selection_restatement_matches_reference(cuda_device, ref_cuda):
    """The oracle's restatement of the reference's tournament selection of negatives against the reference's own function on
    the GPU (no fused operator exists for it here: this pins the restatement such an operator would be checked against)."""
    import torch
    import ge2_oracle as O

    rng = np.random.default_rng(12)
    C, R, N, D, sel = 3, 50, 120, 32, 12
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    k = rng.standard_normal((C, N, D)).astype(np.float32)
    exp_scores, exp_idx = O.tournament_selected_scores(q, k, sel)
    all_scores = np.einsum("crd,cnd->crn", q.astype(np.float64), k.astype(np.float64))
    for groups_per_tile in (1, 5, 12):
        scores, idx = ref_cuda.tournament_selected_scores(torch.from_numpy(q).to(cuda_device), torch.from_numpy(k).to(cuda_device), sel,
                                                          groups_per_tile)
        assert tuple(scores.shape) == (C * R, sel) and tuple(idx.shape) == (C, R * sel)
        scores, idx = scores.cpu().numpy(), idx.cpu().numpy()
        assert np.abs(scores - exp_scores).max() <= 1e-4 * np.abs(exp_scores).max()
        # a different winner is allowed only on a float tie: its score must equal the expected winner's within rounding
        got = np.take_along_axis(all_scores, idx.reshape(C, R, sel), axis=2)
        want = np.take_along_axis(all_scores, exp_idx.reshape(C, R, sel), axis=2)
        assert np.abs(got - want).max() <= 1e-5
        assert (idx != exp_idx).mean() <= 0.01
        assert np.array_equal(idx.reshape(C, R, sel) // (N // sel), np.broadcast_to(np.arange(sel), (C, R, sel)))


@pytest.mark.parametrize("kind,code", [("DOT", 1), ("L2", 2)])
def test_selected_negative_operators_against_reference_gpu(capi, cuda_device, ref_cuda, kind, code):
    """ge2_tournament_select and ge2_selected_neg_scores(_backward) against the reference's own functions on the same device
    tensors; the oracle's restatements of the pair kernels are pinned by the same outputs."""
    import torch
    import ge2_oracle as O

    rng = np.random.default_rng(40 + code)
    C, R, N, D, K = 3, 70, 200, 100, 20
    q = rng.standard_normal((C, R, D)).astype(np.float32)
    n = rng.standard_normal((C, N, D)).astype(np.float32)
    grad = rng.standard_normal((C * R, K)).astype(np.float32)
    tq, tn, tg = (torch.from_numpy(a).to(cuda_device) for a in (q, n, grad))
    ref_scores, ref_idx = ref_cuda.tournament_selected_scores(tq, tn, K, 64)
    scores, idx = capi.tournament_select(tq, tn, K)
    assert (idx != ref_idx).float().mean().item() <= 0.01
    assert (scores - ref_scores).abs().max().item() <= 1e-4 * ref_scores.abs().max().item()
    sel = ref_idx.contiguous()
    ref_out = ref_cuda.selected_neg_scores_forward(tq, tn, sel, code)
    ref_dq, ref_dn = ref_cuda.selected_neg_scores_backward(tg, tq, tn, sel, code)
    out = capi.selected_neg_scores(kind, tq, tn, sel)
    dq, dn = capi.selected_neg_scores_backward(kind, tg, tq, tn, sel)
    exp_out = O.selected_neg_scores(q, n, sel.cpu().numpy(), code)
    exp_dq, exp_dn = O.selected_neg_scores_backward(grad, q, n, sel.cpu().numpy(), code)
    for got, ref, exp in ((out, ref_out, exp_out), (dq, ref_dq, exp_dq), (dn, ref_dn, exp_dn)):
        scale = ref.abs().max().item()
        assert (got - ref).abs().max().item() <= 1e-4 * scale
        assert np.abs(ref.cpu().numpy() - exp).max() <= 1e-4 * scale
