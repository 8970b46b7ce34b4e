"""The C++ libtorch host layer (ge-2_b200/host, module ge2_host): mirrors the reference's map_tensors / Batch / Model /
InMemory interface on top of the C ABI.  CPU part: it loads, has the reference's names, and refuses CPU tensors (there is
no CPU path).  GPU part: one train_batch through the C++ layer against the reference fixtures."""
import importlib
import importlib.util
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import workloads

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"


@pytest.fixture(scope="module")
def host():
    so = ROOT / "ge-2_b200" / "ge2_host.so"
    if not so.exists():
        importlib.import_module("ge-2_b200.build").build_host()
    spec = importlib.util.spec_from_file_location("ge2_host", so)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_interface_names(host):
    for name in ("map_tensors", "map_tensors_unique_inverse_cuda", "Batch", "Model", "InMemory", "GegeRuntimeException"):
        assert hasattr(host, name)
    b = host.Batch()
    for member in ("edges", "unique_node_indices", "node_embeddings", "node_embeddings_state", "node_gradients", "node_state_update",
                   "src_neg_indices_mapping", "dst_neg_indices_mapping", "src_neg_filter", "dst_neg_filter", "accumulateGradients"):
        assert hasattr(b, member)


def test_cpu_tensors_are_rejected(host):
    ids = torch.arange(5)
    with pytest.raises(host.GegeRuntimeException, match="no CPU path"):
        host.map_tensors([ids], True, 10)
    with pytest.raises(host.GegeRuntimeException, match="1D"):
        host.map_tensors([torch.zeros((2, 2), dtype=torch.int64)], True, 10)
    with pytest.raises(host.GegeRuntimeException, match="CUDA device"):
        host.Model(host.DecoderType.DISTMULT, 3, 8, True, 0.1, 0.1, torch.device("cpu"))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(workloads.GOLDEN_CASES))
def test_train_batch_matches_reference_fixture(host, cuda_device, name):
    g = np.load(GOLDEN / f"{name}.npz")
    kind = host.DecoderType.COMPLEX if str(g["kind"]) == "COMPLEX" else host.DecoderType.DISTMULT
    has_rel = "rel" in g
    R = g["rel"].shape[0] if has_rel else 1
    D = g["emb"].shape[1]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    model = host.Model(kind, R, D, "inv_rel" in g, float(g["lr"]), float(g["lr"]), cuda_device, "fp32")
    if has_rel:
        model.relations = t(g["rel"])
        if "inv_rel" in g:
            model.inverse_relations = t(g["inv_rel"])
    batch = host.Batch()
    batch.edges = t(g["edges"])
    batch.node_embeddings = t(g["emb"])
    batch.node_embeddings_state = t(g["state"])
    batch.dst_neg_indices_mapping = t(g["dst_negs"])
    if "src_negs" in g:
        batch.src_neg_indices_mapping = t(g["src_negs"])
        batch.src_neg_filter = t(g["filt"])
    batch.dst_neg_filter = t(g["filt"])
    model.train_batch(batch, True)
    torch.cuda.synchronize()
    rel = lambda a, b: float(np.abs(a - b).max() / (np.abs(b).max() + 1e-30))
    assert abs(float(batch.loss) - float(g["ref_loss"])) <= 1e-4 * abs(float(g["ref_loss"]))
    assert rel(batch.node_gradients.cpu().numpy(), g["ref_node_update"]) < 1e-4      # after accumulateGradients: the embedding update
    assert rel(batch.node_state_update.cpu().numpy(), g["ref_node_state_update"]) < 1e-4
    if has_rel:
        assert rel(model.relations.cpu().numpy(), g["ref_rel_after"]) < 1e-4           # dense Adagrad step applied
        assert rel(model.relations_state.cpu().numpy(), g["ref_rel_state_after"]) < 1e-4


@pytest.mark.gpu
def test_map_tensors_and_storage(host, cuda_device):
    import ge2_oracle as O

    rng = np.random.default_rng(3)
    parts = [rng.integers(0, 5000, n) for n in (1000, 1000, 3000, 3000, 17)]  # five inputs: more than one pack launch
    unique, mapped = host.map_tensors([torch.from_numpy(p).to(cuda_device) for p in parts], True, 5000)
    ou, om = O.map_tensors(parts, 5000)
    assert np.array_equal(unique.cpu().numpy(), ou) and all(np.array_equal(a.cpu().numpy(), b) for a, b in zip(mapped, om))
    # an id outside the domain: the reference falls back to its sort backend; same answer here
    bad = np.array([7, 9000, 7, 3])
    unique, mapped = host.map_tensors([torch.from_numpy(bad).to(cuda_device)], True, 5000)
    assert unique.cpu().tolist() == [3, 7, 9000] and mapped[0].cpu().tolist() == [1, 2, 1, 0]
    table = rng.standard_normal((100, 20)).astype(np.float32)
    st = host.InMemory(torch.from_numpy(table.copy()).to(cuda_device))
    ids = np.array([5, 17, 99])
    assert np.array_equal(st.indexRead(torch.from_numpy(ids).to(cuda_device)).cpu().numpy(), table[ids])
    vals = rng.standard_normal((3, 20)).astype(np.float32)
    st.indexAdd(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(vals).to(cuda_device))
    table[ids] += vals
    assert np.array_equal(st.data.cpu().numpy(), table)
    with pytest.raises(RuntimeError):
        st.indexAdd(torch.from_numpy(ids).to(cuda_device), torch.from_numpy(vals[:2]).to(cuda_device))
