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
    for name in ("map_tensors", "map_tensors_unique_inverse_cuda", "Batch", "Model", "InMemory", "GegeRuntimeException", "MemPartitionBufferStorage",
                 "DataLoader"):
        assert hasattr(host, name)
    for member in ("performNextSwap", "hasSwap", "getNextAdmit", "getNextEvict", "getPartitionToBufferSlotMap", "indexRead", "indexAdd",
                   "setBufferOrdering", "getPartitionSize", "getNumInMemory"):
        assert hasattr(host.MemPartitionBufferStorage, member)
    for member in ("train_batch", "all_reduce", "broadcast", "step", "clear_grad"):
        assert hasattr(host.Model, member)
    assert hasattr(host.DataLoader, "getBatch") and hasattr(host.DataLoader, "updateEmbeddings")
    for name in ("selected_neg_scores", "selected_neg_scores_cuda_forward", "selected_neg_scores_cuda_backward",
                 "distmult_tiled_tournament_selected_scores", "SelectedNegScoreKind"):
        assert hasattr(host, name)
    assert int(host.SelectedNegScoreKind.DOT) == 1 and int(host.SelectedNegScoreKind.L2) == 2  # distmult_selected_neg_cuda.h:5
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


def test_selected_negative_functions_reject_cpu_tensors(host):
    q, n, sel = torch.zeros(1, 2, 4), torch.zeros(1, 3, 4), torch.zeros(1, 2, dtype=torch.int64)
    with pytest.raises(host.GegeRuntimeException, match="no CPU path"):
        host.selected_neg_scores(q, n, sel, host.SelectedNegScoreKind.DOT)
    with pytest.raises(host.GegeRuntimeException, match="no CPU path"):
        host.distmult_tiled_tournament_selected_scores(q, n, q, n, 3, 64)


@pytest.mark.gpu
@pytest.mark.parametrize("kind", ["DOT", "L2"])
def test_selected_neg_scores_autograd_through_the_host_layer(host, cuda_device, kind):
    """selected_neg_scores as the reference's decoder calls it (decoder_methods.cpp:996-998): forward and both gradients against
    the same gather written with torch operators, whose autograd is the comparator."""
    g = torch.Generator(device=cuda_device).manual_seed(5)
    C, R, N, D, K = 3, 40, 60, 100, 6
    q = torch.randn((C, R, D), device=cuda_device, generator=g, requires_grad=True)
    n = torch.randn((C, N, D), device=cuda_device, generator=g, requires_grad=True)
    sel = torch.randint(0, N, (C, R * K), device=cuda_device, generator=g)
    w = torch.randn((C * R, K), device=cuda_device, generator=g)
    out = host.selected_neg_scores(q, n, sel, getattr(host.SelectedNegScoreKind, kind))
    (out * w).sum().backward()
    got = (out.detach(), q.grad.clone(), n.grad.clone())
    q.grad, n.grad = None, None
    picked = n[torch.arange(C, device=cuda_device)[:, None, None], sel.view(C, R, K)]
    if kind == "DOT":
        ref = (q[:, :, None, :] * picked).sum(-1)
    else:
        ref = torch.sqrt(torch.clamp(((q[:, :, None, :] - picked) ** 2).sum(-1), min=1e-8))
    ref = ref.reshape(C * R, K)
    (ref * w).sum().backward()
    for a, b in zip(got, (ref.detach(), q.grad, n.grad)):
        assert (a - b).abs().max().item() <= 1e-4 * max(1.0, b.abs().max().item())
    assert host.selected_neg_status(cuda_device) == 0
    bad = sel.clone()
    bad[1, 3] = N
    host.selected_neg_scores_cuda_forward(q.detach(), n.detach(), bad, 1)
    assert host.selected_neg_status(cuda_device) == 8 and host.selected_neg_status(cuda_device) == 0  # reported once, then cleared


@pytest.mark.gpu
def test_tournament_scores_autograd_through_the_host_layer(host, cuda_device):
    """distmult_tiled_tournament_selected_scores with a selector separate from the scorer: columns chosen by the selector,
    scores and gradients by the scorer (the reference's bmm -> max -> gather, distmult_selected_neg_cuda.cpp:92-106)."""
    g = torch.Generator(device=cuda_device).manual_seed(6)
    C, R, N, D, K = 2, 70, 120, 64, 12
    sq = torch.randn((C, R, D), device=cuda_device, generator=g)
    sn = torch.randn((C, N, D), device=cuda_device, generator=g)
    q = torch.randn((C, R, D), device=cuda_device, generator=g, requires_grad=True)
    n = torch.randn((C, N, D), device=cuda_device, generator=g, requires_grad=True)
    w = torch.randn((C * R, K), device=cuda_device, generator=g)
    scores, cols = host.distmult_tiled_tournament_selected_scores(sq, sn, q, n, K, 64)
    (scores * w).sum().backward()
    got = (scores.detach(), q.grad.clone(), n.grad.clone())
    q.grad, n.grad = None, None
    T = N // K
    sel_scores = sq.bmm(sn.transpose(1, 2)).view(C, R, K, T)
    local = sel_scores.argmax(3)
    ref_cols = local + torch.arange(K, device=cuda_device) * T
    agree = cols.view(C, R, K) == ref_cols
    assert agree.float().mean().item() >= 0.99  # another winner only on a float tie
    ref = q.bmm(n.transpose(1, 2)).gather(2, cols.view(C, R, K)).reshape(C * R, K)  # scored on the columns the kernel kept
    (ref * w).sum().backward()
    for a, b in zip(got, (ref.detach(), q.grad, n.grad)):
        assert (a - b).abs().max().item() <= 1e-4 * max(1.0, b.abs().max().item())
    with pytest.raises(Exception, match="divisible"):
        host.distmult_tiled_tournament_selected_scores(sq, sn, q, n, 7, 64)


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
    # an index outside the table: skipped on the device, reported at the next status check (the reference's index ops throw)
    st.checkStatus()
    got = st.indexRead(torch.tensor([3, 100, 7], device=cuda_device))
    assert np.array_equal(got.cpu().numpy()[[0, 2]], table[[3, 7]]) and float(got[1].abs().max()) == 0.0
    with pytest.raises(host.GegeRuntimeException, match="out of range"):
        st.checkStatus()
    st.checkStatus()  # the word was cleared


def _n_devices():
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def _run_partition_storage(host, devices, P, nodes, D, seed):
    """swaps through every superstep of the schedule, checks what each device holds and changes it, then unloads"""
    partition = importlib.import_module("ge-2_b200.partition")
    rng = np.random.default_rng(seed)
    G = len(devices)
    table = rng.standard_normal((nodes, D)).astype(np.float32)
    expect = table.copy()
    st = host.MemPartitionBufferStorage(nodes, D, P, devices)
    psize = st.getPartitionSize()
    assert psize == -(-nodes // P) and st.getNumInMemory() == 4 * psize
    st.load(torch.from_numpy(table))
    supersteps = partition.make_supersteps(P, G)
    states = [torch.tensor(sorted(lanes[g]) if lanes[g] is not None else [], dtype=torch.int64) for lanes in supersteps for g in range(G)]
    st.setBufferOrdering(states)
    held = [set() for _ in range(G)]
    for k, lanes in enumerate(supersteps):
        for g in range(G):
            want = set(lanes[g] or [])
            assert st.hasSwap(g)
            assert set(st.getNextAdmit(g)) == want - held[g] and set(st.getNextEvict(g)) == held[g] - want
        for g in range(G):  # one host thread serves every device: nothing blocks the host
            st.performNextSwap(g)
        for g in range(G):
            slot_of = st.getPartitionToBufferSlotMap(g).tolist()
            buf = st.activeBuffer(g)
            for p in sorted(lanes[g] or []):
                rows = min(psize, nodes - p * psize)
                slot = slot_of[p]
                assert slot >= 0
                got = buf[slot * psize: slot * psize + rows].cpu().numpy()
                assert np.array_equal(got, expect[p * psize: p * psize + rows]), (k, g, p)
                # train: change two rows of the partition through the storage interface (buffer-local row ids)
                ids = torch.tensor([slot * psize, slot * psize + rows - 1], device=devices[g])
                vals = torch.full((2, D), float(k + 1), device=devices[g])
                st.indexAdd(ids, vals, g)
                expect[p * psize] += k + 1
                expect[p * psize + rows - 1] += k + 1
                assert np.array_equal(st.indexRead(ids[:1], g).cpu().numpy()[0], expect[p * psize])
            assert sorted(i for i, s in enumerate(slot_of) if s >= 0) == sorted(lanes[g] or [])
            held[g] = set(lanes[g] or [])
    for g in range(G):
        assert not st.hasSwap(g)
    out = st.unload()
    assert np.array_equal(out.numpy(), expect)


@pytest.mark.gpu
def test_partition_buffer_storage_one_device(host, cuda_device):
    _run_partition_storage(host, [torch.device("cuda:0")], 8, 1000, 20, 1)
    _run_partition_storage(host, [torch.device("cuda:0")], 4, 397, 12, 2)   # ragged last partition, one state


@pytest.mark.gpu
def test_partition_buffer_storage_two_devices(host, cuda_device):
    if _n_devices() < 2:
        pytest.skip("needs two GPUs")
    _run_partition_storage(host, [torch.device("cuda:0"), torch.device("cuda:1")], 8, 1000, 20, 3)
    _run_partition_storage(host, [torch.device("cuda:0"), torch.device("cuda:1")], 16, 4001, 12, 4)  # G * 4 < P: home slabs in play


@pytest.mark.gpu
@pytest.mark.parametrize("replicas", [1, 2])
def test_all_reduce_over_replicas(host, cuda_device, replicas):
    """Model::broadcast + train_batch(batch, false) on every replica + Model::all_reduce against the oracle's multi-GPU dense
    step, three rounds (both halves of the gradient buffers get used and cleared); in the last round one replica has no batch."""
    import ge2_oracle as O

    if _n_devices() < replicas:
        pytest.skip("needs two GPUs")
    g = np.load(GOLDEN / "complex_d100_deg_padded.npz")
    devices = [torch.device(f"cuda:{i}") for i in range(replicas)]
    R, D, lr = g["rel"].shape[0], g["emb"].shape[1], float(g["lr"])
    model = host.Model(host.DecoderType.COMPLEX, R, D, True, lr, lr, devices[0], "fp32")
    model.relations = torch.from_numpy(g["rel"]).to(devices[0])
    model.inverse_relations = torch.from_numpy(g["inv_rel"]).to(devices[0])
    model.broadcast(devices)
    reps = model.device_models
    assert len(reps) == replicas
    rel, inv = g["rel"].copy(), g["inv_rel"].copy()
    rel_s, inv_s = np.zeros_like(rel), np.zeros_like(inv)
    rng = np.random.default_rng(8)
    for rnd in range(3):
        grads = []
        for i, m in enumerate(reps):
            if rnd == 2 and i == replicas - 1 and replicas > 1:
                grads.append(None)  # a lane without a batch this round
                continue
            t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(devices[i])
            emb = (g["emb"] + 0.05 * rng.standard_normal(g["emb"].shape)).astype(np.float32)
            batch = host.Batch()
            batch.edges, batch.node_embeddings, batch.node_embeddings_state = t(g["edges"]), t(emb), t(g["state"])
            batch.dst_neg_indices_mapping, batch.src_neg_indices_mapping = t(g["dst_negs"]), t(g["src_negs"])
            batch.dst_neg_filter = batch.src_neg_filter = t(g["filt"])
            m.train_batch(batch, False)
            res = O.lp_train_forward_backward("COMPLEX", g["edges"], emb, rel, inv, g["dst_negs"], g["src_negs"], g["filt"], g["filt"])
            grads.append((res.rel_grad, res.inv_rel_grad))
        model.all_reduce()
        O.multi_gpu_dense_step(rel, rel_s, inv, inv_s, grads, lr)
        for m in reps:
            err = lambda a, b: float(np.abs(a.cpu().numpy() - b).max() / (np.abs(b).max() + 1e-30))
            assert err(m.relations, rel) < 1e-4 and err(m.inverse_relations, inv) < 1e-4
            assert err(m.relations_state, rel_s) < 1e-4 and err(m.inverse_relations_state, inv_s) < 1e-4
    model.check_status()
    if replicas > 1:  # the replicas took bit-identical steps
        assert torch.equal(reps[0].relations.cpu(), reps[1].relations.cpu())


@pytest.mark.gpu
def test_data_loader_flow_matches_oracle(host, cuda_device):
    """The reference's unfused per-batch flow through the C++ layer -- getBatch (sample, map_tensors, gather), train_batch,
    updateEmbeddings -- against the oracle's trainer step fed with the same draws."""
    import ge2_oracle as O

    rng = np.random.default_rng(4)
    nodes, R, D, B, C, N = 3000, 20, 50, 500, 5, 200
    edges = np.stack([workloads.zipf_ids(rng, 4 * B, nodes, 1.0), workloads.zipf_ids(rng, 4 * B, R, 1.2), workloads.zipf_ids(rng, 4 * B, nodes, 1.0)], 1).astype(np.int64)
    table = (rng.standard_normal((nodes, D)) * 0.1).astype(np.float32)
    state = np.zeros_like(table)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda_device)
    emb_st, state_st = host.InMemory(t(table)), host.InMemory(t(state))
    model = host.Model(host.DecoderType.DISTMULT, R, D, True, 0.1, 0.1, cuda_device, "fp32")
    loader = host.DataLoader(t(edges), emb_st, state_st, B, C, N, 0.5, True, 11)
    rel, inv = np.ones((R, D), np.float32), np.ones((R, D), np.float32)
    rel_s, inv_s = np.zeros_like(rel), np.zeros_like(rel)
    for step in range(3):
        batch = loader.getBatch()
        uniq = batch.unique_node_indices.cpu().numpy()
        src_negs = uniq[batch.src_neg_indices_mapping.cpu().numpy()]
        dst_negs = uniq[batch.dst_neg_indices_mapping.cpu().numpy()]
        filt = O.deg_negative_local_filter(batch.deg_sample_rows.cpu().numpy(), B)
        model.train_batch(batch, True)
        loader.updateEmbeddings(batch)
        O.train_step("DISTMULT", table, state, rel, rel_s, inv, inv_s, edges[step * B:(step + 1) * B], dst_negs, src_negs, filt, filt, 0.1, nodes)
    err = lambda a, b: float(np.abs(a.cpu().numpy() - b).max() / (np.abs(b).max() + 1e-30))
    assert err(emb_st.data, table) < 1e-4 and err(state_st.data, state) < 1e-4 and err(model.relations, rel) < 1e-4
