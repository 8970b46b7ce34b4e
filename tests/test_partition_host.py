"""Host logic of the partition buffer: schedule, bucket assignment, swap plans, and the swap protocol itself run as
two gloo ranks on CPU (the NCCL path uses the same code with CUDA tensors)."""
import importlib
import os
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path[:0] = [ROOT, os.path.join(ROOT, "oracle")]
import ge2_oracle as O  # noqa: E402

partition = importlib.import_module("ge-2_b200.partition")


@pytest.mark.parametrize("P", [4, 8, 16, 32])
def test_round_robin_covers_all_pairs(P):
    rounds = partition.round_robin_states(P)
    seen = set()
    for rnd in rounds:
        flat = [p for st in rnd for p in st]
        assert sorted(flat) == list(range(P))  # a round uses every partition exactly once: its states are disjoint
        for st in rnd:
            assert len(st) == 4
            seen |= {(a, b) for a in st for b in st}
    assert len(seen) == P * P


@pytest.mark.parametrize("P,world", [(16, 2), (16, 4), (32, 8), (8, 2)])
def test_supersteps_and_bucket_assignment(P, world):
    steps = partition.make_supersteps(P, world)
    for lanes in steps:
        used = [p for st in lanes if st is not None for p in st]
        assert len(used) == len(set(used)) and len(lanes) == world
    owner = partition.assign_buckets(steps, P)
    assert len(owner) == P * P
    for (a, b), (k, r) in owner.items():
        assert a in steps[k][r] and b in steps[k][r]


def test_plan_swap_matches_reference_relay_when_everything_is_resident():
    """world * 4 == P: every admitted partition comes from the rank and slot that hold it now, which is the owner lookup
    of the reference's relay (oracle.relay_swap_plan)."""
    place = partition.Placement.initial(2, 8)
    moves, slots = partition.plan_swap(place, [[0, 1, 2, 3], [4, 5, 6, 7]])
    assert all(m.src_kind == "home" for m in moves) and slots == [[0, 1, 2, 3], [4, 5, 6, 7]]
    place = partition.apply_plan(place, slots)
    nxt = [[0, 1, 4, 5], [2, 3, 6, 7]]
    moves, slots2 = partition.plan_swap(place, nxt)
    ref = O.relay_swap_plan(slots, [sorted(s) for s in nxt])
    ref_src = {p: (sd, ss) for lanes in ref for (_slot, p, sd, ss) in lanes}
    for m in moves:
        assert m.src_kind == "buf" and (m.src_rank, m.src_index) == ref_src[m.partition]
    assert sorted(slots2[0]) == [0, 1, 4, 5] and slots2[0][:2] == [0, 1]  # partitions that stay keep their slot
    with pytest.raises(ValueError):
        partition.plan_swap(place, [[0, 1, 2, 3], [3, 5, 6, 7]])  # overlapping states


def _worker(rank, world, P, rows, D, port, out):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        home_parts = [p for p in range(P) if p % world == rank]
        emb = torch.cat([torch.full((rows, D), float(p * 100)) + torch.arange(rows).view(-1, 1) for p in home_parts])
        state = emb * 0.5
        buf = partition.PartitionBuffer([emb, state], rows, P, rank, world, dist)
        steps = partition.make_supersteps(P, world)
        for k, lanes in enumerate(steps):
            buf.swap(lanes)
            st = lanes[rank]
            if st is not None:
                tab = buf.slot_table()
                for p in st:  # "training": a partition- and superstep-specific update of the resident rows
                    s = tab[p]
                    assert s >= 0
                    buf.buf[0][s * rows:(s + 1) * rows] += (k + 1) * 0.25 + p
                    buf.buf[1][s * rows:(s + 1) * rows] += 1.0
            dist.barrier()
        buf.flush()
        out.put((rank, emb.numpy().copy(), state.numpy().copy()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("P,world", [(8, 2), (16, 2), (16, 4)])
def test_swap_protocol_two_gloo_ranks(P, world):
    rows, D = 3, 2
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + (os.getpid() % 500) + P
    procs = [ctx.Process(target=_worker, args=(r, world, P, rows, D, port, out)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, e, s = out.get(timeout=120)
        got[r] = (e, s)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    # single-process expectation
    steps = partition.make_supersteps(P, world)
    exp_e = {p: np.full((rows, D), p * 100.0, np.float32) + np.arange(rows, dtype=np.float32)[:, None] for p in range(P)}
    exp_s = {p: exp_e[p] * 0.5 for p in range(P)}
    for k, lanes in enumerate(steps):
        for st in lanes:
            if st is None:
                continue
            for p in st:
                exp_e[p] = exp_e[p] + ((k + 1) * 0.25 + p)
                exp_s[p] = exp_s[p] + 1.0
    for r in range(world):
        parts = [p for p in range(P) if p % world == r]
        assert np.array_equal(got[r][0], np.concatenate([exp_e[p] for p in parts]))
        assert np.array_equal(got[r][1], np.concatenate([exp_s[p] for p in parts]))


def test_plan_swap_rejects_claiming_an_idle_ranks_partition():
    place = partition.apply_plan(partition.Placement.initial(2, 8), [[0, 1, 2, 3], [4, 5, 6, 7]])
    with pytest.raises(ValueError, match="idle rank"):
        partition.plan_swap(place, [None, [2, 5, 6, 7]])  # rank 0 idles and keeps partition 2


@pytest.mark.parametrize("P,world", [(8, 1), (8, 2), (16, 2), (32, 8)])
def test_relay_plan_moves_every_partition_exactly_once(P, world):
    """The device-side swap's plan: simulated with numpy slabs it must give every rank exactly its state, leave nothing
    stranded, and agree with the reference's owner lookup (oracle.relay_swap_plan) when everything is resident."""
    rows = 3
    home = {p: np.full((rows, 2), float(p)) for p in range(P)}  # home slab contents = partition id
    bufs = [np.full((partition.CAPACITY * rows, 2), -1.0) for _ in range(world)]
    place = partition.Placement.initial(world, P)
    steps = partition.make_supersteps(P, world)
    for lanes in steps + steps:
        new_slots, pulls = partition.plan_relay(place, lanes)
        if world * partition.CAPACITY == P and place.in_buffer:
            ref = O.relay_swap_plan([list(s) for s in place.slots], [list(s) for s in new_slots])
            ref_src = {p: (sd, ss) for moves in ref for (_slot, p, sd, ss) in moves}
        else:
            ref_src = None
        new_bufs = [b.copy() for b in bufs]
        for r in range(world):
            for src_kind, sr, si, dst_kind, di in pulls[r]:
                slab = bufs[sr][si * rows:(si + 1) * rows] if src_kind == "buf" else home[[p for p in range(P) if p % world == sr and p // world == si][0]]
                if dst_kind == "buf":
                    new_bufs[r][di * rows:(di + 1) * rows] = slab
                    if ref_src is not None and src_kind == "buf":
                        assert ref_src[int(slab[0, 0])] == (sr, si)
                else:
                    home[[p for p in range(P) if p % world == r and p // world == di][0]] = slab.copy()
        bufs = new_bufs
        place = partition.apply_plan(place, new_slots)
        for r, st in enumerate(lanes):
            want = sorted(st) if st is not None else sorted(p for p in place.slots[r] if p >= 0)
            got = [int(bufs[r][k * rows, 0]) for k in range(len(want))]
            assert got == want
    _, pulls = partition.plan_relay(place, [[] for _ in range(world)])  # flush: every resident partition is fetched by its home rank
    assert sorted(p for r in range(world) for p in [(di * world + r) for (_k, _sr, _si, dk, di) in pulls[r] if dk == "home"]) == sorted(place.in_buffer)


def test_state_shuffle_is_a_permutation_and_edge_list_restatement():
    for n in (0, 1, 2, 3, 17, 256, 1000, 65537):
        perm = O.state_shuffle_permutation(n, 5)
        assert sorted(perm.tolist()) == list(range(n))
    assert not np.array_equal(O.state_shuffle_permutation(1000, 5), O.state_shuffle_permutation(1000, 6))
    rng = np.random.default_rng(0)
    P, psize = 4, 50
    e = np.stack([rng.integers(0, P * psize, 2000), rng.integers(0, 5, 2000), rng.integers(0, P * psize, 2000)], 1)
    es, sizes = O.bucket_sort_edges(e, P, psize)
    assert sizes.sum() == 2000 and np.all(np.diff((es[:, 0] // psize) * P + es[:, 2] // psize) >= 0)
    begin = np.concatenate([[0], np.cumsum(sizes)])[:-1]
    slots = np.array([1, -1, 0, -1])
    bk = [0 * P + 2, 2 * P + 0, 2 * P + 2]
    out = O.build_state_edges(es, [int(begin[b]) for b in bk], [int(sizes[b]) for b in bk], slots, psize, 3)
    assert out.shape[0] == sizes[bk].sum() and out[:, [0, 2]].max() < 2 * psize
    # undo the remap: the multiset of rows equals the buckets' rows
    back = out.copy()
    inv = {1: 0, 0: 2}
    for col in (0, 2):
        back[:, col] = np.array([inv[s] for s in out[:, col] // psize]) * psize + out[:, col] % psize
    exp = np.concatenate([es[begin[b]:begin[b] + sizes[b]] for b in bk])
    assert sorted(map(tuple, back.tolist())) == sorted(map(tuple, exp.tolist()))


@pytest.mark.parametrize("P,world", [(8, 2), (16, 2), (16, 4), (32, 8)])
def test_size_aware_bucket_assignment_covers_once_and_is_no_longer_than_greedy(P, world):
    """With bucket sizes every ordered bucket is still trained exactly once, by a state that holds both of its partitions, and
    the epoch (sum over supersteps of the longest lane) is not longer than with the first-fit assignment."""
    import numpy as np

    rng = np.random.default_rng(P * 31 + world)
    w = rng.dirichlet(np.full(P, 0.3))                      # skewed partition weights, like a hub-heavy graph
    sizes = (np.outer(w, w) * 50_000_000).astype(np.int64).reshape(-1)
    steps = partition.make_supersteps(P, world)
    greedy = partition.state_buckets(steps, P)
    balanced = partition.state_buckets(steps, P, sizes)
    seen = sorted(b for lanes in balanced for lane in lanes for b in lane)
    assert seen == list(range(P * P))
    for k, lanes in enumerate(balanced):
        for r, lane in enumerate(lanes):
            st = steps[k][r]
            for b in lane:
                assert st is not None and b // P in st and b % P in st
    length = lambda assign: sum(max(sum(int(sizes[b]) for b in lane) for lane in lanes) for lanes in assign)
    assert length(balanced) <= length(greedy)
