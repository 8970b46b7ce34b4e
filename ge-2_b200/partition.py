"""Partition buffer across GPUs (one process per GPU, torch.distributed for the plumbing): schedule of partition-disjoint
supersteps, bucket assignment, and partition swaps -- RelayBuffer: device-side pulls over NVLink peer memory behind a
device-side barrier (ge2_swap_begin), with the state's edge list rebuilt on the device and a trainer loop around both
(PartitionedTrainer); PartitionBuffer: the same moves as NCCL send/recv, for processes that cannot map each other's memory.

Mirrors, in the reference project (paths relative to gege/src/cpp/src): the partition buffer of
storage/buffer.cpp and storage/storage.cpp:359-757 (MemPartitionBufferStorage, capacity 4, performNextSwap :576-689),
the disjoint per-device states of data/ordering.cpp:1647-1670 / data/dataloader.cpp:709-844, and the relation-gradient
exchange of nn/model.cpp:174-204.  Differences, on purpose:
  * every partition has a home slab on one GPU (p % world), so a swap never touches host memory, also when
    world * capacity < num_partitions (the reference's peer relay requires equality and otherwise stages through the host);
  * an admitted partition is fetched from wherever it currently is -- another rank's active buffer (the reference's relay
    copy) or its home -- and evicted partitions go home; one copy kernel per table (RelayBuffer) or one batch of NCCL
    point-to-point operations (PartitionBuffer);
  * the schedule is a round-robin design over pairs of partitions (every two partitions share a state at least once per
    epoch, states of one superstep are disjoint); the reference's own ordering code can be plugged in instead, the buffer
    only needs the list of states.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

CAPACITY = 4  # buffer_capacity of the reference (buffer.cpp:950,1106; ordering.cpp:1753)


# ----------------------------------------------------------------------------------------------------------------
# schedule
# ----------------------------------------------------------------------------------------------------------------
def round_robin_states(num_partitions: int) -> List[List[List[int]]]:
    """Rounds of pairwise-disjoint 4-partition states such that every two partitions meet in some state.

    Partitions are paired into units (2k, 2k+1); a state is two units; the rounds are the 1-factorisation of the
    complete graph on the units (circle method), so each round uses every partition exactly once.
    Returns rounds[r][s] = sorted list of 4 partition ids.  num_partitions must be a multiple of 4."""
    if num_partitions % 4 != 0 or num_partitions < 4:
        raise ValueError("num_partitions must be a positive multiple of 4")
    units = num_partitions // 2
    if units == 2:
        return [[[0, 1, 2, 3]]]
    ids = list(range(units))
    rounds = []
    for _ in range(units - 1):
        pairs = [(ids[k], ids[units - 1 - k]) for k in range(units // 2)]
        rounds.append([sorted([2 * a, 2 * a + 1, 2 * b, 2 * b + 1]) for a, b in pairs])
        ids = [ids[0]] + [ids[-1]] + ids[1:-1]
    return rounds


def make_supersteps(num_partitions: int, world: int) -> List[List[Optional[List[int]]]]:
    """supersteps[k][rank] = state (4 partition ids) trained by `rank` in superstep k, or None when the lane idles.
    States of one superstep are pairwise disjoint."""
    out = []
    for rnd in round_robin_states(num_partitions):
        for i in range(0, len(rnd), world):
            lane = rnd[i:i + world]
            out.append(lane + [None] * (world - len(lane)))
    return out


def assign_buckets(supersteps, num_partitions: int) -> Dict[Tuple[int, int], Tuple[int, int]]:
    """Every ordered bucket (src partition, dst partition) -> (superstep, rank) of the first state holding both,
    the rule of the reference's greedy bucket assignment (ordering.cpp:1350-1370)."""
    owner = {}
    for k, lanes in enumerate(supersteps):
        for rank, st in enumerate(lanes):
            if st is None:
                continue
            for a in st:
                for b in st:
                    owner.setdefault((a, b), (k, rank))
    missing = [(a, b) for a in range(num_partitions) for b in range(num_partitions) if (a, b) not in owner]
    if missing:
        raise ValueError(f"schedule does not cover buckets {missing[:4]}...")
    return owner


# ----------------------------------------------------------------------------------------------------------------
# swap plan
# ----------------------------------------------------------------------------------------------------------------
@dataclass
class Move:
    partition: int
    src_rank: int
    src_kind: str  # "buf" | "home"
    src_index: int  # buffer slot, or index into the rank's home list
    dst_rank: int
    dst_kind: str
    dst_index: int


@dataclass
class Placement:
    """Where every partition's current data lives, and what each rank's buffer slots hold."""
    world: int
    num_partitions: int
    slots: List[List[int]] = field(default_factory=list)  # slots[rank][slot] = partition or -1
    in_buffer: Dict[int, Tuple[int, int]] = field(default_factory=dict)  # partition -> (rank, slot)

    @staticmethod
    def initial(world: int, num_partitions: int) -> "Placement":
        return Placement(world, num_partitions, [[-1] * CAPACITY for _ in range(world)], {})

    def home_rank(self, p: int) -> int:
        return p % self.world

    def home_index(self, p: int) -> int:
        return p // self.world


def plan_swap(place: Placement, next_states: Sequence[Optional[Sequence[int]]]) -> Tuple[List[Move], List[List[int]]]:
    """Moves that turn the current placement into `next_states` (one state per rank, None = keep the buffer as it is).

    Like the relay branch of performNextSwap (storage.cpp:599-652) each admitted partition is copied from its current
    holder; unlike it a partition that stays on its rank keeps its slot, and partitions nobody holds next go home.
    Returns (moves, new slot tables).  Raises if two ranks claim one partition (states must be disjoint)."""
    world = place.world
    claimed = {}
    for r, st in enumerate(next_states):
        if st is None:
            continue
        if len(st) > CAPACITY or len(set(st)) != len(st):
            raise ValueError("a state holds at most 4 distinct partitions")
        for p in st:
            if p in claimed:
                raise ValueError(f"partition {p} claimed by ranks {claimed[p]} and {r}: states of a superstep must be disjoint")
            claimed[p] = r
    for r, st in enumerate(next_states):
        if st is None:  # an idle rank keeps its partitions: nobody else may claim one of them
            for p in place.slots[r]:
                if p >= 0 and p in claimed:
                    raise ValueError(f"partition {p} stays on idle rank {r} but rank {claimed[p]} claims it")
    new_slots = [list(s) for s in place.slots]
    moves: List[Move] = []
    # 1. evictions: resident partitions that their rank does not keep
    for r in range(world):
        st = next_states[r]
        keep = set(st) if st is not None else set(p for p in place.slots[r] if p >= 0)
        for slot, p in enumerate(place.slots[r]):
            if p >= 0 and p not in keep:
                new_slots[r][slot] = -1
                if p not in claimed:  # nobody needs it next: back to its home slab
                    moves.append(Move(p, r, "buf", slot, place.home_rank(p), "home", place.home_index(p)))
    # 2. admissions into free slots, lowest slot first, partitions in ascending order (deterministic on every rank)
    for r in range(world):
        st = next_states[r]
        if st is None:
            continue
        have = set(p for p in new_slots[r] if p >= 0)
        free = [k for k, p in enumerate(new_slots[r]) if p < 0]
        for p in sorted(st):
            if p in have:
                continue
            slot = free.pop(0)
            new_slots[r][slot] = p
            if p in place.in_buffer:
                sr, ss = place.in_buffer[p]
                moves.append(Move(p, sr, "buf", ss, r, "buf", slot))
            else:
                moves.append(Move(p, place.home_rank(p), "home", place.home_index(p), r, "buf", slot))
    return moves, new_slots


def apply_plan(place: Placement, new_slots: List[List[int]]) -> Placement:
    inb = {p: (r, k) for r, row in enumerate(new_slots) for k, p in enumerate(row) if p >= 0}
    return Placement(place.world, place.num_partitions, [list(s) for s in new_slots], inb)


# ----------------------------------------------------------------------------------------------------------------
# the buffer itself (one per rank)
# ----------------------------------------------------------------------------------------------------------------
class PartitionBuffer:
    """Active buffer [4 * partition_rows, D] plus home slabs for the partitions this rank is home of, for one or more
    tables moved together (embeddings and Adagrad state, graph_storage.h:247-281 of the reference moves both)."""

    def __init__(self, tables_home: Sequence, partition_rows: int, num_partitions: int, rank: int, world: int, dist=None,
                 peer_copies: bool = False):
        """tables_home[t]: tensor [n_home * partition_rows, D] with this rank's home partitions (p % world == rank, ascending).
        dist: torch.distributed module (None for a single process).
        peer_copies (GPUs of one node, one process each): the active buffers are symmetric memory, and a partition that moves
        from one rank's buffer to another's is PULLED by the receiver with a copy kernel that reads the holder's buffer over
        NVLink (the reference's relay copy, storage.cpp:626-652, as a load instead of a peer memcpy), between two host
        barriers; NCCL send/recv then only serves moves from or to home slabs."""
        import torch

        self.rank, self.world, self.dist = rank, world, dist
        self.rows = partition_rows
        self.num_partitions = num_partitions
        self.home = list(tables_home)
        self.peer_buf = None
        if peer_copies and world > 1:
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads only
            import torch.distributed._symmetric_memory as symm_mem

            self.buf, self.peer_buf, self._handles = [], [], []
            for t in self.home:
                shape = (CAPACITY * partition_rows, t.shape[1])
                b = symm_mem.empty(shape, dtype=t.dtype, device=t.device)
                h = symm_mem.rendezvous(b, dist.group.WORLD)
                self.buf.append(b)
                self._handles.append(h)
                self.peer_buf.append([b if r == rank else h.get_buffer(r, shape, t.dtype) for r in range(world)])
        else:
            self.buf = [torch.empty((CAPACITY * partition_rows, t.shape[1]), dtype=t.dtype, device=t.device) for t in self.home]
        self.staging = [torch.empty_like(b) for b in self.buf]
        self.place = Placement.initial(world, num_partitions)

    def _slab(self, kind: str, index: int, t: int, staged: bool = False):
        base = (self.staging[t] if staged else self.buf[t]) if kind == "buf" else self.home[t]
        return base[index * self.rows:(index + 1) * self.rows]

    def swap(self, next_states: Sequence[Optional[Sequence[int]]], stream=None):
        """Performs the swap for every rank's next state (all ranks call this with the same argument).
        Local moves are device copies; moves between ranks are point-to-point sends/receives batched into one group.
        Incoming slabs land in a staging buffer and are copied into place after all outgoing data has left, so a slot
        can be overwritten by the partition that replaces it while its old content is still being sent."""
        import torch

        moves, new_slots = plan_swap(self.place, next_states)
        ops, reqs, local, staged_in = [], [], [], []
        pulls: Dict[int, List[Tuple[int, int]]] = {}
        pull_any = False  # the same on every rank: all ranks see the same plan
        for m in moves:  # same order on every rank: sends and receives pair up per peer in that order
            if self.peer_buf is not None and m.src_kind == "buf" and m.dst_kind == "buf" and m.src_rank != m.dst_rank:
                pull_any = True
                if m.dst_rank == self.rank:  # the receiver fetches it from the holder's buffer
                    pulls.setdefault(m.src_rank, []).append((m.src_index, m.dst_index))
                    staged_in.extend((m, t) for t in range(len(self.home)))
                continue
            for t in range(len(self.home)):
                if m.src_rank == self.rank and m.dst_rank == self.rank:
                    local.append((m, t))
                elif m.src_rank == self.rank:
                    ops.append(("send", self._slab(m.src_kind, m.src_index, t), m.dst_rank))
                elif m.dst_rank == self.rank:
                    dst = self._slab(m.dst_kind, m.dst_index, t, staged=m.dst_kind == "buf")
                    ops.append(("recv", dst, m.src_rank))
                    if m.dst_kind == "buf":
                        staged_in.append((m, t))
        # local moves out of the buffer read the old content: stage them too
        for m, t in local:
            if m.dst_kind == "buf":
                self._slab("buf", m.dst_index, t, staged=True).copy_(self._slab(m.src_kind, m.src_index, t))
                staged_in.append((m, t))
        if pull_any:
            import importlib

            capi = importlib.import_module(__package__ + ".capi")
            # every rank's last training step is complete, so the holders' slabs are final
            torch.cuda.current_stream().synchronize()
            self.dist.barrier()
            for src_rank, pairs in pulls.items():
                for t in range(len(self.home)):
                    capi.copy_slabs(self.peer_buf[t][src_rank], self.staging[t], pairs, self.rows * self.home[t].shape[1])
        if ops:
            d = self.dist
            p2p = [d.P2POp(d.isend if kind == "send" else d.irecv, ten, peer) for kind, ten, peer in ops]
            reqs = d.batch_isend_irecv(p2p)
            for r in reqs:
                r.wait()
        if pull_any:
            # nobody overwrites a slot of its buffer before every rank has fetched what it needs from it
            torch.cuda.current_stream().synchronize()
            self.dist.barrier()
        for m, t in local:
            if m.dst_kind == "home":
                self._slab("home", m.dst_index, t).copy_(self._slab("buf", m.src_index, t))
        for m, t in staged_in:
            self._slab("buf", m.dst_index, t).copy_(self._slab("buf", m.dst_index, t, staged=True))
        self.place = apply_plan(self.place, new_slots)
        return moves

    def flush(self):
        """Sends every resident partition home (end of training / before evaluation), the counterpart of the reference's
        unload(write=true)."""
        return self.swap([[] for _ in range(self.world)])

    def slot_table(self):
        """partition -> slot of this rank's buffer (-1 when not resident): the map mapEdgesWithPartitionSlots_ indexes
        (graph_storage.cpp:270-303 of the reference)."""
        tab = [-1] * self.num_partitions
        for slot, p in enumerate(self.place.slots[self.rank]):
            if p >= 0:
                tab[p] = slot
        return tab


# ----------------------------------------------------------------------------------------------------------------
# the buffer with device-side swaps: two active buffers per table, receiver-side pulls behind a device-side barrier
# ----------------------------------------------------------------------------------------------------------------
def plan_relay(place: Placement, next_states: Sequence[Optional[Sequence[int]]]):
    """Slot tables and pulls of a swap of RelayBuffer: every rank's next buffer is filled slot by slot (the state's
    partitions in ascending order) from wherever each partition is now -- a slot of some rank's current buffer (the
    reference's relay copy, storage.cpp:626-652) or its home slab -- and a resident partition that nobody keeps is pulled
    by its home rank.  A rank whose next state is None keeps its partitions (they still move to its other buffer).
    Returns (new_slots, pulls) with pulls[rank] = list of (src_kind, src_rank, src_index, dst_kind, dst_index)."""
    world = place.world
    states = []
    claimed = {}
    for r in range(world):
        st = next_states[r]
        st = sorted(p for p in place.slots[r] if p >= 0) if st is None else sorted(st)
        if len(st) > CAPACITY or len(set(st)) != len(st):
            raise ValueError("a state holds at most 4 distinct partitions")
        for p in st:
            if p in claimed:
                raise ValueError(f"partition {p} claimed by ranks {claimed[p]} and {r}: states of a superstep must be disjoint")
            claimed[p] = r
        states.append(st)
    new_slots = [st + [-1] * (CAPACITY - len(st)) for st in states]
    pulls = [[] for _ in range(world)]
    for r in range(world):
        for slot, p in enumerate(states[r]):
            if p in place.in_buffer:
                sr, ss = place.in_buffer[p]
                pulls[r].append(("buf", sr, ss, "buf", slot))
            else:
                pulls[r].append(("home", place.home_rank(p), place.home_index(p), "buf", slot))
    for p, (sr, ss) in sorted(place.in_buffer.items()):
        if p not in claimed:  # nobody needs it next: its home rank fetches it
            pulls[place.home_rank(p)].append(("buf", sr, ss, "home", place.home_index(p)))
    return new_slots, pulls


class RelayBuffer:
    """Partition buffer whose swaps run on the device (ge2_swap_begin): two active buffers [4 * partition_rows, D] per table
    that alternate from superstep to superstep, home slabs for the partitions this rank is home of (p % world == rank), all
    of it symmetric memory when world > 1 so that every rank can read every other rank's slabs over NVLink.  A swap reads
    the buffers of the superstep that ended and writes the buffers of the one that begins: no staging copy, no host barrier.

    The counterpart of MemPartitionBufferStorage (storage.cpp:359-757 of the reference) with its peer relay, except that every
    partition also has a home on some GPU, so nothing is staged through the host when world * 4 < num_partitions."""

    def __init__(self, tables_home: Sequence, partition_rows: int, num_partitions: int, rank: int, world: int, dist=None):
        import torch

        from . import capi

        self.capi = capi
        self.rank, self.world, self.dist = rank, world, dist
        self.rows, self.num_partitions = partition_rows, num_partitions
        self.parity = 0
        self.epoch = 0
        self.place = Placement.initial(world, num_partitions)
        dev = tables_home[0].device
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.slab_bytes = [partition_rows * t.shape[1] * t.element_size() for t in tables_home]
        shape = lambda t: (CAPACITY * partition_rows, t.shape[1])
        if world > 1:
            import os

            os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")  # plain peer loads only
            import torch.distributed._symmetric_memory as symm_mem

            self._keep = []

            def shared(sh, dtype, init=None):
                b = symm_mem.empty(sh, dtype=dtype, device=dev)
                if init is None:
                    b.zero_()
                else:
                    b.copy_(init)
                torch.cuda.synchronize(dev)
                h = symm_mem.rendezvous(b, dist.group.WORLD)
                self._keep.append(h)
                return b, [int(x) for x in h.buffer_ptrs]

            self.home, self.home_ptrs, self.bufs, self.buf_ptrs = [], [], [[], []], [[], []]
            for t in tables_home:
                b, ptrs = shared(tuple(t.shape), t.dtype, t)
                self.home.append(b)
                self.home_ptrs.append(ptrs)
                for k in (0, 1):
                    b, ptrs = shared(shape(t), t.dtype)
                    self.bufs[k].append(b)
                    self.buf_ptrs[k].append(ptrs)
            self.flags, self.flag_ptrs = shared((world + 1,), torch.int64)
            dist.barrier()
            torch.cuda.synchronize(dev)
        else:
            self.home = list(tables_home)
            self.home_ptrs = [[t.data_ptr()] for t in self.home]
            self.bufs = [[torch.zeros(shape(t), dtype=t.dtype, device=dev) for t in self.home] for _ in (0, 1)]
            self.buf_ptrs = [[[b.data_ptr()] for b in self.bufs[k]] for k in (0, 1)]
            self.flags, self.flag_ptrs = None, None

    def buf(self, t: int, parity: Optional[int] = None):
        return self.bufs[self.parity if parity is None else parity][t]

    def swap(self, next_states: Sequence[Optional[Sequence[int]]], wait_budget_us: int = 0):
        """Enqueues the swap on the current stream (all ranks call this with the same argument): the barrier kernel, then one
        pull kernel per table.  Afterwards `parity` names the buffers that hold the new state."""
        new_slots, pulls = plan_relay(self.place, next_states)
        self.epoch += 1
        old, new = self.parity, self.parity ^ 1
        for t in range(len(self.home)):
            sb = self.slab_bytes[t]
            lst = []
            for src_kind, sr, si, dst_kind, di in pulls[self.rank]:
                src = (self.buf_ptrs[old][t][sr] if src_kind == "buf" else self.home_ptrs[t][sr]) + si * sb
                dst = (self.bufs[new][t].data_ptr() if dst_kind == "buf" else self.home[t].data_ptr()) + di * sb
                lst.append((src, dst))
            # the barrier goes with the first table's pulls; the others follow it on the same stream
            if t == 0:
                self.capi.swap_begin(self.world, self.rank, self.flag_ptrs, self.epoch, lst, sb, self.status, wait_budget_us)
            elif lst:
                self.capi.swap_begin(1, 0, None, self.epoch, lst, sb, self.status)
        self.parity = new
        self.place = apply_plan(self.place, new_slots)
        return pulls[self.rank]

    def flush(self):
        """Every resident partition goes to its home slab (end of training / before evaluation)."""
        return self.swap([[] for _ in range(self.world)])

    def slot_table(self):
        tab = [-1] * self.num_partitions
        for slot, p in enumerate(self.place.slots[self.rank]):
            if p >= 0:
                tab[p] = slot
        return tab

    def check_status(self):
        import torch

        torch.cuda.synchronize(self.status.device)
        word = int(self.status.item())
        if word:
            raise self.capi.Ge2Error("partition swap: " + self.capi.decode_status(word))


def state_buckets(supersteps, num_partitions: int, bucket_sizes=None):
    """buckets[k][rank] = list of bucket ids (src partition * P + dst partition) trained by `rank` in superstep k.
    Without sizes every ordered bucket goes to the first state that holds both of its partitions (the reference's greedy
    assignment, ordering.cpp:1350-1370).  With bucket_sizes[P * P] the buckets that several states could train (both
    partitions in one unit of the round-robin design: they meet in every round) are dealt out largest first to where they
    lengthen the epoch least -- the epoch's length is the sum over supersteps of the longest lane, the quantity the
    reference's schedule optimizer balances (ordering.cpp:659-728)."""
    P = num_partitions
    where: Dict[Tuple[int, int], List[Tuple[int, int]]] = {}
    for k, lanes in enumerate(supersteps):
        for r, st in enumerate(lanes):
            if st is None:
                continue
            for a in st:
                for b in st:
                    where.setdefault((a, b), []).append((k, r))
    missing = [(a, b) for a in range(P) for b in range(P) if (a, b) not in where]
    if missing:
        raise ValueError(f"schedule does not cover buckets {missing[:4]}...")
    out = [[[] for _ in lanes] for lanes in supersteps]
    if bucket_sizes is None:
        for (a, b), places in sorted(where.items()):
            k, r = places[0]
            out[k][r].append(a * P + b)
        return out
    size = lambda ab: int(bucket_sizes[ab[0] * P + ab[1]])
    load = [[0] * len(lanes) for lanes in supersteps]
    flexible = []
    for ab, places in sorted(where.items()):
        if len(places) == 1:
            k, r = places[0]
            out[k][r].append(ab[0] * P + ab[1])
            load[k][r] += size(ab)
        else:
            flexible.append(ab)
    for ab in sorted(flexible, key=lambda x: (-size(x), x)):
        best = None
        for k, r in where[ab]:
            longest = max(load[k])
            cost = (max(longest, load[k][r] + size(ab)) - longest, load[k][r], k, r)
            if best is None or cost < best:
                best = cost
        _, _, k, r = best
        out[k][r].append(ab[0] * P + ab[1])
        load[k][r] += size(ab)
    for lanes in out:
        for lst in lanes:
            lst.sort()
    return out


class PartitionedTrainer:
    """One epoch over a partitioned graph on this rank: for every superstep swap partitions (RelayBuffer), rebuild the state's
    edge list on the device (ge2_build_state_edges), train its batches through the pipelined step graphs, and -- with several
    ranks -- keep taking part in the relation-gradient exchange until the longest lane of the superstep is done.
    The loop of the reference's multi-GPU trainer (engine/trainer.cpp:779-898) for one lane."""

    def __init__(self, pipe, relay: RelayBuffer, edges_sorted, bucket_sizes, seed: int = 1, bucket_begin=None):
        """edges_sorted: the bucket-sorted training edges on this device (global node ids); bucket_sizes[P * P]: rows of every
        bucket of the graph; bucket_begin[P * P]: first row of each bucket in edges_sorted when the rank holds only the buckets
        it trains (default: the list holds all buckets back to back)."""
        import numpy as np
        import torch

        self.pipe, self.relay = pipe, relay
        self.edges_sorted = edges_sorted
        self.sizes = np.asarray(bucket_sizes, np.int64)
        self.begin = np.concatenate([[0], np.cumsum(self.sizes)])[:-1] if bucket_begin is None else np.asarray(bucket_begin, np.int64)
        P, world = relay.num_partitions, relay.world
        self.supersteps = make_supersteps(P, world)
        self.buckets = state_buckets(self.supersteps, P, self.sizes)
        self.seed = seed
        B = pipe.cfg.B
        self.state_edges_count = [[int(self.sizes[b].sum()) if len(b) else 0 for b in lanes] for lanes in self.buckets]
        cap = max(max(c) for c in self.state_edges_count)
        cap = max(cap, 2 * B)
        dev = edges_sorted.device
        self.state_edges = torch.zeros((cap, edges_sorted.shape[1]), dtype=torch.int64, device=dev)
        self.slot_dev = torch.full((P,), -1, dtype=torch.int64, device=dev)
        self.runners = [None, None]
        self.states_done = 0

    def _runner(self, parity: int):
        """The pipelined step graphs for the tables of buffer `parity` (captured on first use).  Returns (runner, warmed):
        the very first capture of a pipeline runs one host-issued training step (it resolves driver entry points and function
        attributes outside the capture); that step trains a batch of the current state and counts as one of its steps."""
        warmed = False
        if self.runners[parity] is None:
            r = self.relay
            warmed = self.runners[0] is None and self.runners[1] is None
            self.runners[parity] = self.pipe.capture_pipelined(self.state_edges, 1, tables=(r.buf(0, parity), r.buf(1, parity)), warm=warmed)
        return self.runners[parity], warmed

    def run_epoch(self, epoch: int = 0, on_step=None, on_state=None):
        """on_state(k, total): optional callable after the edge list of superstep k is built; on_step(k, i, ids): optional
        callable after step i of superstep k, `ids` being the id set the step trained from (tests replay the step there)."""
        import torch

        from . import capi

        pipe, relay = self.pipe, self.relay
        B = pipe.cfg.B
        for k, lanes in enumerate(self.supersteps):
            relay.swap(lanes)
            mine = self.buckets[k][relay.rank]
            nb = 0
            if lanes[relay.rank] is not None and mine:
                self.slot_dev.copy_(torch.tensor(relay.slot_table(), dtype=torch.int64))
                total = capi.build_state_edges(self.edges_sorted, [int(self.begin[b]) for b in mine], [int(self.sizes[b]) for b in mine],
                                               self.slot_dev, relay.rows, self.state_seed(epoch, k), self.state_edges, pipe.status)
                nb = total // B  # a tail shorter than a batch is left out of this epoch (another tail next epoch: the shuffle differs)
                if on_state is not None:
                    on_state(k, total)
            nb_max = max(c // B for c in self.state_edges_count[k])
            if nb > 0:
                pipe.set_num_batches(nb)
                runner, warmed = self._runner(relay.parity)
                done = 0
                if warmed:
                    done = 1
                    if on_step is not None:
                        on_step(k, 0, pipe.ids[0])
                runner.refill()
                for i in range(done, nb):
                    runner.replay()
                    if on_step is not None:
                        on_step(k, i, pipe.ids[pipe._ids_parity ^ 1])
            if relay.world > 1 and pipe.peer is not None:
                for _ in range(nb_max - nb):
                    pipe.idle_step()
            self.states_done += 1
        relay.flush()

    def state_seed(self, epoch: int, k: int) -> int:
        return self.seed + 7919 * (epoch * len(self.supersteps) + k)
