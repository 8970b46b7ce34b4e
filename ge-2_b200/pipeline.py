"""Per-batch training pipeline on one GPU: the sequence SynchronousTrainer::train runs for every batch
(cpp/src/engine/trainer.cpp:170-211 of the reference project), issued as a fixed list of launches on the current
CUDA stream with no host synchronisation in between:

    sample negatives + pack ids  ->  unique-map  ->  fused decoder forward/loss/backward  ->  sparse Adagrad scatter
    ->  dense Adagrad on the relation tables

Torch tensors are used as device memory only; every arithmetic step is a kernel of libge2_b200.so.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import capi


@dataclass
class PipelineConfig:
    decoder: str            # "DISTMULT" | "COMPLEX" ("DOT" = DISTMULT on 2-column edges)
    B: int                  # batch size
    C: int                  # num_chunks
    N: int                  # negatives_per_positive (per chunk)
    degree_fraction: float  # share of degree-based negatives
    D: int
    R: int                  # number of relations (0/1 => relation-free, 2-column edges)
    domain: int             # nodes resident on the device (rows of the table)
    lr: float = 0.1
    dense_lr: Optional[float] = None
    precision: str = "fp32"
    seed: int = 20260
    inverse: bool = True

    @property
    def has_relations(self):
        return self.R > 1

    @property
    def sides(self):
        return 2 if (self.has_relations and self.inverse) else 1

    @property
    def n_deg(self):
        return int(self.N * self.degree_fraction)  # negative.cpp:945 of the reference project

    @property
    def n_ids(self):
        return 2 * self.B + self.sides * self.C * self.N


class _IdSet:
    """The per-batch id buffers: packed ids, unique map, inverse (and its column slices), device-side count, degree rows,
    relation column.  The pipeline owns two sets so that batch t+1 can be sampled and deduplicated while batch t trains."""

    def __init__(self, cfg: "PipelineConfig", cap: int, dev):
        n_ids, CN, B = cfg.n_ids, cfg.C * cfg.N, cfg.B
        i64 = dict(dtype=torch.int64, device=dev)
        self.packed = torch.empty(n_ids, **i64)
        self.deg_rows = torch.empty((cfg.C, max(cfg.n_deg, 1)), **i64)
        self.unique = torch.empty(cap, **i64)
        self.inverse = torch.empty(n_ids, **i64)
        self.count = torch.zeros(2, dtype=torch.int32, device=dev)
        self.rel_ids = torch.empty(max(B, 1), **i64)  # the batch's relation column, copied by the sampler
        self.loss = torch.zeros(1, dtype=torch.float32, device=dev)  # loss of the batch trained from this set
        self.uws = capi.unique_workspace(cfg.domain, dev)  # one per set: two unique-maps may be in flight at the same time
        self.src_local = self.inverse[0:B]
        self.dst_local = self.inverse[B:2 * B]
        off = 2 * B
        self.src_negs_local = None
        if cfg.sides == 2:
            self.src_negs_local = self.inverse[off:off + CN]
            off += CN
        self.dst_negs_local = self.inverse[off:off + CN]


class PeerGradients:
    """Relation-gradient buffers that every rank of a node can read over NVLink (one process per GPU): the sum over ranks
    and the dense optimizer step then take one launch per rank (ge2_dense_adagrad_peers) instead of a collective call
    between two halves of the step, and the whole multi-GPU step fits in one CUDA graph.  Replaces Model::all_reduce of
    the reference (model.cpp:174-204).  Layout of each rank's buffer: two halves of `numel` floats (the step whose counter
    is t accumulates into half t & 1), then one 8-byte flag per rank, the verdict word and the wait-time counter.

    The buffers are torch symmetric memory: every rank's allocation is mapped into this process's address space with
    access granted to this rank's GPU, which is what a kernel needs to load from it.  (A legacy CUDA IPC import of a
    peer's tensor is mapped in the context of the peer's device and faulted when a kernel of this rank's device read it.)
    No multicast object is bound to the buffers: the kernel uses plain peer loads and stores."""

    def __init__(self, dist, numel: int, device):
        import os

        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        assert numel % 2 == 0, "the flag row behind the two halves must be 8-byte aligned"
        self.rank, self.world, self.numel = dist.get_rank(), dist.get_world_size(), numel
        self.buf = symm_mem.empty(2 * numel + 2 * self.world + 32, dtype=torch.float32, device=device)
        self.buf.zero_()
        torch.cuda.synchronize(device)
        self.handle = symm_mem.rendezvous(self.buf, dist.group.WORLD)  # collective; keeps the peers' mappings alive
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.buf.data_ptr():
            raise RuntimeError("symmetric memory rendezvous returned an unexpected set of buffers")
        dist.barrier()  # every rank has zeroed and mapped every buffer before anybody launches on them
        torch.cuda.synchronize(device)

    def half(self, parity: int):
        return self.buf[parity * self.numel:(parity + 1) * self.numel]

    def waited_ns(self) -> int:
        """nanoseconds this rank's announcing kernels have spent waiting for the slowest rank so far (synchronises)"""
        return int(self.buf[2 * self.numel:2 * self.numel + 2 * self.world + 4].view(torch.int64)[self.world + 1].item())


class BatchPipeline:
    """Owns the per-batch scratch (ids, unique map, gradients, workspaces); tables are owned by the caller."""

    def __init__(self, cfg: PipelineConfig, table, state, rel=None, rel_state=None, inv_rel=None, inv_rel_state=None):
        capi.load_library()
        self.cfg = cfg
        dev = table.device
        self.device = dev
        self.table, self.state = table, state
        self.rel, self.rel_state, self.inv_rel, self.inv_rel_state = rel, rel_state, inv_rel, inv_rel_state
        assert table.is_cuda and table.dtype == torch.float32 and table.shape[1] == cfg.D and table.is_contiguous()
        n_ids, CN = cfg.n_ids, cfg.C * cfg.N
        self.cap = min(n_ids, cfg.domain)
        self.ids = [_IdSet(cfg, self.cap, dev), _IdSet(cfg, self.cap, dev)]
        first = self.ids[0]  # the non-pipelined forms use the first set only; its buffers keep their plain names
        self.packed, self.deg_rows, self.unique, self.inverse, self.count, self.rel_ids = (
            first.packed, first.deg_rows, first.unique, first.inverse, first.count, first.rel_ids)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.node_grad = torch.zeros((self.cap, cfg.D), dtype=torch.float32, device=dev)
        self.loss = first.loss
        self.uws = first.uws
        if cfg.has_relations:
            # one contiguous buffer for both relation-gradient tables: a single all-reduce serves them in the multi-GPU trainer
            self.rel_grads = torch.zeros((cfg.sides,) + tuple(rel.shape), dtype=rel.dtype, device=dev)
            self.rel_grad = self.rel_grads[0]
            self.inv_rel_grad = self.rel_grads[1] if cfg.sides == 2 else None
            # when the caller keeps the two relation tables (and their states) back to back in one allocation, the dense
            # optimizer step is one launch over both
            self._rel_tables_adjacent = False
            if cfg.sides == 2 and rel.is_contiguous() and inv_rel.is_contiguous() and rel_state.is_contiguous() and inv_rel_state.is_contiguous():
                n = rel.numel()
                adj = lambda a, b: (b.data_ptr() == a.data_ptr() + n * a.element_size()
                                    and a.untyped_storage().data_ptr() == b.untyped_storage().data_ptr())
                if adj(rel, inv_rel) and adj(rel_state, inv_rel_state):
                    both = lambda a: torch.as_strided(a, (2,) + tuple(a.shape), (n,) + tuple(a.stride()))
                    self._rel_both, self._rel_state_both = both(rel), both(rel_state)
                    self._rel_tables_adjacent = True
        else:
            self.rel_grad = self.inv_rel_grad = None
            self._rel_tables_adjacent = False
        # device-side batch counters of the graph-replay forms: {t, t + 1}
        self.step_dev = torch.tensor([0, 1], dtype=torch.int64, device=dev)
        self._graph = None
        self._desc = None
        self._ws = None
        self.grad_scale = 1.0  # 1 / #GPUs when relation gradients are all-reduced (model.cpp:188-192 of the reference project)
        self.peer: Optional[PeerGradients] = None
        self._t_host = 0       # host mirror of step_dev[0]; only the peer-gradient form needs it (which half a step writes)
        # number of batches of the resident edge list, on the device: a partition-buffer state replaces the list by one of
        # another length without the captured launches changing (set_num_batches); None = the host-side count is used
        self.nb_dev = None
        self._ids_parity = 0   # which id set holds the batch drawn ahead (shared by every pipelined runner of this pipeline)

    def set_num_batches(self, num_batches: int):
        """Stream-ordered update of the device-side batch count used by the resident / pipelined forms."""
        if self.nb_dev is None:
            self.nb_dev = torch.zeros(1, dtype=torch.int64, device=self.device)
        self.nb_dev.fill_(max(1, int(num_batches)))

    def _sample(self, ids: "_IdSet", edges_all, num_batches: int, counter):
        cfg = self.cfg
        args = (cfg.B, cfg.C, cfg.N, cfg.n_deg, cfg.domain, cfg.sides == 2, cfg.seed, ids.packed, ids.deg_rows if cfg.n_deg > 0 else None,
                ids.rel_ids if cfg.has_relations else None)
        if self.nb_dev is not None:
            capi.sample_batch_dev(edges_all, self.nb_dev, counter, *args)
        else:
            capi.sample_batch(edges_all, num_batches, counter, *args)

    def use_peer_gradients(self, peer: PeerGradients):
        """Multi-GPU: relation gradients go into `peer`'s buffer (alternating halves) and the dense optimizer step sums them
        over the ranks itself.  Supported by enqueue_resident and capture_pipelined; needs the relation tables (and their
        states) back to back when there are two."""
        cfg = self.cfg
        assert cfg.has_relations and (cfg.sides == 1 or self._rel_tables_adjacent)
        assert peer.numel == cfg.sides * self.rel.numel()
        self.peer = peer
        self.grad_scale = 1.0 / peer.world
        self._t_host = int(self.step_dev[0].item())
        self._peer_views = [peer.half(h).view((cfg.sides,) + tuple(self.rel.shape)) for h in (0, 1)]

    def _make_desc(self, edges, rel_ids=None, rel_stride=None, ids: Optional[_IdSet] = None, parity: Optional[int] = None):
        cfg = self.cfg
        ids = ids or self.ids[0]
        rel_grad, inv_rel_grad = self.rel_grad, self.inv_rel_grad
        if self.peer is not None:
            view = self._peer_views[(self._t_host if parity is None else parity) & 1]
            rel_grad, inv_rel_grad = view[0], (view[1] if cfg.sides == 2 else None)
        cols = edges.shape[1]
        if rel_ids is None and cfg.has_relations:
            rel_ids, rel_stride = edges[:, 1], cols
        d = capi.make_lp_desc(
            decoder=cfg.decoder, precision=cfg.precision, B=cfg.B, Cn=cfg.C, N=cfg.N, D=cfg.D, R=cfg.R if cfg.has_relations else 0,
            U=self.cap, node_emb=self.table, row_index=ids.unique, emb_stride=cfg.D, src_ids=ids.src_local, dst_ids=ids.dst_local,
            rel_ids=rel_ids if cfg.has_relations else None, edge_stride=1, rel_stride=rel_stride or 1, dst_negs=ids.dst_negs_local,
            src_negs=ids.src_negs_local, deg_sample_rows=ids.deg_rows if cfg.n_deg > 0 else None, n_deg=cfg.n_deg,
            rel=self.rel, inv_rel=self.inv_rel if cfg.sides == 2 else None, node_grad=self.node_grad, rel_grad=rel_grad,
            inv_rel_grad=inv_rel_grad, loss=ids.loss, status=self.status, node_grad_is_zero=True)
        if self._ws is None:
            self._ws = torch.empty(capi.lp_workspace_bytes(d), dtype=torch.uint8, device=self.device)
        d.workspace, d.workspace_bytes = self._ws.data_ptr(), self._ws.numel()
        return d

    def step(self, edges, batch_index: int, scores_events=None, rel_hook=None):
        """edges: [B, 2|3] int64 device tensor with resident-table row ids (global ids, or buffer-local ids with a
        partition buffer).  Enqueues one training step; returns nothing (loss stays in self.loss).
        scores_events: optional (start, end) torch.cuda.Event pair recorded around the scores kernel alone.
        rel_hook: optional callable run after the backward pass and before the dense optimizer step (the multi-GPU
        trainer all-reduces the relation gradients there, Model::all_reduce of the reference)."""
        cfg = self.cfg
        cols = edges.shape[1]
        assert edges.shape[0] == cfg.B and edges.dtype == torch.int64 and edges.is_contiguous()
        capi.sample_negatives(edges, edges[:, cols - 1], cols, cfg.B, cfg.C, cfg.N, cfg.n_deg, cfg.domain, cfg.sides == 2, cfg.seed,
                              batch_index, self.packed, self.deg_rows if cfg.n_deg > 0 else None)
        capi.unique_bitmap(self.packed, cfg.domain, workspace=self.uws, out_unique=self.unique, out_inverse=self.inverse, out_count=self.count)
        self._backward_and_update(self._make_desc(edges), scores_events, rel_hook)

    def _backward_and_update(self, desc, scores_events=None, rel_hook=None):
        self._backward(desc, scores_events)
        if rel_hook is not None:
            rel_hook(self)
        self._update()

    def _backward(self, desc, scores_events=None):
        if scores_events is None:
            capi.lp_step(desc)
        else:  # same kernels, issued phase by phase so the scores kernel can be bracketed by events
            desc.phases = 1
            capi.lp_step(desc)
            desc.phases = 2
            scores_events[0].record()
            capi.lp_step(desc)
            scores_events[1].record()
            desc.phases = 4
            capi.lp_step(desc)

    def time_scores_phase(self, edges_all, reps: int = 20, phases: int = 2) -> float:
        """Milliseconds per scores phase (the clearing of dK plus the scores launches) as it runs inside a replayed graph:
        `reps` phases captured back to back on the operands the last step left in the workspace, bracketed by events.
        Host-issued launches of the same phase carry a few microseconds of launch gaps that a graph replay does not have.
        (phases: 1 = prepare, 2 = scores, 4 = finish, as in ge2_lp_desc.)"""
        desc = self._make_desc(edges_all, self.ids[0].rel_ids, 1)
        desc.phases = phases
        capi.lp_step(desc)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                capi.lp_step(desc)
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize(self.device)
        desc.phases = 0
        return a.elapsed_time(b) / reps

    def _update(self, ids: Optional[_IdSet] = None):
        self._update_nodes(ids)
        self._update_relations()

    def _update_nodes(self, ids: Optional[_IdSet] = None):
        cfg = self.cfg
        ids = ids or self.ids[0]
        # clear_grad: the rows just consumed are zeroed in the same pass, so the next step needs no memset of the gradient buffer
        capi.adagrad_scatter(self.table, self.state, ids.unique, self.node_grad, cfg.lr, U=self.cap, U_dev=ids.count, clear_grad=True,
                             status=self.status)

    def _update_relations(self):
        cfg = self.cfg
        if cfg.has_relations:
            dl = cfg.lr if cfg.dense_lr is None else cfg.dense_lr
            if self.peer is not None:
                # sum over the ranks' gradient buffers + Adagrad on both tables + clearing of the other half, one launch
                both = cfg.sides == 2
                capi.dense_adagrad_peers(self._rel_both if both else self.rel, self._rel_state_both if both else self.rel_state, self.peer.ptrs,
                                         self.peer.rank, self.peer.numel, self.step_dev, dl, self.status, grad_scale=self.grad_scale)
                return
            if cfg.sides == 2 and self._rel_tables_adjacent:
                # relation and inverse-relation tables (and their states) sit back to back, as the gradients do: one launch
                capi.dense_adagrad(self._rel_both, self._rel_state_both, self.rel_grads, dl, grad_scale=self.grad_scale, clear_grad=True)
                return
            capi.dense_adagrad(self.rel, self.rel_state, self.rel_grad, dl, grad_scale=self.grad_scale, clear_grad=True)
            if cfg.sides == 2:
                capi.dense_adagrad(self.inv_rel, self.inv_rel_state, self.inv_rel_grad, dl, grad_scale=self.grad_scale, clear_grad=True)

    # ---- graph-replay form: the whole step is a fixed launch list that reads its batch index from device memory ----------
    def enqueue_resident(self, edges_all, num_batches: int, scores_events=None, rel_hook=None):
        """One training step on batch (*step_dev % num_batches) of the resident edge list edges_all[num_batches * B, cols];
        advances the device-side counter at the end.  No argument changes from step to step, so the launch list can be
        captured once into a CUDA graph (capture_resident) and replayed."""
        cfg = self.cfg
        self._sample(self.ids[0], edges_all, num_batches, self.step_dev)
        capi.unique_bitmap(self.packed, cfg.domain, workspace=self.uws, out_unique=self.unique, out_inverse=self.inverse, out_count=self.count)
        self._backward_and_update(self._make_desc(edges_all, self.rel_ids, 1), scores_events, rel_hook)
        capi.advance_step(self.step_dev, 2)
        self._t_host += 1
        self._ids_parity = self._t_host & 1  # (a pipelined runner used after this needs refill(): nothing is drawn ahead)

    def capture_resident(self, edges_all, num_batches: int, rel_hook=None):
        """Captures one resident step into a CUDA graph (after one eager step, which also resolves driver entry points and
        function attributes outside the capture).  replay() then costs a single graph launch per step."""
        assert self.peer is None, "the peer-gradient form needs the alternating graphs of capture_pipelined"
        self.enqueue_resident(edges_all, num_batches, rel_hook=rel_hook)
        torch.cuda.synchronize(self.device)
        self._graph_edges = edges_all  # keep the captured pointers alive
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.enqueue_resident(edges_all, num_batches, rel_hook=rel_hook)
        self._graph = g
        return g

    def capture_resident_split(self, edges_all, num_batches: int, rel_hook):
        """Multi-GPU form: the step is captured as two graphs with the relation-gradient all-reduce (rel_hook, a host-issued
        NCCL call) between them -- sample/unique/forward/backward, then the optimizer updates and the counter bump."""
        self.enqueue_resident(edges_all, num_batches, rel_hook=rel_hook)
        torch.cuda.synchronize(self.device)
        self._graph_edges = edges_all
        cfg = self.cfg
        ga, gb = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(ga):
            capi.sample_batch(edges_all, num_batches, self.step_dev, cfg.B, cfg.C, cfg.N, cfg.n_deg, cfg.domain, cfg.sides == 2, cfg.seed,
                              self.packed, self.deg_rows if cfg.n_deg > 0 else None, self.rel_ids if cfg.has_relations else None)
            capi.unique_bitmap(self.packed, cfg.domain, workspace=self.uws, out_unique=self.unique, out_inverse=self.inverse,
                               out_count=self.count)
            self._backward(self._make_desc(edges_all, self.rel_ids, 1))
        with torch.cuda.graph(gb):
            self._update()
            capi.advance_step(self.step_dev, 2)

        class _Split:
            def replay(_self):
                ga.replay()
                rel_hook(self)
                gb.replay()

        self._split = (ga, gb)
        return _Split()

    # ---- pipelined form: batch t+1 is sampled and deduplicated on a side stream while batch t trains -----------------
    def _front(self, ids: _IdSet, edges_all, num_batches: int, counter):
        """sampler + unique-map into one id set; `counter` is the device counter holding the batch number to use"""
        cfg = self.cfg
        self._sample(ids, edges_all, num_batches, counter)
        capi.unique_bitmap(ids.packed, cfg.domain, workspace=ids.uws, out_unique=ids.unique, out_inverse=ids.inverse, out_count=ids.count)

    def idle_step(self):
        """A step of a lane that has no batch (lanes of a superstep have unequal batch counts): the relation-gradient
        exchange alone -- this rank's half of the gradient buffer is zero, so it contributes zeros, as the reference's
        zero-filled gradients do (model.cpp:182-187) -- and the counter bump, so that the replicas of the relation tables
        stay in step with the ranks that train."""
        self._update_relations()
        capi.advance_step(self.step_dev, 2)
        self._t_host += 1
        self._ids_parity = self._t_host & 1

    def capture_pipelined(self, edges_all, num_batches: int, rel_hook=None, front_after_scores: bool = True, tables=None, warm: bool = True):
        """tables: (table, state) to capture the graphs for, when not the pipeline's own -- a partition buffer that alternates
        between two active buffers keeps one runner per buffer; runners of one pipeline are interchangeable from step to
        step (they share the id sets, the counters and the rule "the step whose counter is t uses id set t & 1").
        warm = False skips the host-issued warm-up step (a later capture of a pipeline that has run already).

        Software-pipelined steps: while the decoder step of batch t runs (its scores kernel leaves most SMs idle in its
        second round), the ids of batch t+1 are drawn and deduplicated on a side stream into the other id set; the optimizer
        updates of batch t follow the join, so batch t+1 gathers the updated rows.  Two graphs alternate (one per id set);
        with rel_hook (the multi-GPU all-reduce, host-issued) each step is two graph launches around the hook.
        Returns an object with replay().  The same batches, negatives and arithmetic as the plain resident form."""
        own_tables = (self.table, self.state)
        if tables is not None:
            self.table, self.state = tables
        if warm:
            self.enqueue_resident(edges_all, num_batches, rel_hook=rel_hook)  # warm-up: driver entry points, function attributes
        torch.cuda.synchronize(self.device)
        self._graph_edges = edges_all
        cfg = self.cfg
        ctr_now, ctr_next = self.step_dev[0:1], self.step_dev[1:2]
        self._ids_parity = self._t_host & 1
        self._front(self.ids[self._ids_parity], edges_all, num_batches, ctr_now)  # ids of the first pipelined batch
        torch.cuda.synchronize(self.device)
        # Side streams are made once, outside any capture, and nothing is destroyed while a capture is open (a stream,
        # graph or tensor of an earlier capture dying inside a later one invalidates it): no garbage collection meanwhile.
        import gc

        if getattr(self, "_side_streams", None) is None:
            self._side_streams = (torch.cuda.Stream(device=self.device), torch.cuda.Stream(device=self.device))
        self._make_desc(edges_all, self.ids[0].rel_ids, 1)  # sizes the workspace before the capture
        gc.collect()
        gc_was_on = gc.isenabled()
        gc.disable()
        try:
            graphs = []
            if self.peer is not None:
                assert rel_hook is None and self._t_host == int(self.step_dev[0].item())
            for p in (0, 1):
                cur, nxt = self.ids[p], self.ids[1 - p]
                ga = torch.cuda.CUDAGraph()
                with torch.cuda.graph(ga):
                    main = torch.cuda.current_stream()
                    side, side2 = self._side_streams
                    # graph p trains the steps whose counter has parity p: id set p, half p of the peer gradient buffer
                    desc = self._make_desc(edges_all, cur.rel_ids, 1, ids=cur, parity=p)
                    if front_after_scores:
                        # The scores kernel owns whole SMs (one CTA with all of its shared memory); the small kernels of the next
                        # batch's sampler and unique-map would delay its CTAs, so they are forked after it and run beside the
                        # scatter and the optimizer updates, which leave room on every SM.
                        desc.phases = 3
                        capi.lp_step(desc)
                        side.wait_stream(main)
                        with torch.cuda.stream(side):
                            self._front(nxt, edges_all, num_batches, ctr_next)
                        desc.phases = 4
                        capi.lp_step(desc)
                        desc.phases = 0
                    else:
                        side.wait_stream(main)
                        with torch.cuda.stream(side):
                            self._front(nxt, edges_all, num_batches, ctr_next)
                        self._backward(desc)
                        main.wait_stream(side)
                    if rel_hook is None:
                        # the two optimizer updates touch different tables: the dense one (with its wait for the other ranks'
                        # gradients in the multi-GPU form) runs beside the sparse scatter
                        side2.wait_stream(main)
                        with torch.cuda.stream(side2):
                            self._update_relations()
                        self._update_nodes(cur)
                        main.wait_stream(side2)
                        main.wait_stream(side)
                        capi.advance_step(self.step_dev, 2)
                    if rel_hook is not None and front_after_scores:
                        main.wait_stream(side)
                gb = None
                if rel_hook is not None:
                    gb = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gb):
                        self._update(cur)
                        capi.advance_step(self.step_dev, 2)
                graphs.append((ga, gb))
        finally:
            if gc_was_on:
                gc.enable()
            self.table, self.state = own_tables
        pipe = self

        class _Pipelined:
            def replay(_self):
                ga, gb = graphs[pipe._ids_parity]
                ga.replay()
                if gb is not None:
                    rel_hook(pipe)
                    gb.replay()
                pipe._ids_parity ^= 1
                pipe._t_host += 1

            @property
            def loss(_self):
                """device scalar holding the loss of the batch trained by the last replay"""
                return pipe.ids[pipe._ids_parity ^ 1].loss

            def refill(_self):
                """Draws the ids of the coming batch again (host-issued): call after the resident edge list was replaced,
                e.g. at a partition swap, since the batch sampled ahead came from the old list."""
                pipe._front(pipe.ids[pipe._ids_parity], edges_all, num_batches, ctr_now)

        self._pipelined = graphs
        return _Pipelined()

    def replay(self):
        self._graph.replay()

    def launches_per_step(self, resident: bool = True) -> int:
        """Kernels of libge2_b200.so launched per step (memsets not counted)."""
        cfg = self.cfg
        n = 1 + 3                              # sampler; unique-map: mark, scan, inverse
        n += 1                                 # prepare (gather + relation operator + positive scores + filter words)
        n += 2 if cfg.precision == "f16" else 1  # scores: logsumexp pass + gradient pass (persistent launches), or the fp32 kernel
        n += 1                                 # finish (operator backward + scatter)
        n += 1                                 # sparse Adagrad scatter
        if cfg.has_relations:
            n += 1 if (cfg.sides == 1 or self._rel_tables_adjacent) else 2
        return n + (1 if resident else 0)      # device-side counter bump of the resident / graph forms

    def check_status(self):
        """Synchronises and raises if any kernel flagged bad data (call between epochs, not per batch)."""
        torch.cuda.synchronize(self.device)
        word = int(self.status.item()) | int(self.ids[0].count[1].item()) | int(self.ids[1].count[1].item())
        if word:
            raise capi.Ge2Error("device status: " + capi.decode_status(word))


class HostFeed:
    """Trains batches that arrive in pinned host memory through the pipelined graphs, with the copies off the critical path.

    start(batch0, batch1) trains batch0 (host-issued, also the warm-up the capture needs) and draws the ids of batch1;
    every later step(next_batch, loss_out) trains the batch drawn ahead while, on a side stream, next_batch is drawn.
    The host-to-device copy of next_batch runs on its own stream during the previous step; the 4-byte loss read-back runs on
    a third stream.  Each loss slot and each staging slot is reused every second step; events order the reuse.
    Batches are trained exactly once, in the order given, with the same sampler counters as the resident forms."""

    def __init__(self, pipe: BatchPipeline, cols: int, rel_hook=None):
        self.pipe, self.rel_hook = pipe, rel_hook
        dev = pipe.device
        self.stage = torch.empty((2, pipe.cfg.B, cols), dtype=torch.int64, device=dev)
        self.h2d, self.d2h = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        self.copied = [torch.cuda.Event() for _ in range(2)]
        self.done = [torch.cuda.Event() for _ in range(2)]
        self.read = [torch.cuda.Event() for _ in range(2)]
        self.runner, self.j = None, 0

    def start(self, batch0, batch1, tables=None):
        """tables: (table, state) to train, when not the pipeline's own (a partition buffer's current pair)"""
        pipe = self.pipe
        c = int(pipe.step_dev[0].item())
        self.stage[c % 2].copy_(batch0)
        self.stage[(c + 1) % 2].copy_(batch1)
        self.slot0 = c + 2
        self.runner = pipe.capture_pipelined(self.stage.view(2 * pipe.cfg.B, -1), 2, rel_hook=self.rel_hook, tables=tables)
        torch.cuda.synchronize(pipe.device)
        self.j = 0

    def step(self, next_batch, loss_out=None):
        """next_batch: pinned host tensor [B, cols] (the batch after the one trained by this call);
        loss_out: pinned host tensor of one float receiving this step's loss (valid after a synchronize)."""
        j, main = self.j, torch.cuda.current_stream()
        k = j % 2
        if j >= 2:
            self.h2d.wait_event(self.done[k])  # the sampler of step j-2 was the last reader of this staging slot
        with torch.cuda.stream(self.h2d):
            self.stage[(self.slot0 + j) % 2].copy_(next_batch, non_blocking=True)
            self.copied[k].record()
        main.wait_event(self.copied[k])
        if j >= 2 and loss_out is not None:
            main.wait_event(self.read[k])      # this step overwrites the loss slot read back two steps ago
        self.runner.replay()
        self.done[k].record()
        if loss_out is not None:
            self.d2h.wait_event(self.done[k])
            with torch.cuda.stream(self.d2h):
                loss_out.copy_(self.runner.loss, non_blocking=True)
                self.read[k].record()
        self.j = j + 1

    def drain(self):
        """makes the current stream wait for the loss read-backs still in flight (call before timing stops or before reading them)"""
        torch.cuda.current_stream().wait_stream(self.d2h)

    def refill(self):
        self.runner.refill()
