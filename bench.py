#!/usr/bin/env python
"""Benchmark of the per-batch embedding-training path: train edges/sec.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--precision fp32|f16]

A step is one batch (unique-map -> fused decoder forward/loss/backward -> sparse Adagrad scatter -> dense Adagrad
on the relation tables) of the single-GPU configuration: synthetic knowledge graph with 1,000,000 entities,
1,000 relations, 20,000,000 triples (Zipf 1.1 degrees, Zipf 1.2 relations), ComplEx d=100 fp32, batch 10,000,
1,000 negatives per chunk of 10 (half degree-proportional, half uniform), softmax loss, Adagrad lr 0.1.
With N > 1 every rank trains its own partition-disjoint share of the edges at the same per-GPU batch (weak scaling)
and the relation gradients are all-reduced over NCCL each step.  Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for _p in (ROOT, ROOT / "tests", ROOT / "oracle", ROOT / "oracle" / "_ref"):
    if str(_p) not in sys.path:
        sys.path.insert(0, str(_p))

import numpy as np  # noqa: E402
import torch  # noqa: E402

CFG = dict(name="kg-1M-entities/1k-relations/20M-triples ComplEx d=100 B=10000 neg=10x1000 (50% degree)", nodes=1_000_000, relations=1000,
           triples=20_000_000, decoder="COMPLEX", D=100, B=10_000, C=10, N=1000, degree_fraction=0.5, lr=0.1, alpha_nodes=1.1, alpha_rel=1.2)


# dram__bytes_read.sum + dram__bytes_write.sum of the scores launches of one step on this workload, taken from one ncu
# capture of those launches (operands and partial gradients stay in the 126 MB L2, so it is far below the operand bytes)
NCU_TRAFFIC = {"f16": 22_407_168, "fp32": None}
REPEATS = 9  # the K-step timed region is run this many times; `value` is total steps over total time, the spread is reported


def peaks():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        j = json.loads(f.read_text())
        return dict(hbm=float(j["hbm_gbs"]), tf=float(j["bf16_tflops"]), tf_sustained=float(j.get("bf16_tflops_sustained", j["bf16_tflops"])), src="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, src="fallback")


def zipf_sample_torch(n, domain, alpha, gen, device):
    """ids in [0, domain) with P(rank k) ~ k^-alpha through an inverse-CDF lookup, ranks scattered by a random relabel
    (the preprocessor of the reference project assigns random ids, torch_converter.py:258-261)."""
    w = torch.arange(1, domain + 1, dtype=torch.float64, device=device).pow_(-alpha)
    cdf = torch.cumsum(w, 0)
    cdf /= cdf[-1].clone()
    u = torch.rand(n, dtype=torch.float64, device=device, generator=gen)
    ranks = torch.searchsorted(cdf, u).clamp_(max=domain - 1)
    perm = torch.randperm(domain, device=device, generator=gen)
    return perm[ranks]


def make_graph(cfg, n_edges, seed, device):
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    src = zipf_sample_torch(n_edges, cfg["nodes"], cfg["alpha_nodes"], gen, device)
    dst = zipf_sample_torch(n_edges, cfg["nodes"], cfg["alpha_nodes"], gen, device)
    rel = zipf_sample_torch(n_edges, cfg["relations"], cfg["alpha_rel"], gen, device)
    return torch.stack([src, rel, dst], dim=1).contiguous()


class ClockSampler:
    """Samples SM clocks and clock-event (throttle) reasons while the timed region runs: read-only NVML queries every 2 ms
    from a thread (the timed regions last tens of milliseconds, too short for nvidia-smi's loop), nvidia-smi as fall-back."""
    Q = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    # NVML clock-event reason bits (nvml.h): hw slowdown 0x8, sw thermal 0x20, hw thermal 0x40, sw power cap 0x4
    BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, gpu_index):
        self.idx = gpu_index
        self.proc = None
        self.lines = []
        self.nvml = None
        self.samples = []  # (sm MHz, reasons bitmask)
        self.stop_flag = False

    def _phys_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            parts = [x for x in vis.split(",") if x.strip()]
            if self.idx < len(parts) and parts[self.idx].strip().isdigit():
                return int(parts[self.idx])
        return self.idx

    def start(self):
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self._phys_index())
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.t = threading.Thread(target=self._poll, daemon=True)
            self.t.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self._phys_index())],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _poll(self):
        nv = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    bits = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, bits))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.t.join(timeout=1)
            if not self.samples:
                return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
            reasons = sorted({name for _, bits in self.samples for name, bit in self.BITS if bits & bit})
            return dict(sm_mhz=float(np.median([m for m, _ in self.samples])), sm_max_mhz=self.max_mhz, reasons=reasons,
                        samples=len(self.samples), source="nvml, 2 ms period")
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for ln in self.lines:
            p = [x.strip() for x in ln.split(",")]
            if len(p) < 9:
                continue
            try:
                sm.append(float(p[1]))
                mx.append(float(p[2]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples"])
        return dict(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm), source="nvidia-smi")


# ----------------------------------------------------------------------------------------------------------------
# CPU reference arm: the reference project's own CPU code for the path (oracle/_ref), else the numpy restatement
# ----------------------------------------------------------------------------------------------------------------
class CpuReference:
    def __init__(self, cfg, seed):
        self.cfg = cfg
        self.cores = os.cpu_count() or 1
        torch.set_num_threads(self.cores)
        try:
            import gege_ref  # the reference's CPU sources compiled by oracle/Makefile

            self.ref = gege_ref
            self.kind = "reference"
        except Exception:
            self.ref = None
            self.kind = "port"
        g = torch.Generator().manual_seed(seed)
        n, D, R = cfg["nodes"], cfg["D"], cfg["relations"]
        self.table = (torch.rand((n, D), generator=g) - 0.5) * 0.2
        self.state = torch.zeros((n, D))
        self.edges = make_graph(cfg, 64 * cfg["B"], seed, torch.device("cpu"))
        if self.ref is not None:
            self.model = self.ref.RefModel(cfg["decoder"], R, D, True, cfg["lr"], cfg["lr"])
        else:
            import ge2_oracle as O

            self.O = O
            self.rel = np.zeros((R, D), np.float32)
            self.rel[:, : D // 2] = 1
            self.inv = self.rel.copy()
            self.rs, self.iss = np.zeros_like(self.rel), np.zeros_like(self.rel)
        self.gen = g

    def step(self, i):
        """One batch of SynchronousTrainer's loop on CPU: sample, map_tensors, indexRead, train_batch, indexAdd."""
        cfg = self.cfg
        B, C, N, n = cfg["B"], cfg["C"], cfg["N"], cfg["nodes"]
        nd = int(N * cfg["degree_fraction"])
        e = self.edges[(i % 64) * B:(i % 64 + 1) * B]
        uni = torch.randint(n, (C, N - nd), generator=self.gen)
        rows = torch.randint(0, B, (C, nd), generator=self.gen)
        dst_negs = torch.cat([e[:, 2][rows], uni], 1)
        src_negs = torch.cat([e[:, 0][rows], uni], 1)
        if self.ref is not None:
            filt = self.ref.deg_negative_local_filter(rows, e)
            # map_tensors: the reference's CPU unique (util.cpp:100-111) passes (return_inverse=false, return_counts=true) to
            # unique_consecutive and throws with this torch; torch.unique(sorted, return_inverse) is what it evidently means
            ids = torch.cat([e[:, 0], e[:, 2], src_negs.reshape(-1), dst_negs.reshape(-1)])
            uniq, inv = torch.unique(ids, sorted=True, return_inverse=True)
            local = torch.stack([inv[:B], e[:, 1], inv[B:2 * B]], 1)
            sl = inv[2 * B:2 * B + C * N].reshape(C, N)
            dl = inv[2 * B + C * N:].reshape(C, N)
            emb, st = self.table.index_select(0, uniq), self.state.index_select(0, uniq)
            out = self.model.train_batch(local, emb, st, dl, sl, filt, filt, True, False)
            self.table.index_add_(0, uniq, out["node_update"])
            self.state.index_add_(0, uniq, out["node_state_update"])
            return float(out["loss"])
        filt = self.O.deg_negative_local_filter(rows.numpy(), B)
        loss, _ = self.O.train_step(cfg["decoder"], self.table.numpy(), self.state.numpy(), self.rel, self.rs, self.inv, self.iss, e.numpy(),
                                    dst_negs.numpy(), src_negs.numpy(), filt, filt, cfg["lr"], n)
        return loss

    def timed(self, budget_s, min_steps=2, max_steps=40, warm=1):
        for w in range(warm):
            self.step(w)
        t0 = time.perf_counter()
        k = 0
        while k < max_steps and (k < min_steps or time.perf_counter() - t0 < budget_s):
            self.step(warm + k)
            k += 1
        dt = time.perf_counter() - t0
        return k * self.cfg["B"] / dt, k, dt


def reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = CFG
    cpu = CpuReference(cfg, 20262)
    for w in range(min(args.warmup, 2)):
        cpu.step(w)
    t0 = time.perf_counter()
    cpu.step(100)
    t1 = time.perf_counter() - t0
    steps_run = max(1, min(args.steps, int(200.0 / max(t1, 1e-3))))
    t0 = time.perf_counter()
    for k in range(steps_run):
        cpu.step(200 + k)
    dt = time.perf_counter() - t0
    value = steps_run * cfg["B"] / dt
    sample = f"{steps_run} batches of {cfg['B']} edges of the same workload on CPU ({cpu.kind}: " + (
        "reference C++/libtorch decoder+loss+autograd+accumulateGradients, torch.unique for its broken CPU map_tensors" if cpu.kind == "reference" else "numpy restatement") + ")"
    line = dict(metric="train edges/sec/box", value=value, unit="edges/s", n_gpus=args.gpus, steps=args.steps, warmup=args.warmup,
                ms_per_step=1e3 * dt / steps_run, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32", data="synthetic",
                impl="reference", config=dict(workload=cfg["name"], steps_run=steps_run),
                cpu_baseline=dict(value=value, unit="edges/s", cores=cpu.cores, kind=cpu.kind, sample=sample),
                e2e=dict(value=value, unit="edges/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0))
    print(json.dumps(line), flush=True)


def reference_gpu_ms(cfg, table, state, edges, steps, device):
    """The reference project's OWN GPU code on this GPU and workload (test infrastructure, never the product path):
    oracle/_ref/gege_ref_cuda.so is its sources compiled with -DGEGE_CUDA for sm_100 -- its bitmap unique-map
    (unique_map_cuda.cu:771-882), its DEG filter (negative.cpp:215-263), its decoder / loss / autograd / optimizer steps in the
    order of Model::train_batch (model.cpp:362-404) -- around the ATen calls its dataloader and storage make per batch
    (randint negatives negative.cpp:104-169, index_select storage.cpp:1173-1184, index_add_ storage.cpp:1186-1259).
    Its trainer loop, config system and batch queue are not run, so host-side overheads of the reference are missing
    here: the figure flatters the reference."""
    os.environ.setdefault("GEGE_UNIQUE_BACKEND", "bitmap")
    for k in ("GEGE_CSR_GATHER", "GEGE_CSR_DEBUG", "GEGE_STAGE_DEBUG"):
        os.environ.setdefault(k, "0")
    import gege_ref_cuda as G

    B, C, N, D, n, R = cfg["B"], cfg["C"], cfg["N"], cfg["D"], cfg["nodes"], cfg["relations"]
    nd = int(N * cfg["degree_fraction"])
    model = G.RefModel(cfg["decoder"], R, D, True, cfg["lr"], cfg["lr"], str(device))
    tab, st = table.clone(), state.clone()

    def one(i):
        e = edges[i * B:(i + 1) * B]
        uni = torch.randint(n, (C, N - nd), device=device)
        rows = torch.randint(0, B, (C, nd), device=device)
        dneg, sneg = torch.cat([e[:, 2][rows], uni], 1), torch.cat([e[:, 0][rows], uni], 1)
        filt = G.deg_negative_local_filter(rows, e)
        ids = torch.cat([e[:, 0], e[:, 2], sneg.reshape(-1), dneg.reshape(-1)])
        uniq, inv, _ = G.unique_inverse_cuda(ids, False, n)
        local = torch.stack([inv[:B], e[:, 1], inv[B:2 * B]], 1)
        sl, dl = inv[2 * B:2 * B + C * N].reshape(C, N), inv[2 * B + C * N:].reshape(C, N)
        out = model.train_batch(local, tab.index_select(0, uniq), st.index_select(0, uniq), dl, sl, filt, filt, True, False)
        tab.index_add_(0, uniq, out["node_update"])
        st.index_add_(0, uniq, out["node_state_update"])

    for i in range(3):
        one(i)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for i in range(steps):
        one(3 + i)
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


# ----------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--precision", default=os.environ.get("GE2_PRECISION", "f16"), choices=["fp32", "f16"],
                    help="f16: tcgen05 fp16-operand tiles with fp32 accumulation (1e-2 parity, the designed path); fp32: CUDA-core path (1e-4 parity)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fp32-path", action="store_true", help="skip the side measurement of the fp32 CUDA-core path")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip timing the reference's own GPU code (oracle/_ref/gege_ref_cuda.so) on this GPU")
    ap.add_argument("--steps-per-state", type=int, default=0,
                    help="N > 1: training steps between partition swaps; 0 = what the workload's schedule gives: its triples spread over "
                         "(4N)^2 edge buckets, 16 buckets per state, one batch per step")
    ap.add_argument("--no-epoch", action="store_true", help="N = 1: skip the one-epoch (triples / B steps) timed region")
    ap.add_argument("--no-graph", action="store_true", help="issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--nccl-swaps", action="store_true", help="N > 1: move partitions between ranks with NCCL send/recv instead of peer-memory copies")
    ap.add_argument("--nccl-allreduce", action="store_true",
                    help="N > 1: all-reduce the relation gradients with NCCL between two graphs instead of summing them over peer memory in the dense optimizer kernel")
    ap.add_argument("--no-pipeline", action="store_true", help="do not draw batch t+1 on a side stream while batch t trains")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    if args.impl == "reference":
        reference_arm(args)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=device)

    pkg = importlib.import_module("ge-2_b200")
    pkg.load_library()
    pipeline = importlib.import_module("ge-2_b200.pipeline")
    cfg = CFG
    B, C, N, D, R, nodes = cfg["B"], cfg["C"], cfg["N"], cfg["D"], cfg["relations"], cfg["nodes"]
    K, W = args.steps, args.warmup

    # ---- synthetic data, resident in HBM before the timed region -------------------------------------------
    n_edges = cfg["triples"] if (K + W) * B <= cfg["triples"] else (K + W) * B
    edges = make_graph(cfg, n_edges, 20262 + rank, device)  # each rank: its own edge share (weak scaling)
    edges = edges[torch.randperm(n_edges, device=device)]    # epoch shuffle (dataloader.cpp:613-616 of the reference project)
    gen = torch.Generator(device=device).manual_seed(7 + rank)
    pbuf, supersteps = None, None
    if world == 1:
        table = (torch.rand((nodes, D), device=device, generator=gen) - 0.5) * 0.2
        state = torch.zeros((nodes, D), device=device)
    else:
        # Partition buffer (the reference's multi-GPU layout): 4 * world node partitions, every rank trains on the 4 that are
        # resident in its buffer (same per-GPU domain and batch as the single-GPU run: weak scaling); between supersteps the
        # partitions change hands over NCCL.  Edge endpoints are buffer-local ids, as after the reference's slot remap.
        partition = importlib.import_module("ge-2_b200.partition")
        P, psize = 4 * world, nodes // 4
        home_emb = (torch.rand((4 * psize, D), device=device, generator=gen) - 0.5) * 0.2
        home_state = torch.zeros((4 * psize, D), device=device)
        try:  # partitions that change hands are pulled by the receiver over NVLink peer memory; NCCL send/recv as fall-back
            pbuf = partition.PartitionBuffer([home_emb, home_state], psize, P, rank, world, dist, peer_copies=not args.nccl_swaps)
        except Exception as e:
            print(f"[bench] peer-memory partition copies unavailable ({e!r}); using NCCL send/recv", file=sys.stderr)
            pbuf = partition.PartitionBuffer([home_emb, home_state], psize, P, rank, world, dist)
        supersteps = partition.make_supersteps(P, world)
        for st in supersteps:  # initial load and one pass over the schedule: every connection a swap needs exists before anything is timed
            pbuf.swap(st)
        pbuf.swap(supersteps[0])
        sw0, sw1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        dist.barrier()
        sw0.record()
        pbuf.swap(supersteps[1 % len(supersteps)])  # a full swap, timed on its own (reported beside the step time)
        sw1.record()
        torch.cuda.synchronize()
        swap_ms = sw0.elapsed_time(sw1)
        table, state = pbuf.buf[0], pbuf.buf[1]
    rels = torch.zeros((2, R, D), device=device)  # relation and inverse-relation tables back to back: one optimizer launch for both
    rels[:, :, : D // 2] = 1  # ComplEx relation init (complex.cpp:18-20 of the reference project)
    rel, inv_rel = rels[0], rels[1]
    rel_states = torch.zeros_like(rels)
    pcfg = pipeline.PipelineConfig(cfg["decoder"], B, C, N, cfg["degree_fraction"], D, R, nodes, lr=cfg["lr"], precision=args.precision)
    pipe = pipeline.BatchPipeline(pcfg, table, state, rel, rel_states[0], inv_rel, rel_states[1])
    rel_hook = None
    peer_reduce = world > 1 and not args.nccl_allreduce and not args.no_graph and not args.no_pipeline
    if peer_reduce:
        # Model::all_reduce of the reference (model.cpp:174-204) folded into the dense optimizer launch: every rank reads the
        # other ranks' relation gradients over NVLink (peer memory), so the multi-GPU step stays one graph replay
        try:
            pipe.use_peer_gradients(pipeline.PeerGradients(dist, 2 * R * D, device))
        except Exception as e:  # symmetric memory cannot be set up here: the NCCL form below does the same exchange
            print(f"[bench] peer-memory gradient sum unavailable ({e!r}); using the NCCL all-reduce", file=sys.stderr)
            peer_reduce = False
    if world > 1 and not peer_reduce:
        pipe.grad_scale = 1.0 / world

        def rel_hook(p):  # the same exchange as an NCCL collective between two graphs
            dist.all_reduce(p.rel_grads)  # both tables in one call

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    num_batches = n_edges // B
    use_graph = not args.no_graph  # N > 1: two graphs per step with the host-issued NCCL all-reduce between them
    # steps between swaps: a state holds 16 of the (4N)^2 edge buckets, i.e. triples * 16 / (4N)^2 edges = that many / B batches
    sps = args.steps_per_state if args.steps_per_state > 0 else max(1, int(cfg["triples"] * 16 / (4 * world) ** 2 / B))
    swaps = [0]

    def maybe_swap(i, runner=None):
        """superstep boundary: every `sps` steps the ranks exchange partitions (performNextSwap of the reference)"""
        if pbuf is not None and i > 0 and i % sps == 0:
            swaps[0] += 1
            pbuf.swap(supersteps[(1 + swaps[0]) % len(supersteps)])
            if runner is not None and hasattr(runner, "refill"):
                runner.refill()  # a new state brings a new edge bucket: the batch drawn ahead is drawn again

    # ---- warm-up, then an event-bracketed pass that times the scores kernel alone (roofline) ---------------------
    for i in range(W):
        pipe.enqueue_resident(edges, num_batches, rel_hook=rel_hook)
    pipe.check_status()
    ev_pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    barrier()
    for i in range(K):
        pipe.enqueue_resident(edges, num_batches, scores_events=ev_pairs[i], rel_hook=rel_hook)
    barrier()
    scores_host_ms = float(np.mean([a.elapsed_time(b) for a, b in ev_pairs]))
    # the same phase as it runs in the timed region: inside a replayed graph, without the host's launch gaps
    scores_ms = pipe.time_scores_phase(edges) if use_graph else scores_host_ms

    # ---- device-resident timing (`value`): K steps, one CUDA-graph launch per step -----------------------------------
    pipelined = use_graph and not args.no_pipeline
    if pipelined:
        graph = pipe.capture_pipelined(edges, num_batches, rel_hook=rel_hook)
    elif use_graph:
        graph = pipe.capture_resident(edges, num_batches) if world == 1 else pipe.capture_resident_split(edges, num_batches, rel_hook)
    if use_graph:
        barrier()  # captures take different times on different ranks; start replaying together
        for _ in range(W):
            graph.replay()
    # The clock sampler starts before the barrier (its start-up takes milliseconds and differs between ranks); the barrier and
    # the first event sit back to back.  The K-step region runs REPEATS times, each repeat bracketed by barrier + synchronize
    # on both sides and timed with CUDA events; the step counter runs on across repeats, so at N > 1 partition swaps fall
    # into the timed regions at the rate the workload's schedule gives them.
    clocks = ClockSampler(local_rank)
    clocks.start()
    time.sleep(0.02)
    rep_ms, gstep = [], 0
    for r in range(REPEATS):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(K):
            maybe_swap(gstep, graph if use_graph else None)
            gstep += 1
            if use_graph:
                graph.replay()
            else:
                pipe.enqueue_resident(edges, num_batches, rel_hook=rel_hook)
        end.record()
        barrier()
        rep_ms.append(start.elapsed_time(end))
    swaps_timed = swaps[0]
    pipe.check_status()

    # ---- end-to-end timing (`e2e`): host edges in, loss out, through the same public step call -----------------
    first = int(pipe.step_dev[0].item()) % num_batches
    idx = (first + torch.arange(K)) % num_batches
    host_edges = torch.empty((K, B, 3), dtype=torch.int64).pin_memory()
    host_edges.copy_(edges.reshape(num_batches, B, 3)[idx.to(device)].cpu())
    host_loss = torch.zeros(K, dtype=torch.float32).pin_memory()
    stage = torch.empty((B, 3), dtype=torch.int64, device=device)
    stage.copy_(host_edges[0])
    if pipelined:
        # two staging slots: while batch i trains, the ids of batch i+1 are drawn from the slot copied during step i-1
        graph_e2e = pipeline.HostFeed(pipe, 3, rel_hook=rel_hook)
        graph_e2e.start(host_edges[K - 1], host_edges[0])
    elif use_graph:
        graph_e2e = pipe.capture_resident(stage, 1) if world == 1 else pipe.capture_resident_split(stage, 1, rel_hook)

    e2e_count = [0]

    def e2e_step(i):
        g = e2e_count[0]  # steps since the e2e pass began: partition swaps keep their rhythm across repeats
        e2e_count[0] += 1
        if pipelined:
            maybe_swap(g, graph_e2e)
            graph_e2e.step(host_edges[(i + 1) % K], host_loss[i:i + 1])  # trains batch i, copies and draws batch i+1
            return
        else:
            maybe_swap(g)
            stage.copy_(host_edges[i], non_blocking=True)
            if use_graph:
                graph_e2e.replay()
            else:
                pipe.enqueue_resident(stage, 1, rel_hook=rel_hook)
        host_loss[i:i + 1].copy_(pipe.loss, non_blocking=True)

    barrier()
    for i in range(min(W, K)):
        e2e_step(i)
    rep_e2e = []
    for r in range(REPEATS):
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s2.record()
        for i in range(K):
            e2e_step(i)
        if pipelined:
            graph_e2e.drain()
        e2.record()
        barrier()
        rep_e2e.append(s2.elapsed_time(e2))
    clock_info = clocks.stop()
    pipe.check_status()
    assert bool(torch.isfinite(host_loss).all()) and float(host_loss[-1]) > 0

    t = torch.tensor(rep_ms + rep_e2e + [scores_ms], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every repeat: the slowest rank's device time
    t = t.cpu().tolist()
    rep_ms, rep_e2e, scores_ms = t[:REPEATS], t[REPEATS:2 * REPEATS], t[-1]
    ms, ms_e2e = sum(rep_ms) / REPEATS, sum(rep_e2e) / REPEATS  # mean K-step region = total steps over total time

    # ---- N = 1: one epoch of the workload (its triples / B steps) as a single timed region, clocks sampled across it -----
    epoch_info = None
    if world == 1 and use_graph and not args.no_epoch:
        ep_steps = cfg["triples"] // B
        ck = ClockSampler(local_rank)
        ck.start()
        time.sleep(0.02)
        a_ep, b_ep = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a_ep.record()
        for _ in range(ep_steps):
            graph.replay()
        b_ep.record()
        torch.cuda.synchronize()
        ep_ms = a_ep.elapsed_time(b_ep)
        ci = ck.stop()
        pipe.check_status()
        epoch_info = dict(steps=ep_steps, seconds=ep_ms * 1e-3, value=ep_steps * B / (ep_ms * 1e-3), unit="edges/s", sm_mhz=ci.get("sm_mhz"),
                          reasons=ci.get("reasons"), ms_x_mhz_per_step=(ep_ms / ep_steps) * (ci.get("sm_mhz") or 0.0),
                          note="train edges / epoch seconds, the reference's Edges per Second line (trainer.cpp:229-232), device-resident edges")

    if rank == 0:
        pk = peaks()
        S = pcfg.sides
        flops = 6.0 * S * B * N * D  # forward contraction + the two backward contractions, per side
        achieved = flops / (scores_ms * 1e-3) / 1e12
        line = dict(
            metric="train edges/sec/box", value=world * K * B / (ms * 1e-3), unit="edges/s", n_gpus=world, steps=K, warmup=W,
            ms_per_step=ms / K, higher_is_better=True, scaling="weak", vs_baseline=None, repeats=REPEATS,
            ms_per_step_repeats=dict(min=min(rep_ms) / K, median=float(np.median(rep_ms)) / K, max=max(rep_ms) / K,
                                     note="each repeat = K steps between barrier + synchronize, CUDA events, max over ranks; value = mean"),
            dtype="f32" if args.precision == "fp32" else "f16 tensor tiles, f32 accumulate and storage", data="synthetic",
            config=dict(workload=cfg["name"], per_gpu_batch=B, global_batch=B * world, precision=args.precision,
                        l2="tables (0.8 GB) and edge list larger than L2; rows touched per step are random", parallelism=f"dp{world}" if world > 1 else "single",
                        launch=("one CUDA graph replay per step" if (world == 1 or peer_reduce) else "two CUDA graph replays + one NCCL all-reduce per step") if use_graph else "host-issued launches",
                        pipelined="ids of batch t+1 are drawn and deduplicated on a side stream while batch t trains" if pipelined else None,
                        partitions=None if pbuf is None else dict(count=4 * world, rows=nodes // 4, steps_per_state=sps, swaps_in_timed_region=swaps_timed, steps_in_timed_region=K * REPEATS,
                                                                  swap_ms=swap_ms, swap_ms_per_step_amortized=swap_ms / sps,
                                                                  
                                                                  exchange=("partition slabs pulled over NVLink peer memory" if pbuf.peer_buf is not None else "NCCL send/recv of partition slabs") + "; relation gradients every step: " + ("summed over NVLink peer memory inside the dense optimizer kernel" if peer_reduce else "NCCL all-reduce"))),
            e2e=dict(value=world * K * B / (ms_e2e * 1e-3), unit="edges/s", h2d_bytes_per_step=B * 3 * 8, d2h_bytes_per_step=4,
                     ms_per_step=ms_e2e / K, ms_per_step_median=float(np.median(rep_e2e)) / K,
                     note="pinned host edges -> H2D, step, loss -> pinned host, all stream-ordered; one synchronize at the end of each repeat"
                          + ("; the H2D copy issued in step i carries batch i+1 (drawn ahead while batch i trains) and runs on a copy stream, the loss read-back on another" if pipelined else "")),
            gpu_launches=K * pipe.launches_per_step(), epoch=epoch_info,
            clocks=clock_info,
            roofline=dict(bound="tensor", kernel="lp_scores_%s" % args.precision, achieved=achieved, peak=pk["tf"], unit="TFLOP/s",
                          frac=achieved / pk["tf"], traffic=NCU_TRAFFIC.get(args.precision), peak_source=pk["src"] + " bf16 dense",
                          ms_per_launch=scores_ms, flops_per_launch=flops, ms_host_issued=scores_host_ms,
                          timing="CUDA events around 20 scores phases (dK clear + the scores launches: whole rounds unsplit, leftover blocks as "
                                 "two split launches) replayed as one CUDA graph, as in the timed region; ms_host_issued = the same phase "
                                 "bracketed by events in a host-issued pass of the same K steps (includes launch gaps)"),
        )
        if world == 1 and args.precision == "f16" and not args.no_fp32_path:
            # the same step on the fp32 CUDA-core path (1e-4 parity), for reference next to the headline
            pc32 = pipeline.PipelineConfig(cfg["decoder"], B, C, N, cfg["degree_fraction"], D, R, nodes, lr=cfg["lr"], precision="fp32")
            p32 = pipeline.BatchPipeline(pc32, table, state, rel, torch.zeros_like(rel), inv_rel, torch.zeros_like(inv_rel))
            g32 = p32.capture_resident(edges, num_batches)
            for _ in range(3):
                g32.replay()
            a32, b32 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            k32 = max(10, K // 5)
            torch.cuda.synchronize()
            a32.record()
            for _ in range(k32):
                g32.replay()
            b32.record()
            torch.cuda.synchronize()
            line["fp32_path"] = dict(value=k32 * B / (a32.elapsed_time(b32) * 1e-3), unit="edges/s", ms_per_step=a32.elapsed_time(b32) / k32, steps=k32)
        if world == 1 and not args.no_reference_gpu:
            try:
                ms_ref = reference_gpu_ms(cfg, table, state, edges, min(K, 20), device)
                line["reference_gpu"] = dict(value=B / (ms_ref * 1e-3), unit="edges/s", ms_per_step=ms_ref, speedup_e2e=line["e2e"]["value"] / (B / (ms_ref * 1e-3)),
                                             note="the reference project's own GPU code (its CUDA unique-map, bitmap backend, and its decoder/loss/autograd/"
                                                  "Adagrad translation units compiled for sm_100) on the same GPU and workload, without its trainer loop's "
                                                  "host overheads; test infrastructure, not part of the product path")
            except Exception as ex:  # context only: never let it break the bench line
                line["reference_gpu"] = dict(unavailable=str(ex)[:160])
        if world == 1 and not args.no_cpu_baseline:
            cpu = CpuReference(cfg, 20262)
            v, k, dt = cpu.timed(args.cpu_budget)
            line["cpu_baseline"] = dict(value=v, unit="edges/s", cores=cpu.cores, kind=cpu.kind,
                                        sample=f"{k} batches of {B} edges of the same workload in {dt:.1f} s on the host cores")
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
