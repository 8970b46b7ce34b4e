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

# The partitioned configurations (--config 3|4|5, run with --gpus 2|4|8).  Node ids are drawn from a Zipf law over a random
# relabelling; the rank-frequency exponent alpha stands for the stated degree law (degree exponent g <-> alpha = 1 / (g - 1):
# preferential attachment g = 3 -> 0.5, g = 2.2 -> 0.83).  Seeded synthetic stand-ins with the stated sizes.
PARTITIONED = {
    3: dict(name="social-4.85M-nodes/69M-edges Dot d=100 B=50000 neg=50x1000, 16 partitions", nodes=4_847_571, relations=1, triples=68_993_773,
            decoder="DISTMULT", D=100, B=50_000, C=50, N=1000, degree_fraction=0.0, lr=0.1, alpha_nodes=0.5, alpha_rel=1.2, P=16, gpus=2),
    4: dict(name="follower-41.65M-nodes/1.468B-edges Dot d=100 B=50000 neg=50x1000, 16 partitions", nodes=41_652_230, relations=1,
            triples=1_468_365_182, decoder="DISTMULT", D=100, B=50_000, C=50, N=1000, degree_fraction=0.0, lr=0.1, alpha_nodes=0.83, alpha_rel=1.2,
            P=16, gpus=4),
    5: dict(name="kg-100M-entities/10k-relations/3B-triples DistMult d=128 B=100000 neg=100x2000, 32 partitions", nodes=100_000_000, relations=10_000,
            triples=3_000_000_000, decoder="DISTMULT", D=128, B=100_000, C=100, N=2000, degree_fraction=0.0, lr=0.1, alpha_nodes=1.1, alpha_rel=1.2,
            P=32, gpus=8),
}


# dram__bytes_read.sum + dram__bytes_write.sum of the scores launches of one step on this workload, taken from one ncu
# capture of those launches (operands and partial gradients stay in the 126 MB L2, so it is far below the operand bytes)
NCU_TRAFFIC = {"f16": 38_685_952, "fp32": None}
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
                impl="reference", config=dict(workload=cfg["name"] + (f", weak-scaled: {args.gpus} x nodes and triples, {4 * args.gpus} partitions" if args.gpus > 1 else ""),
                                              steps_run=steps_run, note="the per-batch step of this workload (same batch, negatives and resident-domain sizes) on the host cores"),
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


def host_cpp_ms(cfg, table, state, edges, steps, device, precision):
    """The same steps through the C++ host layer (ge-2_b200/host, the reference's own call sequence: DataLoader::getBatch ->
    Model::train_batch -> DataLoader::updateEmbeddings, unfused, host-issued, one count read-back per batch inside map_tensors
    as a drop-in for the reference's four).  Scratch copies of the tables; ms per step by CUDA events."""
    import importlib.util

    so = ROOT / "ge-2_b200" / "ge2_host.so"
    spec = importlib.util.spec_from_file_location("ge2_host", so)
    H = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(H)
    kind = H.DecoderType.COMPLEX if cfg["decoder"] == "COMPLEX" else H.DecoderType.DISTMULT
    model = H.Model(kind, cfg["relations"], cfg["D"], True, cfg["lr"], cfg["lr"], device, precision)
    emb, st = H.InMemory(table.clone()), H.InMemory(state.clone())
    loader = H.DataLoader(edges, emb, st, cfg["B"], cfg["C"], cfg["N"], cfg["degree_fraction"], True, 20262)

    def one():
        batch = loader.getBatch()
        model.train_batch(batch, True)
        loader.updateEmbeddings(batch)

    for _ in range(3):
        one()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    for _ in range(steps):
        one()
    b.record()
    torch.cuda.synchronize()
    model.check_status()
    return a.elapsed_time(b) / steps


def unique_sweep(device):
    """`--unique-sweep`: ge2_unique_bitmap (graph replay and host-issued) against the reference's own CUDA unique-map (bitmap
    backend, oracle/_ref/gege_ref_cuda.so: test infrastructure) on the (n_ids, domain) pairs of the five configurations,
    uniform random ids, CUDA events over 50 calls.  Prints one JSON line."""
    pkg = importlib.import_module("ge-2_b200")
    pkg.load_library()
    capi = pkg.capi
    os.environ.setdefault("GEGE_UNIQUE_BACKEND", "bitmap")
    for k in ("GEGE_CSR_GATHER", "GEGE_CSR_DEBUG", "GEGE_STAGE_DEBUG"):
        os.environ.setdefault(k, "0")
    try:
        import gege_ref_cuda as G
    except Exception:
        G = None

    def ev(fn, reps=50):
        for _ in range(5):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    rows = []
    for n, dom in ((22_000, 14_951), (40_000, 1_000_000), (150_000, 1_211_896), (150_000, 10_413_060), (600_000, 12_500_000)):
        g = torch.Generator(device=device).manual_seed(n)
        ids = torch.randint(0, dom, (n,), device=device, generator=g)
        ws = capi.unique_workspace(dom, device)
        uq = torch.empty(min(n, dom), dtype=torch.int64, device=device)
        inv = torch.empty(n, dtype=torch.int64, device=device)
        cnt = torch.zeros(2, dtype=torch.int32, device=device)
        call = lambda: capi.unique_bitmap(ids, dom, workspace=ws, out_unique=uq, out_inverse=inv, out_count=cnt)
        host_us = ev(call)
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            call()
        graph_us = ev(gr.replay)
        ref_us = ev(lambda: G.unique_inverse_cuda(ids, False, dom), reps=20) if G is not None else None
        rows.append(dict(n_ids=n, domain=dom, distinct=int(cnt[0]), graph_us=round(graph_us, 1), host_issued_us=round(host_us, 1),
                         reference_kernel_us=None if ref_us is None else round(ref_us, 1),
                         algorithmic_bytes=16 * n + 8 * int(cnt[0])))
    print(json.dumps(dict(unique_sweep=rows)), flush=True)


def selected_sweep(device):
    """`--selected-sweep`: the selected-negative operators (tournament selection; scores of the chosen pairs forward and
    backward) against the reference's own GPU code for them (oracle/_ref/gege_ref_cuda.so: test infrastructure) on batches
    shaped like the benchmarked step (50 000 query rows, 1 000 negatives a chunk, D = 100), CUDA events over 20 calls.
    Algorithmic bytes of the pair kernels: every chosen negative row read once (and, backward, added to once).
    Prints one JSON line."""
    pkg = importlib.import_module("ge-2_b200")
    pkg.load_library()
    capi = pkg.capi
    try:
        import gege_ref_cuda as G
    except Exception:
        G = None

    def ev(fn, reps=20):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    rows = []
    D = 100
    for chunks, R, N, K in ((10, 5000, 1000, 100), (10, 5000, 1000, 10), (50, 1000, 1000, 500)):
        g = torch.Generator(device=device).manual_seed(K)
        q = torch.randn((chunks, R, D), device=device, generator=g) * 0.3
        neg = torch.randn((chunks, N, D), device=device, generator=g) * 0.3
        sel_us = ev(lambda: capi.tournament_select(q, neg, K))
        _, idx = capi.tournament_select(q, neg, K)
        grad = torch.randn((chunks * R, K), device=device, generator=g)
        row = dict(chunks=chunks, rows_per_chunk=R, negatives=N, selected=K, D=D, tournament_us=round(sel_us, 1),
                   tournament_gflop=round(2e-9 * chunks * R * N * D, 2))
        for kind, code in (("DOT", 1), ("L2", 2)):
            row[f"scores_{kind}_us"] = round(ev(lambda: capi.selected_neg_scores(kind, q, neg, idx)), 1)
            row[f"backward_{kind}_us"] = round(ev(lambda: capi.selected_neg_scores_backward(kind, grad, q, neg, idx)), 1)
            if G is not None:
                row[f"reference_scores_{kind}_us"] = round(ev(lambda: G.selected_neg_scores_forward(q, neg, idx, code), reps=5), 1)
                row[f"reference_backward_{kind}_us"] = round(ev(lambda: G.selected_neg_scores_backward(grad, q, neg, idx, code), reps=5), 1)
        row["pair_row_bytes"] = 4 * D * chunks * R * K
        if G is not None:
            row["reference_tournament_us"] = round(ev(lambda: G.tournament_selected_scores(q, neg, K, 64), reps=5), 1)
        rows.append(row)
    print(json.dumps(dict(selected_sweep=rows)), flush=True)


def bucket_sizes_of(cfg, P, psize, seed, device):
    """sizes of all P * P buckets of the graph make_partitioned_edges generates (a counting pass over the same draws)"""
    return make_partitioned_edges(cfg, P, psize, [], seed, device, count_only=True)[1]


_CDF_CACHE = {}


def make_partitioned_edges(cfg, P, psize, keep_buckets, seed, device, chunk=40_000_000, count_only=False):
    """The graph's training edges, generated chunk by chunk with the same seed on every rank; a rank keeps the edges of
    the buckets it will train (keep_buckets) sorted by bucket -- the preprocessor's order
    (torch_partitioner.py:12-31 of the reference project) -- and the sizes of ALL P*P buckets.
    Returns (edges_sorted [n_kept, cols] int64, sizes [P*P] int64 numpy, begin [P*P] int64 numpy, -1 for buckets not kept)."""
    gen = torch.Generator(device=device)
    gen.manual_seed(seed)
    nodes, R = cfg["nodes"], cfg["relations"]
    has_rel = R > 1

    def sampler(domain, alpha):
        key = (domain, alpha, str(device))
        if key not in _CDF_CACHE:
            # powers on the device (element-wise: the same on every rank), the running sum on the host: a device scan adds
            # its tiles in an order that varies from run to run, and every rank and both passes must draw exactly the same graph
            w = torch.arange(1, domain + 1, dtype=torch.float64, device=device).pow_(-alpha).cpu().numpy()
            np.cumsum(w, out=w)
            w /= w[-1]
            _CDF_CACHE[key] = torch.from_numpy(w).to(device)
        cdf = _CDF_CACHE[key]
        perm = torch.randperm(domain, device=device, generator=gen)
        return lambda n: perm[torch.searchsorted(cdf, torch.rand(n, dtype=cdf.dtype, device=device, generator=gen)).clamp_(max=domain - 1)]

    draw_node = sampler(nodes, cfg["alpha_nodes"])
    draw_rel = sampler(R, cfg["alpha_rel"]) if has_rel else None
    keep = torch.zeros(P * P, dtype=torch.bool, device=device)
    if len(keep_buckets):
        keep[torch.tensor(sorted(keep_buckets), dtype=torch.int64, device=device)] = True
    sizes = torch.zeros(P * P, dtype=torch.int64, device=device)
    kept, kept_b = [], []
    left = cfg["triples"]
    while left > 0:
        n = min(chunk, left)
        left -= n
        src, dst = draw_node(n), draw_node(n)
        b = (src // psize) * P + dst // psize
        sizes += torch.bincount(b, minlength=P * P)
        m = keep[b]
        rel_col = draw_rel(n) if has_rel else None  # drawn in both passes: the generator's stream stays the same
        if not count_only:
            cols = [src[m]] + ([rel_col[m]] if has_rel else []) + [dst[m]]
            kept.append(torch.stack(cols, dim=1))
            kept_b.append(b[m])
        del src, dst, b, m, rel_col
    if count_only:
        return None, sizes.cpu().numpy(), None
    e = torch.cat(kept)
    bk = torch.cat(kept_b)
    del kept, kept_b
    order = torch.sort(bk, stable=True).indices
    e = e[order].contiguous()
    sizes_np = sizes.cpu().numpy()
    begin = np.full(P * P, -1, np.int64)
    off = 0
    for bkt in sorted(keep_buckets):
        begin[bkt] = off
        off += int(sizes_np[bkt])
    assert off == e.shape[0]
    return e, sizes_np, begin


def per_kernel_rooflines(pipe, pcfg, capi, edges, num_batches, reps=20):
    """The HBM-bound kernels of the step, each replayed `reps` times as a graph of its own on the buffers a full step left
    behind and bracketed by CUDA events: achieved = algorithmic bytes / time, against the measured copy bandwidth.  The
    working set of one step (ids, fp16 operands, gradient rows) stays in the 126 MB L2 between replays; the embedding rows a
    batch touches are a random 1-2 % of a 0.8 GB table."""
    pk = peaks()
    B, C, N, D, S = pcfg.B, pcfg.C, pcfg.N, pcfg.D, pcfg.sides
    CN, n_ids = C * N, pcfg.n_ids
    U = int(pipe.count[0].item())

    def tg(fn):
        fn()
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(reps):
                fn()
        g.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    ids = pipe.ids[0]  # the id set of the batch trained last
    out = {}

    def add(name, ms, nbytes, what):
        gbs = nbytes / (ms * 1e-3) / 1e9
        out[name] = dict(ms=ms, bytes=nbytes, achieved=gbs, unit="GB/s", peak=pk["hbm"], frac=gbs / pk["hbm"], bound="hbm", bytes_are=what)

    add("unique_map", tg(lambda: capi.unique_bitmap(ids.packed, pcfg.domain, workspace=ids.uws, out_unique=ids.unique, out_inverse=ids.inverse,
                                                      out_count=ids.count)),
        16 * n_ids + 8 * U, "16 B per id (read id, write rank) + 8 B per distinct id; the domain-sized bitset passes (0.19 B per node) not counted")
    add("gather_prepare", pipe.time_scores_phase(edges, reps, 1),
        ((2 + S) * B + S * CN) * D * 4 + (S * pcfg.B + S * CN) * 128 * 2, "embedding / relation rows read (fp32) + fp16 operand rows written")
    add("scatter_finish", pipe.time_scores_phase(edges, reps, 4),
        (B * (6 + 4) + S * CN * 2) * D * 4, "per edge 6 rows in + 4 gradient rows out, per negative 1 row in + 1 out (fp32)")
    t2, s2 = pipe.table.clone(), pipe.state.clone()  # scratch copies: the timing must not train the real tables
    pipe.node_grad.normal_()
    add("adagrad_scatter", tg(lambda: capi.adagrad_scatter(t2, s2, ids.unique, pipe.node_grad, 0.1, U=pipe.cap, U_dev=ids.count,
                                                            clear_grad=False, status=pipe.status)),
        20 * U * D, "per touched row: embedding + state read and written (16 B per float) + gradient read (4 B)")
    pipe.node_grad.zero_()
    del t2, s2
    return out


def scores_roofline(precision, sides, B, N, D, scores_ms, scores_host_ms):
    """roofline object of the dominant kernel (the scores launches): algorithmic flops 6 * S * B * N * D per step (forward
    contraction + the two backward contractions, per side) over the launches' device time, against the measured bf16 peak"""
    pk = peaks()
    flops = 6.0 * sides * B * N * D
    achieved = flops / (scores_ms * 1e-3) / 1e12
    return dict(bound="tensor", kernel="lp_scores_%s" % precision, achieved=achieved, peak=pk["tf"], unit="TFLOP/s", frac=achieved / pk["tf"],
                traffic=NCU_TRAFFIC.get(precision) if (B, N, D, sides) == (CFG["B"], CFG["N"], CFG["D"], 2) else None,
                peak_source=pk["src"] + " bf16 dense", ms_per_launch=scores_ms, flops_per_launch=flops, ms_host_issued=scores_host_ms,
                timing="CUDA events around 20 scores phases (the logsumexp launch + the gradient launch) replayed as one CUDA graph, as in the "
                       "timed region; ms_host_issued = the same phase bracketed by events in a host-issued pass (includes launch gaps)")


def multi_gpu_main(args, rank, world, local_rank, device, dist):
    """N > 1: the partitioned workload.  The graph's nodes are cut into P partitions, four of which are resident per GPU; a
    superstep trains, on every GPU, the edge buckets of its four resident partitions (pairwise disjoint between GPUs: no
    exchange for node embeddings), then the partitions change hands (device-side pulls over NVLink peer memory) and every GPU
    builds its next edge list on the device.  Relation gradients are summed over peer memory inside every step.
    Default: configuration 2 weak-scaled (per-GPU domain, batch and triples as at N = 1, P = 4 N partitions)."""
    pkg = importlib.import_module("ge-2_b200")
    pkg.load_library()
    pipeline = importlib.import_module("ge-2_b200.pipeline")
    partition = importlib.import_module("ge-2_b200.partition")
    capi = pkg.capi
    K, W = args.steps, args.warmup
    if args.config in PARTITIONED:
        cfg = dict(PARTITIONED[args.config])
        if cfg["gpus"] != world:
            raise SystemExit(f"configuration {args.config} is stated for {cfg['gpus']} GPUs (got --gpus {world})")
        P = cfg["P"]
        scaling = "strong"  # a fixed graph; listed for completeness, the driver's scaling run uses the default workload
    else:
        cfg = dict(CFG)
        P = 4 * world
        cfg["nodes"], cfg["triples"] = CFG["nodes"] * world, CFG["triples"] * world
        cfg["name"] = CFG["name"] + f", weak-scaled: {world} x nodes and triples, {P} partitions"
        scaling = "weak"
    B, C, N, D, R = cfg["B"], cfg["C"], cfg["N"], cfg["D"], cfg["relations"]
    has_rel = R > 1
    psize = -(-cfg["nodes"] // P)  # ceil, as the reference sizes its partitions (storage.cpp:368)
    domain = partition.CAPACITY * psize
    supersteps = partition.make_supersteps(P, world)

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    t_setup = time.perf_counter()
    sizes = bucket_sizes_of(cfg, P, psize, 20262, device)   # first pass: the sizes of all buckets (the schedule balances lanes with them)
    chk = torch.from_numpy(sizes).to(device)
    dist.broadcast(chk, 0)
    if not np.array_equal(chk.cpu().numpy(), sizes):
        raise SystemExit("the ranks generated different graphs")
    buckets = partition.state_buckets(supersteps, P, sizes)
    mine = sorted(b for lanes in buckets for b in lanes[rank])
    edges_sorted, sizes2, begin = make_partitioned_edges(cfg, P, psize, mine, 20262, device)
    assert np.array_equal(sizes, sizes2)
    gen = torch.Generator(device=device).manual_seed(7 + rank)
    n_home = len([p for p in range(P) if p % world == rank])
    home_emb = (torch.rand((n_home * psize, D), device=device, generator=gen) - 0.5) * 0.2
    home_state = torch.zeros((n_home * psize, D), device=device)
    relay = partition.RelayBuffer([home_emb, home_state], psize, P, rank, world, dist)
    del home_emb, home_state
    rels = torch.zeros((2, max(R, 1), D), device=device)
    rels[:, :, : D // 2] = 1
    if cfg["decoder"] == "DISTMULT":
        rels[:] = 1  # distmult.cpp:18 of the reference project
    rel_states = torch.zeros_like(rels)
    pcfg = pipeline.PipelineConfig(cfg["decoder"], B, C, N, cfg["degree_fraction"], D, R, domain, lr=cfg["lr"], precision=args.precision)
    pipe = pipeline.BatchPipeline(pcfg, relay.buf(0, 0), relay.buf(1, 0), rels[0] if has_rel else None, rel_states[0] if has_rel else None,
                                  rels[1] if has_rel else None, rel_states[1] if has_rel else None)
    if has_rel:
        pipe.use_peer_gradients(pipeline.PeerGradients(dist, 2 * R * D, device))
    trainer = partition.PartitionedTrainer(pipe, relay, edges_sorted, sizes, seed=31, bucket_begin=begin)
    setup_s = time.perf_counter() - t_setup

    # ---- the schedule's arithmetic: batches per lane and superstep, from the bucket sizes -----------------------------------
    nb = [[c // B for c in lanes] for lanes in trainer.state_edges_count]
    nb_max = [max(x) for x in nb]
    epoch_edges = sum(sum(x) for x in nb) * B
    epoch_steps = sum(nb_max)  # every lane takes part in that many relation-gradient exchanges

    # ---- superstep 0: swap in, build the edge list, capture the step graphs (outside every timed region) ---------------------
    state_no = [0]
    sw_ms, sw_parts = [], []

    def next_state(timed: bool):
        """partition swap + rebuild of this rank's edge list + redraw of the batch sampled ahead, as one device-timed region"""
        k = state_no[0] % len(supersteps)
        state_no[0] += 1
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if timed:
            barrier()
        a.record()
        relay.swap(supersteps[k])
        mid1 = torch.cuda.Event(enable_timing=True)
        mid1.record()
        lane = buckets[k][rank]
        total = 0
        if supersteps[k][rank] is not None and lane:
            trainer.slot_dev.copy_(torch.tensor(relay.slot_table(), dtype=torch.int64))
            total = capi.build_state_edges(edges_sorted, [int(begin[x]) for x in lane], [int(sizes[x]) for x in lane], trainer.slot_dev, psize,
                                           trainer.state_seed(0, k), trainer.state_edges, pipe.status)
        mid2 = torch.cuda.Event(enable_timing=True)
        mid2.record()
        pipe.set_num_batches(max(1, total // B))
        runner, _ = trainer._runner(relay.parity)
        runner.refill()
        b.record()
        if timed:
            barrier()
            sw_ms.append(a.elapsed_time(b))
            sw_parts.append((a.elapsed_time(mid1), mid1.elapsed_time(mid2), mid2.elapsed_time(b)))
        return runner, total

    runner, total0 = next_state(False)
    while total0 // B < 1:  # a lane without a batch in this superstep: move on until this rank has one (all ranks move together)
        runner, total0 = next_state(False)
    barrier()
    for _ in range(W):
        runner.replay()
    pipe.check_status()
    relay.check_status()

    # ---- timed steps: REPEATS regions of K steps inside one state ----------------------------------------------------------------
    clocks = ClockSampler(local_rank)
    clocks.start()
    time.sleep(0.02)
    rep_ms = []
    waited0 = pipe.peer.waited_ns() if has_rel else 0
    for r in range(REPEATS):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(K):
            runner.replay()
        end.record()
        barrier()
        rep_ms.append(start.elapsed_time(end))
    pipe.check_status()
    # how long this rank's announce kernel sat waiting for the slowest rank, per step (the first step of each region also
    # absorbs the host barrier's skew)
    waited_us = torch.tensor([(pipe.peer.waited_ns() - waited0) / (1e3 * REPEATS * K) if has_rel else 0.0], device=device, dtype=torch.float64)
    waited_all = [torch.zeros_like(waited_us) for _ in range(world)]
    dist.all_gather(waited_all, waited_us)
    waited_all = [float(x) for x in waited_all]

    # ---- timed swaps: the next three supersteps' swap + rebuild, each as its own region ---------------------------------------------
    for _ in range(3):
        runner, total = next_state(True)
        for _ in range(2):
            runner.replay()  # the new state trains: graphs of the other buffer, new edge list
    pipe.check_status()
    relay.check_status()

    # ---- end to end: the state's batches from pinned host memory through HostFeed, loss read back every step ----------------------
    cols = edges_sorted.shape[1]
    nb_here = max(1, total // B)
    kk = min(K, nb_here)
    host_edges = torch.empty((kk, B, cols), dtype=torch.int64).pin_memory()
    host_edges.copy_(trainer.state_edges[: kk * B].reshape(kk, B, cols).cpu())
    host_loss = torch.zeros(K, dtype=torch.float32).pin_memory()
    pipe.set_num_batches(2)  # HostFeed trains from a two-slot staging list
    feed = pipeline.HostFeed(pipe, cols)
    feed.start(host_edges[kk - 1], host_edges[0], tables=(relay.buf(0), relay.buf(1)))
    barrier()
    for i in range(min(W, K)):
        feed.step(host_edges[(i + 1) % kk], host_loss[i:i + 1])
    rep_e2e = []
    for r in range(REPEATS):
        s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s2.record()
        for i in range(K):
            feed.step(host_edges[(i + 1) % kk], host_loss[i:i + 1])
        feed.drain()
        e2.record()
        barrier()
        rep_e2e.append(s2.elapsed_time(e2))
    clock_info = clocks.stop()
    pipe.check_status()
    assert bool(torch.isfinite(host_loss).all()) and float(host_loss[-1]) > 0

    scores_ms = pipe.time_scores_phase(trainer.state_edges)  # the scores launches of one step, replayed as a graph of their own
    # The relation-gradient exchange on its own: the announce/wait kernel + the peer-summing optimizer kernel, 20 times back to
    # back (the step counter stands still, so nobody waits: this is the kernels' own time, without the skew between ranks that
    # a real step adds; the half they read was cleared by the last step, so the tables do not move).
    exchange_us = None
    if has_rel:
        barrier()
        g = torch.cuda.CUDAGraph()
        pipe._update_relations()
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for _ in range(20):
                pipe._update_relations()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        g.replay()
        b.record()
        barrier()
        exchange_us = 1e3 * a.elapsed_time(b) / 20
    # the step's kernels on this rank's own state, each timed alone: lanes differ (the buckets of a hub partition repeat a few
    # rows thousands of times), and the exchange makes every step as long as the slowest lane's
    kernel_ms_by_rank = None
    if not args.no_kernel_rooflines:
        barrier()
        mine_ms = per_kernel_rooflines(pipe, pcfg, capi, trainer.state_edges, max(1, total // B))
        names = sorted(mine_ms)
        row = torch.tensor([mine_ms[n]["ms"] for n in names] + [float(pipe.ids[0].count[0].item())], device=device, dtype=torch.float64)
        rows = [torch.zeros_like(row) for _ in range(world)]
        dist.all_gather(rows, row)
        kernel_ms_by_rank = {n: [round(float(r[i]), 5) for r in rows] for i, n in enumerate(names + ["distinct_rows"])}
        kernel_ms_by_rank["scores"] = None  # filled below
    sc_row = torch.tensor([scores_ms], device=device, dtype=torch.float64)
    sc_rows = [torch.zeros_like(sc_row) for _ in range(world)]
    dist.all_gather(sc_rows, sc_row)
    if kernel_ms_by_rank is not None:
        kernel_ms_by_rank["scores"] = [round(float(x), 5) for x in sc_rows]
    t = torch.tensor(rep_ms + rep_e2e + sw_ms + [scores_ms], device=device, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)  # every region: the slowest rank's device time
    t = t.cpu().tolist()
    rep_ms, rep_e2e, sw_ms, scores_ms = t[:REPEATS], t[REPEATS:2 * REPEATS], t[2 * REPEATS:-1], t[-1]
    ms_step = sum(rep_ms) / REPEATS / K
    ms_step_e2e = sum(rep_e2e) / REPEATS / K
    swap_ms = float(np.median(sw_ms))
    n_sw = len(supersteps)
    # one epoch of the schedule: every superstep runs max-over-lanes steps (short lanes idle in the gradient exchange) and ends
    # with a swap + rebuild; value = the epoch's train edges over that time, from the step and swap times measured above
    epoch_ms = epoch_steps * ms_step + n_sw * swap_ms
    epoch_ms_e2e = epoch_steps * ms_step_e2e + n_sw * swap_ms
    if rank == 0:
        line = dict(
            metric="train edges/sec/box", value=epoch_edges / (epoch_ms * 1e-3), unit="edges/s", n_gpus=world, steps=K, warmup=W,
            ms_per_step=ms_step, higher_is_better=True, scaling=scaling, vs_baseline=None, repeats=REPEATS,
            ms_per_step_repeats=dict(min=min(rep_ms) / K, median=float(np.median(rep_ms)) / K, max=max(rep_ms) / K),
            dtype="f32" if args.precision == "fp32" else "f16 tensor tiles, f32 accumulate and storage", data="synthetic",
            config=dict(workload=cfg["name"], per_gpu_batch=B, global_batch=B * world, precision=args.precision, parallelism=f"dp{world}",
                        l2="tables and edge lists larger than L2; rows touched per step are random",
                        launch="one CUDA graph replay per step (relation gradients summed over NVLink peer memory inside it)",
                        value_is="one epoch of the partition schedule: its train edges / (its steps x the measured step time + its swaps x "
                                 "the measured swap + edge-list rebuild time); steps and swaps are timed in this run on the device, max over ranks",
                        partitions=dict(count=P, rows=psize, resident_per_gpu=partition.CAPACITY, supersteps=n_sw, epoch_steps_per_lane=epoch_steps,
                                        epoch_train_edges=epoch_edges, steps_per_superstep_mean=epoch_steps / n_sw,
                                        lane_balance=epoch_edges / (epoch_steps * B * world), exchange_wait_us_per_step_by_rank=waited_all if has_rel else None, kernel_ms_by_rank=kernel_ms_by_rank, swap_ms=swap_ms, swap_ms_all=sw_ms, swap_parts_ms_rank0=[dict(pulls=x, edge_list=y, refill=z) for x, y, z in sw_parts],
                                        swap_share_of_epoch=n_sw * swap_ms / epoch_ms, slab_mb=psize * D * 4 / 1e6,
                                        exchange_us_per_step=exchange_us, step_only_value=world * B / (ms_step * 1e-3),
                                        swap="receiver-side pulls over NVLink peer memory behind a device-side barrier, two alternating active "
                                             "buffers, edge list of the new state built on the device (bucket gather + slot remap + shuffle)"),
                        setup_seconds=setup_s),
            e2e=dict(value=epoch_edges / (epoch_ms_e2e * 1e-3), unit="edges/s", h2d_bytes_per_step=B * cols * 8, d2h_bytes_per_step=4,
                     ms_per_step=ms_step_e2e, note="the same epoch arithmetic with the step time measured through HostFeed: the batch arrives in "
                                                    "pinned host memory (already in buffer-local ids), H2D copy, step, loss read back, every step"),
            gpu_launches=K * pipe.launches_per_step(), clocks=clock_info,
            roofline=scores_roofline(args.precision, pcfg.sides, B, N, D, scores_ms, None),
        )
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()


# ----------------------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5],
                    help="2: the single-GPU configuration (weak-scaled over partitions at N > 1); 3, 4, 5: the stated partitioned configurations "
                         "(need --gpus 2, 4, 8)")
    ap.add_argument("--precision", default=os.environ.get("GE2_PRECISION", "f16"), choices=["fp32", "f16"],
                    help="f16: tcgen05 fp16-operand tiles with fp32 accumulation (1e-2 parity, the designed path); fp32: CUDA-core path (1e-4 parity)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-fp32-path", action="store_true", help="skip the side measurement of the fp32 CUDA-core path")
    ap.add_argument("--no-reference-gpu", action="store_true", help="skip timing the reference's own GPU code (oracle/_ref/gege_ref_cuda.so) on this GPU")
    ap.add_argument("--no-host-cpp", action="store_true", help="N = 1: skip the side measurement through the C++ host layer")
    ap.add_argument("--no-epoch", action="store_true", help="N = 1: skip the one-epoch (triples / B steps) timed region")
    ap.add_argument("--no-kernel-rooflines", action="store_true", help="N = 1: skip the per-kernel timings behind roofline_kernels")
    ap.add_argument("--no-graph", action="store_true", help="N = 1: issue every launch from the host instead of replaying a CUDA graph")
    ap.add_argument("--no-pipeline", action="store_true", help="N = 1: do not draw batch t+1 on a side stream while batch t trains")
    ap.add_argument("--cpu-budget", type=float, default=15.0)
    ap.add_argument("--unique-sweep", action="store_true", help="time the unique-map on the five (n_ids, domain) pairs against the reference's kernel and exit")
    ap.add_argument("--selected-sweep", action="store_true", help="time the selected-negative operators against the reference's GPU code and exit")
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
    if args.unique_sweep:
        if rank == 0:
            unique_sweep(device)
        return
    if args.selected_sweep:
        if rank == 0:
            selected_sweep(device)
        return
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=device)
        multi_gpu_main(args, rank, world, local_rank, device, dist)
        return
    if args.config != 2:
        raise SystemExit(f"configuration {args.config} is stated for {PARTITIONED[args.config]['gpus']} GPUs: run it with --gpus {PARTITIONED[args.config]['gpus']}")

    pkg = importlib.import_module("ge-2_b200")
    pkg.load_library()
    pipeline = importlib.import_module("ge-2_b200.pipeline")
    capi = pkg.capi
    cfg = CFG
    B, C, N, D, R, nodes = cfg["B"], cfg["C"], cfg["N"], cfg["D"], cfg["relations"], cfg["nodes"]
    K, W = args.steps, args.warmup

    # ---- synthetic data, resident in HBM before the timed region -------------------------------------------
    n_edges = cfg["triples"] if (K + W) * B <= cfg["triples"] else (K + W) * B
    edges = make_graph(cfg, n_edges, 20262, device)
    edges = edges[torch.randperm(n_edges, device=device)]    # epoch shuffle (dataloader.cpp:613-616 of the reference project)
    gen = torch.Generator(device=device).manual_seed(7)
    table = (torch.rand((nodes, D), device=device, generator=gen) - 0.5) * 0.2
    state = torch.zeros((nodes, D), device=device)
    rels = torch.zeros((2, R, D), device=device)  # relation and inverse-relation tables back to back: one optimizer launch for both
    rels[:, :, : D // 2] = 1  # ComplEx relation init (complex.cpp:18-20 of the reference project)
    rel, inv_rel = rels[0], rels[1]
    rel_states = torch.zeros_like(rels)
    pcfg = pipeline.PipelineConfig(cfg["decoder"], B, C, N, cfg["degree_fraction"], D, R, nodes, lr=cfg["lr"], precision=args.precision)
    pipe = pipeline.BatchPipeline(pcfg, table, state, rel, rel_states[0], inv_rel, rel_states[1])

    def barrier():
        torch.cuda.synchronize()

    num_batches = n_edges // B
    use_graph = not args.no_graph

    # ---- warm-up, then an event-bracketed pass that times the scores kernel alone (roofline) ---------------------
    for i in range(W):
        pipe.enqueue_resident(edges, num_batches)
    pipe.check_status()
    ev_pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    barrier()
    for i in range(K):
        pipe.enqueue_resident(edges, num_batches, scores_events=ev_pairs[i])
    barrier()
    scores_host_ms = float(np.mean([a.elapsed_time(b) for a, b in ev_pairs]))
    # the same phase as it runs in the timed region: inside a replayed graph, without the host's launch gaps
    scores_ms = pipe.time_scores_phase(edges) if use_graph else scores_host_ms
    kernel_rooflines = None if (args.no_kernel_rooflines or not use_graph) else per_kernel_rooflines(pipe, pcfg, capi, edges, num_batches)

    # ---- device-resident timing (`value`): K steps, one CUDA-graph launch per step -----------------------------------
    pipelined = use_graph and not args.no_pipeline
    if pipelined:
        graph = pipe.capture_pipelined(edges, num_batches)
    elif use_graph:
        graph = pipe.capture_resident(edges, num_batches)
    if use_graph:
        for _ in range(W):
            graph.replay()
    # The clock sampler starts before the first timed region (its start-up takes milliseconds).  The K-step region runs
    # REPEATS times, each repeat bracketed by a synchronize on both sides and timed with CUDA events.
    clocks = ClockSampler(local_rank)
    clocks.start()
    time.sleep(0.02)
    rep_ms = []
    for r in range(REPEATS):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        start.record()
        for i in range(K):
            if use_graph:
                graph.replay()
            else:
                pipe.enqueue_resident(edges, num_batches)
        end.record()
        barrier()
        rep_ms.append(start.elapsed_time(end))
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
        graph_e2e = pipeline.HostFeed(pipe, 3)
        graph_e2e.start(host_edges[K - 1], host_edges[0])
    elif use_graph:
        graph_e2e = pipe.capture_resident(stage, 1)

    def e2e_step(i):
        if pipelined:
            graph_e2e.step(host_edges[(i + 1) % K], host_loss[i:i + 1])  # trains batch i, copies and draws batch i+1
            return
        stage.copy_(host_edges[i], non_blocking=True)
        if use_graph:
            graph_e2e.replay()
        else:
            pipe.enqueue_resident(stage, 1)
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
    ms, ms_e2e = sum(rep_ms) / REPEATS, sum(rep_e2e) / REPEATS  # mean K-step region = total steps over total time

    # ---- one epoch of the workload (its triples / B steps) as a single timed region, clocks sampled across it -----
    epoch_info = None
    if use_graph and not args.no_epoch:
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

    world = 1
    if rank == 0:
        S = pcfg.sides
        line = dict(
            metric="train edges/sec/box", value=K * B / (ms * 1e-3), unit="edges/s", n_gpus=1, steps=K, warmup=W,
            ms_per_step=ms / K, higher_is_better=True, scaling="weak", vs_baseline=None, repeats=REPEATS,
            ms_per_step_repeats=dict(min=min(rep_ms) / K, median=float(np.median(rep_ms)) / K, max=max(rep_ms) / K,
                                     note="each repeat = K steps between synchronizes, CUDA events; value = mean"),
            dtype="f32" if args.precision == "fp32" else "f16 tensor tiles, f32 accumulate and storage", data="synthetic",
            config=dict(workload=cfg["name"], per_gpu_batch=B, global_batch=B, precision=args.precision,
                        l2="tables (0.8 GB) and edge list larger than L2; rows touched per step are random", parallelism="single",
                        launch="one CUDA graph replay per step" if use_graph else "host-issued launches",
                        pipelined="ids of batch t+1 are drawn and deduplicated on a side stream while batch t trains" if pipelined else None),
            e2e=dict(value=K * B / (ms_e2e * 1e-3), unit="edges/s", h2d_bytes_per_step=B * 3 * 8, d2h_bytes_per_step=4,
                     ms_per_step=ms_e2e / K, ms_per_step_median=float(np.median(rep_e2e)) / K,
                     note="pinned host edges -> H2D, step, loss -> pinned host, all stream-ordered; one synchronize at the end of each repeat"
                          + ("; the H2D copy issued in step i carries batch i+1 (drawn ahead while batch i trains) and runs on a copy stream, the loss read-back on another" if pipelined else "")),
            gpu_launches=K * pipe.launches_per_step(), epoch=epoch_info,
            clocks=clock_info,
            roofline=scores_roofline(args.precision, S, B, N, D, scores_ms, scores_host_ms),
            roofline_kernels=kernel_rooflines,
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
        if world == 1 and not args.no_host_cpp:
            try:
                ms_cpp = host_cpp_ms(cfg, table, state, edges, min(K, 20), device, args.precision)
                line["host_cpp"] = dict(value=B / (ms_cpp * 1e-3), unit="edges/s", ms_per_step=ms_cpp,
                                        note="the reference's call sequence through the C++ host layer (getBatch -> train_batch -> updateEmbeddings), "
                                             "unfused and host-issued with one count read-back per batch; the headline path is the fused, "
                                             "graph-replayed launch sequence over the same C ABI")
            except Exception as ex:
                line["host_cpp"] = dict(unavailable=str(ex)[:160])
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


if __name__ == "__main__":
    main()
