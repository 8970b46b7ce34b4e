"""ctypes binding of the C ABI declared in include/ge2_b200.h.

Thin by design: tensors are torch CUDA tensors used as device memory, every wrapper passes raw pointers and the
current CUDA stream, checks the int status and raises Ge2Error.  No arithmetic happens on this side.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Optional

PKG = Path(__file__).resolve().parent

GE2_OK = 0
DECODER = {"DISTMULT": 0, "DOT": 0, "COMPLEX": 1}
PRECISION = {"fp32": 0, "f16": 1}
STATUS_BITS = {1: "id out of range", 2: "scan timeout", 4: "filter collision", 8: "bad index", 16: "pipeline timeout", 32: "peer timeout"}

EXPORTS = [
    "ge2_version", "ge2_last_cuda_error", "ge2_status_string", "ge2_check_device", "ge2_unique_workspace_bytes",
    "ge2_unique_bitmap", "ge2_pack_ids", "ge2_lp_workspace_bytes", "ge2_lp_step", "ge2_sparse_adagrad", "ge2_index_read",
    "ge2_index_add", "ge2_adagrad_scatter", "ge2_dense_adagrad", "ge2_sample_negatives", "ge2_remap_edges_to_slots",
    "ge2_copy_slabs", "ge2_unique_bitmap_static", "ge2_sample_batch", "ge2_advance_step", "ge2_dense_adagrad_peers",
    "ge2_enable_peer_access", "ge2_build_state_edges", "ge2_swap_begin", "ge2_swap_wait", "ge2_sample_batch_dev",
    "ge2_eval_workspace_bytes", "ge2_eval_ranks", "ge2_selected_neg_scores", "ge2_selected_neg_scores_backward",
    "ge2_tournament_select",
]


class Ge2Error(RuntimeError):
    pass


class LpDesc(C.Structure):
    _fields_ = [
        ("decoder", C.c_int32), ("has_relations", C.c_int32), ("use_inverse", C.c_int32), ("precision", C.c_int32),
        ("B", C.c_int32), ("C", C.c_int32), ("N", C.c_int32), ("D", C.c_int32), ("R", C.c_int32), ("phases", C.c_int32),
        ("U", C.c_int64),
        ("node_emb", C.c_void_p), ("row_index", C.c_void_p), ("emb_stride", C.c_int64),
        ("src_ids", C.c_void_p), ("rel_ids", C.c_void_p), ("dst_ids", C.c_void_p), ("edge_stride", C.c_int64), ("rel_stride", C.c_int64),
        ("dst_negs", C.c_void_p), ("src_negs", C.c_void_p),
        ("dst_filter", C.c_void_p), ("dst_filter_n", C.c_int64), ("src_filter", C.c_void_p), ("src_filter_n", C.c_int64),
        ("deg_sample_rows", C.c_void_p), ("n_deg", C.c_int32), ("flags", C.c_int32),
        ("rel", C.c_void_p), ("inv_rel", C.c_void_p),
        ("node_grad", C.c_void_p), ("rel_grad", C.c_void_p), ("inv_rel_grad", C.c_void_p), ("loss", C.c_void_p),
        ("pos_scores", C.c_void_p), ("neg_scores", C.c_void_p), ("inv_pos_scores", C.c_void_p), ("inv_neg_scores", C.c_void_p),
        ("status", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class EvalDesc(C.Structure):
    _fields_ = [
        ("decoder", C.c_int32), ("has_relations", C.c_int32), ("use_inverse", C.c_int32), ("D", C.c_int32),
        ("B", C.c_int64), ("num_nodes", C.c_int64), ("R", C.c_int64),
        ("node_emb", C.c_void_p), ("emb_stride", C.c_int64),
        ("src_ids", C.c_void_p), ("rel_ids", C.c_void_p), ("dst_ids", C.c_void_p), ("edge_stride", C.c_int64), ("rel_stride", C.c_int64),
        ("rel", C.c_void_p), ("inv_rel", C.c_void_p), ("neg_ids", C.c_void_p), ("num_negs", C.c_int64),
        ("dst_filter", C.c_void_p), ("dst_filter_n", C.c_int64), ("src_filter", C.c_void_p), ("src_filter_n", C.c_int64),
        ("dst_ranks", C.c_void_p), ("src_ranks", C.c_void_p), ("pos_scores", C.c_void_p), ("inv_pos_scores", C.c_void_p),
        ("status", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
    ]


class SwapDesc(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("flag_rows", C.POINTER(C.c_void_p)), ("epoch", C.c_uint64),
                ("wait_budget_us", C.c_uint32), ("num_pulls", C.c_int32), ("pull_src", C.POINTER(C.c_void_p)), ("pull_dst", C.POINTER(C.c_void_p)),
                ("slab_bytes", C.c_int64), ("status", C.c_void_p)]


_lib = None


def lib_path() -> Path:
    return Path(os.environ.get("GE2_B200_LIB", PKG / "libge2_b200.so"))


def load_library():
    """Loads libge2_b200.so (once).  Raises Ge2Error when it has not been built: there is no fallback path."""
    global _lib
    if _lib is not None:
        return _lib
    path = lib_path()
    if not path.exists():
        raise Ge2Error(f"{path} is missing: build it with `python ge-2_b200/build.py` (needs nvcc); no CPU fallback exists")
    lib = C.CDLL(str(path))
    lib.ge2_version.restype = C.c_char_p
    lib.ge2_status_string.restype = C.c_char_p
    lib.ge2_status_string.argtypes = [C.c_int]
    lib.ge2_unique_workspace_bytes.restype = C.c_size_t
    lib.ge2_unique_workspace_bytes.argtypes = [C.c_int64]
    lib.ge2_unique_bitmap.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_unique_bitmap_static.argtypes = [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_pack_ids.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_void_p, C.c_void_p]
    lib.ge2_lp_workspace_bytes.argtypes = [C.POINTER(LpDesc), C.POINTER(C.c_size_t)]
    lib.ge2_lp_step.argtypes = [C.POINTER(LpDesc), C.c_void_p]
    lib.ge2_sparse_adagrad.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_float, C.c_void_p]
    lib.ge2_index_read.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_index_add.argtypes = [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_adagrad_scatter.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_void_p, C.c_int32, C.c_float,
                                        C.c_int32, C.c_void_p, C.c_void_p]
    lib.ge2_dense_adagrad.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_float, C.c_float, C.c_float, C.c_int32, C.c_void_p]
    lib.ge2_dense_adagrad_peers.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_int32, C.c_int32, C.c_int64, C.c_void_p, C.c_float,
                                            C.c_float, C.c_float, C.c_uint32, C.c_void_p, C.c_void_p]
    lib.ge2_enable_peer_access.argtypes = [C.c_int32]
    lib.ge2_sample_negatives.argtypes = [C.c_void_p, C.c_void_p, C.c_int64, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                         C.c_uint64, C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_sample_batch.argtypes = [C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                     C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_sample_batch_dev.argtypes = [C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int64, C.c_int32,
                                         C.c_uint64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_build_state_edges.argtypes = [C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.POINTER(C.c_int64), C.c_int32, C.c_void_p, C.c_int32, C.c_int64,
                                          C.c_uint64, C.c_void_p, C.POINTER(C.c_int64), C.c_void_p, C.c_void_p]
    lib.ge2_swap_begin.argtypes = [C.POINTER(SwapDesc), C.c_void_p]
    lib.ge2_swap_wait.argtypes = [C.c_void_p, C.c_void_p]
    lib.ge2_advance_step.argtypes = [C.c_void_p, C.c_int32, C.c_void_p]
    lib.ge2_remap_edges_to_slots.argtypes = [C.c_void_p, C.c_int64, C.c_int32, C.c_void_p, C.c_int32, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_copy_slabs.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_int32), C.c_int32, C.c_int64, C.c_void_p]
    lib.ge2_check_device.argtypes = [C.c_int]
    lib.ge2_selected_neg_scores.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                            C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_selected_neg_scores_backward.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                                     C.c_int64, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]
    lib.ge2_tournament_select.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64, C.c_int,
                                          C.c_void_p, C.c_void_p, C.c_void_p]
    _lib = lib
    return lib


def check(rc: int, what: str):
    if rc != GE2_OK:
        lib = load_library()
        msg = lib.ge2_status_string(rc).decode()
        extra = f" (cudaError {lib.ge2_last_cuda_error()})" if rc == 2 else ""
        raise Ge2Error(f"{what}: {msg}{extra}")


def ptr(t) -> Optional[int]:
    return None if t is None else t.data_ptr()


def cur_stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def decode_status(word: int) -> str:
    return ", ".join(name for bit, name in STATUS_BITS.items() if word & bit) or "clean"


# ------------------------------------------------------------------------------------------------------------
# wrappers (device tensors in, device tensors out; nothing is synchronised)
# ------------------------------------------------------------------------------------------------------------
def unique_workspace(domain: int, device):
    import torch

    return torch.empty(load_library().ge2_unique_workspace_bytes(domain), dtype=torch.uint8, device=device)


def unique_bitmap(ids, domain: int, workspace=None, out_unique=None, out_inverse=None, out_count=None):
    """ids: int64 CUDA [n].  Returns (unique[capacity], inverse[n], count[2] int32) -- count[0] distinct ids (device)."""
    import torch

    lib = load_library()
    n = ids.numel()
    dev = ids.device
    if workspace is None:
        workspace = unique_workspace(domain, dev)
    if out_unique is None:
        out_unique = torch.empty(max(1, min(n, domain)), dtype=torch.int64, device=dev)
    if out_inverse is None:
        out_inverse = torch.empty(max(1, n), dtype=torch.int64, device=dev)
    if out_count is None:
        out_count = torch.empty(2, dtype=torch.int32, device=dev)
    check(lib.ge2_unique_bitmap(ptr(ids), n, domain, ptr(workspace), workspace.numel(), ptr(out_unique), ptr(out_inverse), ptr(out_count),
                                cur_stream()), "ge2_unique_bitmap")
    return out_unique, out_inverse[:n], out_count


UNIQUE_STATIC_MAX_DOMAIN = 4194304


def unique_bitmap_static(ids, domain: int, out_unique, out_inverse, out_count):
    """Unique-map with the library's built-in scratch: for callers that may not allocate device memory.  Every buffer is
    supplied by the caller; domain is limited to UNIQUE_STATIC_MAX_DOMAIN.  Calls that overlap on the GPU race."""
    check(load_library().ge2_unique_bitmap_static(ptr(ids), ids.numel(), domain, ptr(out_unique), ptr(out_inverse), ptr(out_count),
                                                  cur_stream()), "ge2_unique_bitmap_static")


def make_lp_desc(*, decoder, precision, B, Cn, N, D, R, U, node_emb, row_index=None, emb_stride=None, src_ids, dst_ids, rel_ids=None,
                 edge_stride=1, rel_stride=1, dst_negs, src_negs=None, dst_filter=None, src_filter=None, deg_sample_rows=None, n_deg=0,
                 rel=None, inv_rel=None, node_grad, rel_grad=None, inv_rel_grad=None, loss, pos_scores=None, neg_scores=None,
                 inv_pos_scores=None, inv_neg_scores=None, status=None, workspace=None, node_grad_is_zero=False) -> LpDesc:
    d = LpDesc()
    d.decoder = DECODER[decoder] if isinstance(decoder, str) else decoder
    d.precision = PRECISION[precision] if isinstance(precision, str) else precision
    d.has_relations = 1 if rel_ids is not None else 0
    d.use_inverse = 1 if (src_negs is not None and inv_rel is not None) else 0
    d.B, d.C, d.N, d.D, d.R, d.U = B, Cn, N, D, R, U
    d.node_emb, d.row_index = ptr(node_emb), ptr(row_index)
    d.emb_stride = emb_stride if emb_stride is not None else D
    d.src_ids, d.rel_ids, d.dst_ids = ptr(src_ids), ptr(rel_ids), ptr(dst_ids)
    d.edge_stride, d.rel_stride = edge_stride, rel_stride
    d.dst_negs, d.src_negs = ptr(dst_negs), ptr(src_negs)
    d.dst_filter, d.dst_filter_n = ptr(dst_filter), (0 if dst_filter is None else dst_filter.shape[0])
    d.src_filter, d.src_filter_n = ptr(src_filter), (0 if src_filter is None else src_filter.shape[0])
    if d.dst_filter_n == 0:
        d.dst_filter = None
    if d.src_filter_n == 0:
        d.src_filter = None
    d.deg_sample_rows, d.n_deg = ptr(deg_sample_rows), n_deg
    d.flags = 1 if node_grad_is_zero else 0
    d.rel, d.inv_rel = ptr(rel), ptr(inv_rel)
    d.node_grad, d.rel_grad, d.inv_rel_grad, d.loss = ptr(node_grad), ptr(rel_grad), ptr(inv_rel_grad), ptr(loss)
    d.pos_scores, d.neg_scores = ptr(pos_scores), ptr(neg_scores)
    d.inv_pos_scores, d.inv_neg_scores = ptr(inv_pos_scores), ptr(inv_neg_scores)
    d.status = ptr(status)
    if workspace is not None:
        d.workspace, d.workspace_bytes = ptr(workspace), workspace.numel()
    return d


def lp_workspace_bytes(desc: LpDesc) -> int:
    out = C.c_size_t(0)
    check(load_library().ge2_lp_workspace_bytes(C.byref(desc), C.byref(out)), "ge2_lp_workspace_bytes")
    return out.value


def lp_step(desc: LpDesc):
    check(load_library().ge2_lp_step(C.byref(desc), cur_stream()), "ge2_lp_step")


def sparse_adagrad(grad, state_local, lr: float, out_delta=None, out_state_update=None, rows_dev=None):
    import torch

    rows, D = grad.shape
    if out_delta is None:
        out_delta = torch.empty_like(grad)
    if out_state_update is None:
        out_state_update = torch.empty_like(grad)
    check(load_library().ge2_sparse_adagrad(ptr(grad), ptr(state_local), ptr(out_delta), ptr(out_state_update), rows, ptr(rows_dev), D, lr,
                                            cur_stream()), "ge2_sparse_adagrad")
    return out_delta, out_state_update


def index_read(table, ids, n_dev=None, out=None, status=None):
    import torch

    n, D = ids.numel(), table.shape[1]
    if out is None:
        out = torch.empty((n, D), dtype=table.dtype, device=table.device)
    check(load_library().ge2_index_read(ptr(table), table.shape[0], ptr(ids), n, ptr(n_dev), D, ptr(out), ptr(status), cur_stream()),
          "ge2_index_read")
    return out


def index_add(table, ids, values, n_dev=None, status=None):
    n, D = ids.numel(), table.shape[1]
    check(load_library().ge2_index_add(ptr(table), table.shape[0], ptr(ids), n, ptr(n_dev), D, ptr(values), ptr(status), cur_stream()),
          "ge2_index_add")


def adagrad_scatter(table, state, unique_ids, node_grad, lr: float, U=None, U_dev=None, clear_grad=False, status=None):
    D = table.shape[1]
    U = unique_ids.numel() if U is None else U
    check(load_library().ge2_adagrad_scatter(ptr(table), ptr(state), table.shape[0], ptr(unique_ids), U, ptr(U_dev), ptr(node_grad), D, lr,
                                             1 if clear_grad else 0, ptr(status), cur_stream()), "ge2_adagrad_scatter")


def dense_adagrad(param, sum_state, grad, lr: float, eps: float = 1e-10, grad_scale: float = 1.0, clear_grad=False):
    check(load_library().ge2_dense_adagrad(ptr(param), ptr(sum_state), ptr(grad), param.numel(), lr, eps, grad_scale, 1 if clear_grad else 0,
                                           cur_stream()), "ge2_dense_adagrad")


def dense_adagrad_peers(param, sum_state, peer_ptrs, rank: int, numel: int, step_dev, lr: float, status, eps: float = 1e-10,
                        grad_scale: float = 1.0, wait_budget_us: int = 0):
    """peer_ptrs: list of device addresses (ints), one per rank, of the ranks' gradient buffers as mapped in this process.
    wait_budget_us: how long to wait for the other ranks' announcements (0 = the library's default of 4 s)."""
    arr = (C.c_void_p * len(peer_ptrs))(*peer_ptrs)
    check(load_library().ge2_dense_adagrad_peers(ptr(param), ptr(sum_state), arr, len(peer_ptrs), rank, numel, ptr(step_dev), lr, eps, grad_scale,
                                                 wait_budget_us, ptr(status), cur_stream()), "ge2_dense_adagrad_peers")


def enable_peer_access(peer_device: int):
    check(load_library().ge2_enable_peer_access(peer_device), "ge2_enable_peer_access")


def sample_negatives(src_ids, dst_ids, edge_stride, B, Cn, N, n_deg, domain, want_src, seed, batch_index, out_packed, out_deg_rows):
    check(load_library().ge2_sample_negatives(ptr(src_ids), ptr(dst_ids), edge_stride, B, Cn, N, n_deg, domain, 1 if want_src else 0, seed,
                                              batch_index, ptr(out_packed), ptr(out_deg_rows), cur_stream()), "ge2_sample_negatives")


def sample_batch(edges, num_batches, step_dev, B, Cn, N, n_deg, domain, want_src, seed, out_packed, out_deg_rows, out_rel):
    check(load_library().ge2_sample_batch(ptr(edges), edges.shape[1], num_batches, ptr(step_dev), B, Cn, N, n_deg, domain, 1 if want_src else 0,
                                          seed, ptr(out_packed), ptr(out_deg_rows), ptr(out_rel), cur_stream()), "ge2_sample_batch")


def sample_batch_dev(edges, num_batches_dev, step_dev, B, Cn, N, n_deg, domain, want_src, seed, out_packed, out_deg_rows, out_rel):
    """sample_batch with the number of batches of the resident edge list read from device memory (int64 scalar tensor)."""
    check(load_library().ge2_sample_batch_dev(ptr(edges), edges.shape[1], ptr(num_batches_dev), ptr(step_dev), B, Cn, N, n_deg, domain,
                                              1 if want_src else 0, seed, ptr(out_packed), ptr(out_deg_rows), ptr(out_rel), cur_stream()),
          "ge2_sample_batch_dev")


def build_state_edges(edges_sorted, bucket_begin, bucket_len, partition_to_slot, partition_size: int, seed: int, out_edges, status=None) -> int:
    """Edge list of one partition-buffer state: the named buckets of the bucket-sorted list, concatenated, remapped to buffer
    slots and shuffled, in one launch.  bucket_begin / bucket_len: Python lists.  Returns the number of rows written."""
    nb = len(bucket_begin)
    beg = (C.c_int64 * max(nb, 1))(*bucket_begin)
    ln = (C.c_int64 * max(nb, 1))(*bucket_len)
    total = C.c_int64(0)
    assert sum(bucket_len) <= out_edges.shape[0]
    check(load_library().ge2_build_state_edges(ptr(edges_sorted), edges_sorted.shape[1], beg, ln, nb, ptr(partition_to_slot), partition_to_slot.numel(),
                                               partition_size, seed, ptr(out_edges), C.byref(total), ptr(status), cur_stream()), "ge2_build_state_edges")
    return total.value


def swap_begin(world: int, rank: int, flag_row_ptrs, epoch: int, pulls, slab_bytes: int, status, wait_budget_us: int = 0, stream=None):
    """pulls: list of (src address, dst address) ints.  flag_row_ptrs: list of `world` addresses (None when world == 1)."""
    d = SwapDesc()
    d.world, d.rank, d.epoch, d.wait_budget_us = world, rank, epoch, wait_budget_us
    rows = (C.c_void_p * max(world, 1))(*(flag_row_ptrs or [None]))
    d.flag_rows = C.cast(rows, C.POINTER(C.c_void_p))
    n = len(pulls)
    src = (C.c_void_p * max(n, 1))(*[p[0] for p in pulls])
    dst = (C.c_void_p * max(n, 1))(*[p[1] for p in pulls])
    d.num_pulls, d.pull_src, d.pull_dst = n, C.cast(src, C.POINTER(C.c_void_p)), C.cast(dst, C.POINTER(C.c_void_p))
    d.slab_bytes, d.status = slab_bytes, ptr(status)
    check(load_library().ge2_swap_begin(C.byref(d), cur_stream() if stream is None else stream), "ge2_swap_begin")


def eval_ranks(decoder, node_emb, edges, rel=None, inv_rel=None, dst_filter=None, src_filter=None, neg_ids=None, status=None):
    """Ranks of edges[B, 2|3] (rows of node_emb) against every node (or the rows neg_ids lists): (dst_ranks, src_ranks or None).
    Filter pairs are [F, 2] int64 (edge row, candidate column)."""
    import torch

    lib = load_library()
    lib.ge2_eval_workspace_bytes.restype = C.c_size_t
    lib.ge2_eval_workspace_bytes.argtypes = [C.POINTER(EvalDesc)]
    lib.ge2_eval_ranks.argtypes = [C.POINTER(EvalDesc), C.c_void_p]
    B, cols = edges.shape
    dev = node_emb.device
    d = EvalDesc()
    d.decoder = {"DISTMULT": 0, "DOT": 0, "COMPLEX": 1}[decoder]
    d.has_relations = int(cols == 3 and rel is not None)
    d.use_inverse = int(d.has_relations and inv_rel is not None)
    d.D, d.B, d.num_nodes = node_emb.shape[1], B, node_emb.shape[0]
    d.R = rel.shape[0] if rel is not None else 0
    d.node_emb, d.emb_stride = ptr(node_emb), node_emb.stride(0)
    d.src_ids, d.dst_ids = ptr(edges), edges.data_ptr() + 8 * (cols - 1)
    d.rel_ids = edges.data_ptr() + 8 if d.has_relations else None
    d.edge_stride = d.rel_stride = cols
    d.rel, d.inv_rel = ptr(rel), ptr(inv_rel) if d.use_inverse else None
    d.neg_ids, d.num_negs = ptr(neg_ids), (neg_ids.numel() if neg_ids is not None else 0)
    d.dst_filter, d.dst_filter_n = ptr(dst_filter), (dst_filter.shape[0] if dst_filter is not None else 0)
    d.src_filter, d.src_filter_n = ptr(src_filter), (src_filter.shape[0] if src_filter is not None else 0)
    dst_ranks = torch.zeros(B, dtype=torch.int64, device=dev)
    src_ranks = torch.zeros(B, dtype=torch.int64, device=dev) if d.use_inverse else None
    d.dst_ranks, d.src_ranks = ptr(dst_ranks), ptr(src_ranks)
    d.status = ptr(status)
    ws = torch.empty(int(lib.ge2_eval_workspace_bytes(C.byref(d))), dtype=torch.uint8, device=dev)
    d.workspace, d.workspace_bytes = ws.data_ptr(), ws.numel()
    check(lib.ge2_eval_ranks(C.byref(d), cur_stream()), "ge2_eval_ranks")
    return dst_ranks, src_ranks


SELECTED_KINDS = {"DOT": 1, "L2": 2}


def _selected_shapes(chunked, negatives, selected):
    chunks, rows, D = chunked.shape
    assert negatives.shape[0] == chunks and negatives.shape[2] == D and selected.shape[0] == chunks
    assert chunked.is_contiguous() and negatives.is_contiguous() and selected.is_contiguous()
    K = selected.shape[1] // max(rows, 1)
    assert selected.shape[1] == rows * K, "selected must be [chunks, rows_per_chunk * num_selected]"
    return chunks, rows, negatives.shape[1], K, D


def selected_neg_scores(kind, chunked, negatives, selected, status=None):
    """Scores [chunks * rows, K] of chunked [chunks, rows, D] against negatives[chunk, selected[chunk, row * K + k]]."""
    import torch

    chunks, rows, N, K, D = _selected_shapes(chunked, negatives, selected)
    out = torch.empty((chunks * rows, K), dtype=torch.float32, device=chunked.device)
    check(load_library().ge2_selected_neg_scores(SELECTED_KINDS[kind], ptr(chunked), ptr(negatives), ptr(selected), chunks, rows, N, K, D,
                                                 ptr(out), ptr(status), cur_stream()), "ge2_selected_neg_scores")
    return out


def selected_neg_scores_backward(kind, grad_out, chunked, negatives, selected, status=None):
    """(grad_chunked, grad_negatives) of selected_neg_scores for grad_out [chunks * rows, K]."""
    import torch

    chunks, rows, N, K, D = _selected_shapes(chunked, negatives, selected)
    assert tuple(grad_out.shape) == (chunks * rows, K) and grad_out.is_contiguous()
    grad_chunked, grad_negatives = torch.empty_like(chunked), torch.empty_like(negatives)
    check(load_library().ge2_selected_neg_scores_backward(SELECTED_KINDS[kind], ptr(grad_out), ptr(chunked), ptr(negatives), ptr(selected),
                                                          chunks, rows, N, K, D, ptr(grad_chunked), ptr(grad_negatives), ptr(status),
                                                          cur_stream()), "ge2_selected_neg_scores_backward")
    return grad_chunked, grad_negatives


def tournament_select(chunked, negatives, num_selected, score_chunked=None, score_negatives=None):
    """Per row and group of num_negs / num_selected consecutive negatives the best-scoring one: (scores [chunks * rows,
    num_selected], columns [chunks, rows * num_selected]).  score_* default to the selector's tensors."""
    import torch

    chunks, rows, D = chunked.shape
    N = negatives.shape[1]
    assert negatives.shape[0] == chunks and negatives.shape[2] == D and chunked.is_contiguous() and negatives.is_contiguous()
    for t, like in ((score_chunked, chunked), (score_negatives, negatives)):
        assert t is None or (t.shape == like.shape and t.is_contiguous())
    scores = torch.empty((chunks * rows, num_selected), dtype=torch.float32, device=chunked.device)
    idx = torch.empty((chunks, rows * num_selected), dtype=torch.int64, device=chunked.device)
    check(load_library().ge2_tournament_select(ptr(chunked), ptr(negatives), ptr(score_chunked), ptr(score_negatives), chunks, rows, N,
                                               num_selected, D, ptr(scores), ptr(idx), cur_stream()), "ge2_tournament_select")
    return scores, idx


def swap_wait(swap_stream: int, compute_stream: int):
    check(load_library().ge2_swap_wait(swap_stream, compute_stream), "ge2_swap_wait")


def advance_step(step_dev, n=1):
    check(load_library().ge2_advance_step(ptr(step_dev), n, cur_stream()), "ge2_advance_step")


def remap_edges_to_slots(edges, partition_to_slot, partition_size, out=None, status=None):
    import torch

    n, cols = edges.shape
    if out is None:
        out = torch.empty_like(edges)
    check(load_library().ge2_remap_edges_to_slots(ptr(edges), n, cols, ptr(partition_to_slot), partition_to_slot.numel(), partition_size,
                                                  ptr(out), ptr(status), cur_stream()), "ge2_remap_edges_to_slots")
    return out


def copy_slabs(src, dst, moves, slab_floats):
    arr = (C.c_int32 * (2 * len(moves)))(*[v for m in moves for v in m])
    check(load_library().ge2_copy_slabs(ptr(src), ptr(dst), arr, len(moves), slab_floats, cur_stream()), "ge2_copy_slabs")
