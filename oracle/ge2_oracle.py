"""CPU restatement of the reference's per-batch embedding-training path.  TEST INFRASTRUCTURE ONLY.

Only tests/, the smoke check and the CPU-baseline leg of bench.py may import this module; the product
path never does (it fails loudly when the CUDA library is missing).

Every function cites the reference file:line it follows (paths relative to gege/src/ of the reference
project).  Integer work is restated bit-exactly; floating-point work is restated in float32 with the same
operation order wherever the reference's order is defined (element-wise ops), and in float64-accumulated
form for the contractions, whose accumulation order inside the BLAS the reference calls is unspecified.

Parity pin: the reference has no golden vectors or known-answer tests for this path.  The restatement is
pinned instead against outputs of the reference's own code run on CPU (oracle/_ref, built by
oracle/Makefile from the reference sources); tests/golden/ holds fixtures generated that way by
tests/golden/make_golden.py.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np

MASK_VALUE = np.float32(-1e9)  # cpp/src/data/samplers/negative.cpp:572
ADAGRAD_EPS = np.float32(1e-10)  # cpp/src/data/batch.cpp:266, python/tools/configuration/datatypes.py:58


# --------------------------------------------------------------------------------------------------
# (1) unique-map
# --------------------------------------------------------------------------------------------------
def unique_map_bitmap(ids: np.ndarray, domain: int):
    """Bitmap backend of map_tensors_unique_inverse_cuda (cuda/src/common/unique_map_cuda.cu:446-517,771-882).

    mark bit `key` in a domain-sized bitset (:446-459); popcount per 64-bit word (:461-466); exclusive scan
    of the word counts (:825-830); emit ids in ascending order per word (:468-479);
    inverse[i] = word_offset[key>>6] + popc(word & lowmask(key&63)) (:481-517).
    Returns (unique_ids int64 ascending, inverse int64, invalid flag).  invalid=True (an id outside
    [0, domain)) is where the reference falls back to its sort backend (:841-844).
    """
    ids = np.asarray(ids, dtype=np.int64).reshape(-1)
    n = ids.shape[0]
    if n == 0:
        return np.empty(0, np.int64), np.empty(0, np.int64), False
    invalid = bool(((ids < 0) | (ids >= domain)).any())
    if invalid:
        return None, None, True
    num_words = (domain + 63) >> 6
    words = np.zeros(num_words, dtype=np.uint64)
    np.bitwise_or.at(words, ids >> 6, np.uint64(1) << (ids & 63).astype(np.uint64))
    bits = np.unpackbits(words.view(np.uint8).reshape(num_words, 8), axis=1, bitorder="little")  # [W,64], bit b of word w
    counts = bits.sum(axis=1).astype(np.int64)
    offsets = np.zeros(num_words, dtype=np.int64)
    np.cumsum(counts[:-1], out=offsets[1:])
    w_idx, b_idx = np.nonzero(bits)  # row-major => ascending (word, bit)
    unique_ids = (w_idx.astype(np.int64) << 6) + b_idx.astype(np.int64)
    below = np.cumsum(bits, axis=1) - bits  # popc(word & lowmask(bit)) for every bit position
    inverse = offsets[ids >> 6] + below[ids >> 6, ids & 63].astype(np.int64)
    return unique_ids, inverse, False


def unique_map_sort(ids: np.ndarray):
    """unique_with_inverse_compat (cpp/src/common/util.cpp:100-111): sort, unique_consecutive, scatter ranks back.
    This is the reference's CPU path and the fallback of every CUDA backend; same result as the bitmap backend."""
    ids = np.asarray(ids, dtype=np.int64).reshape(-1)
    u, inv = np.unique(ids, return_inverse=True)
    return u.astype(np.int64), inv.astype(np.int64).reshape(-1)


def map_tensors(id_lists, domain: int = -1):
    """map_tensors (cpp/src/common/util.cpp:311-387): concatenate the 1-D id tensors (:113-159), unique-map them,
    split the inverse back into one mapped tensor per input (:375-380)."""
    flat = [np.asarray(t, dtype=np.int64).reshape(-1) for t in id_lists]
    all_ids = np.concatenate(flat) if flat else np.empty(0, np.int64)
    if domain > 0:
        u, inv, invalid = unique_map_bitmap(all_ids, domain)
        if invalid:
            u, inv = unique_map_sort(all_ids)
    else:
        u, inv = unique_map_sort(all_ids)
    out, off = [], 0
    for t in flat:
        out.append(inv[off : off + t.shape[0]])
        off += t.shape[0]
    return u, out


# --------------------------------------------------------------------------------------------------
# negative-sample bookkeeping (producer side; kept by the reference, restated for the parity harness)
# --------------------------------------------------------------------------------------------------
def chunk_size(batch: int, num_chunks: int) -> int:
    """ceil(B / C): decoder_methods.cpp:772 and comparators.cpp:64 use float, negative.cpp:223 double."""
    return int(math.ceil(np.float32(batch) / np.float32(num_chunks)))


def deg_negative_local_filter(sample_edge_ids: np.ndarray, batch: int) -> np.ndarray:
    """deg_negative_local_filter (cpp/src/data/samplers/negative.cpp:215-263).

    sample_edge_ids [C, N_deg]: batch row each degree-based negative was drawn from.  An entry whose row lies in
    the chunk that sampled it gives a filter pair (row, column); nonzero() order is row-major over [C, N_deg]."""
    s = np.asarray(sample_edge_ids, dtype=np.int64)
    if s.size == 0:
        return np.empty((0, 2), np.int64)
    C, nd = s.shape
    cs = int(math.ceil(float(batch) / C))
    chunk_ids = np.floor(s.astype(np.float64) / float(cs)).astype(np.int64)
    mask = chunk_ids == np.arange(C, dtype=np.int64)[:, None]
    c_idx, col = np.nonzero(mask)
    rows = s.reshape(-1)[c_idx * nd + col]
    return np.stack([rows, col], axis=1).astype(np.int64)


def materialize_negatives(edges: np.ndarray, uniform_ids: Optional[np.ndarray], sample_edge_ids: Optional[np.ndarray], inverse: bool):
    """materialize_negative_output (negative.cpp:136-169, degree samples :97-102): ids = cat(deg, uniform) along dim 1;
    degree ids are the dst column (src column when corrupting sources) of the sampled batch edges."""
    parts = []
    if sample_edge_ids is not None and sample_edge_ids.size:
        col = edges[:, 0] if inverse else edges[:, -1]
        parts.append(col[sample_edge_ids.reshape(-1)].reshape(sample_edge_ids.shape))
    if uniform_ids is not None and uniform_ids.size:
        parts.append(uniform_ids)
    return np.concatenate(parts, axis=1).astype(np.int64)


# --------------------------------------------------------------------------------------------------
# (2) decoder forward + softmax-CE loss + backward
# --------------------------------------------------------------------------------------------------
def _apply_relation(kind: str, e: np.ndarray, r: Optional[np.ndarray]) -> np.ndarray:
    """HadamardOperator / ComplexHadamardOperator (cpp/src/nn/decoders/edge/relation_operators.cpp:3-31)."""
    if r is None:
        return e
    if kind == "DISTMULT":
        return e * r
    D = e.shape[1]
    h = D // 2
    out = np.zeros_like(e)
    out[:, :h] = e[:, :h] * r[:, :h] - e[:, h:] * r[:, h:]
    out[:, h:] = e[:, :h] * r[:, h:] + e[:, h:] * r[:, :h]
    return out


def _apply_relation_backward(kind: str, e, r, d_out):
    """Gradient of _apply_relation w.r.t. (e, r): what autograd derives from relation_operators.cpp:3-31."""
    if kind == "DISTMULT":
        return d_out * r, d_out * e
    D = e.shape[1]
    h = D // 2
    gr, gi = d_out[:, :h], d_out[:, h:]
    de = np.empty_like(e)
    dr = np.empty_like(e)
    de[:, :h] = gr * r[:, :h] + gi * r[:, h:]
    de[:, h:] = -gr * r[:, h:] + gi * r[:, :h]
    dr[:, :h] = gr * e[:, :h] + gi * e[:, h:]
    dr[:, h:] = -gr * e[:, h:] + gi * e[:, :h]
    return de, dr


def _side(Q, other, neg_emb, filt, C, acc):
    """One corruption side: positive scores, chunked negative scores, mask, softmax-CE, gradients.

    DotCompare (comparators.cpp:128-138) with pad_and_reshape (:62-75): rows padded with zero rows up to C*ceil(B/C);
    pos padded with 0 (decoder_methods.cpp:1089-1097); apply_score_filter (negative.cpp:570-575) writes -1e9;
    SoftmaxCrossEntropy with SUM reduction (loss.cpp:46-63): l_i = -pos_i + log(exp(pos_i) + sum_j exp(neg_ij)).
    """
    B, D = Q.shape
    N = neg_emb.shape[1]
    npc = chunk_size(B, C)
    Bp = npc * C
    Qp = np.zeros((Bp, D), acc)
    Qp[:B] = Q
    pos = np.zeros(Bp, acc)
    pos[:B] = (Q.astype(acc) * other.astype(acc)).sum(-1)
    Qc = Qp.reshape(C, npc, D)
    neg = np.einsum("cid,cjd->cij", Qc, neg_emb.astype(acc)).reshape(Bp, N)
    neg32 = neg.astype(np.float32)
    pos32 = pos.astype(np.float32)
    if filt is not None and len(filt):
        neg[filt[:, 0], filt[:, 1]] = acc(MASK_VALUE)
        neg32[filt[:, 0], filt[:, 1]] = MASK_VALUE
    m = np.maximum(neg.max(axis=1), pos)
    z = np.exp(pos - m) + np.exp(neg - m[:, None]).sum(axis=1)
    lse = m + np.log(z)
    loss = (lse - pos).sum()
    d_pos = np.exp(pos - lse) - 1.0
    d_neg = np.exp(neg - lse[:, None])
    if filt is not None and len(filt):
        d_neg[filt[:, 0], filt[:, 1]] = 0.0  # index_put_ overwrote those entries: no gradient flows to them
    d_negc = d_neg.reshape(C, npc, N)
    dQ = np.einsum("cij,cjd->cid", d_negc, neg_emb.astype(acc)).reshape(Bp, D)[:B] + d_pos[:B, None] * other.astype(acc)
    d_other = d_pos[:B, None] * Q.astype(acc)
    d_negemb = np.einsum("cij,cid->cjd", d_negc, Qc)
    return pos32[:Bp], neg32, loss, dQ, d_other, d_negemb


@dataclass
class LPResult:
    pos_scores: np.ndarray
    neg_scores: np.ndarray
    inv_pos_scores: Optional[np.ndarray]
    inv_neg_scores: Optional[np.ndarray]
    loss: float
    node_grad: np.ndarray
    rel_grad: Optional[np.ndarray]
    inv_rel_grad: Optional[np.ndarray]


def lp_train_forward_backward(kind, edges, node_emb, rel, inv_rel, dst_negs, src_negs=None, dst_filter=None, src_filter=None,
                              acc=np.float64) -> LPResult:
    """Model::train_batch's forward_lp + loss + backward for CORRUPT_NODE / RNS (cpp/src/nn/model.cpp:318-397;
    cpp/src/nn/decoders/edge/decoder_methods.cpp:724-806,933-946).

    kind: "DISTMULT" | "COMPLEX"; a 2-column edge list is the relation-free ("Dot") case (decoder_methods.cpp:717-719).
    edges: [B,2|3] int64 batch-local ids (src[,rel],dst); node_emb: [U,D] f32; rel/inv_rel: [R,D] f32 or None;
    dst_negs/src_negs: [C,N] int64 batch-local ids; filters: [F,2] int64 (row, col) or None.
    Gradients are reduced over duplicate ids exactly as index_select's backward does (sum).
    """
    edges = np.asarray(edges, np.int64)
    has_rel = edges.shape[1] == 3
    src_ids, dst_ids = edges[:, 0], edges[:, -1]
    E = node_emb.astype(np.float32)
    U, D = E.shape
    C, N = dst_negs.shape
    src, dst = E[src_ids], E[dst_ids]
    node_grad = np.zeros((U, D), acc)
    rel_grad = inv_rel_grad = None

    r = rel[edges[:, 1]] if has_rel else None
    Q = _apply_relation(kind, src, r)
    pos, neg, loss, dQ, d_dst, d_neg = _side(Q, dst, E[dst_negs.reshape(-1)].reshape(C, N, D), dst_filter, C, acc)
    if has_rel:
        d_src, d_r = _apply_relation_backward(kind, src.astype(acc), r.astype(acc), dQ)
        rel_grad = np.zeros(rel.shape, acc)
        np.add.at(rel_grad, edges[:, 1], d_r)
    else:
        d_src = dQ
    np.add.at(node_grad, src_ids, d_src)
    np.add.at(node_grad, dst_ids, d_dst)
    np.add.at(node_grad, dst_negs.reshape(-1), d_neg.reshape(C * N, D))

    ipos = ineg = None
    if has_rel and inv_rel is not None and src_negs is not None:
        ir = inv_rel[edges[:, 1]]
        Qi = _apply_relation(kind, dst, ir)
        ipos, ineg, iloss, dQi, d_src2, d_neg2 = _side(Qi, src, E[src_negs.reshape(-1)].reshape(C, N, D), src_filter, C, acc)
        loss = iloss + loss  # model.cpp:386 lhs + rhs
        d_dst2, d_ir = _apply_relation_backward(kind, dst.astype(acc), ir.astype(acc), dQi)
        inv_rel_grad = np.zeros(inv_rel.shape, acc)
        np.add.at(inv_rel_grad, edges[:, 1], d_ir)
        np.add.at(node_grad, dst_ids, d_dst2)
        np.add.at(node_grad, src_ids, d_src2)
        np.add.at(node_grad, src_negs.reshape(-1), d_neg2.reshape(C * N, D))

    f32 = lambda a: None if a is None else a.astype(np.float32)
    return LPResult(pos, neg, ipos, ineg, float(loss), f32(node_grad), f32(rel_grad), f32(inv_rel_grad))


# --------------------------------------------------------------------------------------------------
# (3) sparse Adagrad + scatter, dense Adagrad
# --------------------------------------------------------------------------------------------------
def sparse_adagrad(grad: np.ndarray, state: np.ndarray, lr: float):
    """Batch::accumulateGradients (cpp/src/data/batch.cpp:264-266), float32, same operation order:
    upd = g*g; state_local = state + upd; delta = -lr * (g / (sqrt(state_local) + 1e-10)).
    Returns (delta, upd): what indexAdd adds to the embedding table and to the state table."""
    g = grad.astype(np.float32)
    upd = g * g
    st = state.astype(np.float32) + upd
    delta = np.float32(-np.float32(lr)) * (g / (np.sqrt(st) + ADAGRAD_EPS))
    return delta.astype(np.float32), upd


def index_add(table: np.ndarray, ids: np.ndarray, values: np.ndarray):
    """InMemory::indexAdd CPU branch (cpp/src/storage/storage.cpp:1233-1246): table[ids[i]][j] += values[i][j]."""
    np.add.at(table, ids, values)
    return table


def dense_adagrad(param, grad, state, lr: float, eps: float = 1e-10):
    """AdagradOptimizer::step (cpp/src/nn/optim.cpp:109-143) with weight_decay = lr_decay = 0:
    sum += g*g; param += (-lr) * g / (sqrt(sum) + eps).  Float32 in place; returns (param, state)."""
    g = grad.astype(np.float32)
    state += g * g
    std = np.sqrt(state) + np.float32(eps)
    param += np.float32(-lr) * (g / std)
    return param, state


# --------------------------------------------------------------------------------------------------
# (4) partition buffer bookkeeping
# --------------------------------------------------------------------------------------------------
def map_edges_with_partition_slots(edges, partition_to_slot, partition_size: int):
    """GraphModelStorage::mapEdgesWithPartitionSlots_ (cpp/src/storage/graph_storage.cpp:270-303):
    local = slot[id // partition_size] * partition_size + id % partition_size for the src and dst columns.
    Raises when an endpoint's partition is not resident (slot < 0), as the reference throws."""
    edges = np.asarray(edges, np.int64)
    out = edges.copy()
    for col in (0, edges.shape[1] - 1):
        ids = edges[:, col]
        part = np.floor(ids.astype(np.float64) / float(partition_size)).astype(np.int64)
        slot = np.asarray(partition_to_slot, np.int64)[part]
        if (slot < 0).any():
            raise RuntimeError("Encountered edge endpoint outside current partition buffer state during arithmetic remap")
        out[:, col] = slot * partition_size + (ids - part * partition_size)
    return out


_M64 = (1 << 64) - 1


def _mix64(x: np.ndarray) -> np.ndarray:
    """splitmix64 finaliser on uint64 arrays (wrap-around arithmetic)."""
    with np.errstate(over="ignore"):
        x = x + np.uint64(0x9E3779B97F4A7C15)
        x = (x ^ (x >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        x = (x ^ (x >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return x ^ (x >> np.uint64(31))


def state_shuffle_permutation(n: int, seed: int) -> np.ndarray:
    """The permutation DataLoader::setActiveEdges draws with randperm (cpp/src/data/dataloader.cpp:613-616), restated as the
    fixed bijection the device path uses so that both sides can be compared bit for bit: four Feistel rounds over the
    smallest even number of bits covering n, walked until the value falls below n.  perm[j] = source row of output row j."""
    if n == 0:
        return np.empty(0, np.int64)
    bits = 2
    while bits < 62 and (1 << bits) < n:
        bits += 1
    if bits & 1:
        bits += 1
    half = np.uint64(bits // 2)
    mask = np.uint64((1 << (bits // 2)) - 1)
    key = np.uint64((seed * 0x9E3779B97F4A7C15 + 0x632BE59BD9B4E019) & _M64)
    x = np.arange(n, dtype=np.uint64)
    todo = np.ones(n, bool)
    with np.errstate(over="ignore"):
        while todo.any():
            v = x[todo]
            l, r = v >> half, v & mask
            for rnd in range(4):
                f = _mix64(key + np.uint64((rnd * 0xD1342543DE82EF95) & _M64) + r) & mask
                l, r = r, l ^ f
            v = (l << half) | r
            x[todo] = v
            todo[todo] = v >= np.uint64(n)
    return x.astype(np.int64)


def build_state_edges(edges_sorted, bucket_begin, bucket_len, partition_to_slot, partition_size: int, seed: int):
    """GraphModelStorage::updateInMemorySubGraph_ + DataLoader::setActiveEdges for one state
    (cpp/src/storage/graph_storage.cpp:938-1240, cpp/src/data/dataloader.cpp:524-633): the state's buckets of the bucket-sorted
    edge list concatenated in the given order, endpoints remapped to buffer slots (:270-303), rows shuffled."""
    parts = [np.asarray(edges_sorted[b:b + l]) for b, l in zip(bucket_begin, bucket_len)]
    cat = np.concatenate(parts, axis=0) if parts else np.empty((0, edges_sorted.shape[1]), np.int64)
    perm = state_shuffle_permutation(cat.shape[0], seed)
    return map_edges_with_partition_slots(cat[perm], partition_to_slot, partition_size)


def bucket_sort_edges(edges, num_partitions: int, partition_size: int):
    """The preprocessor's partitioned edge order (python/tools/preprocess/converters/partitioners/torch_partitioner.py:12-31):
    edges sorted (stably) by bucket id = src partition * P + dst partition, plus the P*P bucket sizes."""
    edges = np.asarray(edges, np.int64)
    b = (edges[:, 0] // partition_size) * num_partitions + edges[:, -1] // partition_size
    order = np.argsort(b, kind="stable")
    sizes = np.bincount(b, minlength=num_partitions * num_partitions).astype(np.int64)
    return edges[order], sizes


def relay_swap_plan(current_states, next_states):
    """Owner lookup of MemPartitionBufferStorage::performNextSwap, peer-relay branch (cpp/src/storage/storage.cpp:599-652).

    current_states / next_states: one list of resident partition ids per device (slot order).
    Returns, per device, a list of (slot, partition, src_device, src_slot): every slot of the next state is filled
    from the device and slot that hold the partition now.  Raises when a needed partition has no owner (:622-624)."""
    owner = {}
    for dev, st in enumerate(current_states):
        for slot, p in enumerate(st):
            owner[int(p)] = (dev, slot)
    plan = []
    for dev, st in enumerate(next_states):
        moves = []
        for slot, p in enumerate(st):
            if int(p) not in owner:
                raise RuntimeError(f"Peer relay could not find current owner for partition {int(p)}")
            moves.append((slot, int(p), owner[int(p)][0], owner[int(p)][1]))
        plan.append(moves)
    return plan


def relay_swap_apply(buffers, current_states, next_states, partition_rows):
    """Data movement of the peer-relay swap (storage.cpp:626-652, pointer flip :673): buffers[d] is device d's
    [capacity*partition_rows, D] slab array; returns the new per-device arrays (staging tensors)."""
    plan = relay_swap_plan(current_states, next_states)
    new = [np.empty_like(b) for b in buffers]
    for dev, moves in enumerate(plan):
        for slot, _p, sdev, sslot in moves:
            new[dev][slot * partition_rows : (slot + 1) * partition_rows] = buffers[sdev][sslot * partition_rows : (sslot + 1) * partition_rows]
    return new


def allreduce_relation_grads(grads_per_device):
    """Model::all_reduce (cpp/src/nn/model.cpp:174-204): each replica's gradient is divided by the device count, then
    summed over devices; a replica with no gradient contributes zeros (:182-187)."""
    g = len(grads_per_device)
    shape = next(x.shape for x in grads_per_device if x is not None)
    tot = np.zeros(shape, np.float32)
    for x in grads_per_device:
        if x is not None:
            tot += x.astype(np.float32) / np.float32(g)
    return tot


# --------------------------------------------------------------------------------------------------
# evaluation metric (used for the MRR parity check only)
# --------------------------------------------------------------------------------------------------
def ranks_from_scores(pos: np.ndarray, neg: np.ndarray) -> np.ndarray:
    """cpp/src/reporting/reporting.cpp:52-54: rank = (neg >= pos).sum(1) + 1."""
    return (neg >= pos[:, None]).sum(axis=1) + 1


def mrr(ranks: np.ndarray) -> float:
    """cpp/src/reporting/reporting.cpp:28: mean of float32 reciprocals."""
    return float((np.float32(1.0) / ranks.astype(np.float32)).mean())


def _fma_chain_scores(q: np.ndarray, e: np.ndarray) -> np.ndarray:
    """scores[i, n] = the float32 chain acc = fma(q[i, d], e[n, d], acc), d ascending.  Emulated through float64: the product
    of two float32 values is exact there, and rounding the float64 sum to float32 differs from a fused multiply-add only
    when that sum sits within 2^-29 of a float32 midpoint."""
    acc = np.zeros((q.shape[0], e.shape[0]), np.float32)
    q64, e64 = q.astype(np.float64), e.astype(np.float64)
    for d in range(q.shape[1]):
        acc = (acc.astype(np.float64) + q64[:, d, None] * e64[None, :, d]).astype(np.float32)
    return acc


def _fma_chain_rows(q: np.ndarray, e: np.ndarray) -> np.ndarray:
    acc = np.zeros(q.shape[0], np.float32)
    q64, e64 = q.astype(np.float64), e.astype(np.float64)
    for d in range(q.shape[1]):
        acc = (acc.astype(np.float64) + q64[:, d] * e64[:, d]).astype(np.float32)
    return acc


def eval_ranks(kind, table, rel, inv_rel, edges, dst_filter=None, src_filter=None, neg_ids=None):
    """Filtered link-prediction ranks of `edges` (global ids) against all nodes or the rows `neg_ids` lists.
    node_corrupt_forward (cpp/src/nn/decoders/edge/decoder_methods.cpp:597-659) -> apply_score_filter
    (cpp/src/data/samplers/negative.cpp:570-575: filtered scores become -1e9) -> computeRanks
    (cpp/src/reporting/reporting.cpp:52-54).  The reference contracts through its BLAS (order unspecified); here every score
    is a float32 chain in ascending column order, which is what the device kernel evaluates.
    Returns (dst_ranks, src_ranks or None)."""
    has_rel = edges.shape[1] == 3 and rel is not None
    src, dst = table[edges[:, 0]], table[edges[:, -1]]
    cand = table if neg_ids is None else table[neg_ids]
    out = []
    for side, filt in ((0, dst_filter), (1, src_filter)):
        if side == 1 and not (has_rel and inv_rel is not None):
            out.append(None)
            continue
        a, b = (src, dst) if side == 0 else (dst, src)
        r = (rel if side == 0 else inv_rel)[edges[:, 1]] if has_rel else None
        q = _apply_relation(kind, a, r).astype(np.float32)
        pos = _fma_chain_rows(q, b)
        neg = _fma_chain_scores(q, cand)
        if filt is not None and len(filt):
            neg[filt[:, 0], filt[:, 1]] = np.float32(-1e9)
        out.append(ranks_from_scores(pos, neg).astype(np.int64))
    return out[0], out[1]


def tournament_selected_scores(chunked: np.ndarray, negatives: np.ndarray, selected: int):
    """The reference's tournament selection of negatives, selector = scorer
    (cpp/src/nn/decoders/edge/distmult_selected_neg_cuda.cpp:46-121): chunked [C, rows, D] query rows, negatives [C, N, D];
    the N negatives of a chunk form `selected` groups of N / selected consecutive ones, and every row keeps, per group, the
    negative that scores highest against it (first one on a tie).  Returns (scores [C * rows, selected] float32,
    indices [C, rows * selected] int64, the column of the kept negative in its chunk).  The training step then runs its
    softmax over these `selected` scores instead of all N, and gradients reach only the kept negatives."""
    C, R, D = chunked.shape
    N = negatives.shape[1]
    if N % selected:
        raise ValueError("negatives_num must be divisible by selected_negatives_num")
    T = N // selected
    scores = np.einsum("crd,cnd->crn", chunked.astype(np.float64), negatives.astype(np.float64)).astype(np.float32)
    view = scores.reshape(C, R, selected, T)
    local = view.argmax(axis=3)
    kept = np.take_along_axis(view, local[..., None], axis=3)[..., 0]
    idx = local + np.arange(selected, dtype=np.int64)[None, None, :] * T
    return kept.reshape(C * R, selected), idx.reshape(C, R * selected).astype(np.int64)


SELECTED_DOT, SELECTED_L2 = 1, 2  # the reference's SelectedNegScoreKind (distmult_selected_neg_cuda.h:5)
_SELECTED_L2_TOL = 1e-8


def _selected_rows(chunked, negatives, selected):
    C, R, D = chunked.shape
    K = selected.shape[1] // max(R, 1)
    idx = selected.reshape(C, R, K)
    picked = negatives[np.arange(C)[:, None, None], idx]  # [C, R, K, D]
    return C, R, D, K, idx, picked.astype(np.float64)


def selected_neg_scores(chunked: np.ndarray, negatives: np.ndarray, selected: np.ndarray, kind: int) -> np.ndarray:
    """Scores of every query row against the negatives chosen for it
    (cuda/src/nn/decoders/edge/distmult_selected_neg_cuda.cu:15-85): chunked [C, R, D], negatives [C, N, D], selected
    [C, R * K] columns of the row's chunk; DOT: q . n, L2: sqrt(max(|q - n|^2, 1e-8)).  Returns [C * R, K] float32."""
    C, R, D, K, _, picked = _selected_rows(chunked, negatives, selected)
    q = chunked.astype(np.float64)[:, :, None, :]
    if kind == SELECTED_DOT:
        out = (q * picked).sum(-1)
    else:
        out = np.sqrt(np.maximum(((q - picked) ** 2).sum(-1), _SELECTED_L2_TOL))
    return out.reshape(C * R, K).astype(np.float32)


def selected_neg_scores_backward(grad_out: np.ndarray, chunked: np.ndarray, negatives: np.ndarray, selected: np.ndarray, kind: int):
    """Gradients of selected_neg_scores (distmult_selected_neg_cuda.cu:88-202): (grad_chunked [C, R, D], grad_negatives
    [C, N, D]).  DOT: dq += g n, dn += g q.  L2: dq += g (q - n) / |q - n|, dn -= the same, nothing when |q - n|^2 <= 1e-8."""
    C, R, D, K, idx, picked = _selected_rows(chunked, negatives, selected)
    q = chunked.astype(np.float64)[:, :, None, :]
    g = grad_out.astype(np.float64).reshape(C, R, K, 1)
    if kind == SELECTED_DOT:
        dq_pair, dn_pair = g * picked, g * np.broadcast_to(q, picked.shape)
    else:
        diff = q - picked
        sq = (diff ** 2).sum(-1, keepdims=True)
        coeff = np.where(sq > _SELECTED_L2_TOL, g / np.sqrt(np.maximum(sq, 1e-300)), 0.0)
        dq_pair, dn_pair = coeff * diff, -coeff * diff
    grad_neg = np.zeros(negatives.shape, np.float64)
    for c in range(C):
        np.add.at(grad_neg[c], idx[c].reshape(-1), dn_pair[c].reshape(-1, D))
    return dq_pair.sum(2).astype(np.float32), grad_neg.astype(np.float32)


def global_filter(all_edges: np.ndarray, edges: np.ndarray, inverse: bool) -> np.ndarray:
    """compute_filter_corruption with global = true (cpp/src/data/samplers/negative.cpp:421-568): for evaluation edge i all
    (i, n) such that replacing its destination (inverse: its source) by n gives an edge of `all_edges` (same relation when the
    edges carry one).  Rows in the reference's order: by edge, neighbours in the order of the sorted edge list."""
    has_rel = edges.shape[1] == 3
    keep, corrupt = (edges.shape[1] - 1, 0) if inverse else (0, edges.shape[1] - 1)
    order = np.argsort(all_edges[:, keep], kind="stable")
    sorted_edges = all_edges[order]
    starts = np.searchsorted(sorted_edges[:, keep], edges[:, keep], side="left")
    ends = np.searchsorted(sorted_edges[:, keep], edges[:, keep], side="right")
    rows = []
    for i in range(len(edges)):
        nb = sorted_edges[starts[i]:ends[i]]
        if has_rel:
            nb = nb[nb[:, 1] == edges[i, 1]]
        rows.append(np.stack([np.full(len(nb), i, np.int64), nb[:, corrupt].astype(np.int64)], 1))
    return np.concatenate(rows) if rows else np.zeros((0, 2), np.int64)


# --------------------------------------------------------------------------------------------------
# one full reference training step on global tables (the shape bench.py's CPU "port" leg times)
# --------------------------------------------------------------------------------------------------
def train_step(kind, table, state, rel, rel_state, inv_rel, inv_rel_state, edges_global, dst_neg_global, src_neg_global,
               dst_filter, src_filter, lr, domain, dense_lr=None, rel_grads_out=None):
    """SynchronousTrainer's loop body (cpp/src/engine/trainer.cpp:170-211) on CPU: map_tensors -> indexRead ->
    train_batch -> accumulateGradients -> indexAdd.  Updates table/state/rel tables in place; returns (loss, U).
    rel_grads_out: a list; when given, the relation gradients are appended to it as (rel_grad, inv_rel_grad) and the dense
    optimizer step is left to the caller (the multi-GPU trainer averages them over the devices first, multi_gpu_dense_step)."""
    has_rel = edges_global.shape[1] == 3
    lists = [edges_global[:, 0], edges_global[:, -1]]
    if src_neg_global is not None:
        lists.append(src_neg_global.reshape(-1))
    lists.append(dst_neg_global.reshape(-1))  # order of dataloader.cpp:1225-1237: src, dst, src_neg, dst_neg
    uniq, mapped = map_tensors(lists, domain)
    k = 2
    src_neg_l = None
    if src_neg_global is not None:
        src_neg_l = mapped[k].reshape(src_neg_global.shape)
        k += 1
    dst_neg_l = mapped[k].reshape(dst_neg_global.shape)
    if has_rel:
        e_local = np.stack([mapped[0], edges_global[:, 1], mapped[1]], axis=1)
    else:
        e_local = np.stack([mapped[0], mapped[1]], axis=1)
    emb = table[uniq]
    st = state[uniq]
    res = lp_train_forward_backward(kind, e_local, emb, rel, inv_rel, dst_neg_l, src_neg_l, dst_filter, src_filter)
    if has_rel and rel_grads_out is not None:
        rel_grads_out.append((res.rel_grad, res.inv_rel_grad))
    elif has_rel:
        dl = lr if dense_lr is None else dense_lr
        dense_adagrad(rel, res.rel_grad, rel_state, dl)
        if inv_rel is not None:
            dense_adagrad(inv_rel, res.inv_rel_grad, inv_rel_state, dl)
    delta, upd = sparse_adagrad(res.node_grad, st, lr)
    index_add(table, uniq, delta)
    index_add(state, uniq, upd)
    return res.loss, uniq.shape[0]


def multi_gpu_dense_step(rel, rel_state, inv_rel, inv_rel_state, grads_per_device, lr):
    """Model::all_reduce + step_all (cpp/src/nn/model.cpp:174-204; barrier cpp/src/engine/trainer.cpp:846-883) for one batch
    round: grads_per_device[j] = (rel_grad, inv_rel_grad) of device j, or None for a device without a batch (its gradients are
    zero-filled, :182-187).  Every gradient is divided by the number of devices, summed, and every replica takes the same
    Adagrad step: one table stands for all replicas."""
    g = allreduce_relation_grads([None if x is None else x[0] for x in grads_per_device])
    dense_adagrad(rel, g, rel_state, lr)
    if inv_rel is not None:
        gi = allreduce_relation_grads([None if x is None else x[1] for x in grads_per_device])
        dense_adagrad(inv_rel, gi, inv_rel_state, lr)
