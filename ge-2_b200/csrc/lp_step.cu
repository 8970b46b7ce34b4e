// Link-prediction training step (forward scores, softmax cross-entropy, backward) -- gather / scatter halves.
// The contraction-heavy middle lives in lp_scores_fp32.cu / lp_scores_f16.cu.
//
// Follows, in the reference project: Model::train_batch up to loss.backward() (cpp/src/nn/model.cpp:362-397),
// mod_node_corrupt_forward RNS branch (cpp/src/nn/decoders/edge/decoder_methods.cpp:724-806,933-946,1089-1097),
// relation operators (relation_operators.cpp:3-31), apply_score_filter (cpp/src/data/samplers/negative.cpp:570-575)
// and SoftmaxCrossEntropy with SUM reduction (cpp/src/nn/loss.cpp:46-63).
#include "lp_internal.cuh"

namespace ge2 {
namespace {

__device__ __forceinline__ const float* emb_row(const ge2_lp_desc& d, int64_t local) {
    const int64_t row = d.row_index != nullptr ? __ldg(&d.row_index[local]) : local;
    return d.node_emb + row * d.emb_stride;
}


// ---------------------------------------------------------------------------------------------------
// mask: one int per (side, chunk, column) = the batch row whose score there is overwritten with -1e9
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) mask_from_pairs_kernel(const int64_t* __restrict__ pairs, int64_t F, int npc, int Bp, int N,
                                                              int32_t* __restrict__ mask, int32_t* status) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t f = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; f < F; f += stride) {
        const int64_t row = pairs[2 * f], col = pairs[2 * f + 1];
        if (row < 0 || row >= Bp || col < 0 || col >= N) {
            or_status(status, GE2_STATUS_BAD_INDEX);
            continue;
        }
        const int c = (int)(row / npc);
        const int32_t old = atomicCAS(&mask[(int64_t)c * N + col], -1, (int32_t)row);
        if (old != -1 && old != (int32_t)row) or_status(status, GE2_STATUS_FILTER_COLLISION);
    }
}

// four consecutive columns [k, k+4) of a row of length D; columns past D read as zero.  `vec` = the row start is
// 16-byte aligned and D % 4 == 0, so one vector load serves; otherwise 8-byte pairs (k even) or scalars.
__device__ __forceinline__ float4 load4(const float* __restrict__ row, int k, int D, bool vec) {
    if (vec && k + 3 < D) return __ldg(reinterpret_cast<const float4*>(row + k));
    float4 v;
    if ((k & 1) == 0 && k + 3 < D && (((uintptr_t)(row + k)) & 7) == 0) {
        const float2 a = __ldg(reinterpret_cast<const float2*>(row + k)), b = __ldg(reinterpret_cast<const float2*>(row + k + 2));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    v.x = k < D ? __ldg(row + k) : 0.f;
    v.y = k + 1 < D ? __ldg(row + k + 1) : 0.f;
    v.z = k + 2 < D ? __ldg(row + k + 2) : 0.f;
    v.w = k + 3 < D ? __ldg(row + k + 3) : 0.f;
    return v;
}

__device__ __forceinline__ void store_half4(__half* dst, float4 v) {
    const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
    uint2 pk;
    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(dst) = pk;
}

// ---------------------------------------------------------------------------------------------------
// prep: eight lanes per output row (four rows in flight per warp, so the dependent loads id -> row index -> embedding
// row overlap), each lane 4 columns at a time.  Rows [0, S*Bp) are query rows, rows [S*Bp, S*Bp + S*CN) negative rows.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) lp_prep_kernel(LpKernelArgs a) {
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x;
    const int gl = tid & 7;                              // lane within the row group
    const unsigned gmask = 0xFFu << ((tid & 31) & ~7);   // the 8 lanes of this group inside the warp
    const int64_t groups = ((int64_t)gridDim.x * blockDim.x) >> 3;
    const int64_t q_rows = (int64_t)L.S * L.Bp;
    const int64_t total = q_rows + (int64_t)L.S * L.CN;
    const int64_t total_pad = round_up<int64_t>(total, 4);  // whole warps stay in the loop for the shuffles
    const int D = d.D, h = D / 2, ld = L.ld;
    const bool vec_e = (d.emb_stride % 4 == 0) && (((uintptr_t)d.node_emb) & 15) == 0 && D % 4 == 0;
    const bool vec_r = D % 4 == 0 && ((((uintptr_t)d.rel) | ((uintptr_t)d.inv_rel)) & 15) == 0;
    const bool write_k32 = d.precision != GE2_PRECISION_F16;  // the tensor path reads only the fp16 copy of the negatives
    griddep_wait();
    if (blockIdx.x == 0 && tid == 0) *L.loss_acc = 0.0;        // the scores kernel of this step adds every row's loss term to it
    if (blockIdx.x == 0 && L.item_ctr != nullptr)               // arrival counters of the tensor path's logsumexp pass start at zero
        for (int k = tid; k < L.n_items + 2; k += blockDim.x) L.item_ctr[k] = 0;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + tid) >> 3; w < total_pad; w += groups) {
        if (w >= total) continue;
        if (w < q_rows) {
            const int s = (int)(w / L.Bp);
            const int i = (int)(w - (int64_t)s * L.Bp);
            float* q = L.Q + ((int64_t)s * L.Bp + i) * ld;
            __half* qh = L.Qh != nullptr ? L.Qh + ((int64_t)s * L.Bp + i) * ld : nullptr;
            bool ok = i < d.B;  // rows past B: zero rows appended by pad_and_reshape; their positive score is padded with 0
            int64_t sid = 0, did = 0, rid = 0;
            if (ok) {
                sid = d.src_ids[(int64_t)i * d.edge_stride];
                did = d.dst_ids[(int64_t)i * d.edge_stride];
                ok = sid >= 0 && sid < d.U && did >= 0 && did < d.U;
                if (d.has_relations) {
                    rid = d.rel_ids[(int64_t)i * d.rel_stride];
                    ok = ok && rid >= 0 && rid < d.R;
                }
                if (!ok && gl == 0) or_status(d.status, GE2_STATUS_BAD_INDEX);
            }
            const float* ea = ok ? emb_row(d, s == 0 ? sid : did) : nullptr;  // the endpoint the relation is applied to
            const float* eb = ok ? emb_row(d, s == 0 ? did : sid) : nullptr;  // the endpoint it is compared with
            const float* r = (ok && d.has_relations) ? (s == 0 ? d.rel : d.inv_rel) + rid * D : nullptr;
            float dot = 0.f;
            for (int k = gl * 4; k < ld; k += 32) {
                float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
                if (ok) {
                    const float4 x = load4(ea, k, D, vec_e);
                    if (r == nullptr) {
                        v = x;
                    } else {
                        const float4 rr = load4(r, k, D, vec_r);
                        if (d.decoder == GE2_DECODER_DISTMULT) {
                            v = make_float4(x.x * rr.x, x.y * rr.y, x.z * rr.z, x.w * rr.w);
                        } else {
                            // complex Hadamard: columns [0, h) real, [h, D) imaginary; the partner component comes from the
                            // same two rows (just loaded, so these scalar reads hit L1)
                            float xv[4] = {x.x, x.y, x.z, x.w}, rv[4] = {rr.x, rr.y, rr.z, rr.w}, o[4];
#pragma unroll
                            for (int e2 = 0; e2 < 4; e2++) {
                                const int c = k + e2;
                                o[e2] = 0.f;
                                if (c < D) {
                                    const int cp = c < h ? c + h : c - h;
                                    const float xp = __ldg(ea + cp), rp = __ldg(r + cp);
                                    o[e2] = c < h ? xv[e2] * rv[e2] - xp * rp   // real: e_re r_re - e_im r_im
                                                  : xp * rv[e2] + xv[e2] * rp;  // imaginary: e_re r_im + e_im r_re
                                }
                            }
                            v = make_float4(o[0], o[1], o[2], o[3]);
                        }
                    }
                    const float4 y = load4(eb, k, D, vec_e);
                    dot += v.x * y.x + v.y * y.y + v.z * y.z + v.w * y.w;
                }
                if (write_k32) *reinterpret_cast<float4*>(q + k) = v;  // only the fp32 scores kernel reads the fp32 copies
                if (qh != nullptr) store_half4(qh + k, v);
            }
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) dot += __shfl_xor_sync(gmask, dot, o);
            if (gl == 0) L.pos[(int64_t)s * L.Bp + i] = dot;
        } else {
            const int64_t e = w - q_rows;
            const int s = (int)(e / L.CN);
            const int64_t j = e - (int64_t)s * L.CN;
            const int64_t id = (s == 0 ? d.dst_negs : d.src_negs)[j];
            const bool bad = id < 0 || id >= d.U;
            if (bad && gl == 0) or_status(d.status, GE2_STATUS_BAD_INDEX);
            if (gl == 0 && d.deg_sample_rows != nullptr) {
                // the filter word of this (side, chunk, column): deg_negative_local_filter on the device (negative.cpp:215-263 of
                // the reference): entry (c, col) masks row deg_rows[c][col] when that row belongs to chunk c; the same for both
                // sides (the reference shares one filter tensor, negative.cpp:1049-1056)
                const int c = (int)(j / d.N), col = (int)(j - (int64_t)c * d.N);
                int32_t m = -1;
                if (col < d.n_deg) {
                    const int64_t r = d.deg_sample_rows[(int64_t)c * d.n_deg + col];
                    if (r < 0 || r >= d.B) or_status(d.status, GE2_STATUS_BAD_INDEX);
                    else if ((int)(r / L.npc) == c) m = (int32_t)r;
                }
                L.mask[e] = m;
            }
            const float* src = bad ? nullptr : emb_row(d, id);
            for (int k = gl * 4; k < ld; k += 32) {
                const float4 v = bad ? make_float4(0.f, 0.f, 0.f, 0.f) : load4(src, k, D, vec_e);
                if (write_k32) *reinterpret_cast<float4*>(L.K + e * ld + k) = v;
                if (L.Kh != nullptr) store_half4(L.Kh + e * ld + k, v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// finish: relation-operator backward and the scatter of every gradient row.
// One warp per row: an edge (both corruption sides at once) or one negative.  Lanes run along the embedding, so every
// load and every atomic of a warp covers one contiguous 128-byte piece of a row, and the loads of a row (two endpoints, two
// relation rows, two rows of dQ) are all issued before the first one is needed.  For ComplEx a lane holds the real and the
// imaginary component of the same complex coordinate, so the operator's backward needs no second pass over the rows.
// A CTA walks a contiguous range of rows and folds the gradients of relation rows (few rows, hit by every edge) into a
// small shared-memory table that is flushed once at the end; node rows go straight to global memory (the batch-local
// gradient buffer lives in L2).  Sums are the same as the reference's index_add backward up to fp32 addition order.
// ---------------------------------------------------------------------------------------------------
constexpr int kFinSlots = 32;     // relation rows cached per CTA
constexpr int kFinWarps = 8;
constexpr long long kFinEmpty = -1;

constexpr int kFinEdgeBatch = 64;  // edges whose scalars (ids, table rows, d loss / d pos, table slots) are fetched together
constexpr int kFinHotSlots = 8;    // node rows cached per CTA: rows that occur more than once among a batch's endpoints

struct FinishSmem {
    float acc[kFinSlots][128];
    long long tag[kFinSlots];  // (1 + side) << 40 | relation id
    // per edge of the current batch: filled by one thread per edge, so the chain id -> row index -> ... is walked for
    // 64 edges at once instead of once per warp and edge
    long long sid[kFinEdgeBatch], did[kFinEdgeBatch], srow[kFinEdgeBatch], drow[kFinEdgeBatch];
    int rid[kFinEdgeBatch], slot[2][kFinEdgeBatch];  // rid < 0: skip the edge (bad ids, flagged by prep)
    float dpos[2][kFinEdgeBatch];
    // Hub rows: in a skewed graph one node can be an endpoint of a tenth of the batch, and thousands of atomics on the same
    // 128 bytes of its gradient row serialise in L2.  A row seen twice among the 128 endpoints of an edge batch gets a
    // shared-memory row (first come, kept until the end of the CTA) and reaches global memory once per CTA.
    float hot[kFinHotSlots][128];
    long long hot_tag[kFinHotSlots];      // batch-local node id, or kFinEmpty
    int hot_slot[2][kFinEdgeBatch];      // per edge: slot of its source / destination row, or -1
};

__device__ __forceinline__ int fin_slot_of(long long key) { return (int)(((unsigned long long)key * 0x9E3779B97F4A7C15ull) >> 59); }  // top 5 bits

__global__ void __launch_bounds__(kFinWarps * 32) lp_finish_kernel(LpKernelArgs a, int edges_per_cta, int negs_per_cta) {
    __shared__ FinishSmem sm;
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int64_t e_rows = d.B;  // one row per edge (both sides), then one per negative
    const int64_t total = e_rows + (int64_t)L.S * L.CN;
    const int D = d.D, h = D / 2, ld = L.ld;
    const bool cplx = d.has_relations && d.decoder == GE2_DECODER_COMPLEX;
    const int n_el = cplx ? h : D;       // coordinates a lane loop runs over: complex pairs, or plain columns
    const int off2 = cplx ? h : 0;       // where the second component of a coordinate lives
    const bool vec_g = (D % 4 == 0) && (((uintptr_t)d.node_grad) & 15) == 0;
    const float gs = L.grad_unscale;  // the tensor path leaves dQ / dK scaled by a power of two

    if (d.has_relations) {
        for (int k = tid; k < kFinSlots * 128; k += kFinWarps * 32) (&sm.acc[0][0])[k] = 0.f;
        if (tid < kFinSlots) sm.tag[tid] = kFinEmpty;
    }
    for (int k = tid; k < kFinHotSlots * 128; k += kFinWarps * 32) (&sm.hot[0][0])[k] = 0.f;
    if (tid < kFinHotSlots) sm.hot_tag[tid] = kFinEmpty;
    griddep_wait();  // the shared-memory set-up above overlaps the tail of the scores kernel
    // loss = sum over sides and padded rows of (lse - pos), accumulated in double by the scores kernel that ran before
    if (blockIdx.x == 0 && tid == 0) *d.loss = (float)*L.loss_acc;
    __syncthreads();

    // Every CTA takes a contiguous share of the edges (heavy rows: six input rows, four output rows each) and a contiguous
    // share of the negatives (one row in, one out), so the heavy rows are spread over the whole grid.
    const int64_t e_begin = (int64_t)blockIdx.x * edges_per_cta;
    const int64_t e_end = e_begin + edges_per_cta < e_rows ? e_begin + edges_per_cta : e_rows;
    const int64_t n_begin = e_rows + (int64_t)blockIdx.x * negs_per_cta;
    const int64_t n_end = n_begin + negs_per_cta < total ? n_begin + negs_per_cta : total;

    // the negatives of this CTA: one row of dK each, added to the gradient row of the node it was drawn as
    auto scatter_negatives = [&]() {
        // A row whose node holds a shared-memory row (claimed by the edges of this CTA: a hub) is summed there: with
        // negatives drawn by degree a hub node owns thousands of these rows, and their atomics would serialise in L2.
        for (int64_t w = n_begin + warp; w < n_end; w += kFinWarps) {
            const int64_t e = w - e_rows;
            const int s = (int)(e / L.CN);
            const int64_t j = e - (int64_t)s * L.CN;
            const int64_t id = (s == 0 ? d.dst_negs : d.src_negs)[j];
            if (id < 0 || id >= d.U) continue;
            const float* dk = L.dK + e * ld;
            const int sidx = (int)(((unsigned long long)id * 0x9E3779B97F4A7C15ull) >> 61);
            if (sm.hot_tag[sidx] == id) {
                for (int k = lane; k < D; k += 32) {
                    const float v = dk[k] * gs;
                    if (v != 0.f) atomicAdd(&sm.hot[sidx][k], v);
                }
                continue;
            }
            float* grow = d.node_grad + id * D;
            if (vec_g) {
                for (int k = lane * 4; k < D; k += 128) {
                    float4 v = *reinterpret_cast<const float4*>(dk + k);
                    v.x *= gs, v.y *= gs, v.z *= gs, v.w *= gs;
                    if (v.x != 0.f || v.y != 0.f || v.z != 0.f || v.w != 0.f) atomicAdd(reinterpret_cast<float4*>(grow + k), v);
                }
            } else {
                for (int k = lane; k < D; k += 32) {
                    const float v = dk[k] * gs;
                    if (v != 0.f) atomicAdd(grow + k, v);
                }
            }
        }
    };
    bool negs_done = false;
    for (int64_t base = e_begin; base < e_end; base += kFinEdgeBatch) {
        const int nb = (int)(e_end - base < kFinEdgeBatch ? e_end - base : kFinEdgeBatch);
        if (tid < nb) {
            const int64_t i = base + tid;
            const int64_t sid = d.src_ids[i * d.edge_stride];
            const int64_t did = d.dst_ids[i * d.edge_stride];
            bool ok = sid >= 0 && sid < d.U && did >= 0 && did < d.U;
            int64_t rid = 0;
            if (d.has_relations) {
                rid = d.rel_ids[i * d.rel_stride];
                ok = ok && rid >= 0 && rid < d.R;
            }
            sm.rid[tid] = ok ? (int)rid : -1;
            if (ok) {
                sm.sid[tid] = sid;
                sm.did[tid] = did;
                sm.srow[tid] = d.row_index != nullptr ? __ldg(&d.row_index[sid]) : sid;
                sm.drow[tid] = d.row_index != nullptr ? __ldg(&d.row_index[did]) : did;
                for (int s = 0; s < L.S; s++) {
                    const int64_t qrow = (int64_t)s * L.Bp + i;
                    sm.dpos[s][tid] = __expf(L.pos[qrow] - L.lse[qrow]) - 1.0f;  // d loss / d pos_i = softmax prob of the positive - 1
                    int slot = -1;
                    if (d.has_relations) {  // claim (or find) the shared slot of this relation row; -1 when it belongs to another row
                        const long long key = ((long long)(1 + s) << 40) | rid;
                        const int sidx = fin_slot_of(key);
                        const long long old = (long long)atomicCAS((unsigned long long*)&sm.tag[sidx], (unsigned long long)kFinEmpty, (unsigned long long)key);
                        slot = (old == kFinEmpty || old == key) ? sidx : -1;
                    }
                    sm.slot[s][tid] = slot;
                }
            }
        }
        __syncthreads();
        if (tid < 2 * kFinEdgeBatch) {  // thread (side, k): does the row of this endpoint occur again in the batch, or hold a slot already?
            const int side = tid / kFinEdgeBatch, k = tid % kFinEdgeBatch;
            int hs = -1;
            if (k < nb && sm.rid[k] >= 0) {
                const long long id = side == 0 ? sm.sid[k] : sm.did[k];
                const int sidx = (int)(((unsigned long long)id * 0x9E3779B97F4A7C15ull) >> 61);  // top 3 bits
                if (sm.hot_tag[sidx] == id) {
                    hs = sidx;
                } else if (sm.hot_tag[sidx] == kFinEmpty) {
                    int seen = 0;
                    for (int j = 0; j < nb; j++)
                        if (sm.rid[j] >= 0) seen += (sm.sid[j] == id) + (sm.did[j] == id);
                    if (seen > 1) {
                        const long long old = (long long)atomicCAS((unsigned long long*)&sm.hot_tag[sidx], (unsigned long long)kFinEmpty, (unsigned long long)id);
                        if (old == kFinEmpty || old == id) hs = sidx;
                    }
                }
            }
            sm.hot_slot[side][k] = hs;
        }
        __syncthreads();
        for (int k = warp; k < nb; k += kFinWarps) {
            // one edge, both corruption sides at once: side 0 applies the relation to the source and compares with the
            // destination, side 1 the inverse relation to the destination and compares with the source, so each endpoint
            // receives one combined row instead of two
            const int64_t i = base + k;
            const int rid = sm.rid[k];
            if (rid < 0) continue;  // bad rows were flagged by prep
            const int64_t sid = sm.sid[k], did = sm.did[k];
            const float* es = d.node_emb + sm.srow[k] * d.emb_stride;
            const float* ed = d.node_emb + sm.drow[k] * d.emb_stride;
            const float* r[2] = {nullptr, nullptr};
            const float* dq[2] = {nullptr, nullptr};
            float* rg[2] = {nullptr, nullptr};
            int slot_r[2] = {-1, -1};
            float dpos[2] = {0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 2; s++) {
                if (s >= L.S) break;
                dq[s] = L.dQ + ((int64_t)s * L.Bp + i) * ld;
                dpos[s] = sm.dpos[s][k];
                if (d.has_relations) {
                    r[s] = (s == 0 ? d.rel : d.inv_rel) + (int64_t)rid * D;
                    rg[s] = (s == 0 ? d.rel_grad : d.inv_rel_grad) + (int64_t)rid * D;
                    slot_r[s] = sm.slot[s][k];
                }
            }
            // generic pointers: a shared-memory row for a hub, the global gradient row otherwise (the atomics below take either)
            const int hs_s = sm.hot_slot[0][k], hs_d = sm.hot_slot[1][k];
            float* gsrc = hs_s >= 0 ? sm.hot[hs_s] : d.node_grad + sid * D;
            float* gdst = hs_d >= 0 ? sm.hot[hs_d] : d.node_grad + did * D;
            for (int c = lane; c < n_el; c += 32) {
                // components 0 / 1 of coordinate c: (real, imaginary) for ComplEx, otherwise only component 0 is used
                const int c2 = c + off2;
                const float s0 = __ldg(es + c), d0 = __ldg(ed + c);
                const float s1 = cplx ? __ldg(es + c2) : 0.f, d1 = cplx ? __ldg(ed + c2) : 0.f;
                float gs0 = 0.f, gs1 = 0.f, gd0 = 0.f, gd1 = 0.f;  // gradient of the source / destination row at this coordinate
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    if (s >= L.S) break;
                    const float a0 = s == 0 ? s0 : d0, a1 = s == 0 ? s1 : d1;  // endpoint the relation is applied to
                    const float b0 = s == 0 ? d0 : s0, b1 = s == 0 ? d1 : s1;  // endpoint it is compared with
                    // gradient with respect to the relation-adjusted embedding q = op(a, r): from the negatives (dQ) and the positive
                    const float g0 = dq[s][c] * gs + dpos[s] * b0;
                    const float g1 = cplx ? dq[s][c2] * gs + dpos[s] * b1 : 0.f;
                    float ga0, ga1 = 0.f, gb0, gb1 = 0.f, vr0 = 0.f, vr1 = 0.f;
                    if (r[s] == nullptr) {            // Dot: q = a
                        gb0 = dpos[s] * a0;
                        ga0 = g0;
                    } else if (!cplx) {               // DistMult: q = a * r
                        const float r0 = __ldg(r[s] + c);
                        gb0 = dpos[s] * (a0 * r0);
                        ga0 = g0 * r0;
                        vr0 = g0 * a0;
                    } else {                          // ComplEx: q = a x r (complex product), backward through both factors
                        const float r0 = __ldg(r[s] + c), r1 = __ldg(r[s] + c2);
                        gb0 = dpos[s] * (a0 * r0 - a1 * r1);
                        gb1 = dpos[s] * (a0 * r1 + a1 * r0);
                        ga0 = g0 * r0 + g1 * r1;
                        ga1 = -g0 * r1 + g1 * r0;
                        vr0 = g0 * a0 + g1 * a1;
                        vr1 = -g0 * a1 + g1 * a0;
                    }
                    if (s == 0) {
                        gs0 += ga0; gs1 += ga1; gd0 += gb0; gd1 += gb1;
                    } else {
                        gd0 += ga0; gd1 += ga1; gs0 += gb0; gs1 += gb1;
                    }
                    if (rg[s] != nullptr) {
                        if (slot_r[s] >= 0) {
                            atomicAdd(&sm.acc[slot_r[s]][c], vr0);
                            if (cplx) atomicAdd(&sm.acc[slot_r[s]][c2], vr1);
                        } else {
                            atomicAdd(rg[s] + c, vr0);
                            if (cplx) atomicAdd(rg[s] + c2, vr1);
                        }
                    }
                }
                atomicAdd(gsrc + c, gs0);
                atomicAdd(gdst + c, gd0);
                if (cplx) {
                    atomicAdd(gsrc + c2, gs1);
                    atomicAdd(gdst + c2, gd1);
                }
            }
        }
        if (!negs_done) {  // after the first batch of edges, whose endpoints have claimed the shared-memory rows of the hubs
            scatter_negatives();
            negs_done = true;
        }
        __syncthreads();  // the batch's scalars are overwritten by the next batch
    }
    if (!negs_done) scatter_negatives();
    __syncthreads();
    for (int slot = warp; slot < kFinHotSlots; slot += kFinWarps) {  // hub rows: one pass over global memory per CTA
        const long long id = sm.hot_tag[slot];
        if (id == kFinEmpty) continue;
        float* grow = d.node_grad + id * D;
        for (int k = lane; k < D; k += 32) {
            const float v = sm.hot[slot][k];
            if (v != 0.f) atomicAdd(grow + k, v);
        }
    }
    if (!d.has_relations) return;
    // flush: warp w writes slots w, w + 8, ...
    for (int slot = warp; slot < kFinSlots; slot += kFinWarps) {
        const long long key = sm.tag[slot];
        if (key == kFinEmpty) continue;
        const int kind = (int)(key >> 40);
        const long long id = key & ((1ll << 40) - 1);
        float* grow = (kind == 1 ? d.rel_grad : d.inv_rel_grad) + id * D;
        for (int k = lane; k < D; k += 32) {
            const float v = sm.acc[slot][k];
            if (v != 0.f) atomicAdd(grow + k, v);
        }
    }
}

__global__ void __launch_bounds__(256) copy_pos_kernel(const float* __restrict__ pos, int Bp, float* __restrict__ out0, float* __restrict__ out1,
                                                       int S) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < Bp) {
        if (out0 != nullptr) out0[i] = pos[i];
        if (S == 2 && out1 != nullptr) out1[i] = pos[Bp + i];
    }
}

int validate(const ge2_lp_desc* d) {
    if (d == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if (d->B <= 0 || d->C <= 0 || d->N <= 0 || d->D <= 0 || d->U <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (d->decoder != GE2_DECODER_DISTMULT && d->decoder != GE2_DECODER_COMPLEX) return GE2_ERR_INVALID_ARGUMENT;
    if (d->precision != GE2_PRECISION_FP32 && d->precision != GE2_PRECISION_F16) return GE2_ERR_INVALID_ARGUMENT;
    if (d->use_inverse && !d->has_relations) return GE2_ERR_INVALID_ARGUMENT;
    if (d->D > 128) return GE2_ERR_UNSUPPORTED;
    // the reference's complex operator splits the row in D/2 and D - D/2 columns and multiplies them element-wise: D must be even
    if (d->decoder == GE2_DECODER_COMPLEX && d->has_relations && (d->D & 1)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->node_emb == nullptr || d->src_ids == nullptr || d->dst_ids == nullptr || d->dst_negs == nullptr || d->node_grad == nullptr ||
        d->loss == nullptr || d->edge_stride <= 0 || d->emb_stride < d->D)
        return GE2_ERR_INVALID_ARGUMENT;
    if (d->has_relations && (d->rel_stride <= 0 || d->rel_ids == nullptr || d->rel == nullptr || d->rel_grad == nullptr || d->R <= 0)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->use_inverse && (d->src_negs == nullptr || d->inv_rel == nullptr || d->inv_rel_grad == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->dst_filter_n < 0 || d->src_filter_n < 0 || (d->dst_filter_n > 0 && d->dst_filter == nullptr) ||
        (d->src_filter_n > 0 && d->src_filter == nullptr))
        return GE2_ERR_INVALID_ARGUMENT;
    if (d->deg_sample_rows != nullptr && (d->n_deg <= 0 || d->n_deg > d->N)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->deg_sample_rows != nullptr && (d->dst_filter_n > 0 || d->src_filter_n > 0)) return GE2_ERR_INVALID_ARGUMENT;
    return GE2_OK;
}

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" int ge2_lp_workspace_bytes(const ge2_lp_desc* desc, size_t* bytes) {
    if (bytes == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    int rc = validate(desc);
    if (rc != GE2_OK) return rc;
    *bytes = lp_make_layout(*desc, nullptr).bytes;
    return GE2_OK;
}

extern "C" int ge2_lp_step(const ge2_lp_desc* desc, ge2_stream_t stream_) {
    int rc = validate(desc);
    if (rc != GE2_OK) return rc;
    LpKernelArgs a;
    a.d = *desc;
    if (desc->workspace == nullptr || ((uintptr_t)desc->workspace & 255) != 0) return GE2_ERR_WORKSPACE;
    a.L = lp_make_layout(*desc, desc->workspace);
    if (desc->workspace_bytes < a.L.bytes) return GE2_ERR_WORKSPACE;
    const LpLayout& L = a.L;
    cudaStream_t stream = as_stream(stream_);

    const int phases = desc->phases == 0 ? 7 : desc->phases;
    // fp32 path: dK is reduced with atomics and starts from zero; the tensor path stores whole tiles and clears nothing
    if ((phases & 2) && desc->precision == GE2_PRECISION_FP32) GE2_CUDA_TRY(cudaMemsetAsync(L.dK, 0, L.zero_bytes, stream));
    if ((phases & 4) && !(desc->flags & GE2_LP_NODE_GRAD_IS_ZERO))
        GE2_CUDA_TRY(cudaMemsetAsync(desc->node_grad, 0, (size_t)desc->U * desc->D * 4, stream));
    if (phases & 1) {
    if (desc->deg_sample_rows == nullptr) {  // (with the degree-sample plan the prepare kernel writes every filter word itself)
        GE2_CUDA_TRY(cudaMemsetAsync(L.mask, 0xFF, (size_t)L.S * L.CN * 4, stream));
        if (desc->dst_filter_n > 0) {
            mask_from_pairs_kernel<<<stream_grid(desc->dst_filter_n, 256), 256, 0, stream>>>(desc->dst_filter, desc->dst_filter_n, L.npc, L.Bp,
                                                                                           desc->N, L.mask, desc->status);
            GE2_LAUNCH_CHECK();
        }
        if (L.S == 2 && desc->src_filter_n > 0) {
            mask_from_pairs_kernel<<<stream_grid(desc->src_filter_n, 256), 256, 0, stream>>>(desc->src_filter, desc->src_filter_n, L.npc, L.Bp,
                                                                                           desc->N, L.mask + L.CN, desc->status);
            GE2_LAUNCH_CHECK();
        }
    }

    const int64_t prep_rows = (int64_t)L.S * L.Bp + (int64_t)L.S * L.CN;
    GE2_CUDA_TRY(launch_after(lp_prep_kernel, dim3((unsigned)stream_grid(prep_rows, 32, 8)), dim3(256), 0, stream, a));
    }

    if (phases & 2) {
        rc = desc->precision == GE2_PRECISION_F16 ? lp_scores_f16(a, stream) : lp_scores_fp32(a, stream);
        if (rc != GE2_OK) return rc;
    }
    if (!(phases & 4)) return GE2_OK;

    const int64_t fin_rows = (int64_t)desc->B + (int64_t)L.S * L.CN;
    // about four CTAs per SM, each with a contiguous share of the edges (whose relation rows meet in its shared table) and of the negatives
    const int64_t neg_rows = (int64_t)L.S * L.CN;
    int fin_ctas = (int)std::min<int64_t>((int64_t)kNumSMs * 4, ceil_div<int64_t>(fin_rows, 8));
    if (fin_ctas < 1) fin_ctas = 1;
    const int edges_per_cta = (int)ceil_div<int64_t>(desc->B, fin_ctas), negs_per_cta = (int)ceil_div<int64_t>(neg_rows, fin_ctas);
    GE2_CUDA_TRY(launch_after(lp_finish_kernel, dim3((unsigned)fin_ctas), dim3(256), 0, stream, a, edges_per_cta, negs_per_cta));
    if (desc->pos_scores != nullptr || desc->inv_pos_scores != nullptr) {
        copy_pos_kernel<<<ceil_div(L.Bp, 256), 256, 0, stream>>>(L.pos, L.Bp, desc->pos_scores, desc->inv_pos_scores, L.S);
        GE2_LAUNCH_CHECK();
    }
    return GE2_OK;
}
