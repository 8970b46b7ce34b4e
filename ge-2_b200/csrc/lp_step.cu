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

// deg_negative_local_filter on the device (negative.cpp:215-263): entry (c, j) masks row deg_rows[c][j] when that
// row belongs to chunk c.  Same mask for both sides (the reference shares one filter tensor, negative.cpp:1049-1056).
__global__ void __launch_bounds__(256) mask_from_deg_rows_kernel(const int64_t* __restrict__ deg_rows, int C, int n_deg, int npc, int B,
                                                                 int N, int S, int64_t CN, int32_t* __restrict__ mask, int32_t* status) {
    const int64_t total = (int64_t)C * n_deg;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        const int c = (int)(e / n_deg), j = (int)(e % n_deg);
        const int64_t row = deg_rows[e];
        if (row < 0 || row >= B) {
            or_status(status, GE2_STATUS_BAD_INDEX);
            continue;
        }
        if ((int)(row / npc) == c) {
            for (int s = 0; s < S; s++) mask[s * CN + (int64_t)c * N + j] = (int32_t)row;
        }
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
    if (blockIdx.x == 0 && tid == 0) *L.loss_acc = 0.0;        // the scores kernel of this step adds every row's loss term to it
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
// finish: relation-operator backward and the duplicate-reducing scatter of every gradient row.
// Eight lanes share a row (16 columns each for ld = 128), so a warp has four rows in flight and the chain of dependent
// loads (ids -> row index -> embedding row) overlaps four ways.  A CTA walks a contiguous range of rows and first folds
// gradients for frequently hit rows (hub nodes under a power-law degree distribution, popular relations) into a small
// shared-memory table; what does not find a slot goes to global memory with 16-byte vector atomics, and the table is
// flushed once at the end.  Sums are the same as the reference's index_add backward up to fp32 addition order.
// ---------------------------------------------------------------------------------------------------
constexpr int kFinSlots = 32;     // hot rows cached per CTA
constexpr int kFinLanes = 8;      // lanes per row
constexpr long long kFinEmpty = -1;

struct FinishSmem {
    float acc[kFinSlots][128];
    long long tag[kFinSlots];  // 0 <= key < 2^40: node row; (1 + side) << 40 | relation id: relation row
};

__device__ __forceinline__ int fin_slot_of(long long key) { return (int)(((unsigned long long)key * 0x9E3779B97F4A7C15ull) >> 59); }  // top 5 bits

__global__ void __launch_bounds__(256) lp_finish_kernel(LpKernelArgs a, int rows_per_cta) {
    __shared__ FinishSmem sm;
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x;
    const int gl = tid & (kFinLanes - 1);                 // lane within the row group
    const int group = tid / kFinLanes;                    // 32 groups per CTA
    const unsigned gmask = 0xFFu << ((tid & 31) & ~7);    // the 8 lanes of this group inside the warp
    const int gleader = (tid & 31) & ~7;
    const int64_t e_rows = d.B;  // one row group per edge (both sides), then one per negative
    const int64_t total = e_rows + (int64_t)L.S * L.CN;
    const int D = d.D, h = D / 2, ld = L.ld;
    const bool vec4 = (D % 4 == 0) && (((uintptr_t)d.node_grad | (uintptr_t)d.rel_grad | (uintptr_t)d.inv_rel_grad) & 15) == 0;
    const bool vec_e = (d.emb_stride % 4 == 0) && (((uintptr_t)d.node_emb) & 15) == 0 && D % 4 == 0;
    const bool vec_r = D % 4 == 0 && ((((uintptr_t)d.rel) | ((uintptr_t)d.inv_rel)) & 15) == 0;

    // loss = sum over sides and padded rows of (lse - pos), accumulated in double by the scores kernel that ran before
    if (blockIdx.x == 0 && tid == 0) *d.loss = (float)*L.loss_acc;
    for (int k = tid; k < kFinSlots * 128; k += 256) (&sm.acc[0][0])[k] = 0.f;
    if (tid < kFinSlots) sm.tag[tid] = kFinEmpty;
    __syncthreads();

    // claims (or finds) the shared slot of `key`; -1 when the slot belongs to another row.  Group-uniform result.
    auto claim = [&](long long key) -> int {
        int slot = -1;
        if ((tid & 31) == gleader) {
            const int sidx = fin_slot_of(key);
            const long long old = (long long)atomicCAS((unsigned long long*)&sm.tag[sidx], (unsigned long long)kFinEmpty, (unsigned long long)key);
            slot = (old == kFinEmpty || old == key) ? sidx : -1;
        }
        return __shfl_sync(gmask, slot, gleader);
    };
    // adds four consecutive columns [k, k+4) of a gradient row either into the shared slot or straight into global memory
    auto add4 = [&](int slot, float* grow, int k, float4 v) {
        if (v.x == 0.f && v.y == 0.f && v.z == 0.f && v.w == 0.f) return;
        if (slot >= 0) {
            atomicAdd(&sm.acc[slot][k], v.x);
            atomicAdd(&sm.acc[slot][k + 1], v.y);
            atomicAdd(&sm.acc[slot][k + 2], v.z);
            atomicAdd(&sm.acc[slot][k + 3], v.w);
        } else if (vec4) {
            atomicAdd(reinterpret_cast<float4*>(grow + k), v);
        } else {
            if (k < D) atomicAdd(grow + k, v.x);
            if (k + 1 < D) atomicAdd(grow + k + 1, v.y);
            if (k + 2 < D) atomicAdd(grow + k + 2, v.z);
            if (k + 3 < D) atomicAdd(grow + k + 3, v.w);
        }
    };

    const int64_t row_begin = (int64_t)blockIdx.x * rows_per_cta;
    const int64_t row_end = row_begin + rows_per_cta < total ? row_begin + rows_per_cta : total;
    for (int64_t w0 = row_begin; w0 < row_end; w0 += 32) {
        const int64_t w = w0 + group;  // whole warps stay in the loop (shuffles below), rows past the end do nothing
        const bool live = w < row_end;
        if (live && w < e_rows) {
            // one edge, both corruption sides at once: side 0 applies the relation to the source and compares with the
            // destination, side 1 the inverse relation to the destination and compares with the source, so each endpoint
            // receives one combined row instead of two
            const int i = (int)w;
            const int64_t sid = d.src_ids[(int64_t)i * d.edge_stride];
            const int64_t did = d.dst_ids[(int64_t)i * d.edge_stride];
            bool ok = sid >= 0 && sid < d.U && did >= 0 && did < d.U;
            int64_t rid = 0;
            if (d.has_relations) {
                rid = d.rel_ids[(int64_t)i * d.rel_stride];
                ok = ok && rid >= 0 && rid < d.R;
            }
            if (ok) {  // bad rows were flagged by prep
                const float* es = emb_row(d, sid);
                const float* ed = emb_row(d, did);
                const int slot_s = claim(sid), slot_d = claim(did);
                int slot_r[2] = {-1, -1};
                const float *r[2] = {nullptr, nullptr}, *dq[2];
                float* rg[2] = {nullptr, nullptr};
                float dpos[2];
#pragma unroll
                for (int s = 0; s < 2; s++) {
                    if (s >= L.S) break;
                    const int64_t qrow = (int64_t)s * L.Bp + i;
                    dq[s] = L.dQ + qrow * ld;
                    dpos[s] = __expf(L.pos[qrow] - L.lse[qrow]) - 1.0f;  // d loss / d pos_i = softmax prob of the positive - 1
                    if (d.has_relations) {
                        r[s] = (s == 0 ? d.rel : d.inv_rel) + rid * D;
                        rg[s] = (s == 0 ? d.rel_grad : d.inv_rel_grad) + rid * D;
                        slot_r[s] = claim(((long long)(1 + s) << 40) | rid);
                    }
                }
                for (int k = gl * 4; k < D; k += kFinLanes * 4) {
                    const float4 s4 = load4(es, k, D, vec_e), d4 = load4(ed, k, D, vec_e);
                    const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
                    float gs[4] = {0.f, 0.f, 0.f, 0.f}, gd[4] = {0.f, 0.f, 0.f, 0.f};  // gradient rows of the source / destination node
#pragma unroll
                    for (int s = 0; s < 2; s++) {
                        if (s >= L.S) break;
                        const float* ea = s == 0 ? es : ed;            // endpoint the relation is applied to
                        const float* eb = s == 0 ? ed : es;            // endpoint it is compared with
                        const float* eav = s == 0 ? sv : dv;
                        const float* ebv = s == 0 ? dv : sv;
                        float* ga = s == 0 ? gs : gd;
                        float* gb = s == 0 ? gd : gs;
                        // the relation-adjusted embedding q = op(ea, r) is recomputed from rows that are loaded anyway
                        const float4 dq4 = *reinterpret_cast<const float4*>(dq[s] + k);
                        const float dqv[4] = {dq4.x, dq4.y, dq4.z, dq4.w};
                        float vr[4] = {0.f, 0.f, 0.f, 0.f};
                        float rv[4] = {0.f, 0.f, 0.f, 0.f};
                        if (r[s] != nullptr) {
                            const float4 r4 = load4(r[s], k, D, vec_r);
                            rv[0] = r4.x; rv[1] = r4.y; rv[2] = r4.z; rv[3] = r4.w;
                        }
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int c = k + e;
                            const float g = dqv[e] + dpos[s] * ebv[e];  // d loss / d adjusted embedding
                            if (r[s] == nullptr) {
                                gb[e] += dpos[s] * eav[e];
                                ga[e] += g;
                            } else if (d.decoder == GE2_DECODER_DISTMULT) {
                                gb[e] += dpos[s] * (eav[e] * rv[e]);
                                ga[e] += g * rv[e];
                                vr[e] = g * eav[e];
                            } else if (c < D) {
                                // complex Hadamard forward and backward: both need the partner component
                                const int cp = c < h ? c + h : c - h;
                                const float gp = dq[s][cp] + dpos[s] * __ldg(eb + cp);
                                const float rp = __ldg(r[s] + cp), eap = __ldg(ea + cp);
                                if (c < h) {  // real component: g = g_re, gp = g_im
                                    gb[e] += dpos[s] * (eav[e] * rv[e] - eap * rp);
                                    ga[e] += g * rv[e] + gp * rp;
                                    vr[e] = g * eav[e] + gp * eap;
                                } else {  // imaginary component: g = g_im, gp = g_re
                                    gb[e] += dpos[s] * (eap * rv[e] + eav[e] * rp);
                                    ga[e] += -gp * rv[e] + g * rp;
                                    vr[e] = -gp * eav[e] + g * eap;
                                }
                            }
                        }
                        if (rg[s] != nullptr) add4(slot_r[s], rg[s], k, make_float4(vr[0], vr[1], vr[2], vr[3]));
                    }
                    add4(slot_s, d.node_grad + sid * D, k, make_float4(gs[0], gs[1], gs[2], gs[3]));
                    add4(slot_d, d.node_grad + did * D, k, make_float4(gd[0], gd[1], gd[2], gd[3]));
                }
            }
        } else if (live) {
            const int64_t e = w - e_rows;
            const int s = (int)(e / L.CN);
            const int64_t j = e - (int64_t)s * L.CN;
            const int64_t id = (s == 0 ? d.dst_negs : d.src_negs)[j];
            if (id >= 0 && id < d.U) {
                const float* dk = L.dK + e * ld;
                const int slot = claim(id);
                for (int k = gl * 4; k < D; k += kFinLanes * 4) add4(slot, d.node_grad + id * D, k, *reinterpret_cast<const float4*>(dk + k));
            }
        }
    }
    __syncthreads();
    // flush: group g writes slot g
    if (group < kFinSlots) {
        const long long key = sm.tag[group];
        if (key != kFinEmpty) {
            const int kind = (int)(key >> 40);
            const long long id = key & ((1ll << 40) - 1);
            float* grow = kind == 0 ? d.node_grad + id * D : (kind == 1 ? d.rel_grad : d.inv_rel_grad) + id * D;
            for (int k = gl * 4; k < D; k += kFinLanes * 4)
                add4(-1, grow, k, make_float4(sm.acc[group][k], sm.acc[group][k + 1], sm.acc[group][k + 2], sm.acc[group][k + 3]));
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
    if (phases & 2) GE2_CUDA_TRY(cudaMemsetAsync(L.dK, 0, L.zero_bytes, stream));
    if ((phases & 4) && !(desc->flags & GE2_LP_NODE_GRAD_IS_ZERO))
        GE2_CUDA_TRY(cudaMemsetAsync(desc->node_grad, 0, (size_t)desc->U * desc->D * 4, stream));
    if (phases & 1) {
    GE2_CUDA_TRY(cudaMemsetAsync(L.mask, 0xFF, (size_t)L.S * L.CN * 4, stream));
    if (desc->deg_sample_rows != nullptr) {
        mask_from_deg_rows_kernel<<<stream_grid((int64_t)desc->C * desc->n_deg, 256), 256, 0, stream>>>(
            desc->deg_sample_rows, desc->C, desc->n_deg, L.npc, desc->B, desc->N, L.S, L.CN, L.mask, desc->status);
        GE2_LAUNCH_CHECK();
    } else {
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
    lp_prep_kernel<<<stream_grid(prep_rows, 32, 8), 256, 0, stream>>>(a);
    GE2_LAUNCH_CHECK();
    }

    if (phases & 2) {
        rc = desc->precision == GE2_PRECISION_F16 ? lp_scores_f16(a, stream) : lp_scores_fp32(a, stream);
        if (rc != GE2_OK) return rc;
    }
    if (!(phases & 4)) return GE2_OK;

    const int64_t fin_rows = (int64_t)desc->B + (int64_t)L.S * L.CN;
    // contiguous row ranges per CTA (so that repeated rows meet in a CTA's shared table), two CTAs per SM worth of ranges
    const int fin_ctas = (int)(fin_rows < (int64_t)kNumSMs * 4 * 32 ? ceil_div<int64_t>(fin_rows, 32) : (int64_t)kNumSMs * 4);
    const int rows_per_cta = (int)round_up<int64_t>(ceil_div<int64_t>(fin_rows, fin_ctas), 32);
    lp_finish_kernel<<<(unsigned)ceil_div<int64_t>(fin_rows, rows_per_cta), 256, 0, stream>>>(a, rows_per_cta);
    GE2_LAUNCH_CHECK();
    if (desc->pos_scores != nullptr || desc->inv_pos_scores != nullptr) {
        copy_pos_kernel<<<ceil_div(L.Bp, 256), 256, 0, stream>>>(L.pos, L.Bp, desc->pos_scores, desc->inv_pos_scores, L.S);
        GE2_LAUNCH_CHECK();
    }
    return GE2_OK;
}
