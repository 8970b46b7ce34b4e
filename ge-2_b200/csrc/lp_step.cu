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

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
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

// ---------------------------------------------------------------------------------------------------
// prep: one warp per output row.  Rows [0, S*Bp) are query rows, rows [S*Bp, S*Bp + S*CN) negative rows.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) lp_prep_kernel(LpKernelArgs a) {
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t q_rows = (int64_t)L.S * L.Bp;
    const int64_t total = q_rows + (int64_t)L.S * L.CN;
    const int D = d.D, h = D / 2, ld = L.ld;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
        if (w < q_rows) {
            const int s = (int)(w / L.Bp);
            const int i = (int)(w - (int64_t)s * L.Bp);
            float* q = L.Q + ((int64_t)s * L.Bp + i) * ld;
            __half* qh = L.Qh != nullptr ? L.Qh + ((int64_t)s * L.Bp + i) * ld : nullptr;
            if (i >= d.B) {  // zero rows appended by pad_and_reshape; their positive score is padded with 0
                for (int k = lane; k < ld; k += 32) {
                    q[k] = 0.f;
                    if (qh != nullptr) qh[k] = __float2half_rn(0.f);
                }
                if (lane == 0) L.pos[(int64_t)s * L.Bp + i] = 0.f;
                continue;
            }
            const int64_t sid = d.src_ids[(int64_t)i * d.edge_stride];
            const int64_t did = d.dst_ids[(int64_t)i * d.edge_stride];
            bool ok = sid >= 0 && sid < d.U && did >= 0 && did < d.U;
            int64_t rid = 0;
            if (d.has_relations) {
                rid = d.rel_ids[(int64_t)i * d.rel_stride];
                ok = ok && rid >= 0 && rid < d.R;
            }
            if (!ok) {
                if (lane == 0) or_status(d.status, GE2_STATUS_BAD_INDEX);
                for (int k = lane; k < ld; k += 32) {
                    q[k] = 0.f;
                    if (qh != nullptr) qh[k] = __float2half_rn(0.f);
                }
                if (lane == 0) L.pos[(int64_t)s * L.Bp + i] = 0.f;
                continue;
            }
            const float* ea = emb_row(d, s == 0 ? sid : did);  // the endpoint the relation is applied to
            const float* eb = emb_row(d, s == 0 ? did : sid);  // the endpoint it is compared with
            const float* r = d.has_relations ? (s == 0 ? d.rel : d.inv_rel) + rid * D : nullptr;
            float dot = 0.f;
            for (int k = lane; k < ld; k += 32) {
                float v = 0.f;
                if (k < D) {
                    if (r == nullptr) {
                        v = ea[k];
                    } else if (d.decoder == GE2_DECODER_DISTMULT) {
                        v = ea[k] * r[k];
                    } else if (k < h) {
                        v = ea[k] * r[k] - ea[k + h] * r[k + h];
                    } else {
                        v = ea[k - h] * r[k] + ea[k] * r[k - h];
                    }
                    dot += v * eb[k];
                }
                q[k] = v;
                if (qh != nullptr) qh[k] = __float2half_rn(v);
            }
            dot = warp_sum(dot);
            if (lane == 0) L.pos[(int64_t)s * L.Bp + i] = dot;
        } else {
            const int64_t e = w - q_rows;
            const int s = (int)(e / L.CN);
            const int64_t j = e - (int64_t)s * L.CN;
            const int64_t id = (s == 0 ? d.dst_negs : d.src_negs)[j];
            float* krow = L.K + e * ld;
            __half* khrow = L.Kh != nullptr ? L.Kh + e * ld : nullptr;
            const bool bad = id < 0 || id >= d.U;
            if (bad && lane == 0) or_status(d.status, GE2_STATUS_BAD_INDEX);
            const float* src = bad ? nullptr : emb_row(d, id);
            for (int k = lane; k < ld; k += 32) {
                const float v = (!bad && k < D) ? src[k] : 0.f;
                krow[k] = v;
                if (khrow != nullptr) khrow[k] = __float2half_rn(v);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// finish: one warp per edge row and side, then one warp per negative row.
// ---------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) lp_finish_kernel(LpKernelArgs a) {
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const int64_t e_rows = (int64_t)L.S * d.B;
    const int64_t total = e_rows + (int64_t)L.S * L.CN;
    const int D = d.D, h = D / 2, ld = L.ld;
    const bool vec4 = (D % 4 == 0) && (((uintptr_t)d.node_grad | (uintptr_t)d.rel_grad | (uintptr_t)d.inv_rel_grad) & 15) == 0;
    for (int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; w < total; w += warps) {
        if (w < e_rows) {
            const int s = (int)(w / d.B);
            const int i = (int)(w - (int64_t)s * d.B);
            const int64_t sid = d.src_ids[(int64_t)i * d.edge_stride];
            const int64_t did = d.dst_ids[(int64_t)i * d.edge_stride];
            bool ok = sid >= 0 && sid < d.U && did >= 0 && did < d.U;
            int64_t rid = 0;
            if (d.has_relations) {
                rid = d.rel_ids[(int64_t)i * d.rel_stride];
                ok = ok && rid >= 0 && rid < d.R;
            }
            if (!ok) continue;  // already flagged by prep
            const int64_t aid = s == 0 ? sid : did, bid = s == 0 ? did : sid;
            const float* ea = emb_row(d, aid);
            const float* eb = emb_row(d, bid);
            const float* r = d.has_relations ? (s == 0 ? d.rel : d.inv_rel) + rid * D : nullptr;
            float* rg = d.has_relations ? (s == 0 ? d.rel_grad : d.inv_rel_grad) + rid * D : nullptr;
            const int64_t qrow = (int64_t)s * L.Bp + i;
            const float* q = L.Q + qrow * ld;
            const float* dq = L.dQ + qrow * ld;
            const float dpos = __expf(L.pos[qrow] - L.lse[qrow]) - 1.0f;  // d loss / d pos_i = softmax prob of the positive - 1
            float* ga = d.node_grad + aid * D;
            float* gb = d.node_grad + bid * D;
            // per column k: contribution to the compared endpoint (gb), the relation-adjusted endpoint (ga) and the relation row (gr)
            auto column = [&](int k, float& vb, float& va, float& vr) {
                vb = dpos * q[k];
                const float g = dq[k] + dpos * eb[k];  // d loss / d adjusted embedding
                if (r == nullptr) {
                    va = g;
                    vr = 0.f;
                } else if (d.decoder == GE2_DECODER_DISTMULT) {
                    va = g * r[k];
                    vr = g * ea[k];
                } else {
                    // complex Hadamard backward: needs the gradient of the partner component too
                    const int kp = k < h ? k + h : k - h;
                    const float gp = dq[kp] + dpos * eb[kp];
                    if (k < h) {  // real component: g = g_re, gp = g_im
                        va = g * r[k] + gp * r[kp];
                        vr = g * ea[k] + gp * ea[kp];
                    } else {  // imaginary component: g = g_im, gp = g_re
                        va = -gp * r[k] + g * r[kp];
                        vr = -gp * ea[k] + g * ea[kp];
                    }
                }
            };
            if (vec4) {  // 16-byte vector reductions: a quarter of the atomic operations
                for (int k = lane * 4; k < D; k += 128) {
                    float vb[4], va[4], vr[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) column(k + e, vb[e], va[e], vr[e]);
                    atomicAdd(reinterpret_cast<float4*>(gb + k), make_float4(vb[0], vb[1], vb[2], vb[3]));
                    atomicAdd(reinterpret_cast<float4*>(ga + k), make_float4(va[0], va[1], va[2], va[3]));
                    if (rg != nullptr) atomicAdd(reinterpret_cast<float4*>(rg + k), make_float4(vr[0], vr[1], vr[2], vr[3]));
                }
            } else {
                for (int k = lane; k < D; k += 32) {
                    float vb, va, vr;
                    column(k, vb, va, vr);
                    atomicAdd(&gb[k], vb);
                    atomicAdd(&ga[k], va);
                    if (rg != nullptr) atomicAdd(&rg[k], vr);
                }
            }
        } else {
            const int64_t e = w - e_rows;
            const int s = (int)(e / L.CN);
            const int64_t j = e - (int64_t)s * L.CN;
            const int64_t id = (s == 0 ? d.dst_negs : d.src_negs)[j];
            if (id < 0 || id >= d.U) continue;
            const float* dk = L.dK + e * ld;
            float* g = d.node_grad + id * D;
            if (vec4) {
                for (int k = lane * 4; k < D; k += 128) {
                    const float4 v = *reinterpret_cast<const float4*>(dk + k);
                    if (v.x != 0.f || v.y != 0.f || v.z != 0.f || v.w != 0.f) atomicAdd(reinterpret_cast<float4*>(g + k), v);
                }
            } else {
                for (int k = lane; k < D; k += 32) {
                    const float v = dk[k];
                    if (v != 0.f) atomicAdd(&g[k], v);
                }
            }
        }
    }
}

// loss = sum over sides and padded rows of (lse - pos); fixed reduction order so the value is reproducible
__global__ void __launch_bounds__(1024) lp_loss_kernel(const float* __restrict__ lse, const float* __restrict__ pos, int64_t n,
                                                       float* __restrict__ loss) {
    __shared__ double s_part[32];
    double acc = 0.0;
    for (int64_t i = threadIdx.x; i < n; i += blockDim.x) acc += (double)lse[i] - (double)pos[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x < 32) {
        double v = threadIdx.x < (blockDim.x >> 5) ? s_part[threadIdx.x] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        if (threadIdx.x == 0) *loss = (float)v;
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
    if (phases & 4) GE2_CUDA_TRY(cudaMemsetAsync(desc->node_grad, 0, (size_t)desc->U * desc->D * 4, stream));
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
    lp_prep_kernel<<<stream_grid(prep_rows, 8, 8), 256, 0, stream>>>(a);
    GE2_LAUNCH_CHECK();
    }

    if (phases & 2) {
        rc = desc->precision == GE2_PRECISION_F16 ? lp_scores_f16(a, stream) : lp_scores_fp32(a, stream);
        if (rc != GE2_OK) return rc;
    }
    if (!(phases & 4)) return GE2_OK;

    const int64_t fin_rows = (int64_t)L.S * desc->B + (int64_t)L.S * L.CN;
    lp_finish_kernel<<<stream_grid(fin_rows, 8, 8), 256, 0, stream>>>(a);
    GE2_LAUNCH_CHECK();
    lp_loss_kernel<<<1, 1024, 0, stream>>>(L.lse, L.pos, (int64_t)L.S * L.Bp, desc->loss);
    GE2_LAUNCH_CHECK();
    if (desc->pos_scores != nullptr || desc->inv_pos_scores != nullptr) {
        copy_pos_kernel<<<ceil_div(L.Bp, 256), 256, 0, stream>>>(L.pos, L.Bp, desc->pos_scores, desc->inv_pos_scores, L.S);
        GE2_LAUNCH_CHECK();
    }
    return GE2_OK;
}
