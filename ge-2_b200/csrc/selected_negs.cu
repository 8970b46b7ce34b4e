// Selected-negative scoring for the DNS / GAN / tournament samplers: a query row is scored against the few negatives chosen
// for it instead of against its whole chunk.
//
// Follows, in the reference project:
//   scores of chosen pairs, forward     gege/src/cuda/src/nn/decoders/edge/distmult_selected_neg_cuda.cu:15-85
//                                       (one thread per (row, chosen negative) walking D; dot product, or
//                                       sqrt(max(|q - n|^2, 1e-8)) for the L2 comparator)
//   ... backward                        same file :88-202 (query gradient: a thread per (row, d) looping the chosen negatives;
//                                       negative gradient: an atomic add per (row, chosen, d); L2: one thread per pair)
//   tournament selection                gege/src/cpp/src/nn/decoders/edge/distmult_selected_neg_cuda.cpp:46-121 (per tile of
//                                       groups: bmm -> view [.., groups, T] -> max(3) -> gather; the negatives of a chunk form
//                                       `selected` groups of T = N / selected consecutive ones, a row keeps the best of each)
//
// Here a warp owns a query row: the row sits in registers (D <= 128, four values a lane), every chosen negative row is read
// once with coalesced (16-byte, where the rows allow it) loads and serves the score, the query gradient and the negative gradient of its pair in one pass
// (the reference's backward reads every pair twice, in two launches).  The tournament never stores the [rows x N] scores:
// a CTA holds 128 query rows in shared memory, streams 128-column tiles whose edges fall on group boundaries, and scans each
// tile for the group winners.  fp32 on the CUDA cores: the winner of a group is decided by comparing nearly equal scores.
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"

namespace ge2 {
namespace {

constexpr int kMaxD = 128;
constexpr int kPairThreads = 256, kPairWarps = kPairThreads / 32;
constexpr float kL2Floor = 1e-8f;  // the reference's kSelectedNegL2Tol, compared in float

struct PairArgs {
    const float* chunked;     // [chunks * R, D]
    const float* negatives;   // [chunks, N, D]
    const int64_t* selected;  // [chunks * R, K] columns of the row's chunk
    int64_t rows, R, N, K;
    int D, kind;
    int32_t* status;
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// A row of D <= 128 floats over the 32 lanes, four values a lane.  VEC (D a multiple of 4, 16-byte aligned rows): lane l holds
// elements 4l .. 4l+3, one 16-byte access; else lane l holds elements l, l+32, l+64, l+96.  Values past D are 0.
template <bool VEC>
__device__ __forceinline__ void load_row(float (&v)[4], const float* __restrict__ p, int lane, int D) {
    if (VEC) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (lane * 4 < D) t = __ldg(reinterpret_cast<const float4*>(p) + lane);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = lane + 32 * j < D ? __ldg(p + lane + 32 * j) : 0.f;
    }
}

template <bool VEC>
__device__ __forceinline__ void store_row(float* __restrict__ p, const float (&v)[4], int lane, int D) {
    if (VEC) {
        if (lane * 4 < D) reinterpret_cast<float4*>(p)[lane] = make_float4(v[0], v[1], v[2], v[3]);
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (lane + 32 * j < D) p[lane + 32 * j] = v[j];
    }
}

template <bool VEC>
__device__ __forceinline__ void add_row(float* __restrict__ p, const float (&v)[4], int lane, int D) {
    if (VEC) {
        if (lane * 4 < D) atomicAdd(reinterpret_cast<float4*>(p) + lane, make_float4(v[0], v[1], v[2], v[3]));  // four element-wise adds, one request
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++)
            if (lane + 32 * j < D) atomicAdd(p + lane + 32 * j, v[j]);
    }
}

// this lane's share of q . n (DOT) or |q - n|^2 (L2); lanes past D hold zeros in both
template <int KIND>
__device__ __forceinline__ float pair_partial(const float (&q)[4], const float (&n)[4]) {
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        if (KIND == GE2_SELECTED_DOT) {
            part = __fmaf_rn(q[j], n[j], part);
        } else {
            const float diff = q[j] - n[j];
            part = __fmaf_rn(diff, diff, part);
        }
    }
    return part;
}

template <int KIND>
__device__ __forceinline__ float finish_score(float sum) {
    return KIND == GE2_SELECTED_DOT ? sum : sqrtf(fmaxf(sum, kL2Floor));
}

// out[row, k] = score(chunked[row], negatives[chunk(row), selected[row, k]]); an index outside [0, N) scores 0 and sets BAD_INDEX.
// Four pairs a turn: their partial sums are folded across the warp together (6 shuffles for 4 sums instead of 20), lanes 0, 8,
// 16 and 24 end up with the totals of pairs 0, 1, 2 and 3.
template <bool VEC, int KIND>
__global__ void __launch_bounds__(kPairThreads) selected_scores_kernel(PairArgs a, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * kPairWarps;
    const bool hi = (lane & 16) != 0, mid = (lane & 8) != 0;
    const int my_pair = (hi ? 2 : 0) + (mid ? 1 : 0);
    for (int64_t row = (int64_t)blockIdx.x * kPairWarps + (threadIdx.x >> 5); row < a.rows; row += warps) {
        const int64_t c = row / a.R;
        float qv[4];
        load_row<VEC>(qv, a.chunked + row * a.D, lane, a.D);
        const int64_t* sel = a.selected + row * a.K;
        const float* negs = a.negatives + c * a.N * a.D;
        float* out_row = out + row * a.K;
        int64_t k = 0;
        for (; k + 4 <= a.K; k += 4) {
            float v[4];
            unsigned ok = 0u;  // one address per load for the warp: the columns and everything decided by them are warp-uniform
#pragma unroll
            for (int p = 0; p < 4; p++) {
                int64_t idx = __ldg(sel + k + p);
                if (idx >= 0 && idx < a.N) ok |= 1u << p;
                else idx = 0;  // a stand-in row for the loads; its score is dropped below
                float nv[4];
                load_row<VEC>(nv, negs + idx * a.D, lane, a.D);
                v[p] = pair_partial<KIND>(qv, nv);
            }
            const float r0 = (hi ? v[2] : v[0]) + __shfl_xor_sync(0xffffffffu, hi ? v[0] : v[2], 16);
            const float r1 = (hi ? v[3] : v[1]) + __shfl_xor_sync(0xffffffffu, hi ? v[1] : v[3], 16);
            float sum = (mid ? r1 : r0) + __shfl_xor_sync(0xffffffffu, mid ? r0 : r1, 8);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            if ((lane & 7) == 0) out_row[k + my_pair] = ((ok >> my_pair) & 1u) ? finish_score<KIND>(sum) : 0.f;
            if (ok != 0xFu && lane == 0) or_status(a.status, GE2_STATUS_BAD_INDEX);
        }
        for (; k < a.K; k++) {
            const int64_t idx = __ldg(sel + k);
            const bool ok = idx >= 0 && idx < a.N;
            float nv[4];
            load_row<VEC>(nv, negs + (ok ? idx : 0) * a.D, lane, a.D);
            const float sum = warp_sum(pair_partial<KIND>(qv, nv));
            if (lane == 0) {
                if (!ok) or_status(a.status, GE2_STATUS_BAD_INDEX);
                out_row[k] = ok ? finish_score<KIND>(sum) : 0.f;
            }
        }
    }
}

// grad_chunked[row] = sum_k d score / d q; grad_negatives (zeroed by the caller of the kernel) += d score / d n per pair.
// dot: dq = g n, dn = g q.  L2: dq = g (q - n) / |q - n|, dn = -dq, nothing when |q - n|^2 <= 1e-8.
template <bool VEC, int KIND>
__global__ void __launch_bounds__(kPairThreads) selected_scores_backward_kernel(PairArgs a, const float* __restrict__ grad_out,
                                                                                float* __restrict__ grad_chunked,
                                                                                float* __restrict__ grad_negatives) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = (int64_t)gridDim.x * kPairWarps;
    for (int64_t row = (int64_t)blockIdx.x * kPairWarps + (threadIdx.x >> 5); row < a.rows; row += warps) {
        const int64_t c = row / a.R;
        float qv[4], acc[4] = {0.f, 0.f, 0.f, 0.f};
        load_row<VEC>(qv, a.chunked + row * a.D, lane, a.D);
        const int64_t* sel = a.selected + row * a.K;
        const float* g_row = grad_out + row * a.K;
        for (int64_t k = 0; k < a.K; k++) {
            const int64_t idx = __ldg(sel + k);
            if (idx < 0 || idx >= a.N) {  // warp-uniform
                if (lane == 0) or_status(a.status, GE2_STATUS_BAD_INDEX);
                continue;
            }
            const float g = __ldg(g_row + k);
            const int64_t n_off = (c * a.N + idx) * a.D;
            float nv[4], dn[4];
            load_row<VEC>(nv, a.negatives + n_off, lane, a.D);
            if (KIND == GE2_SELECTED_DOT) {
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    acc[j] = __fmaf_rn(g, nv[j], acc[j]);
                    dn[j] = g * qv[j];
                }
            } else {
                const float sq = warp_sum(pair_partial<KIND>(qv, nv));
                if (sq <= kL2Floor) continue;  // warp-uniform: every lane holds the same sum
                const float coeff = g / sqrtf(sq);
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const float v = coeff * (qv[j] - nv[j]);
                    acc[j] += v;
                    dn[j] = -v;
                }
            }
            add_row<VEC>(grad_negatives + n_off, dn, lane, a.D);
        }
        store_row<VEC>(grad_chunked + row * a.D, acc, lane, a.D);
    }
}

// ---------------------------------------------------------------------------------------------------------------------------
// tournament selection
// ---------------------------------------------------------------------------------------------------------------------------
constexpr int kTile = 128, kHalf = kTile / 2, kChunkD = 32, kTourThreads = 256;
constexpr int kTileStride = kTile + 4;  // floats between the rows of Qt and Et: 16-byte aligned, banks shifted by 4 a row
constexpr int kStStride = kTile + 1;
constexpr int kFetch = kTile * kChunkD / kTourThreads;  // values of a negative slice a thread moves: 16 consecutive of one row

struct TourArgs {
    const float* chunked;    // [chunks, R, D]
    const float* negatives;  // [chunks, N, D]
    int64_t R, N, K, T;      // T = N / K negatives in a group
    int64_t units;           // work items of a (chunk, row tile): T <= 128: tiles of groups_per_unit whole groups; else one group
    int64_t units_per_cta;   // a CTA takes this many consecutive units
    int groups_per_unit;
    int D;
    float* out_scores;       // [chunks * R, K]
    int64_t* out_idx;        // [chunks * R, K] column of the winner in its chunk
};

inline size_t tour_smem_bytes(int D) { return (size_t)(D * kTileStride + kChunkD * kTileStride + kHalf * kStStride) * sizeof(float); }

// the slice [c0, c0 + 32) of 128 negative rows starting at column n0: a thread holds 16 consecutive values of one row
__device__ __forceinline__ void tour_fetch(float (&r)[kFetch], const float* __restrict__ Nc, int64_t n0, int64_t col_end, int c0, int D, int tid) {
    const int64_t col = n0 + (tid >> 1);
    const int d0 = c0 + (tid & 1) * kFetch;
    const float* row = Nc + col * D;
    const bool in = col < col_end;
#pragma unroll
    for (int k = 0; k < kFetch; k++) r[k] = (in && d0 + k < D) ? __ldg(row + d0 + k) : 0.f;
}

// grid: x = tiles of 128 query rows, y = shares of the units, z = chunk.  256 threads as 16 x 16; a thread owns rows
// {ty*4 .. +3} and {64 + ty*4 .. +3} and columns {tx*4 .. +3} and {64 + tx*4 .. +3} of the 128 x 128 tile: 64 multiply-adds
// for four 16-byte shared-memory loads a step.  The slices of the negative tiles go global -> registers -> shared memory, the
// next slice (of this tile or of the CTA's next tile) in flight while the current one is multiplied.  The tile's scores pass
// through shared memory 64 rows at a time for the scan of the group winners.
__global__ void __launch_bounds__(kTourThreads, 2) tournament_kernel(TourArgs a) {
    extern __shared__ __align__(16) float tour_smem[];
    float* Qt = tour_smem;                    // [D][132]: the CTA's query rows, transposed
    float* Et = Qt + a.D * kTileStride;       // [32][132]: a slice of the negative tile, transposed
    float* St = Et + kChunkD * kTileStride;   // [64][129]: half of the tile's scores
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int D = a.D;
    const int64_t c = blockIdx.z, r0 = (int64_t)blockIdx.x * kTile;
    const int rows_here = (int)(a.R - r0 < kTile ? a.R - r0 : kTile);
    const float* Q = a.chunked + (c * a.R + r0) * D;
    for (int k = tid; k < kTile * D; k += kTourThreads) {
        const int row = k / D, cc = k - row * D;
        Qt[cc * kTileStride + row] = row < rows_here ? __ldg(Q + k) : 0.f;
    }
    const float* Nc = a.negatives + c * a.N * D;
    const bool whole_groups = a.T <= kTile;  // every group of a unit lies inside its one tile
    const int64_t u_first = (int64_t)blockIdx.y * a.units_per_cta;
    const int64_t u_last = u_first + a.units_per_cta < a.units ? u_first + a.units_per_cta : a.units;
    auto unit_groups = [&](int64_t u) { return (int)(a.K - u * a.groups_per_unit < a.groups_per_unit ? a.K - u * a.groups_per_unit : a.groups_per_unit); };
    float pre[kFetch];
    if (u_first < u_last) tour_fetch(pre, Nc, u_first * a.groups_per_unit * a.T, (u_first * a.groups_per_unit + unit_groups(u_first)) * a.T, 0, D, tid);
    for (int64_t u = u_first; u < u_last; u++) {
        const int64_t g_begin = u * a.groups_per_unit;
        const int g_count = unit_groups(u);
        const int64_t col_begin = g_begin * a.T, col_end = col_begin + (int64_t)g_count * a.T;
        // a group wider than a tile: thread t < 64 keeps the running winners of rows t and 64 + t over the group's tiles
        float best_v[2] = {-CUDART_INF_F, -CUDART_INF_F};
        int64_t best_i[2] = {col_begin, col_begin};
        for (int64_t n0 = col_begin; n0 < col_end; n0 += kTile) {
            float acc[8][8];
#pragma unroll
            for (int i = 0; i < 8; i++)
#pragma unroll
                for (int j = 0; j < 8; j++) acc[i][j] = 0.f;
            for (int c0 = 0; c0 < D; c0 += kChunkD) {
                {
                    const int node = tid >> 1, cc = (tid & 1) * kFetch;
#pragma unroll
                    for (int k = 0; k < kFetch; k++) Et[(cc + k) * kTileStride + node] = pre[k];
                }
                __syncthreads();  // also orders the writes of Qt before its first use
                // what comes after this slice: the tile's next slice, the unit's next tile, or the CTA's next unit
                if (c0 + kChunkD < D) {
                    tour_fetch(pre, Nc, n0, col_end, c0 + kChunkD, D, tid);
                } else if (n0 + kTile < col_end) {
                    tour_fetch(pre, Nc, n0 + kTile, col_end, 0, D, tid);
                } else if (u + 1 < u_last) {
                    const int64_t nb = (u + 1) * a.groups_per_unit * a.T;
                    tour_fetch(pre, Nc, nb, nb + (int64_t)unit_groups(u + 1) * a.T, 0, D, tid);
                }
                const int kmax = D - c0 < kChunkD ? D - c0 : kChunkD;
                for (int k = 0; k < kmax; k++) {
                    const float* qrow = Qt + (c0 + k) * kTileStride + ty * 4;
                    const float* erow = Et + k * kTileStride + tx * 4;
                    const float4 q0 = *reinterpret_cast<const float4*>(qrow), q1 = *reinterpret_cast<const float4*>(qrow + kHalf);
                    const float4 e0 = *reinterpret_cast<const float4*>(erow), e1 = *reinterpret_cast<const float4*>(erow + kHalf);
                    const float qv[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
                    const float ev[8] = {e0.x, e0.y, e0.z, e0.w, e1.x, e1.y, e1.z, e1.w};
#pragma unroll
                    for (int i = 0; i < 8; i++)
#pragma unroll
                        for (int j = 0; j < 8; j++) acc[i][j] = __fmaf_rn(qv[i], ev[j], acc[i][j]);
                }
                __syncthreads();
            }
            // the scores of rows [64 h, 64 h + 64) go through St, then the (row, group) winners are read off it
#pragma unroll
            for (int h = 0; h < 2; h++) {
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 8; j++)
                        St[(ty * 4 + i) * kStStride + (j < 4 ? tx * 4 + j : kHalf + tx * 4 + j - 4)] = acc[h * 4 + i][j];
                __syncthreads();
                if (whole_groups) {
                    // one (row, group) per thread and turn; groups vary fastest, so a warp writes runs of adjacent winners
                    const int T = (int)a.T;
                    for (int it = tid; it < kHalf * g_count; it += kTourThreads) {
                        const int lr = it / g_count, g = it - lr * g_count, row = h * kHalf + lr;
                        const float* sc = St + lr * kStStride + g * T;
                        float bv = sc[0];
                        int bi = 0;
                        for (int j = 1; j < T; j++)
                            if (sc[j] > bv) {  // the first of equal scores wins
                                bv = sc[j];
                                bi = j;
                            }
                        if (row < rows_here) {
                            const int64_t o = (c * a.R + r0 + row) * a.K + g_begin + g;
                            a.out_scores[o] = bv;
                            a.out_idx[o] = n0 + (int64_t)g * T + bi;
                        }
                    }
                } else if (tid < kHalf) {
                    const int len = (int)(col_end - n0 < kTile ? col_end - n0 : kTile);
                    const float* sc = St + tid * kStStride;
                    for (int j = 0; j < len; j++)
                        if (sc[j] > best_v[h]) {
                            best_v[h] = sc[j];
                            best_i[h] = n0 + j;
                        }
                }
                __syncthreads();  // the other half, or the next tile, overwrites St
            }
        }
        if (!whole_groups && tid < kHalf) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int row = h * kHalf + tid;
                if (row < rows_here) {
                    const int64_t o = (c * a.R + r0 + row) * a.K + g_begin;
                    a.out_scores[o] = best_v[h];
                    a.out_idx[o] = best_i[h];
                }
            }
        }
    }
}

int check_pairs(int kind, const void* chunked, const void* negatives, const void* selected, int64_t chunks, int64_t rows_per_chunk,
                int64_t num_negs, int64_t num_selected, int D) {
    if (kind != GE2_SELECTED_DOT && kind != GE2_SELECTED_L2) return GE2_ERR_INVALID_ARGUMENT;
    if (chunks < 0 || rows_per_chunk < 0 || num_negs <= 0 || num_selected < 0 || D <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (D > kMaxD) return GE2_ERR_UNSUPPORTED;
    if (chunks * rows_per_chunk * num_selected > 0 && (chunked == nullptr || negatives == nullptr || selected == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    return GE2_OK;
}

// 16-byte accesses to rows: D a multiple of 4 and every table that is touched 16-byte aligned
bool rows_are_vectors(int D, const void* p0, const void* p1, const void* p2, const void* p3) {
    return (D & 3) == 0 && (((uintptr_t)p0 | (uintptr_t)p1 | (uintptr_t)p2 | (uintptr_t)p3) & 15) == 0;
}

PairArgs pair_args(int kind, const float* chunked, const float* negatives, const int64_t* selected, int64_t chunks, int64_t rows_per_chunk,
                   int64_t num_negs, int64_t num_selected, int D, int32_t* status) {
    PairArgs a;
    a.chunked = chunked;
    a.negatives = negatives;
    a.selected = selected;
    a.rows = chunks * rows_per_chunk;
    a.R = rows_per_chunk;
    a.N = num_negs;
    a.K = num_selected;
    a.D = D;
    a.kind = kind;
    a.status = status;
    return a;
}

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" int ge2_selected_neg_scores(int kind, const float* chunked, const float* negatives, const int64_t* selected, int64_t chunks,
                                       int64_t rows_per_chunk, int64_t num_negs, int64_t num_selected, int D, float* out_scores,
                                       int32_t* status, ge2_stream_t stream_) {
    const int rc = check_pairs(kind, chunked, negatives, selected, chunks, rows_per_chunk, num_negs, num_selected, D);
    if (rc != GE2_OK) return rc;
    const int64_t rows = chunks * rows_per_chunk;
    if (rows * num_selected == 0) return GE2_OK;
    if (out_scores == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    const PairArgs a = pair_args(kind, chunked, negatives, selected, chunks, rows_per_chunk, num_negs, num_selected, D, status);
    const bool vec = rows_are_vectors(D, chunked, negatives, nullptr, nullptr);
    const dim3 grid((unsigned)stream_grid(rows, kPairWarps));
    cudaStream_t stream = as_stream(stream_);
    if (kind == GE2_SELECTED_DOT) {
        if (vec) selected_scores_kernel<true, GE2_SELECTED_DOT><<<grid, kPairThreads, 0, stream>>>(a, out_scores);
        else selected_scores_kernel<false, GE2_SELECTED_DOT><<<grid, kPairThreads, 0, stream>>>(a, out_scores);
    } else {
        if (vec) selected_scores_kernel<true, GE2_SELECTED_L2><<<grid, kPairThreads, 0, stream>>>(a, out_scores);
        else selected_scores_kernel<false, GE2_SELECTED_L2><<<grid, kPairThreads, 0, stream>>>(a, out_scores);
    }
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_selected_neg_scores_backward(int kind, const float* grad_out, const float* chunked, const float* negatives,
                                                const int64_t* selected, int64_t chunks, int64_t rows_per_chunk, int64_t num_negs,
                                                int64_t num_selected, int D, float* grad_chunked, float* grad_negatives, int32_t* status,
                                                ge2_stream_t stream_) {
    const int rc = check_pairs(kind, chunked, negatives, selected, chunks, rows_per_chunk, num_negs, num_selected, D);
    if (rc != GE2_OK) return rc;
    const int64_t rows = chunks * rows_per_chunk;
    cudaStream_t stream = as_stream(stream_);
    if (chunks > 0) {
        if (grad_negatives == nullptr) return GE2_ERR_INVALID_ARGUMENT;
        GE2_CUDA_TRY(cudaMemsetAsync(grad_negatives, 0, (size_t)(chunks * num_negs * D) * sizeof(float), stream));
    }
    if (rows == 0) return GE2_OK;
    if (grad_chunked == nullptr || (num_selected > 0 && grad_out == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    // with nothing selected the kernel still writes the zero query gradient
    const PairArgs a = pair_args(kind, chunked, negatives, selected, chunks, rows_per_chunk, num_negs, num_selected, D, status);
    const bool vec = rows_are_vectors(D, chunked, negatives, grad_chunked, grad_negatives);
    const dim3 grid((unsigned)stream_grid(rows, kPairWarps));
    if (kind == GE2_SELECTED_DOT) {
        if (vec) selected_scores_backward_kernel<true, GE2_SELECTED_DOT><<<grid, kPairThreads, 0, stream>>>(a, grad_out, grad_chunked, grad_negatives);
        else selected_scores_backward_kernel<false, GE2_SELECTED_DOT><<<grid, kPairThreads, 0, stream>>>(a, grad_out, grad_chunked, grad_negatives);
    } else {
        if (vec) selected_scores_backward_kernel<true, GE2_SELECTED_L2><<<grid, kPairThreads, 0, stream>>>(a, grad_out, grad_chunked, grad_negatives);
        else selected_scores_backward_kernel<false, GE2_SELECTED_L2><<<grid, kPairThreads, 0, stream>>>(a, grad_out, grad_chunked, grad_negatives);
    }
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_tournament_select(const float* selector_chunked, const float* selector_negatives, const float* score_chunked,
                                     const float* score_negatives, int64_t chunks, int64_t rows_per_chunk, int64_t num_negs,
                                     int64_t num_selected, int D, float* out_scores, int64_t* out_idx, ge2_stream_t stream_) {
    if (chunks < 0 || rows_per_chunk < 0 || num_negs <= 0 || num_selected <= 0 || D <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (num_negs % num_selected != 0) return GE2_ERR_INVALID_ARGUMENT;  // the reference's TORCH_CHECK
    if (D > kMaxD || chunks > 65535) return GE2_ERR_UNSUPPORTED;
    if (chunks * rows_per_chunk == 0) return GE2_OK;
    if (selector_chunked == nullptr || selector_negatives == nullptr || out_scores == nullptr || out_idx == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if (score_chunked == nullptr) score_chunked = selector_chunked;
    if (score_negatives == nullptr) score_negatives = selector_negatives;
    cudaStream_t stream = as_stream(stream_);

    TourArgs a;
    a.chunked = selector_chunked;
    a.negatives = selector_negatives;
    a.R = rows_per_chunk;
    a.N = num_negs;
    a.K = num_selected;
    a.T = num_negs / num_selected;
    a.D = D;
    a.groups_per_unit = a.T <= kTile ? (int)(kTile / a.T) : 1;
    a.units = ceil_div<int64_t>(num_selected, a.groups_per_unit);
    a.out_scores = out_scores;
    a.out_idx = out_idx;
    const int64_t row_tiles = ceil_div<int64_t>(rows_per_chunk, kTile);
    if (row_tiles > 0x7fffffffLL) return GE2_ERR_UNSUPPORTED;
    const size_t smem = tour_smem_bytes(D);
    // How many CTAs share the units of a (row tile, chunk): the split with the shortest bound on the makespan of CTAs handed
    // out greedily to `slots` resident places -- all work / slots + the work of one CTA, its query-tile load counted as a third
    // of a unit.  Two CTAs an SM by registers.
    const int64_t per_sm = std::max<int64_t>(1, std::min<int64_t>(2, (int64_t)(227 * 1024) / (int64_t)(smem + 1024)));
    const int64_t slots = (int64_t)kNumSMs * per_sm, base = row_tiles * chunks;
    int64_t shares = 1;
    double best_cost = 0.0;
    for (int64_t s = 1; s <= std::min<int64_t>(a.units, 64); s++) {
        const int64_t per = ceil_div<int64_t>(a.units, s), used = ceil_div<int64_t>(a.units, per);  // `used` CTAs get work
        const double cost = ((double)(base * used) / (double)slots + 1.0) * ((double)per + 0.33);
        if (s == 1 || cost < best_cost - 1e-9) {
            best_cost = cost;
            shares = used;
            a.units_per_cta = per;
        }
    }
    // per-device function attribute; setting it on every call keeps multi-device processes correct and is not a stream operation
    GE2_CUDA_TRY(cudaFuncSetAttribute(tournament_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)row_tiles, (unsigned)shares, (unsigned)chunks);
    tournament_kernel<<<grid, kTourThreads, smem, stream>>>(a);
    GE2_LAUNCH_CHECK();
    if (score_chunked != selector_chunked || score_negatives != selector_negatives) {
        // a selector separate from the scorer: the winners are scored again with the scorer's rows
        return ge2_selected_neg_scores(GE2_SELECTED_DOT, score_chunked, score_negatives, out_idx, chunks, rows_per_chunk, num_negs, num_selected,
                                       D, out_scores, nullptr, stream_);
    }
    return GE2_OK;
}
