// Internal layout shared by the kernels of the link-prediction training step (ge2_lp_step).
//
// Data flow of one step (S = corruption sides, Bp = C * ceil(B/C) padded batch rows, ld = padded row length):
//   prep     : gather src/dst/relation rows, apply the relation operator        -> Q[S][Bp][ld], pos[S][Bp]
//              gather negative rows                                              -> K[S][C*N][ld]
//   scores   : per (side, chunk): S = Q K^T, mask, row logsumexp with the positive score,
//              P = exp(S - lse), dQ = P K, dK = P^T Q  (score tiles never leave the SM)   -> lse, dQ, dK
//   finish   : relation-operator backward, d pos terms, duplicate-reducing scatter into node_grad / rel_grad, loss
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace ge2 {

constexpr float kLpF16GradUnscale = 1.0f / 16384.0f;  // the tensor path leaves dQ and dK scaled by 2^14 (its W tiles are)

struct LpLayout {
    int S;        // sides
    int npc;      // rows per chunk = ceil(B / C)
    int Bp;       // C * npc
    int ld;       // padded row length of Q / K / dQ / dK (floats)
    int64_t CN;   // C * N
    // workspace sections
    float* Q;         // [S][Bp][ld]
    float* K;         // [S][CN][ld]
    float* dQ;        // [S][Bp][ld]
    float* dK;        // [S][CN][ld]   fp32 path: zeroed every step, reduced with atomics; tensor path: stored tile by tile
    float* pos;       // [S][Bp]
    float* lse;       // [S][Bp]
    int32_t* mask;    // [S][CN]  batch row whose score in this (chunk, column) is masked, or -1
    __half* Qh;       // [S][Bp][ld]  fp16 copy of Q, operand of the tensor-core path (null on the fp32 path)
    __half* Kh;       // [S][CN][ld]  fp16 copy of K
    double* loss_acc; // [1] sum over rows of (lse - pos): zeroed by the prepare kernel, added to by the scores kernels
    float* part;      // [S][Bp][8][2] per-row partial (max, sum) of the logsumexp pass when a row block's tiles are split over CTAs
    float* lse2s;     // [S*C][row_blocks*128] row logsumexp in base-2 units minus the probability scale exponent; 1e30 for rows past the chunk
    int32_t* item_ctr;  // [S*C*row_blocks] arrivals of the CTAs sharing a row block in the logsumexp pass, then arrivals at and
                        // departures from the barrier between the two passes; all zero between steps
    int n_items;        // S * C * row_blocks
    float grad_unscale; // factor the scatter kernel applies to what it reads from dQ / dK: 1, or 2^-14 on the tensor path
    size_t bytes;
    size_t zero_begin, zero_bytes;  // dK range
};

struct LpKernelArgs {
    ge2_lp_desc d;
    LpLayout L;
};

inline size_t lp_align(size_t x) { return (x + 255) & ~(size_t)255; }

inline int lp_row_ld(int D) { return D <= 64 ? 64 : 128; }

inline LpLayout lp_make_layout(const ge2_lp_desc& d, void* base) {
    LpLayout L;
    L.S = (d.has_relations && d.use_inverse) ? 2 : 1;
    L.npc = rows_per_chunk(d.B, d.C);
    L.Bp = d.C * L.npc;
    L.ld = lp_row_ld(d.D);
    L.CN = (int64_t)d.C * d.N;
    char* p = (char*)base;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off += lp_align(bytes);
        return o;
    };
    size_t oQ = take((size_t)L.S * L.Bp * L.ld * 4);
    size_t oK = take((size_t)L.S * L.CN * L.ld * 4);
    size_t odQ = take((size_t)L.S * L.Bp * L.ld * 4);
    size_t odK = take((size_t)L.S * L.CN * L.ld * 4);
    size_t opos = take((size_t)L.S * L.Bp * 4);
    size_t olse = take((size_t)L.S * L.Bp * 4);
    size_t omask = take((size_t)L.S * L.CN * 4);
    size_t oloss = take(8);
    const bool half_copies = d.precision == GE2_PRECISION_F16;
    size_t oQh = half_copies ? take((size_t)L.S * L.Bp * L.ld * 2) : 0;
    size_t oKh = half_copies ? take((size_t)L.S * L.CN * L.ld * 2) : 0;
    size_t opart = half_copies ? take((size_t)L.S * L.Bp * 16 * 4) : 0;
    const int row_blocks = (L.npc + 127) / 128;
    L.n_items = L.S * d.C * row_blocks;
    size_t olse2 = half_copies ? take((size_t)L.n_items * 128 * 4) : 0;
    size_t octr = half_copies ? take((size_t)(L.n_items + 2) * 4) : 0;  // + the two counters of the grid barrier
    L.Q = (float*)(p + oQ);
    L.K = (float*)(p + oK);
    L.dQ = (float*)(p + odQ);
    L.dK = (float*)(p + odK);
    L.pos = (float*)(p + opos);
    L.lse = (float*)(p + olse);
    L.mask = (int32_t*)(p + omask);
    L.loss_acc = (double*)(p + oloss);
    L.Qh = half_copies ? (__half*)(p + oQh) : nullptr;
    L.Kh = half_copies ? (__half*)(p + oKh) : nullptr;
    L.part = half_copies ? (float*)(p + opart) : nullptr;
    L.grad_unscale = half_copies ? kLpF16GradUnscale : 1.0f;
    L.lse2s = half_copies ? (float*)(p + olse2) : nullptr;
    L.item_ctr = half_copies ? (int32_t*)(p + octr) : nullptr;
    L.zero_begin = odK;
    L.zero_bytes = (size_t)L.S * L.CN * L.ld * 4;
    L.bytes = off;
    return L;
}

// scores kernels (one per precision); both fill lse, dQ, dK (+ optional score dumps) from Q, K, pos, mask
int lp_scores_fp32(const LpKernelArgs& a, cudaStream_t stream);
int lp_scores_f16(const LpKernelArgs& a, cudaStream_t stream);

}  // namespace ge2
