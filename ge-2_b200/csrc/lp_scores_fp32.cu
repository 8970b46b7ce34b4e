// fp32 (CUDA-core FFMA) scores kernel of the link-prediction step: the 1e-4-parity path.
//
// One CTA = (side, chunk, 64-row block).  It keeps its 64 query rows in shared memory and streams the chunk's
// negatives past them twice, 64 at a time:
//   sweep 1: S = Q K^T per tile, mask, running (max, sum-exp) per row            -> lse (with the positive score folded in)
//   sweep 2: S again, P = exp(S - lse); dQ += P K (registers, whole sweep); dK tile = P^T Q -> atomics into dK
// The [rows x N] score matrix only ever exists as 64x64 tiles in registers / shared memory.
// Stands in for the reference's bmm + logsumexp + cross_entropy + autograd chain
// (cpp/src/nn/decoders/edge/comparators.cpp:128-138, cpp/src/nn/loss.cpp:46-63 of the reference project).
#include <math.h>

#include "lp_internal.cuh"

namespace ge2 {
namespace {

constexpr int BM = 64;        // query rows per CTA
constexpr int BN = 64;        // negatives per tile
constexpr int kThreads = 256; // 16 x 16 threads, 4 x 4 scores each
constexpr float kMasked = -1e9f;

template <int DP>
struct Smem {
    float q[BM][DP + 4];
    float k[BN][DP + 4];
    float p[BM][BN + 4];
    float lse[BM];
    float loss[BM];  // per-row lse - pos, summed by one thread
    int32_t mask[BN];
};

template <int DP>
__device__ __forceinline__ void load_rows(float (*dst)[DP + 4], const float* __restrict__ src, int valid_rows, int tid) {
    // 64 rows x DP floats, float4 granularity; rows >= valid_rows are zero-filled
    constexpr int V = DP / 4;
    for (int e = tid; e < 64 * V; e += kThreads) {
        const int r = e / V, c = e - r * V;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < valid_rows) v = __ldg(reinterpret_cast<const float4*>(src + (int64_t)r * DP) + c);
        *reinterpret_cast<float4*>(&dst[r][c * 4]) = v;
    }
}

template <int DP>
__device__ __forceinline__ void score_tile(const Smem<DP>& sm, int ty, int tx, float (&acc)[4][4]) {
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int c = 0; c < 4; c++) acc[r][c] = 0.f;
#pragma unroll 4
    for (int d4 = 0; d4 < DP / 4; d4++) {
        float4 a[4], b[4];
#pragma unroll
        for (int r = 0; r < 4; r++) a[r] = *reinterpret_cast<const float4*>(&sm.q[ty + 16 * r][d4 * 4]);
#pragma unroll
        for (int c = 0; c < 4; c++) b[c] = *reinterpret_cast<const float4*>(&sm.k[tx + 16 * c][d4 * 4]);
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                acc[r][c] = fmaf(a[r].x, b[c].x, acc[r][c]);
                acc[r][c] = fmaf(a[r].y, b[c].y, acc[r][c]);
                acc[r][c] = fmaf(a[r].z, b[c].z, acc[r][c]);
                acc[r][c] = fmaf(a[r].w, b[c].w, acc[r][c]);
            }
    }
}

template <int DP>
__global__ void __launch_bounds__(kThreads, 2) lp_scores_fp32_kernel(LpKernelArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem<DP>& sm = *reinterpret_cast<Smem<DP>*>(smem_raw);
    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int s = blockIdx.z, c = blockIdx.y;
    const int row0 = blockIdx.x * BM;                 // first row of this block inside the chunk
    const int valid_rows = min(BM, L.npc - row0);      // rows past the chunk end do not exist
    const int64_t grow0 = (int64_t)s * L.Bp + (int64_t)c * L.npc + row0;  // row in the [S*Bp] arrays
    const float* Kc = L.K + ((int64_t)s * L.CN + (int64_t)c * d.N) * DP;
    const int32_t* maskc = L.mask + (int64_t)s * L.CN + (int64_t)c * d.N;
    float* dKc = L.dK + ((int64_t)s * L.CN + (int64_t)c * d.N) * DP;
    float* dump = s == 0 ? d.neg_scores : d.inv_neg_scores;  // optional [Bp, N] score dump

    load_rows<DP>(sm.q, L.Q + grow0 * DP, valid_rows, tid);
    const int n_tiles = (d.N + BN - 1) / BN;

    // ---- sweep 1: row-wise logsumexp over the negatives --------------------------------------------
    float run_m[4], run_l[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        run_m[r] = -INFINITY;
        run_l[r] = 0.f;
    }
    for (int t = 0; t < n_tiles; t++) {
        const int n0 = t * BN;
        const int valid_n = min(BN, d.N - n0);
        __syncthreads();  // previous tile fully consumed (also orders the q load before first use)
        load_rows<DP>(sm.k, Kc + (int64_t)n0 * DP, valid_n, tid);
        if (tid < BN) sm.mask[tid] = tid < valid_n ? maskc[n0 + tid] : -1;
        __syncthreads();
        float acc[4][4];
        score_tile<DP>(sm, ty, tx, acc);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int lr = ty + 16 * r;
            const int brow = c * L.npc + row0 + lr;  // batch row (padded numbering), what the filter names
            float v[4];
            float tmax = -INFINITY;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const int lc = tx + 16 * cc;
                float sc = acc[r][cc];
                if (sm.mask[lc] == brow) sc = kMasked;
                v[cc] = lc < valid_n ? sc : -INFINITY;
                tmax = fmaxf(tmax, v[cc]);
                if (dump != nullptr && lr < valid_rows && lc < valid_n) dump[(int64_t)brow * d.N + n0 + lc] = sc;
            }
            if (tmax > -INFINITY) {
                const float nm = fmaxf(run_m[r], tmax);
                float add = 0.f;
#pragma unroll
                for (int cc = 0; cc < 4; cc++) add += expf(v[cc] - nm);  // exp(-inf) = 0 for absent columns
                run_l[r] = run_l[r] * expf(run_m[r] - nm) + add;
                run_m[r] = nm;
            }
        }
    }
    // combine the 16 threads that share a row (consecutive lanes of a half warp), fold in the positive score
#pragma unroll
    for (int r = 0; r < 4; r++) {
        float m = run_m[r], l = run_l[r];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, m, o);
            const float ol = __shfl_xor_sync(0xffffffffu, l, o);
            const float nm = fmaxf(m, om);
            if (nm > -INFINITY) {
                l = l * expf(m - nm) + ol * expf(om - nm);
                m = nm;
            }
        }
        const int lr = ty + 16 * r;
        if (tx == 0) {
            float lse = 0.f;
            if (lr < valid_rows) {
                const float pos = L.pos[grow0 + lr];
                const float nm = fmaxf(m, pos);
                const float z = l * expf(m - nm) + expf(pos - nm);
                lse = nm + logf(z);
                L.lse[grow0 + lr] = lse;
                sm.loss[lr] = lse - pos;
            } else {
                sm.loss[lr] = 0.f;
            }
            sm.lse[lr] = lse;
        }
    }

    __syncthreads();
    if (tid == 0) {  // one double-precision add per CTA into the step's loss
        double acc = 0.0;
        for (int r = 0; r < BM; r++) acc += (double)sm.loss[r];
        atomicAdd(L.loss_acc, acc);
    }
    // ---- sweep 2: probabilities, dQ and dK ---------------------------------------------------------
    constexpr int H = DP / 64;  // column groups of 64 floats; thread owns columns tx*4 + 64*h
    float dq[4][H][4];
#pragma unroll
    for (int r = 0; r < 4; r++)
#pragma unroll
        for (int hh = 0; hh < H; hh++)
#pragma unroll
            for (int e = 0; e < 4; e++) dq[r][hh][e] = 0.f;

    for (int t = 0; t < n_tiles; t++) {
        const int n0 = t * BN;
        const int valid_n = min(BN, d.N - n0);
        __syncthreads();  // previous tile's K / P fully consumed; sm.lse visible
        load_rows<DP>(sm.k, Kc + (int64_t)n0 * DP, valid_n, tid);
        if (tid < BN) sm.mask[tid] = tid < valid_n ? maskc[n0 + tid] : -1;
        __syncthreads();
        float acc[4][4];
        score_tile<DP>(sm, ty, tx, acc);
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int lr = ty + 16 * r;
            const int brow = c * L.npc + row0 + lr;
            const float lse = sm.lse[lr];
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {
                const int lc = tx + 16 * cc;
                float pr = 0.f;  // masked entries were overwritten in place: no gradient reaches them
                if (lr < valid_rows && lc < valid_n && sm.mask[lc] != brow) pr = expf(acc[r][cc] - lse);
                sm.p[lr][lc] = pr;
            }
        }
        __syncthreads();
        // dQ[rows ty+16r][cols] += sum_j P[row][j] * K[j][cols]
#pragma unroll 2
        for (int j4 = 0; j4 < BN / 4; j4++) {
            float4 pa[4];
#pragma unroll
            for (int r = 0; r < 4; r++) pa[r] = *reinterpret_cast<const float4*>(&sm.p[ty + 16 * r][j4 * 4]);
#pragma unroll
            for (int q = 0; q < 4; q++) {
#pragma unroll
                for (int hh = 0; hh < H; hh++) {
                    const float4 kb = *reinterpret_cast<const float4*>(&sm.k[j4 * 4 + q][tx * 4 + 64 * hh]);
#pragma unroll
                    for (int r = 0; r < 4; r++) {
                        const float pv = q == 0 ? pa[r].x : q == 1 ? pa[r].y : q == 2 ? pa[r].z : pa[r].w;
                        dq[r][hh][0] = fmaf(pv, kb.x, dq[r][hh][0]);
                        dq[r][hh][1] = fmaf(pv, kb.y, dq[r][hh][1]);
                        dq[r][hh][2] = fmaf(pv, kb.z, dq[r][hh][2]);
                        dq[r][hh][3] = fmaf(pv, kb.w, dq[r][hh][3]);
                    }
                }
            }
        }
        // dK[negatives ty*4+r][cols] = sum_i P[i][neg] * Q[i][cols]
        float dk[4][H][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int hh = 0; hh < H; hh++)
#pragma unroll
                for (int e = 0; e < 4; e++) dk[r][hh][e] = 0.f;
#pragma unroll 4
        for (int i = 0; i < BM; i++) {
            const float4 pa = *reinterpret_cast<const float4*>(&sm.p[i][ty * 4]);
#pragma unroll
            for (int hh = 0; hh < H; hh++) {
                const float4 qb = *reinterpret_cast<const float4*>(&sm.q[i][tx * 4 + 64 * hh]);
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const float pv = r == 0 ? pa.x : r == 1 ? pa.y : r == 2 ? pa.z : pa.w;
                    dk[r][hh][0] = fmaf(pv, qb.x, dk[r][hh][0]);
                    dk[r][hh][1] = fmaf(pv, qb.y, dk[r][hh][1]);
                    dk[r][hh][2] = fmaf(pv, qb.z, dk[r][hh][2]);
                    dk[r][hh][3] = fmaf(pv, qb.w, dk[r][hh][3]);
                }
            }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const int ln = ty * 4 + r;
            if (ln < valid_n) {
#pragma unroll
                for (int hh = 0; hh < H; hh++) {
                    const int col = tx * 4 + 64 * hh;
                    if (col < d.D) {  // padded columns of Q are zero: nothing to add there
                        float4* dst = reinterpret_cast<float4*>(dKc + (int64_t)(n0 + ln) * DP + col);
                        atomicAdd(dst, make_float4(dk[r][hh][0], dk[r][hh][1], dk[r][hh][2], dk[r][hh][3]));
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const int lr = ty + 16 * r;
        if (lr < valid_rows) {
#pragma unroll
            for (int hh = 0; hh < H; hh++) {
                const int col = tx * 4 + 64 * hh;
                *reinterpret_cast<float4*>(L.dQ + (grow0 + lr) * DP + col) = make_float4(dq[r][hh][0], dq[r][hh][1], dq[r][hh][2], dq[r][hh][3]);
            }
        }
    }
}

template <int DP>
int launch(const LpKernelArgs& a, cudaStream_t stream) {
    const size_t smem = sizeof(Smem<DP>);
    // per-device function attribute; setting it on every launch keeps multi-device processes correct and is not a stream operation
    GE2_CUDA_TRY(cudaFuncSetAttribute(lp_scores_fp32_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)ceil_div(a.L.npc, BM), (unsigned)a.d.C, (unsigned)a.L.S);
    lp_scores_fp32_kernel<DP><<<grid, kThreads, smem, stream>>>(a);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

}  // namespace

int lp_scores_fp32(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.ld == 64) return launch<64>(a, stream);
    if (a.L.ld == 128) return launch<128>(a, stream);
    return GE2_ERR_UNSUPPORTED;
}

}  // namespace ge2
