// Tensor-core scores kernel of the link-prediction step: tcgen05.mma kind::f16 (fp16 operands, the 11-bit significand
// of TF32) with fp32 accumulators in tensor memory, operands staged in shared memory by TMA (plain tiled loads, no
// multicast).  The 1e-2-parity path; everything outside the three contractions stays fp32.
//
// One CTA = (side, chunk, 128-row block).  Shared memory holds the query block Q [128 x DP], one tile of negatives
// K [128 x DP] and one tile of probabilities P [128 x 128] as fp16, all in the 128-byte-swizzled layout TMA writes
// (64-element column blocks of 128 rows at a 128-byte pitch).  That one layout serves every contraction, because a
// block read along its rows is a K-major operand and read along its columns an MN-major operand:
//   S  [row, n] = Q  K^T   A = Q  (K-major, k = d)    B = K (K-major, k = d)      -> TMEM columns [0, 128)
//   dQ [row, d] += P  K    A = P  (K-major, k = n)    B = K (MN-major, k = n)     -> TMEM columns [128, 128 + DP)
//   dK [n, d]   = P^T Q    A = P  (MN-major, k = row) B = Q (MN-major, k = row)   -> TMEM columns [256, 256 + DP)
// (32-bit tf32 operands cannot do this: the hardware transposes them only from a different, 32-byte-atom swizzle, so
// every tile would be needed twice and the set no longer fits in shared memory.)
// Sweep 1 runs the first contraction alone to get each row's logsumexp; sweep 2 recomputes S, turns it into
// P = exp(S - lse) in registers, writes P to shared memory and issues the two gradient contractions.
// The [rows x N] score matrix never leaves the SM.  Replaces the reference's bmm + logsumexp + cross_entropy +
// autograd chain (cpp/src/nn/decoders/edge/comparators.cpp:128-138, cpp/src/nn/loss.cpp:46-63 of the reference project).
//
// Threads: warps 0-3 own one accumulator row each (TMEM lane = thread), warp 4 allocates tensor memory and its
// lane 0 issues every TMA load and MMA.  Steps are separated by block-wide barriers; each mbarrier wait is bounded
// and a wait that runs out raises GE2_STATUS_PIPE_TIMEOUT, after which the CTA drains and frees its tensor memory.
#include "lp_internal.cuh"
#include "tc_ptx.cuh"

namespace ge2 {
namespace {

using namespace tc;

constexpr int BM = 128;                 // query rows per CTA  (MMA M)
constexpr int BN = 128;                 // negatives per tile  (MMA N of the score contraction)
constexpr int kThreads = 160;           // 4 row warps + 1 control warp
constexpr int kCtl = 128;               // the thread that issues TMA and MMA
constexpr int kBlockBytes = 128 * 128;  // one 64-half column block of 128 rows
constexpr int kMmaK = 16;               // k extent of one kind::f16 MMA (32 bytes)
constexpr uint32_t kTmemCols = 512;
constexpr float kMasked = -1e9f;

template <int DP>
struct Layout {
    static constexpr int NB = DP / 64;               // column blocks of Q / K
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + NB * kBlockBytes;
    static constexpr int kP = kK + NB * kBlockBytes;
    static constexpr int kBars = kP + (BN / 64) * kBlockBytes;  // two mbarriers
    static constexpr int kTmem = kBars + 16;                      // tensor memory base address
    static constexpr int kAbort = kTmem + 4;
    static constexpr int kMask = kAbort + 12;                     // BN int32
    static constexpr int kEnd = kMask + BN * 4;
    // 1024 bytes of slack to align the base; at least 120 KB so that one CTA owns the SM and its tensor memory
    static constexpr int kDynamic = (kEnd + 1024) > 120 * 1024 ? (kEnd + 1024) : 120 * 1024;
};

// K-major operand: k-step `ks` (16 halves = 32 bytes) sits in column block ks/4 at byte (ks%4)*32; 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile, int ks) {
    return smem_desc_sw128(tile + (ks >> 2) * kBlockBytes + (ks & 3) * 32, 16, 1024);
}
// MN-major operand: k-step `ks` is rows [16 ks, 16 ks + 16) = two 8-row groups of 1024 bytes; the 64-element MN blocks are
// kBlockBytes apart
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile, int ks) { return smem_desc_sw128(tile + ks * 2048, kBlockBytes, 1024); }

// byte offset of the 16-byte chunk holding halves [col, col + 8) of row `row` in the swizzled block layout (col % 8 == 0)
__device__ __forceinline__ uint32_t swz_chunk_offset(int row, int col) {
    const int chunk = (col & 63) >> 3;
    return (uint32_t)((col >> 6) * kBlockBytes + row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int DP>
__global__ void __launch_bounds__(kThreads, 1)
    lp_scores_f16_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, LpKernelArgs a) {
    using LY = Layout<DP>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem + LY::kQ;
    unsigned char* sK = smem + LY::kK;
    unsigned char* sP = smem + LY::kP;
    uint64_t* bar_tma = (uint64_t*)(smem + LY::kBars);
    uint64_t* bar_mma = bar_tma + 1;
    uint32_t* s_tmem = (uint32_t*)(smem + LY::kTmem);
    volatile int* s_abort = (volatile int*)(smem + LY::kAbort);
    int32_t* s_mask = (int32_t*)(smem + LY::kMask);

    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int s = blockIdx.z, c = blockIdx.y;
    const int row0 = blockIdx.x * BM;
    const int valid_rows = min(BM, L.npc - row0);
    const int zc = s * d.C + c;  // third TMA coordinate: (side, chunk)
    const int64_t grow0 = (int64_t)s * L.Bp + (int64_t)c * L.npc + row0;
    const int32_t* maskc = L.mask + (int64_t)s * L.CN + (int64_t)c * d.N;
    float* dKc = L.dK + ((int64_t)s * L.CN + (int64_t)c * d.N) * DP;
    float* dump = s == 0 ? d.neg_scores : d.inv_neg_scores;
    const int n_tiles = (d.N + BN - 1) / BN;
    constexpr int NB = LY::NB;
    constexpr uint32_t kTileBytes = NB * kBlockBytes;

    if (tid == 0) {
        mbar_init(bar_tma, 1);
        mbar_init(bar_mma, 1);
        *s_abort = 0;
        mbar_init_fence();
    }
    if (warp == 4) {
        tmem_alloc(s_tmem, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    const uint32_t tS = tmem, tdQ = tmem + 128, tdK = tmem + 256;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // this warp's quarter of the 128 TMEM lanes
    const uint32_t aQ = smem_u32(sQ), aK = smem_u32(sK), aP = smem_u32(sP);
    constexpr uint32_t kIdescS = idesc_f16(BM, BN, 0, 0);
    constexpr uint32_t kIdescDQ = idesc_f16(BM, DP, 0, 1);
    constexpr uint32_t kIdescDK = idesc_f16(BN, DP, 1, 1);
    uint32_t ph_tma = 0, ph_mma = 0;

    // wait on a barrier phase; on timeout flag the CTA for an orderly exit (everybody still reaches the next __syncthreads)
    auto wait_phase = [&](uint64_t* bar, uint32_t& phase) {
        if (!mbar_wait(bar, phase)) {
            *s_abort = 1;
            or_status(d.status, GE2_STATUS_PIPE_TIMEOUT);
        }
        phase ^= 1;
    };
    auto load_k_tile = [&](int n0) {  // control thread only
        mbar_expect_tx(bar_tma, kTileBytes);
#pragma unroll
        for (int b = 0; b < NB; b++) tma_load_3d(sK + b * kBlockBytes, &tmK, b * 64, n0, zc, bar_tma);
    };
    auto issue_scores = [&]() {  // control thread only: S = Q K^T
        tc_fence_after();
#pragma unroll
        for (int ks = 0; ks < DP / kMmaK; ks++) mma_f16_ss(tS, desc_kmajor(aQ, ks), desc_kmajor(aK, ks), kIdescS, ks > 0);
        mma_commit(bar_mma);
    };

    // ---- query block -------------------------------------------------------------------------------------------
    if (tid == kCtl) {
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        mbar_expect_tx(bar_tma, kTileBytes);
#pragma unroll
        for (int b = 0; b < NB; b++) tma_load_3d(sQ + b * kBlockBytes, &tmQ, b * 64, row0, zc, bar_tma);
    }
    wait_phase(bar_tma, ph_tma);

    const int my_row = tid;                      // row warps: accumulator row / TMEM lane
    const int brow = c * L.npc + row0 + my_row;  // batch row in the padded numbering the filter uses
    float run_m = -INFINITY, run_l = 0.f, lse = 0.f;

    // ---- sweep 1: logsumexp --------------------------------------------------------------------------------------
    for (int t = 0; t < n_tiles; t++) {
        const int n0 = t * BN;
        const int valid_n = min(BN, d.N - n0);
        if (tid < BN) s_mask[tid] = tid < valid_n ? maskc[n0 + tid] : -1;
        if (tid == kCtl) load_k_tile(n0);
        wait_phase(bar_tma, ph_tma);
        if (tid == kCtl) issue_scores();
        wait_phase(bar_mma, ph_mma);
        tc_fence_after();
        __syncthreads();
        if (*s_abort) break;
        if (warp < 4) {
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; cb++) {
                float v[32];
                tmem_ld_32x32(tS + lane_sel + cb * 32, v);
                float tmax = -INFINITY;
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int col = cb * 32 + j;
                    float sc = v[j];
                    if (s_mask[col] == brow) sc = kMasked;
                    if (dump != nullptr && my_row < valid_rows && col < valid_n) dump[(int64_t)brow * d.N + n0 + col] = sc;
                    v[j] = col < valid_n ? sc : -INFINITY;
                    tmax = fmaxf(tmax, v[j]);
                }
                if (tmax > -INFINITY) {
                    const float nm = fmaxf(run_m, tmax);
                    float add = 0.f;
#pragma unroll
                    for (int j = 0; j < 32; j++) add += __expf(v[j] - nm);
                    run_l = run_l * __expf(run_m - nm) + add;
                    run_m = nm;
                }
            }
        }
        tc_fence_before();
        __syncthreads();  // S and the K tile are free again
    }
    if (warp < 4 && my_row < valid_rows) {
        const float pos = L.pos[grow0 + my_row];
        const float nm = fmaxf(run_m, pos);
        lse = nm + __logf(run_l * __expf(run_m - nm) + __expf(pos - nm));
        L.lse[grow0 + my_row] = lse;
    }

    // ---- sweep 2: probabilities, dQ and dK -------------------------------------------------------------------------
    for (int t = 0; t < n_tiles; t++) {
        if (*s_abort) break;
        const int n0 = t * BN;
        const int valid_n = min(BN, d.N - n0);
        if (tid < BN) s_mask[tid] = tid < valid_n ? maskc[n0 + tid] : -1;
        if (tid == kCtl) load_k_tile(n0);
        wait_phase(bar_tma, ph_tma);
        if (tid == kCtl) issue_scores();
        wait_phase(bar_mma, ph_mma);
        tc_fence_after();
        __syncthreads();
        if (*s_abort) break;
        if (warp < 4) {
#pragma unroll 1
            for (int cb = 0; cb < BN / 32; cb++) {
                float v[32];
                tmem_ld_32x32(tS + lane_sel + cb * 32, v);
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int col = cb * 32 + j;
                    // masked entries were overwritten in place by the reference: no gradient reaches them
                    const bool live = my_row < valid_rows && col < valid_n && s_mask[col] != brow;
                    v[j] = live ? __expf(v[j] - lse) : 0.f;
                }
#pragma unroll
                for (int q = 0; q < 4; q++) {  // 8 halves = one 16-byte chunk
                    uint4 pk;
                    pk.x = pack_half2(v[8 * q + 0], v[8 * q + 1]);
                    pk.y = pack_half2(v[8 * q + 2], v[8 * q + 3]);
                    pk.z = pack_half2(v[8 * q + 4], v[8 * q + 5]);
                    pk.w = pack_half2(v[8 * q + 6], v[8 * q + 7]);
                    *reinterpret_cast<uint4*>(sP + swz_chunk_offset(my_row, cb * 32 + q * 8)) = pk;
                }
            }
            fence_proxy_async_smem();  // P was written with ordinary stores; the MMA reads it through the async proxy
        }
        tc_fence_before();
        __syncthreads();
        if (tid == kCtl) {
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < BN / kMmaK; ks++)  // dQ += P K, k runs over the tile's negatives
                mma_f16_ss(tdQ, desc_kmajor(aP, ks), desc_mnmajor(aK, ks), kIdescDQ, (t > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
            for (int ks = 0; ks < BM / kMmaK; ks++)  // dK = P^T Q, k runs over the block's rows
                mma_f16_ss(tdK, desc_mnmajor(aP, ks), desc_mnmajor(aQ, ks), kIdescDK, ks > 0);
            mma_commit(bar_mma);
        }
        wait_phase(bar_mma, ph_mma);
        tc_fence_after();
        __syncthreads();
        if (*s_abort) break;
        if (warp < 4) {  // here a TMEM lane is a negative of the tile
            float* dst = dKc + (int64_t)(n0 + my_row) * DP;
#pragma unroll 1
            for (int cb = 0; cb < DP / 32; cb++) {
                float v[32];
                tmem_ld_32x32(tdK + lane_sel + cb * 32, v);  // warp-collective: lanes past the tile's end take part too
                if (my_row < valid_n) {
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const int col = cb * 32 + q * 4;
                        if (col < d.D) atomicAdd(reinterpret_cast<float4*>(dst + col), make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();  // dK accumulator, P and the K tile are free again
    }
    if (warp < 4 && !*s_abort) {
#pragma unroll 1
        for (int cb = 0; cb < DP / 32; cb++) {
            float v[32];
            tmem_ld_32x32(tdQ + lane_sel + cb * 32, v);
            if (my_row < valid_rows) {
                float* dst = L.dQ + (grow0 + my_row) * DP + cb * 32;
#pragma unroll
                for (int q = 0; q < 8; q++) *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
            }
        }
    }
    // ---- teardown: nothing of this CTA may still be in flight when tensor memory is released ----------------------
    tc_fence_before();
    __syncthreads();
    if (*s_abort && tid == kCtl) {
        // a wait ran out: give outstanding copies / MMAs one more bounded chance to land before the memory is reused
        mbar_wait(bar_tma, ph_tma ^ 1, 1u << 16);
        mbar_wait(bar_mma, ph_mma ^ 1, 1u << 16);
    }
    __syncthreads();
    if (warp == 4) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup: the library does not link libcuda, so it still
// loads on a machine without a driver
EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
        fn = (EncodeTiledFn)p;
    }
    return fn;
}

// [S*C matrices][rows][ld halves] viewed as a 3-D tensor; box = 64 halves x 128 rows of one matrix, 128-byte swizzle,
// rows past the matrix end read as zero
int make_map(CUtensorMap* map, __half* base, int ld, int rows, int mats) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return GE2_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)ld, (cuuint64_t)rows, (cuuint64_t)mats};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 2, (cuuint64_t)rows * ld * 2};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return GE2_ERR_CUDA;
    }
    return GE2_OK;
}

template <int DP>
int launch(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.Qh == nullptr || a.L.Kh == nullptr) return GE2_ERR_WORKSPACE;
    CUtensorMap tmQ, tmK;
    int rc = make_map(&tmQ, a.L.Qh, DP, a.L.npc, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    rc = make_map(&tmK, a.L.Kh, DP, a.d.N, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    const int smem = Layout<DP>::kDynamic;
    GE2_CUDA_TRY(cudaFuncSetAttribute(lp_scores_f16_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    dim3 grid((unsigned)ceil_div(a.L.npc, BM), (unsigned)a.d.C, (unsigned)a.L.S);
    lp_scores_f16_kernel<DP><<<grid, kThreads, smem, stream>>>(tmQ, tmK, a);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

}  // namespace

int lp_scores_f16(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.ld == 64) return launch<64>(a, stream);
    if (a.L.ld == 128) return launch<128>(a, stream);
    return GE2_ERR_UNSUPPORTED;
}

}  // namespace ge2
