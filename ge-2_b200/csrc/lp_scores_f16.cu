// Tensor-core scores kernels of the link-prediction step: tcgen05.mma kind::f16 (fp16 operands, the 11-bit significand
// of TF32) with fp32 accumulators in tensor memory, operands staged in shared memory by TMA (every CTA issues its own
// plain tiled loads).  The 1e-2-parity path; everything outside the contractions stays fp32.
// Replaces the reference's bmm + logsumexp + cross_entropy + autograd chain (cpp/src/nn/decoders/edge/comparators.cpp:128-138,
// cpp/src/nn/loss.cpp:46-63 of the reference project).
//
// Per (side, chunk) the work is Q [rows x D] against K [negatives x D]: S = Q K^T, row logsumexp (with the positive score),
// P = exp(S - lse), dQ = P K, dK = P^T Q.  The [rows x negatives] matrices never leave the SM.  Two launches:
//
//   lp_lse_kernel   S tile by tile, running (max, sum) per row in the exp2 domain                          -> lse, loss
//   lp_grad_kernel  a block X of 128 query rows (Q) stays in shared memory and the tiles Y of 128 negatives (K) of its chunk
//                   stream past it: S = X Y^T is recomputed (cheaper than storing it), W = exp2(S log2 e - lse) * 2^14 is
//                   packed to fp16, dQ += W Y accumulates in tensor memory over the block's whole stream and is written
//                   once; dK_tile = W^T X is produced per tile and added into global dK (the row blocks of a chunk meet
//                   there) by TMA reduce-adds.
//
// Both launches are persistent: the (block, tile) units of the whole step are numbered consecutively and dealt to the
// CTAs (one per SM) as contiguous ranges of equal length, so every SM is busy to the end whatever the number of blocks.
// A block whose units straddle a CTA boundary is finished by two (rarely more) CTAs: in the logsumexp pass each leaves a
// per-row partial (max, sum) and the gradient pass combines them; in the gradient pass each adds its part of dQ into the
// output rows with TMA reduce-adds (those rows are cleared by the first launch); whole blocks are written with plain TMA
// stores.
//
// Shared memory holds X [128 x DP], a ring of Y tiles [128 x DP] (five in the logsumexp pass, three in the gradient pass)
// and, in the gradient pass, one W tile [128 x 128] and the drain warps' staging slabs; X, Y and W are fp16 in the
// 128-byte-swizzled layout TMA writes (64-element column blocks of 128 rows at a 128-byte pitch).  That one layout serves
// every contraction, because a block read along its rows is a K-major operand and read along its columns an MN-major
// operand:
//   S  [x, y] = X Y^T    A = X (K-major, k = d)    B = Y (K-major, k = d)
//   dQ [x, d] += W Y     A = W (K-major, k = y)    B = Y (MN-major, k = y)
//   dK [y, d] = W^T X    A = W (MN-major, k = x)   B = X (MN-major, k = x)
// Tensor memory (512 columns), gradient pass: S at 0, dQ at 128, two dK accumulators at 256 and 384 that alternate from
// tile to tile, so the contraction of one tile runs while the other's result is drained.  Logsumexp pass: two score
// accumulators at 0 and 128.
// (32-bit tf32 operands cannot do this: the hardware transposes them only from a different, 32-byte-atom swizzle.)
// W is scaled by 2^14 before it is packed to fp16, so that probabilities down to 2^-38 keep their full significand instead
// of falling into fp16's subnormal range; dQ and dK leave this kernel with that factor still on them and the scatter
// kernel, their only reader, takes it off (LpLayout::grad_unscale).
//
// Warp roles, connected by mbarrier pipelines (no block-wide barrier inside the loops):
//   warps 0-15  softmax: thread = accumulator row (tensor-memory lane).  lse pass: two groups of 8 warps take alternate
//               tiles (64 columns per warp).  Gradient pass: all 16 warps on every tile (32 columns per warp): scores ->
//               registers (the accumulator is handed back at once) -> W in shared memory
//   warps 16-19 lse pass: warp 16 combines the softmax warps' partials at the end of a block; warps 17-19 clear dK and
//               the dQ rows of split blocks.  Gradient pass: drain (with warps 23-26): accumulator -> swizzled staging
//               slab -> TMA store / reduce-add, each warp its lane quarter and every second 32-column slab
//   warp  20    lane 0: TMA producer (X at the start of a block, the Y ring)
//   warp  21    lane 0: issues the score contractions; the warp also allocates and frees tensor memory
//   warp  22    lane 0: issues the dK and dQ contractions of the gradient pass
//   warps 23-26 gradient pass only (864 threads): the second set of drain warps
// Every mbarrier wait is bounded; a wait that runs out raises GE2_STATUS_PIPE_TIMEOUT and sets a block-wide abort flag
// that every other wait polls, so all roles fall through to the common exit where tensor memory is released.
#include <stdlib.h>

#include <algorithm>

#include "lp_internal.cuh"
#include "tc_ptx.cuh"

namespace ge2 {
namespace {

using namespace tc;

constexpr int BM = 128;                 // rows of the stationary block (MMA M)
constexpr int BN = 128;                 // rows of a streamed tile (MMA N of the score contraction)
constexpr int kSoftmaxWarps = 16;       // 4 row quarters (tensor-memory lane groups) x 4 groups of 32 columns
constexpr int kThreads = 736;           // lse pass: 16 softmax warps + 4 combine / clearing warps + TMA warp + two MMA warps
constexpr int kThreadsB = 864;          // gradient pass: 16 softmax warps + 8 drain warps (16-19 and 23-26) + TMA warp + two MMA warps
constexpr int kDrainWarps = 8;
constexpr int kDrainWarp0 = kSoftmaxWarps, kTmaWarp = kDrainWarp0 + 4, kMmaWarp = kTmaWarp + 1, kGradWarp = kMmaWarp + 1;
constexpr int kBlockBytes = 128 * 128;  // one 64-half column block of 128 rows
constexpr int kMmaK = 16;               // k extent of one kind::f16 MMA (32 bytes)
constexpr int kStages = 3;              // Y ring depth of the gradient pass (shared memory is full there: X, 3 Y, W, 16 staging slabs)
constexpr int kStagesA = 5;             // Y ring depth of the lse pass (no W tiles: room for a deeper ring, which the load latency wants)
constexpr int kMaxStages = kStagesA;
constexpr int kMaxParts = 8;            // most CTAs that can share one row block in the lse pass; size of a row's partial list
constexpr uint32_t kTmemCols = 512;
constexpr float kMasked = -1e9f;
constexpr float kLog2e = 1.4426950408889634f, kLn2 = 0.6931471805599453f;
constexpr int kWShift = 14;             // W = P * 2^14 in fp16; undone by the reader of dQ / dK (kLpF16GradUnscale)
constexpr float kDeadRow = 1e30f;       // "lse" of a row past the end of its chunk: exp2(anything - 1e30) = 0

// mbarrier slots (a superset; the lse pass uses the first group and the exchange barriers)
enum Bar { kBarXFull = 0, kBarXEmpty, kBarYFull, kBarYEmpty = kBarYFull + kMaxStages, kBarSFull = kBarYEmpty + kMaxStages, kBarSEmpty = kBarSFull + 2,
           kBarWFull = kBarSEmpty + 2, kBarWEmpty = kBarWFull + 2, kBarAccFull = kBarWEmpty + 2, kBarAccEmpty = kBarAccFull + 2,
           kBarXch = kBarAccEmpty + 2, kBarXchFree = kBarXch + 2, kBarDkFull = kBarXchFree + 2, kBarDkEmpty = kBarDkFull + 2,
           kNumBars = kBarDkEmpty + 2 };

// How the units of a launch are dealt to its CTAs: CTA k takes units [k * units / grid, (k + 1) * units / grid).
struct Sched {
    int RB, T, ZC;       // row blocks per chunk, negative tiles per chunk, sides * chunks
    int unitsA, gridA;   // lse pass: unit = (zc, row block, tile), numbered (zc * RB + rb) * T + tile
    int unitsB, gridB;   // gradient pass: the same units (X = Q block, stream over the K tiles)
};
__host__ __device__ __forceinline__ int range_begin(int k, int units, int grid) { return (int)(((long long)k * units) / grid); }
__host__ __device__ __forceinline__ int cta_of_unit(int u, int units, int grid) { return (int)((((long long)u + 1) * grid - 1) / units); }

template <int DP>
struct Layout {
    static constexpr int NB = DP / 64;               // column blocks of X / Y
    static constexpr int kTileBytes = NB * kBlockBytes;
    static constexpr int kWBytes = (BN / 64) * kBlockBytes;
    static constexpr int kX = 0;
    static constexpr int kY = kX + kTileBytes;
    static constexpr int kW = kY + kStages * kTileBytes;
    // --- gradient pass ---
    static constexpr int kMiscB = kW + kWBytes;                   // barriers, tensor-memory address, abort flag
    static constexpr int kDrain = kMiscB + 2048;                  // 8 drain warps x 2 slabs (32 rows x 128 bytes), 128-byte swizzled
    static constexpr int kEndB = kDrain + kDrainWarps * 2 * 4096;
    static constexpr int kDynamicB = kEndB + 1024;                // 1024 bytes of slack to align the base
    // --- lse pass (no W tiles) ---
    static constexpr int kMiscA = kY + kStagesA * kTileBytes;
    static constexpr int kXch = kMiscA + 1024;                    // 2 halves x 4 partial slots x 128 rows x (max, sum)
    static constexpr int kEndA = kXch + 2 * 4 * 128 * 8;
    // at least 120 KB so that one CTA owns the SM and its tensor memory
    static constexpr int kDynamicA = (kEndA + 1024) > 120 * 1024 ? (kEndA + 1024) : 120 * 1024;
    static_assert(kNumBars * 8 + 16 <= 512, "barrier block overflows its slot");
    static_assert(kDynamicB <= 227 * 1024, "gradient pass exceeds the shared memory of an SM");
};

// Descriptors are built once per tile; a k-step only adds its byte offset (>> 4) to the start-address field, which cannot
// carry out of the field because shared-memory addresses stay below 256 KB.
// K-major operand: k-step `ks` (16 halves = 32 bytes) sits in column block ks/4 at byte (ks%4)*32; 8-row groups are 1024 bytes apart
__device__ __forceinline__ uint64_t desc_kmajor_base(uint32_t tile) { return smem_desc_sw128(tile, 16, 1024); }
__host__ __device__ constexpr uint64_t koff_kmajor(int ks) { return (uint64_t)(((ks >> 2) * kBlockBytes + (ks & 3) * 32) >> 4); }
// MN-major operand: k-step `ks` is rows [16 ks, 16 ks + 16) = two 8-row groups of 1024 bytes; the 64-element MN blocks are
// kBlockBytes apart
__device__ __forceinline__ uint64_t desc_mnmajor_base(uint32_t tile) { return smem_desc_sw128(tile, kBlockBytes, 1024); }
__host__ __device__ constexpr uint64_t koff_mnmajor(int ks) { return (uint64_t)((ks * 2048) >> 4); }

// byte offset of the 16-byte chunk holding halves [col, col + 8) of row `row` in the swizzled block layout (col % 8 == 0)
__device__ __forceinline__ uint32_t swz_chunk_offset(int row, int col) {
    const int chunk = (col & 63) >> 3;
    return (uint32_t)((col >> 6) * kBlockBytes + row * 128 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ float exp2f_fast(float x) {  // one MUFU.EX2; 2^-inf = 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// Bounded wait that also gives up as soon as another role has raised the abort flag.
__device__ __forceinline__ bool pipe_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int32_t* status) {
    for (uint32_t i = 0; i < (1u << 20); i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);  // long waits (a role idle for a whole block) must not eat issue slots
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    or_status(status, GE2_STATUS_PIPE_TIMEOUT);
    return false;
}

// what a CTA needs to know about one unit of the lse pass
struct UnitA {
    int item, tile, rb, zc;
};
__device__ __forceinline__ UnitA decode_a(int u, const Sched& sc) {
    UnitA r;
    r.item = u / sc.T;
    r.tile = u - r.item * sc.T;
    r.zc = r.item / sc.RB;
    r.rb = r.item - r.zc * sc.RB;
    return r;
}
// The loops walk their units with these instead of decoding every index (no divisions inside the pipelines).
struct IterA {
    int item, tile, rb, zc;
    __device__ __forceinline__ IterA(int u, const Sched& sc) {
        const UnitA un = decode_a(u, sc);
        item = un.item, tile = un.tile, rb = un.rb, zc = un.zc;
    }
    __device__ __forceinline__ void next(const Sched& sc) {
        if (++tile == sc.T) {
            tile = 0;
            item++;
            if (++rb == sc.RB) rb = 0, zc++;
        }
    }
};
// =====================================================================================================================
// launch 1: row logsumexp
// =====================================================================================================================
template <int DP>
__global__ void __launch_bounds__(kThreads, 1)
    lp_lse_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, LpKernelArgs a, Sched sc) {
    using LY = Layout<DP>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sX = smem + LY::kX;
    unsigned char* sY = smem + LY::kY;
    uint64_t* bars = (uint64_t*)(smem + LY::kMiscA);
    uint32_t* s_tmem = (uint32_t*)(smem + LY::kMiscA + kNumBars * 8);
    volatile int* s_abort = (volatile int*)(smem + LY::kMiscA + kNumBars * 8 + 4);
    float2* s_xch = reinterpret_cast<float2*>(smem + LY::kXch);

    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ub = range_begin(blockIdx.x, sc.unitsA, gridDim.x), ue = range_begin(blockIdx.x + 1, sc.unitsA, gridDim.x);
    const int n_iter = ue - ub;
    constexpr int NB = LY::NB;
    auto wait = [&](int bar, uint32_t parity) { return pipe_wait(&bars[bar], parity, s_abort, d.status); };
    auto warp_wait = [&](int bar, uint32_t parity) -> bool {  // one lane polls; then every lane observes the completed phase itself
        if (__all_sync(0xffffffffu, mbar_try_wait(&bars[bar], parity) ? 1 : 0)) return true;  // usually complete already
        int ok = 1;
        if (lane == 0) ok = wait(bar, parity) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) ok = mbar_try_wait(&bars[bar], parity) ? 1 : 0;
        return __all_sync(0xffffffffu, ok) != 0;
    };
    // TMA producer state: runs a few units before the block-wide barrier (their latency overlaps the allocation of tensor
    // memory), the rest afterwards
    int tma_it = 0, tma_sg = -1;
    IterA tma_un(ub, sc);  // unit of iteration tma_it
    auto produce = [&](int it) -> bool {
        const IterA& un = tma_un;
        if (it == 0 || un.tile == 0) {  // a new block: X may be overwritten once the score contractions of the last one are done
            tma_sg++;
            if (!wait(kBarXEmpty, (tma_sg & 1) ^ 1)) return false;
            mbar_expect_tx(&bars[kBarXFull], LY::kTileBytes);
#pragma unroll
            for (int b = 0; b < NB; b++) tma_load_3d(sX + b * kBlockBytes, &tmQ, b * 64, un.rb * BM, un.zc, &bars[kBarXFull]);
        }
        const int st = it % kStagesA, use = it / kStagesA;
        if (!wait(kBarYEmpty + st, (use & 1) ^ 1)) return false;
        mbar_expect_tx(&bars[kBarYFull + st], LY::kTileBytes);
#pragma unroll
        for (int b = 0; b < NB; b++) tma_load_3d(sY + st * LY::kTileBytes + b * kBlockBytes, &tmK, b * 64, un.tile * BN, un.zc, &bars[kBarYFull + st]);
        tma_un.next(sc);
        return true;
    };
    if (warp == kTmaWarp && lane == 0) {
        mbar_init(&bars[kBarXFull], 1);
        mbar_init(&bars[kBarXEmpty], 1);
        for (int k = 0; k < kStagesA; k++) {
            mbar_init(&bars[kBarYFull + k], 1);
            mbar_init(&bars[kBarYEmpty + k], 1);
        }
        for (int k = 0; k < 2; k++) {
            mbar_init(&bars[kBarSFull + k], 1);
            mbar_init(&bars[kBarSEmpty + k], kSoftmaxWarps / 2);  // one arrival per warp of the group that owns the tile
            mbar_init(&bars[kBarXch + k], kSoftmaxWarps);
            mbar_init(&bars[kBarXchFree + k], 1);
        }
        *s_abort = 0;
        mbar_init_fence();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        griddep_wait();  // the operands come from the kernel before this one
        // early loads: the first two tiles, and only while no wait can depend on another role (first block)
        while (tma_it < n_iter && tma_it < 2 && (tma_it == 0 || tma_un.tile != 0)) {
            produce(tma_it);
            tma_it++;
        }
    }
    if (warp == kMmaWarp) {
        tmem_alloc(s_tmem, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();  // set-up done; from here on global memory written by the preceding kernel is read and its buffers rewritten
    const uint32_t tmem = *s_tmem;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // this warp's quarter of the 128 tensor-memory lanes

    if (warp == kTmaWarp) {
        if (lane == 0) {
            for (; tma_it < n_iter; tma_it++)
                if (!produce(tma_it)) break;
        }
    } else if (warp == kMmaWarp) {
        // ================================ score contractions ================================
        if (lane == 0) {
            const uint32_t aX = smem_u32(sX), aY0 = smem_u32(sY);
            constexpr uint32_t kIdescS = idesc_f16(BM, BN, 0, 0);
            const uint64_t dXk = desc_kmajor_base(aX);
            int sg = -1;
            IterA un(ub, sc);
            for (int it = 0; it < n_iter; it++, un.next(sc)) {
                if (it == 0 || un.tile == 0) {
                    sg++;
                    if (!wait(kBarXFull, sg & 1)) break;
                }
                const int st = it % kStagesA, use = it / kStagesA, sb = it & 1, su = it >> 1;
                if (!wait(kBarYFull + st, use & 1)) break;
                if (!wait(kBarSEmpty + sb, (su & 1) ^ 1)) break;
                tc_fence_after();
                const uint64_t dYk = desc_kmajor_base(aY0 + st * LY::kTileBytes);
#pragma unroll
                for (int ks = 0; ks < DP / kMmaK; ks++) mma_f16_ss(tmem + sb * 128, dXk + koff_kmajor(ks), dYk + koff_kmajor(ks), kIdescS, ks > 0);
                mma_commit(&bars[kBarSFull + sb]);
                mma_commit(&bars[kBarYEmpty + st]);
                if (it == n_iter - 1 || un.tile == sc.T - 1) mma_commit(&bars[kBarXEmpty]);
            }
        }
    } else if (warp == kDrainWarp0) {
        // ================================ combine warp ================================
        // At the end of every block: the four partial (max, sum) pairs of each row (two softmax groups x two column
        //     halves) meet in shared memory; a block this CTA ran alone is finished here, a block shared with other CTAs
        //     leaves its partial in global memory and the last CTA to arrive finishes it.
        int sg = 0;
        for (int u = ub; u < ue; sg++) {
            const UnitA un = decode_a(u, sc);
            const int seg_end = min(ue, (un.item + 1) * sc.T);
            const bool whole = un.tile == 0 && seg_end == (un.item + 1) * sc.T;
            const int h = sg & 1;
            const int s = un.zc / d.C, c = un.zc - s * d.C;
            const int row0 = un.rb * BM;
            const int valid_rows = min(BM, L.npc - row0);
            const int64_t grow0 = (int64_t)s * L.Bp + (int64_t)c * L.npc + row0;
            float pos4[4];  // fetched before the wait for the block's last tile: off the tail of the kernel
#pragma unroll
            for (int q = 0; q < 4; q++) pos4[q] = q * 32 + lane < valid_rows ? __ldg(&L.pos[grow0 + q * 32 + lane]) : 0.f;
            if (!warp_wait(kBarXch + h, (sg >> 1) & 1)) break;
            float m4[4], l4[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const int r = q * 32 + lane;
                float2 pr[4];
                float nm = -INFINITY;
#pragma unroll
                for (int k = 0; k < 4; k++) {
                    pr[k] = s_xch[(h * 4 + k) * 128 + r];
                    nm = fmaxf(nm, pr[k].x);
                }
                float l = 0.f;
                if (nm > -INFINITY) {
#pragma unroll
                    for (int k = 0; k < 4; k++) l += pr[k].y * exp2f_fast(pr[k].x - nm);  // an empty partial has sum 0 and max -inf
                }
                m4[q] = nm;
                l4[q] = l;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarXchFree + h]);  // the softmax warps may write this half again
            if (!whole) {
                // shared with a neighbouring CTA: leave this CTA's partial; every CTA of the gradient pass that needs the block's
                // lse combines the partials itself
                const int p_first = cta_of_unit(un.item * sc.T, sc.unitsA, (int)gridDim.x);
                const int my_part = (int)blockIdx.x - p_first;
                float2* part = reinterpret_cast<float2*>(L.part);
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int r = q * 32 + lane;
                    if (r < valid_rows && my_part < kMaxParts) part[(grow0 + r) * kMaxParts + my_part] = make_float2(m4[q], l4[q]);
                }
            }
            const bool finish = whole;
            if (finish) {
                float loss = 0.f;
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int r = q * 32 + lane;
                    float shifted = kDeadRow;
                    if (r < valid_rows) {
                        const float pos2 = pos4[q] * kLog2e;
                        const float nm2 = fmaxf(m4[q], pos2);
                        const float lse2 = nm2 + __log2f(l4[q] * exp2f_fast(m4[q] - nm2) + exp2f_fast(pos2 - nm2));
                        L.lse[grow0 + r] = lse2 * kLn2;
                        loss += (lse2 - pos2) * kLn2;
                        shifted = lse2 - (float)kWShift;
                    }
                    L.lse2s[(int64_t)un.item * BM + r] = shifted;
                }
                // the step's loss = sum over rows of (lse - pos): one double-precision atomic per block
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, o);
                if (lane == 0) atomicAdd(L.loss_acc, (double)loss);
            }
            u = seg_end;
        }
    } else if (warp > kDrainWarp0 && warp < kTmaWarp) {
        // ================================ warps 17-19: clear what the gradient pass will reduce into ================================
        // dK (every row block of a chunk adds its part: this CTA clears its share of the whole array) and the dQ rows of every
        // block whose stream the gradient pass cuts at a CTA boundary (boundary j of that launch is looked after by CTA
        // (j - 1) % gridDim.x of this one).
        const int wz = warp - kDrainWarp0 - 1;
        {
            const int64_t n4 = (int64_t)sc.ZC * d.N * (DP / 4);
            const int64_t z0 = n4 * blockIdx.x / gridDim.x, z1 = n4 * (blockIdx.x + 1) / gridDim.x;
            float4* p4 = reinterpret_cast<float4*>(L.dK);
            for (int64_t k = z0 + wz * 32 + lane; k < z1; k += 96) p4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
        for (int j = 1 + (int)blockIdx.x; j < sc.gridB; j += (int)gridDim.x) {
            const int u = range_begin(j, sc.unitsB, sc.gridB);
            if (u <= 0 || u >= sc.unitsB) continue;
            const UnitA un = decode_a(u, sc);
            if (un.tile == 0) continue;  // the boundary falls between two blocks: nothing is split
            float* base = L.dQ + ((int64_t)un.zc * L.npc + (int64_t)un.rb * BM) * DP;
            const int rows = min(BM, L.npc - un.rb * BM);
            float4* p4 = reinterpret_cast<float4*>(base);
            for (int k = wz * 32 + lane; k < rows * (DP / 4); k += 96) p4[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    } else if (warp < kSoftmaxWarps) {
        // ================================ softmax warps (0-15) ================================
        // Two groups of 8 warps take alternate tiles: group g = warp / 8 owns the local iterations with (it & 1) == g, so
        // while one group waits for its scores the other keeps the exp unit busy.  Within a group, warp w takes rows
        // 32*(w & 3) ... + 31 (its quarter of the tensor-memory lanes) and columns 64*((w >> 2) & 1) ... + 63 of the tile,
        // as two passes of 32 columns.
        const int grp = warp >> 3;
        const int ch = (warp >> 2) & 1;
        const int slot = grp * 2 + ch;  // where this warp's partial (max, sum) goes in the exchange
        const int my_row = tid & 127;   // accumulator row / tensor-memory lane
        // The filter is sparse: a tile has at most one masked row per column and few of them fall in this warp's 32 rows.
        // Lane l looks at columns l and l + 32 of the warp's 64; an entry that names a row of this warp is handed to that
        // row's thread, which ends up with one bit per masked column of its own row.  The words of the group's next tile
        // are fetched while the current one is processed.
        auto load_mask = [&](int it, const IterA& un, int32_t (&m)[2]) {
            m[0] = m[1] = -1;
            if (it < n_iter) {
                const int32_t* maskc = L.mask + (int64_t)un.zc * d.N;  // mask is [S][C][N] = [zc][N]
                const int n0 = un.tile * BN;
                const int vn = min(BN, d.N - n0);
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int idx = ch * 64 + k * 32 + lane;
                    if (idx < vn) m[k] = __ldg(&maskc[n0 + idx]);
                }
            }
        };
        int32_t mnext[2];
        IterA un(ub, sc), pre(ub, sc);  // `pre`: the unit whose filter words are fetched next (this group's tile after the current one)
        if (grp == 1) pre.next(sc);
        load_mask(grp, pre, mnext);
        pre.next(sc);
        pre.next(sc);
        float run_m = -INFINITY, run_l = 0.f;
        int sg = -1;
        bool alive = true;
        for (int it = 0; alive && it < n_iter; it++, un.next(sc)) {
            if (it == 0 || un.tile == 0) {
                sg++;
                run_m = -INFINITY;
                run_l = 0.f;
            }
            if ((it & 1) == grp) {
                const int s = un.zc / d.C, c = un.zc - s * d.C;
                const int row0 = un.rb * BM;
                const int brow = c * L.npc + row0 + my_row;            // batch row in the padded numbering the filter uses
                const int wrow0 = c * L.npc + row0 + (warp & 3) * 32;  // first batch row of this warp
                const bool row_live = my_row < min(BM, L.npc - row0);
                float* dump = s == 0 ? d.neg_scores : d.inv_neg_scores;
                const int n0 = un.tile * BN;
                uint32_t mb[2], wor[2];
                {
                    const int32_t mcur[2] = {mnext[0], mnext[1]};
                    load_mask(it + 2, pre, mnext);  // `pre` is the unit of iteration it + 2
                    pre.next(sc);
                    pre.next(sc);
#pragma unroll
                    for (int k = 0; k < 2; k++) {
                        mb[k] = 0u;  // bit j = column ch*64 + 32k + j of this tile is masked for my row
                        unsigned ballot = __ballot_sync(0xffffffffu, (unsigned)(mcur[k] - wrow0) < 32u);
                        while (ballot != 0) {
                            const int src = __ffs(ballot) - 1;
                            ballot &= ballot - 1;
                            if (__shfl_sync(0xffffffffu, mcur[k], src) == brow) mb[k] |= 1u << src;
                        }
                        wor[k] = __reduce_or_sync(0xffffffffu, mb[k]);  // which 8-column groups hold a masked entry for any row of this warp
                    }
                }
                const int sb = it & 1;
                if (!warp_wait(kBarSFull + sb, (it >> 1) & 1)) { alive = false; break; }  // warp-uniform: tcgen05.ld is collective
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int nv = min(BN, d.N - n0) - ch * 64 - k * 32;  // live columns among these 32
                    float v[32];
                    tmem_ld_32x32(tmem + sb * 128 + ch * 64 + k * 32 + lane_sel, v);
                    if (k == 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars[kBarSEmpty + sb]);  // the tile is in registers: this accumulator is free again
                    }
                    if (nv <= 0) continue;
                    if (nv < 32 || dump != nullptr) {  // ragged last tile, or the score dump of the tests
#pragma unroll
                        for (int j = 0; j < 32; j++) {
                            float sc_ = ((mb[k] >> j) & 1u) ? kMasked : v[j];
                            if (dump != nullptr && row_live && j < nv) dump[(int64_t)brow * d.N + n0 + ch * 64 + k * 32 + j] = sc_;
                            v[j] = j < nv ? sc_ : -INFINITY;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            if ((wor[k] >> (q * 8)) & 0xffu) {  // warp-uniform
#pragma unroll
                                for (int j = 8 * q; j < 8 * q + 8; j++) v[j] = ((mb[k] >> j) & 1u) ? kMasked : v[j];
                            }
                        }
                    }
                    float mx[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) mx[q] = v[q];
#pragma unroll
                    for (int j = 4; j < 32; j++) mx[j & 3] = fmaxf(mx[j & 3], v[j]);
                    const float tmax = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
                    const float nm = fmaxf(run_m, tmax * kLog2e);
                    float add[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                    for (int j = 0; j < 32; j++) add[j & 3] += exp2f_fast(fmaf(v[j], kLog2e, -nm));  // 2^-inf = 0 for absent columns
                    run_l = fmaf(run_l, exp2f_fast(run_m - nm), (add[0] + add[1]) + (add[2] + add[3]));
                    run_m = nm;
                }
            }
            if (it == n_iter - 1 || un.tile == sc.T - 1) {
                // end of the block (or of this CTA's share of it): hand the partial to the combine warp
                const int h = sg & 1;
                if (!warp_wait(kBarXchFree + h, ((sg >> 1) & 1) ^ 1)) { alive = false; break; }
                s_xch[(h * 4 + slot) * 128 + my_row] = make_float2(run_m, run_l);
                __syncwarp();
                if (lane == 0) mbar_arrive(&bars[kBarXch + h]);
            }
        }
    }
    // ---- common exit: every role ends here, normally or after an abort; then tensor memory is released ----------
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        if (*s_abort && lane == 0) {
            // a wait ran out somewhere: give copies still in flight a bounded chance to land before the SM's shared and
            // tensor memory are handed to the next CTA
            for (int k = 0; k < kStagesA; k++) mbar_wait(&bars[kBarYFull + k], 0, 1u << 14);
        }
        __syncwarp();
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
}

// =====================================================================================================================
// launch 2: both gradients
// =====================================================================================================================
template <int DP>
__global__ void __launch_bounds__(kThreadsB, 1)
    lp_grad_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmDK,
                   const __grid_constant__ CUtensorMap tmDKt, const __grid_constant__ CUtensorMap tmDQ,
                   const __grid_constant__ CUtensorMap tmDQt, LpKernelArgs a, Sched sc) {
    using LY = Layout<DP>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sX = smem + LY::kX;
    unsigned char* sY = smem + LY::kY;
    unsigned char* sW = smem + LY::kW;
    uint64_t* bars = (uint64_t*)(smem + LY::kMiscB);
    uint32_t* s_tmem = (uint32_t*)(smem + LY::kMiscB + kNumBars * 8);
    volatile int* s_abort = (volatile int*)(smem + LY::kMiscB + kNumBars * 8 + 4);

    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int ub = range_begin(blockIdx.x, sc.unitsB, gridDim.x), ue = range_begin(blockIdx.x + 1, sc.unitsB, gridDim.x);
    const int n_iter = ue - ub;
    constexpr int NB = LY::NB;
    auto wait = [&](int bar, uint32_t parity) { return pipe_wait(&bars[bar], parity, s_abort, d.status); };
    auto warp_wait = [&](int bar, uint32_t parity) -> bool {
        if (__all_sync(0xffffffffu, mbar_try_wait(&bars[bar], parity) ? 1 : 0)) return true;  // usually complete already
        int ok = 1;
        if (lane == 0) ok = wait(bar, parity) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) ok = mbar_try_wait(&bars[bar], parity) ? 1 : 0;
        return __all_sync(0xffffffffu, ok) != 0;
    };
    constexpr int kBarDqFull = kBarAccFull, kBarDqEmpty = kBarAccEmpty;
    // Only real columns of dQ / dK leave the SM: D / 32 full slabs of 32 columns, then one narrow slab (its own tensor map,
    // dense rows of `tail` floats) for the remainder rounded up to 4.  Worker warp w drains slab w / 4 of its lane quarter.
    int full_slabs = d.D / 32, tail = ((d.D % 32) + 3) & ~3;
    if (tail == 32) {
        full_slabs++;
        tail = 0;
    }
    const int drain_slabs = full_slabs + (tail > 0 ? 1 : 0);
    int tma_it = 0, tma_sg = -1;
    IterA tma_un(ub, sc);  // unit of iteration tma_it
    auto produce = [&](int it) -> bool {
        const IterA& un = tma_un;
        if (it == 0 || un.tile == 0) {
            tma_sg++;
            if (!wait(kBarXEmpty, (tma_sg & 1) ^ 1)) return false;
            mbar_expect_tx(&bars[kBarXFull], LY::kTileBytes);
#pragma unroll
            for (int b = 0; b < NB; b++) tma_load_3d(sX + b * kBlockBytes, &tmQ, b * 64, un.rb * BM, un.zc, &bars[kBarXFull]);
        }
        const int st = it % kStages, use = it / kStages;
        if (!wait(kBarYEmpty + st, (use & 1) ^ 1)) return false;
        mbar_expect_tx(&bars[kBarYFull + st], LY::kTileBytes);
#pragma unroll
        for (int b = 0; b < NB; b++) tma_load_3d(sY + st * LY::kTileBytes + b * kBlockBytes, &tmK, b * 64, un.tile * BN, un.zc, &bars[kBarYFull + st]);
        tma_un.next(sc);
        return true;
    };
    if (warp == kTmaWarp && lane == 0) {
        mbar_init(&bars[kBarXFull], 1);
        mbar_init(&bars[kBarXEmpty], 1);
        for (int k = 0; k < kStages; k++) {
            mbar_init(&bars[kBarYFull + k], 1);
            mbar_init(&bars[kBarYEmpty + k], 1);
        }
        mbar_init(&bars[kBarSFull], 1);
        mbar_init(&bars[kBarSEmpty], kSoftmaxWarps);  // one arrival per worker warp: the score tile is in registers
        mbar_init(&bars[kBarWFull], kSoftmaxWarps);
        mbar_init(&bars[kBarWEmpty], 1);
        for (int k = 0; k < 2; k++) {
            mbar_init(&bars[kBarDkFull + k], 1);                 // dK of a tile complete
            mbar_init(&bars[kBarDkEmpty + k], kDrainWarps);      // ... and read by the drain warps
        }
        mbar_init(&bars[kBarDqFull], 1);                         // dQ of a block complete
        mbar_init(&bars[kBarDqEmpty], kDrainWarps);
        *s_abort = 0;
        mbar_init_fence();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        griddep_wait();  // the operands come from the kernel before this one
        // early loads: the first two tiles, and only while no wait can depend on another role (first block)
        while (tma_it < n_iter && tma_it < 2 && (tma_it == 0 || tma_un.tile != 0)) {
            produce(tma_it);
            tma_it++;
        }
    }
    if (warp == kMmaWarp) {
        tmem_alloc(s_tmem, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    griddep_wait();  // set-up done; from here on global memory written by the preceding kernel is read and its buffers rewritten
    const uint32_t tmem = *s_tmem;
    // tensor memory: the score accumulator at 0, dQ at 128 (accumulated over the block's whole stream), two dK accumulators at
    // 256 and 384 that alternate from tile to tile, so the contraction of one tile runs while the other's result is drained
    const uint32_t tS = tmem, tdQ = tmem + 128, tdK0 = tmem + 256;
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;

    if (warp == kTmaWarp) {
        if (lane == 0) {
            for (; tma_it < n_iter; tma_it++)
                if (!produce(tma_it)) break;
        }
    } else if (warp == kMmaWarp) {
        // ================================ MMA issuer 1: score contractions S = Q K^T ================================
        if (lane == 0) {
            const uint32_t aX = smem_u32(sX), aY0 = smem_u32(sY);
            constexpr uint32_t kIdescS = idesc_f16(BM, BN, 0, 0);
            const uint64_t dXk = desc_kmajor_base(aX);
            int sg = -1;
            IterA un(ub, sc);
            for (int it = 0; it < n_iter; it++, un.next(sc)) {
                if (it == 0 || un.tile == 0) {
                    sg++;
                    if (!wait(kBarXFull, sg & 1)) break;
                }
                const int st = it % kStages, use = it / kStages;
                if (!wait(kBarYFull + st, use & 1)) break;
                if (!wait(kBarSEmpty, (it & 1) ^ 1)) break;  // every worker warp holds the previous tile's scores in registers
                tc_fence_after();
                const uint64_t dYk = desc_kmajor_base(aY0 + st * LY::kTileBytes);
#pragma unroll
                for (int ks = 0; ks < DP / kMmaK; ks++) mma_f16_ss(tS, dXk + koff_kmajor(ks), dYk + koff_kmajor(ks), kIdescS, ks > 0);
                mma_commit(&bars[kBarSFull]);
            }
        }
    } else if (warp == kGradWarp) {
        // ================================ MMA issuer 2: dQ += W K, dK = W^T Q ================================
        // A thread of its own, so that the score contraction of the next tile is issued while this one still waits for
        // the W of the current tile.
        if (lane == 0) {
            const uint32_t aX = smem_u32(sX), aY0 = smem_u32(sY), aW0 = smem_u32(sW);
            // the embedding dimension rounded up to the MMA k step, not to the 64-column block: D = 100 costs 7/8 of DP = 128
            const int D16 = ((d.D + kMmaK - 1) / kMmaK) * kMmaK;
            const uint32_t kIdescDQ = idesc_f16(BM, D16, 0, 1);
            const uint32_t kIdescDK = idesc_f16(BN, D16, 1, 1);
            const uint64_t dXm = desc_mnmajor_base(aX);
            int sg = -1;
            bool fresh = true;
            IterA un(ub, sc);
            for (int it = 0; it < n_iter; it++, un.next(sc)) {
                if (it == 0 || un.tile == 0) {
                    sg++;
                    fresh = true;
                    if (!wait(kBarDqEmpty, (sg & 1) ^ 1)) break;  // the drain of the previous block has read dQ
                }
                const int st = it % kStages, pb = it & 1;
                // (no wait on X or the Y stage: W was made from scores that were made from them)
                if (!wait(kBarWFull, it & 1)) break;
                if (!wait(kBarDkEmpty + pb, ((it >> 1) & 1) ^ 1)) break;  // the tile before last has been drained out of this accumulator
                tc_fence_after();
                const uint32_t tdK = tdK0 + pb * 128;
                const uint32_t aW = aW0;
                const uint64_t dWk = desc_kmajor_base(aW), dWm = desc_mnmajor_base(aW), dYm = desc_mnmajor_base(aY0 + st * LY::kTileBytes);
#pragma unroll
                for (int ks = 0; ks < BM / kMmaK; ks++)  // dK = W^T Q, k runs over the block's rows; first, so that its drain starts early
                    mma_f16_ss(tdK, dWm + koff_mnmajor(ks), dXm + koff_mnmajor(ks), kIdescDK, ks > 0);
                mma_commit(&bars[kBarDkFull + pb]);
#pragma unroll
                for (int ks = 0; ks < BN / kMmaK; ks++)  // dQ += W K, k runs over the tile's negatives
                    mma_f16_ss(tdQ, dWk + koff_kmajor(ks), dYm + koff_mnmajor(ks), kIdescDQ, (!fresh || ks > 0) ? 1u : 0u);
                fresh = false;
                mma_commit(&bars[kBarYEmpty + st]);
                mma_commit(&bars[kBarWEmpty]);
                if (it == n_iter - 1 || un.tile == sc.T - 1) {
                    mma_commit(&bars[kBarDqFull]);
                    mma_commit(&bars[kBarXEmpty]);  // Q is an operand of the score and the dK contractions; those of this block are all behind this point
                }
            }
        }
    } else if (warp < kSoftmaxWarps) {
        // ================================ softmax warps (0-15): W = exp2(S log2 e - lse) * 2^14 ================================
        // All sixteen work on the same tile: warp w takes rows 32*(w & 3) ... + 31 (its quarter of the tensor-memory lanes) and
        // columns 32*(w >> 2) ... + 31: one tensor-memory load, after which the score accumulator is handed back at once.
        const int cg = warp >> 2;      // column group of the score tile
        const int wq = warp & 3;       // lane quarter
        const int my_row = tid & 127;
        float lrow = kDeadRow;  // (shifted, base-2) lse of my row of the current block
        auto load_mask_q = [&](int it, const IterA& un) -> int32_t {  // filter word of column cg*32 + lane of the K tile
            if (it < n_iter) {
                const int n0 = un.tile * BN;
                const int idx = cg * 32 + lane;
                if (idx < min(BN, d.N - n0)) return __ldg(&L.mask[(int64_t)un.zc * d.N + n0 + idx]);
            }
            return -1;
        };
        IterA un(ub, sc), pre(ub, sc);  // `pre`: the unit whose filter word is fetched next
        int32_t mnext = load_mask_q(0, pre);
        pre.next(sc);
        int row_base = 0;  // batch row (padded numbering, as the filter uses it) of row 0 of the current block
        for (int it = 0; it < n_iter; it++, un.next(sc)) {
            if (it == 0 || un.tile == 0) {
                const int s = un.zc / d.C, c = un.zc - s * d.C;
                row_base = c * L.npc + un.rb * BM;
                // was the block run by one CTA of the lse pass (that launch's grid and ranges are known here)?
                const int p_first = cta_of_unit(un.item * sc.T, sc.unitsA, sc.gridA);
                const int nparts = cta_of_unit(un.item * sc.T + sc.T - 1, sc.unitsA, sc.gridA) - p_first + 1;
                if (nparts == 1) {
                    lrow = __ldg(&L.lse2s[(int64_t)un.item * BM + my_row]);
                } else {
                    // A block that the lse pass split between CTAs: combine the partial (max, sum) pairs its sharers left;
                    // the CTA of this launch that starts the block also writes the lse for the scatter kernel and adds the
                    // rows' loss terms.
                    const int64_t grow = (int64_t)s * L.Bp + row_base + my_row;
                    const bool live = my_row < min(BM, L.npc - un.rb * BM);
                    const bool writer = un.tile == 0 && warp < 4;
                    float loss = 0.f;
                    lrow = kDeadRow;
                    if (live) {
                        const float2* part = reinterpret_cast<const float2*>(L.part) + grow * kMaxParts;
                        float m = -INFINITY, l = 0.f;
                        for (int k = 0; k < nparts && k < kMaxParts; k++) {
                            const float2 pk = __ldg(&part[k]);
                            const float nm = fmaxf(m, pk.x);
                            if (nm > -INFINITY) {
                                l = l * exp2f_fast(m - nm) + pk.y * exp2f_fast(pk.x - nm);
                                m = nm;
                            }
                        }
                        const float pos2 = __ldg(&L.pos[grow]) * kLog2e;
                        const float nm2 = fmaxf(m, pos2);
                        const float lse2 = nm2 + __log2f(l * exp2f_fast(m - nm2) + exp2f_fast(pos2 - nm2));
                        lrow = lse2 - (float)kWShift;
                        if (writer) {
                            L.lse[grow] = lse2 * kLn2;
                            loss = (lse2 - pos2) * kLn2;
                        }
                    }
                    if (writer) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) loss += __shfl_xor_sync(0xffffffffu, loss, o);
                        if (lane == 0) atomicAdd(L.loss_acc, (double)loss);
                    }
                }
            }
            uint32_t mb = 0u;  // bit j = column cg*32 + j of this tile is masked for my row
            {
                const int32_t mcur = mnext;
                mnext = load_mask_q(it + 1, pre);
                pre.next(sc);
                const int brow = row_base + my_row, wrow0 = row_base + wq * 32;
                unsigned ballot = __ballot_sync(0xffffffffu, (unsigned)(mcur - wrow0) < 32u);
                while (ballot != 0) {
                    const int src = __ffs(ballot) - 1;
                    ballot &= ballot - 1;
                    if (__shfl_sync(0xffffffffu, mcur, src) == brow) mb |= 1u << src;
                }
            }
            const uint32_t wor = __reduce_or_sync(0xffffffffu, mb);  // which 8-column groups hold a masked entry for any row of this warp
            if (!warp_wait(kBarSFull, it & 1)) break;
            tc_fence_after();
            float v[32];
            tmem_ld_32x32(tS + cg * 32 + lane_sel, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarSEmpty]);  // the piece is in registers: the score accumulator is free for the next tile
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = exp2f_fast(fmaf(v[j], kLog2e, -lrow));
            // Columns past the chunk's last negative: their zero scores are in no row's lse, so exp2 could overflow fp16
            // and meet the zero row of K as inf * 0 in dQ (their dK rows are clipped by the tensor map).
            const int nv = min(BN, d.N - un.tile * BN) - cg * 32;
            if (nv < 32) {
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = j < nv ? v[j] : 0.f;
            }
            // Masked entries were overwritten in place by the reference: no gradient reaches them.  Nothing else needs
            // zeroing: rows of Q past the chunk's end carry the dead-row lse (W = 0).
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if ((wor >> (q * 8)) & 0xffu) {  // warp-uniform
#pragma unroll
                    for (int j = 8 * q; j < 8 * q + 8; j++) v[j] = ((mb >> j) & 1u) ? 0.f : v[j];
                }
            }
            // One W buffer: the contractions of the previous tile must have read it.  They were issued when that tile's W was
            // complete and ran while this tile's scores were loaded and exponentiated, so the wait is short.
            if (!warp_wait(kBarWEmpty, (it & 1) ^ 1)) break;
#pragma unroll
            for (int q = 0; q < 4; q++) {  // 8 halves = one 16-byte chunk
                uint4 pk;
                pk.x = pack_half2(v[8 * q + 0], v[8 * q + 1]);
                pk.y = pack_half2(v[8 * q + 2], v[8 * q + 3]);
                pk.z = pack_half2(v[8 * q + 4], v[8 * q + 5]);
                pk.w = pack_half2(v[8 * q + 6], v[8 * q + 7]);
                *reinterpret_cast<uint4*>(sW + swz_chunk_offset(my_row, cg * 32 + q * 8)) = pk;
            }
            fence_proxy_async_smem();  // W was written with ordinary stores; the MMA reads it through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarWFull]);
        }
    } else {
        // ================================ drain warps (16-19 and 23-26) ================================
        // Every tile: the dK accumulator [128 negatives x D] (two alternate, so the contraction of the next tile runs
        // meanwhile) goes through per-warp staging slabs in shared memory (128-byte rows, 16-byte chunks XOR-swizzled by
        // row: conflict-free stores, and the layout a SWIZZLE_128B tensor map expects) and from there into global dK as one
        // TMA reduce-add per 32 x 32 slab: the row blocks of a chunk add up there (dK is cleared by the first launch).  At
        // the end of a block dQ leaves the same way: a plain store when this CTA ran the block's whole stream, a reduce-add
        // when the stream was cut at a CTA boundary.  Rows past the chunk's end are clipped by the tensor maps.  Drain warp
        // dw takes lane quarter dw & 3 and the slabs of parity dw >> 2; two staging slabs alternate, so a slab is written
        // while the TMA engine still reads the previous one.
        // a warp reaches only the tensor-memory lanes 32 * (warp % 4) ... + 31: each set of four consecutive warps covers all quarters
        const int wq = warp & 3, half = warp < kTmaWarp ? 0 : 1;
        const int dw = half * 4 + wq;
        unsigned char* scr0 = smem + LY::kDrain + dw * 8192;
        int slab = 0;  // counts this warp's TMA operations: consecutive ones alternate between the two staging slabs
        int my_last = -1;  // the last slab this warp drains (-1: none)
        for (int cb = half; cb < drain_slabs; cb += 2) my_last = cb;
        // one accumulator -> global memory; `release` is arrived on as soon as this warp's last slab is in registers
        auto drain = [&](uint32_t tacc, const CUtensorMap* map_full, const CUtensorMap* map_tail, int y, int z, bool reduce, int release) {
            // The coordinates are pinned in ordinary registers here, where the whole warp is active: taken straight from the
            // index arithmetic into the one-lane section below, the third coordinate was seen to reach the store as 0.
            asm volatile("" : "+r"(y), "+r"(z));
            if (my_last < 0) {
                if (lane == 0) mbar_arrive(&bars[release]);
                return;
            }
#pragma unroll 1
            for (int cb = half; cb < drain_slabs; cb += 2) {
                float v[32];
                tmem_ld_32x32(tacc + lane_sel + cb * 32, v);  // warp-collective
                if (cb == my_last) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[release]);
                }
                unsigned char* scr = scr0 + (slab++ & 1) * 4096;
                if (lane == 0) bulk_wait_group_read<1>();  // the operation that last used this slab (two operations ago) has read it
                __syncwarp();
                const bool narrow = cb == full_slabs;
                if (!narrow) {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *reinterpret_cast<float4*>(scr + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if (q * 4 < tail)
                            *reinterpret_cast<float4*>(scr + lane * (tail * 4) + q * 16) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const CUtensorMap* map = narrow ? map_tail : map_full;
                    if (reduce) tma_reduce_add_3d(map, cb * 32, y, z, scr);
                    else tma_store_3d(map, cb * 32, y, z, scr);
                    bulk_commit_group();
                }
            }
        };
        int sg = -1;
        bool ok = true, whole = false;
        IterA un(ub, sc);
        for (int it = 0; ok && it < n_iter; it++, un.next(sc)) {
            if (it == 0 || un.tile == 0) {
                sg++;
                // this CTA runs the whole stream of the block iff it starts at tile 0 and the block's last tile is in its range
                whole = un.tile == 0 && (ub + it + sc.T <= ue);
            }
            if (!warp_wait(kBarDkFull + (it & 1), (it >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            drain(tdK0 + (it & 1) * 128, &tmDK, &tmDKt, un.tile * BN + wq * 32, un.zc, true, kBarDkEmpty + (it & 1));
            if (it == n_iter - 1 || un.tile == sc.T - 1) {
                if (!warp_wait(kBarDqFull, sg & 1)) { ok = false; break; }
                tc_fence_after();
                drain(tdQ, &tmDQ, &tmDQt, un.rb * BM + wq * 32, un.zc, !whole, kBarDqEmpty);
            }
        }
        if (lane == 0) bulk_wait_group<0>();  // all of this warp's stores have landed before the CTA can exit
        __syncwarp();
    }
    // ---- common exit: every role ends here, normally or after an abort; then tensor memory is released ----------
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        if (*s_abort && lane == 0) {
            for (int k = 0; k < kStages; k++) mbar_wait(&bars[kBarYFull + k], 0, 1u << 14);
            for (int k = 0; k < 2; k++) mbar_wait(&bars[kBarDkFull + k], 0, 1u << 14);
            mbar_wait(&bars[kBarDqFull], 0, 1u << 14);
        }
        __syncwarp();
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

// dK / dQ [S*C][rows][ld floats] as a 3-D tensor for the stores: box = 32 floats x 32 rows with the 128-byte swizzle, or
// (narrow slab) box_cols < 32 floats x 32 rows, dense
int make_map_f32_slab(CUtensorMap* map, float* base, int ld, int rows, int mats, int box_cols = 32) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return GE2_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)ld, (cuuint64_t)rows, (cuuint64_t)mats};
    cuuint64_t strides[2] = {(cuuint64_t)ld * 4, (cuuint64_t)rows * ld * 4};
    cuuint32_t box[3] = {(cuuint32_t)box_cols, 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        g_last_cuda_error = (int)r;
        return GE2_ERR_CUDA;
    }
    return GE2_OK;
}

int env_int(const char* name, int fallback) {
    const char* e = getenv(name);
    return e != nullptr ? atoi(e) : fallback;
}

template <int DP>
int launch(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.Qh == nullptr || a.L.Kh == nullptr || a.L.lse2s == nullptr || a.L.item_ctr == nullptr) return GE2_ERR_WORKSPACE;
    const int ZC = a.L.S * a.d.C;
    CUtensorMap tmQ, tmK;
    int rc = make_map(&tmQ, a.L.Qh, DP, a.L.npc, ZC);
    if (rc != GE2_OK) return rc;
    rc = make_map(&tmK, a.L.Kh, DP, a.d.N, ZC);
    if (rc != GE2_OK) return rc;
    CUtensorMap tmDK;
    rc = make_map_f32_slab(&tmDK, a.L.dK, DP, a.d.N, ZC);
    if (rc != GE2_OK) return rc;
    CUtensorMap tmDKt = tmDK;  // narrow slab for the last D % 32 columns (rounded up to 4), when there are any
    const int tail_cols = ((a.d.D % 32) + 3) & ~3;
    if (tail_cols > 0 && tail_cols < 32) {
        rc = make_map_f32_slab(&tmDKt, a.L.dK, DP, a.d.N, ZC, tail_cols);
        if (rc != GE2_OK) return rc;
    }
    // dQ [S*C chunks][rows per chunk][ld floats]: the same slab shapes
    CUtensorMap tmDQ, tmDQt;
    rc = make_map_f32_slab(&tmDQ, a.L.dQ, DP, a.L.npc, ZC);
    if (rc != GE2_OK) return rc;
    tmDQt = tmDQ;
    if (tail_cols > 0 && tail_cols < 32) {
        rc = make_map_f32_slab(&tmDQt, a.L.dQ, DP, a.L.npc, ZC, tail_cols);
        if (rc != GE2_OK) return rc;
    }
    Sched sc;
    sc.RB = ceil_div(a.L.npc, BM);
    sc.T = ceil_div(a.d.N, BN);
    sc.ZC = ZC;
    const long long unitsA = (long long)ZC * sc.RB * sc.T;
    if (2 * unitsA > 0x3fffffff) return GE2_ERR_UNSUPPORTED;
    sc.unitsA = (int)unitsA;
    sc.unitsB = sc.unitsA;
    const int sms = std::max(1, std::min(kNumSMs, env_int("GE2_F16_CTAS", kNumSMs)));  // development switch: fewer CTAs than SMs
    // every CTA's range is at least ceil(T / 7) units long, so a row block is shared by at most kMaxParts CTAs
    sc.gridA = std::max(1, std::min(sms, sc.unitsA / ceil_div(sc.T, kMaxParts - 1)));
    sc.gridB = std::max(1, std::min(sms, sc.unitsB));
    GE2_CUDA_TRY(cudaFuncSetAttribute(lp_lse_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<DP>::kDynamicA));
    GE2_CUDA_TRY(cudaFuncSetAttribute(lp_grad_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, Layout<DP>::kDynamicB));
    const int only = env_int("GE2_F16_ONLY", 0);  // development switch: 1 = logsumexp pass alone, 2 = gradient pass alone (on a workspace a full step left behind)
    if (only != 2) {
        GE2_CUDA_TRY(launch_after(lp_lse_kernel<DP>, dim3((unsigned)sc.gridA), dim3(kThreads), Layout<DP>::kDynamicA, stream, tmQ, tmK, a, sc));
    }
    if (only != 1) {
        GE2_CUDA_TRY(launch_after(lp_grad_kernel<DP>, dim3((unsigned)sc.gridB), dim3(kThreadsB), Layout<DP>::kDynamicB, stream, tmQ, tmK, tmDK, tmDKt, tmDQ,
                                  tmDQt, a, sc));
    }
    return GE2_OK;
}

}  // namespace

int lp_scores_f16(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.ld == 64) return launch<64>(a, stream);
    if (a.L.ld == 128) return launch<128>(a, stream);
    return GE2_ERR_UNSUPPORTED;
}

}  // namespace ge2
