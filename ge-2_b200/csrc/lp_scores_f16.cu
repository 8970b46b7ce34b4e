// Tensor-core scores kernel of the link-prediction step: tcgen05.mma kind::f16 (fp16 operands, the 11-bit significand
// of TF32) with fp32 accumulators in tensor memory, operands staged in shared memory by TMA (every CTA issues its own plain tiled
// loads).  The 1e-2-parity path; everything outside the three contractions stays fp32.
//
// One CTA = (side, chunk, 128-row block) -- or, when the grid would otherwise leave SMs idle in its last round, a share of
// that block's tiles (see choose_nsplit).  Shared memory holds the query block Q [128 x DP], a ring of three tiles of
// negatives K [128 x DP] and two tiles of probabilities P [128 x 128] as fp16, all in the 128-byte-swizzled layout TMA
// writes (64-element column blocks of 128 rows at a 128-byte pitch).  That one layout serves every contraction, because
// a block read along its rows is a K-major operand and read along its columns an MN-major operand:
//   S  [row, n] = Q  K^T   A = Q  (K-major, k = d)    B = K (K-major, k = d)      -> TMEM columns [0, 128)
//   dQ [row, d] += P  K    A = P  (K-major, k = n)    B = K (MN-major, k = n)     -> TMEM columns [128, 128 + DP)
//   dK [n, d]   = P^T Q    A = P  (MN-major, k = row) B = Q (MN-major, k = row)   -> TMEM columns [256, ..) and [384, ..), alternating
// (32-bit tf32 operands cannot do this: the hardware transposes them only from a different, 32-byte-atom swizzle, so
// every tile would be needed twice and the set no longer fits in shared memory.)
// The chunk's negatives stream past the query block twice: sweep 1 runs the first contraction alone to get each row's
// logsumexp; sweep 2 recomputes S, turns it into P = exp(S - lse) in registers, writes P to shared memory and issues the
// two gradient contractions.  The [rows x N] score matrix never leaves the SM.  Replaces the reference's bmm +
// logsumexp + cross_entropy + autograd chain (cpp/src/nn/decoders/edge/comparators.cpp:128-138,
// cpp/src/nn/loss.cpp:46-63 of the reference project).
//
// Warp roles, connected by mbarrier pipelines (no block-wide barrier inside the loops):
//   warps 0-15  softmax: thread = accumulator row (TMEM lane).  Sweep 1: two groups of 8 warps take alternate tiles (64
//               columns per warp), S -> registers -> running max/sum in the exp2 domain.  Sweep 2: all 16 warps on every tile
//               (32 columns per warp), S -> registers (the accumulator is handed back at once) -> P in shared memory
//   warps 16-19 drain: dK accumulator -> swizzled staging in shared memory -> one TMA reduce-add per 32 x 32 slab into
//               global dK (row blocks of a chunk add up there); at the end dQ accumulator -> global dQ the same way (TMA
//               stores, or reduce-adds when the block's tiles are shared between CTAs)
//   warp  20    lane 0: TMA producer for the K ring (and the one-off Q load)
//   warp  21    lane 0: issues the score contractions; the warp also allocates and frees tensor memory
//   warp  22    lane 0: issues the gradient contractions of sweep 2
// Two issuing threads, because one thread would sit in the wait for the probabilities of tile i while the score
// contraction of tile i+1 could already run; with two dK accumulators the drain of tile i overlaps the contractions of
// tile i+1, and in sweep 1 (no gradient accumulators yet) the scores alternate between two accumulators.
// Every mbarrier wait is bounded; a wait that runs out raises GE2_STATUS_PIPE_TIMEOUT and sets a block-wide abort flag
// that every other wait polls, so all roles fall through to the common exit where tensor memory is released.
#include <stdlib.h>

#include "lp_internal.cuh"
#include "tc_ptx.cuh"

namespace ge2 {
namespace {

using namespace tc;

constexpr int BM = 128;                 // query rows per CTA  (MMA M)
constexpr int BN = 128;                 // negatives per tile  (MMA N of the score contraction)
constexpr int kSoftmaxWarps = 16;       // 4 row quarters (tensor-memory lane groups) x 4 groups of 32 columns
constexpr int kColGroups = kSoftmaxWarps / 4;
constexpr int kThreads = 736;           // 16 softmax warps + 4 drain warps + TMA warp + two MMA warps
constexpr int kDrainWarp0 = kSoftmaxWarps, kTmaWarp = kDrainWarp0 + 4, kMmaWarp = kTmaWarp + 1, kGradWarp = kMmaWarp + 1;
constexpr int kBlockBytes = 128 * 128;  // one 64-half column block of 128 rows
constexpr int kMmaK = 16;               // k extent of one kind::f16 MMA (32 bytes)
constexpr int kStagesK = 3;             // K ring depth
constexpr int kMaxSplit = 8;            // most CTAs that share one (side, chunk, row block); size of a row's partial list
constexpr uint32_t kTmemCols = 512;
constexpr float kMasked = -1e9f;

// mbarrier slots
enum Bar { kBarQ = 0, kBarKFull = 1, kBarKEmpty = kBarKFull + kStagesK, kBarSFull = kBarKEmpty + kStagesK, kBarSEmpty = kBarSFull + 3,
           kBarPFull = kBarSEmpty + 3, kBarPEmpty = kBarPFull + 2, kBarDkFull = kBarPEmpty + 2, kBarDkEmpty = kBarDkFull + 2, kBarDqFull = kBarDkEmpty + 2,
           kBarXch, kNumBars };

template <int DP>
struct Layout {
    static constexpr int NB = DP / 64;               // column blocks of Q / K
    static constexpr int kTileBytes = NB * kBlockBytes;
    static constexpr int kPBytes = (BN / 64) * kBlockBytes;
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + kTileBytes;
    static constexpr int kP = kK + kStagesK * kTileBytes;
    static constexpr int kBars = kP + 2 * kPBytes;
    static constexpr int kTmem = kBars + kNumBars * 8;           // tensor memory base address
    static constexpr int kAbort = kTmem + 4;
    // 4 drain warps x 2 buffers x (32 rows x 128 bytes): staging for the TMA reductions of dK, 128-byte swizzled.
    // The per-column-group (max, sum) exchange at the end of sweep 1 (4 x 128 float2) borrows the same bytes: no drain runs before sweep 2.
    static constexpr int kDrain = ((kAbort + 4 + 1023) / 1024) * 1024;
    static constexpr int kXch = kDrain;
    static constexpr int kEnd = kDrain + 4 * 2 * 4096;
    // 1024 bytes of slack to align the base; at least 120 KB so that one CTA owns the SM and its tensor memory
    static constexpr int kDynamic = (kEnd + 1024) > 120 * 1024 ? (kEnd + 1024) : 120 * 1024;
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
        if (i > 64) __nanosleep(i > 4096 ? 256 : 32);  // long waits (a role idle for a whole sweep) must not eat issue slots
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    or_status(status, GE2_STATUS_PIPE_TIMEOUT);
    return false;
}


template <int DP>
__global__ void __launch_bounds__(kThreads, 1)
    lp_scores_f16_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmDK,
                         const __grid_constant__ CUtensorMap tmDKt, const __grid_constant__ CUtensorMap tmDQ,
                         const __grid_constant__ CUtensorMap tmDQt, LpKernelArgs a, int mode, int nsplit, int item_begin) {
    using LY = Layout<DP>;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* sQ = smem + LY::kQ;
    unsigned char* sK = smem + LY::kK;
    unsigned char* sP = smem + LY::kP;
    uint64_t* bars = (uint64_t*)(smem + LY::kBars);
    uint32_t* s_tmem = (uint32_t*)(smem + LY::kTmem);
    volatile int* s_abort = (volatile int*)(smem + LY::kAbort);

    const ge2_lp_desc& d = a.d;
    const LpLayout& L = a.L;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // blockIdx.x = (item - item_begin) * nsplit + h, item = (side * C + chunk) * row_blocks + row block: with nsplit > 1 the
    // chunk's negative tiles are dealt round-robin to nsplit CTAs
    const int row_blocks = (L.npc + BM - 1) / BM;
    const int item = item_begin + (int)blockIdx.x / nsplit;
    const int split_h = blockIdx.x % nsplit;
    const int rb = item % row_blocks;
    const int c = (item / row_blocks) % d.C, s = item / (row_blocks * d.C);
    const int row0 = rb * BM;
    const int valid_rows = min(BM, L.npc - row0);
    const int zc = s * d.C + c;  // third TMA coordinate: (side, chunk)
    const int64_t grow0 = (int64_t)s * L.Bp + (int64_t)c * L.npc + row0;
    const int T_all = (d.N + BN - 1) / BN;                         // tiles of the chunk
    const int T_loc = (T_all - split_h + nsplit - 1) / nsplit;       // tiles of this CTA: split_h, split_h + nsplit, ...
    // mode 0: both sweeps in one launch (nsplit == 1); mode 1: sweep 1 only, leaves per-row partial (max, sum);
    // mode 2: sweep 2 only, starts from the partials.  Iteration i < nA is sweep 1 on local tile i, later ones sweep 2.
    const int nA = mode == 2 ? 0 : T_loc, nB = mode == 1 ? 0 : T_loc;
    const int n_iter = nA + nB;
    // The row blocks of one chunk run side by side and all reduce into the same dK rows; each starts its sweeps at a
    // different tile so that at any moment they touch different rows instead of queueing on the same L2 lines.
    const int rot = rb % T_loc;
    auto tile_n0 = [&](int i) {
        int lt = (i < nA ? i : i - nA) + rot;  // both terms are below T_loc: one conditional subtraction instead of a modulo
        lt = lt >= T_loc ? lt - T_loc : lt;
        return (split_h + nsplit * lt) * BN;
    };
    constexpr int NB = LY::NB;

    // The TMA thread sets the barriers up and starts the first loads at once, so their latency overlaps the allocation of
    // tensor memory and the block-wide barrier below (a fresh "empty" barrier needs no wait).
    const int n_early = n_iter < kStagesK ? n_iter : kStagesK;
    if (warp == kTmaWarp && lane == 0) {
        mbar_init(&bars[kBarQ], 1);
        for (int k = 0; k < kStagesK; k++) {
            mbar_init(&bars[kBarKFull + k], 1);
            mbar_init(&bars[kBarKEmpty + k], 1);
        }
        for (int k = 0; k < 2; k++) {
            mbar_init(&bars[kBarDkFull + k], 1);
            mbar_init(&bars[kBarDkEmpty + k], 4);  // one arrival per drain warp
            mbar_init(&bars[kBarPFull + k], kSoftmaxWarps);
            mbar_init(&bars[kBarPEmpty + k], 1);
        }
        for (int k = 0; k < 2; k++) {
            mbar_init(&bars[kBarSFull + k], 1);
            mbar_init(&bars[kBarSEmpty + k], kSoftmaxWarps / 2);  // sweep 1: one arrival per warp of the group that owns the tile
        }
        mbar_init(&bars[kBarSFull + 2], 1);               // sweep 2: every softmax warp takes part in every tile
        mbar_init(&bars[kBarSEmpty + 2], kSoftmaxWarps);
        mbar_init(&bars[kBarDqFull], 1);
        mbar_init(&bars[kBarXch], kSoftmaxWarps);  // the column groups of every row exchange their (max, sum) once, after sweep 1
        *s_abort = 0;
        mbar_init_fence();
        prefetch_tensormap(&tmQ);
        prefetch_tensormap(&tmK);
        mbar_expect_tx(&bars[kBarQ], LY::kTileBytes);
#pragma unroll
        for (int b = 0; b < LY::NB; b++) tma_load_3d(sQ + b * kBlockBytes, &tmQ, b * 64, row0, zc, &bars[kBarQ]);
        for (int i = 0; i < n_early; i++) {
            mbar_expect_tx(&bars[kBarKFull + i], LY::kTileBytes);
            const int n0 = tile_n0(i);
#pragma unroll
            for (int b = 0; b < LY::NB; b++) tma_load_3d(sK + i * LY::kTileBytes + b * kBlockBytes, &tmK, b * 64, n0, zc, &bars[kBarKFull + i]);
        }
    }
    if (warp == kMmaWarp) {
        tmem_alloc(s_tmem, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *s_tmem;
    // tensor memory: S [0,128); dQ [128, 128+DP), which sweep 1 borrows as a second S buffer so the score contraction of
    // tile i+1 never waits for the softmax warps; two dK accumulators at 256 and 384 so the drain of tile t overlaps the
    // contractions of tile t+1
    const uint32_t tS = tmem, tdQ = tmem + 128, tdK = tmem + 256;
    // S buffer and its use count for iteration i: sweep 1 alternates two buffers, sweep 2 has only the first
    const int s_uses1 = (nA + 1) >> 1;  // uses of buffer 0 during sweep 1
    auto s_buf = [&](int i) { return i < nA ? (i & 1) : 0; };
    auto s_use = [&](int i) { return i < nA ? (i >> 1) : s_uses1 + (i - nA); };
    const uint32_t lane_sel = (uint32_t)((warp & 3) * 32) << 16;  // this warp's quarter of the 128 TMEM lanes
    auto wait = [&](int bar, uint32_t parity) { return pipe_wait(&bars[bar], parity, s_abort, d.status); };
    // Whole-warp wait: one lane polls until the phase completes (32 lanes polling the same mbarrier slow every other role's
    // polls down); then every lane observes the completed phase with a single try_wait of its own, which the ordering of
    // its later tensor-memory and shared-memory reads hangs on.
    auto warp_wait = [&](int bar, uint32_t parity) -> bool {
        int ok = 1;
        if (lane == 0) ok = wait(bar, parity) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) ok = mbar_try_wait(&bars[bar], parity) ? 1 : 0;
        return __all_sync(0xffffffffu, ok) != 0;
    };

    if (warp == kTmaWarp) {
        // ================================ TMA producer ================================
        if (lane == 0) {
            for (int i = n_early; i < n_iter; i++) {  // the first loads went out before the block-wide barrier
                const int st = i % kStagesK, use = i / kStagesK;
                if (!wait(kBarKEmpty + st, (use & 1) ^ 1)) break;
                mbar_expect_tx(&bars[kBarKFull + st], LY::kTileBytes);
                const int n0 = tile_n0(i);
#pragma unroll
                for (int b = 0; b < NB; b++) tma_load_3d(sK + st * LY::kTileBytes + b * kBlockBytes, &tmK, b * 64, n0, zc, &bars[kBarKFull + st]);
            }
        }
    } else if (warp == kMmaWarp) {
        // ================================ MMA issuer 1: score contractions ================================
        if (lane == 0) {
            const uint32_t aQ = smem_u32(sQ), aK0 = smem_u32(sK);
            constexpr uint32_t kIdescS = idesc_f16(BM, BN, 0, 0);
            bool ok = wait(kBarQ, 0);
            const uint64_t dQk = desc_kmajor_base(aQ);
            for (int i = 0; ok && i < n_iter; i++) {
                const int st = i % kStagesK, use = i / kStagesK;
                const int sb = s_buf(i), su = s_use(i);
                if (!wait(kBarKFull + st, use & 1)) break;
                if (i < nA) {
                    if (!wait(kBarSEmpty + sb, (su & 1) ^ 1)) break;
                } else {
                    // sweep 2 writes the first accumulator only: its last sweep-1 tile must have been read, then tile by tile
                    if (i == nA && nA > 0 && !wait(kBarSEmpty + 0, (s_uses1 - 1) & 1)) break;
                    if (!wait(kBarSEmpty + 2, ((i - nA) & 1) ^ 1)) break;
                }
                tc_fence_after();
                const uint64_t dKk = desc_kmajor_base(aK0 + st * LY::kTileBytes);
#pragma unroll
                for (int ks = 0; ks < DP / kMmaK; ks++) mma_f16_ss(tS + sb * 128, dQk + koff_kmajor(ks), dKk + koff_kmajor(ks), kIdescS, ks > 0);
                mma_commit(&bars[i < nA ? kBarSFull + (i & 1) : kBarSFull + 2]);
                if (i < nA) mma_commit(&bars[kBarKEmpty + st]);  // sweep 1 needs the tile for nothing else
            }
        }
    } else if (warp == kGradWarp) {
        // ================================ MMA issuer 2: gradient contractions of sweep 2 ================================
        // A thread of its own, so that the score contraction of the next tile is issued while this one still waits for
        // the probabilities of the current tile.
        if (lane == 0 && nB > 0) {
            const uint32_t aQ = smem_u32(sQ), aK0 = smem_u32(sK), aP0 = smem_u32(sP);
            // the embedding dimension rounded up to the MMA k step, not to the 64-column block: D = 100 costs 7/8 of DP = 128
            const int D16 = ((d.D + kMmaK - 1) / kMmaK) * kMmaK;
            const uint32_t kIdescDQ = idesc_f16(BM, D16, 0, 1);
            const uint32_t kIdescDK = idesc_f16(BN, D16, 1, 1);
            bool ok = wait(kBarQ, 0);
            const uint64_t dQm = desc_mnmajor_base(aQ);
            for (int t = 0; ok && t < nB; t++) {
                const int j = nA + t, pb = t & 1, st = j % kStagesK;
                // (no wait on the K stage: the probabilities were made from scores that were made from it)
                if (!wait(kBarPFull + pb, (t >> 1) & 1)) break;
                if (!wait(kBarDkEmpty + (t & 1), ((t >> 1) & 1) ^ 1)) break;
                tc_fence_after();
                const uint32_t aK = aK0 + st * LY::kTileBytes, aP = aP0 + pb * LY::kPBytes;
                const uint64_t dPk = desc_kmajor_base(aP), dPm = desc_mnmajor_base(aP), dKm = desc_mnmajor_base(aK);
#pragma unroll
                for (int ks = 0; ks < BN / kMmaK; ks++)  // dQ += P K, k runs over the tile's negatives
                    mma_f16_ss(tdQ, dPk + koff_kmajor(ks), dKm + koff_mnmajor(ks), kIdescDQ, (t > 0 || ks > 0) ? 1u : 0u);
#pragma unroll
                for (int ks = 0; ks < BM / kMmaK; ks++)  // dK = P^T Q, k runs over the block's rows
                    mma_f16_ss(tdK + (t & 1) * 128, dPm + koff_mnmajor(ks), dQm + koff_mnmajor(ks), kIdescDK, ks > 0);
                mma_commit(&bars[kBarKEmpty + st]);
                mma_commit(&bars[kBarPEmpty + pb]);
                mma_commit(&bars[kBarDkFull + (t & 1)]);
                if (t == nB - 1) mma_commit(&bars[kBarDqFull]);
            }
        }
    } else if (warp < kDrainWarp0) {
        // ================================ softmax warps (0-15) ================================
        // Two groups of 8 warps take alternate tiles: group g = warp / 8 owns the tiles with (tile index & 1) == g of each
        // sweep, so while one group waits for its scores or stores its probabilities the other keeps the exp unit busy (all 16
        // warps on one tile would move through the same phase at the same time and leave the unit idle between tiles).
        // Within a group, warp w takes rows 32*(w & 3) ... + 31 (its quarter of the tensor-memory lanes) and columns
        // 64*((w >> 2) & 1) ... + 63 of the tile, as two passes of 32 columns.
        const int grp = warp >> 3;                       // which tiles
        const int ch = (warp >> 2) & 1;                  // which 64 columns of a tile
        const int slot = grp * 2 + ch;                   // where this warp's partial (max, sum) goes in the exchange
        const int my_row = tid & 127;                    // accumulator row / TMEM lane
        const int brow = c * L.npc + row0 + my_row;      // batch row in the padded numbering the filter uses
        const int wrow0 = c * L.npc + row0 + (warp & 3) * 32;  // first batch row of this warp
        const int32_t* maskc = L.mask + (int64_t)s * L.CN + (int64_t)c * d.N;
        float* dump = s == 0 ? d.neg_scores : d.inv_neg_scores;
        constexpr float kLog2e = 1.4426950408889634f;
        const bool row_live = my_row < valid_rows;
        // running max / sum of exp2 in the base-2 domain (scores pre-multiplied by log2 e): one FFMA + one MUFU per score
        float run_m = -INFINITY, run_l = 0.f, lse2 = 0.f, my_loss = 0.f;
        // fetched now (written by the kernel before this one), needed when the two sweeps meet
        const float pos_mine = (mode != 1 && row_live) ? __ldg(&L.pos[grow0 + my_row]) : 0.f;
        // the step's loss = sum over rows of (lse - pos): one double-precision atomic per warp
        auto add_row_loss = [&](float v) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0) atomicAdd(L.loss_acc, (double)v);
        };
        if (mode == 2 && row_live) {  // sweep 1 ran in an earlier launch: combine its partial (max, sum) pairs
            float m = -INFINITY, l = 0.f;
            const float2* part = reinterpret_cast<const float2*>(L.part) + (grow0 + my_row) * kMaxSplit;
            for (int k = 0; k < nsplit; k++) {
                const float2 pk = part[k];
                const float nm = fmaxf(m, pk.x);
                if (nm > -INFINITY) {
                    l = l * exp2f_fast(m - nm) + pk.y * exp2f_fast(pk.x - nm);
                    m = nm;
                }
            }
            const float pos2 = pos_mine * kLog2e;
            const float nm = fmaxf(m, pos2);
            lse2 = nm + __log2f(l * exp2f_fast(m - nm) + exp2f_fast(pos2 - nm));
            if (split_h == 0 && slot == 0) L.lse[grow0 + my_row] = lse2 * 0.6931471805599453f;
            my_loss = (lse2 - pos2) * 0.6931471805599453f;
        }
        // The filter is sparse: a tile has at most one masked row per column and few of them fall in this warp's 32 rows.
        // Lane l looks at columns l and l + 32 of the warp's 64; an entry that names a row of this warp is handed to that
        // row's thread, which ends up with one bit per masked column of its own row.  The words of the group's next tile
        // are fetched while the current one is processed.
        auto load_mask = [&](int i, int32_t (&m)[2]) {
            if (i < n_iter) {
                const int n0 = tile_n0(i);
                const int vn = min(BN, d.N - n0);
#pragma unroll
                for (int k = 0; k < 2; k++) {
                    const int idx = ch * 64 + k * 32 + lane;
                    m[k] = idx < vn ? __ldg(&maskc[n0 + idx]) : -1;
                }
            } else {
                m[0] = m[1] = -1;
            }
        };
        // per-tile preamble shared by both sweeps: mask bits of my row, then the wait for the tile's scores
        uint32_t mb[2], wor[2];
        int32_t mnext[2] = {-1, -1};
        auto mask_bits = [&](int next_i) {
            const int32_t mcur[2] = {mnext[0], mnext[1]};
            load_mask(next_i, mnext);
#pragma unroll
            for (int k = 0; k < 2; k++) {
                mb[k] = 0u;  // bit j = column ch*64 + 32k + j of this tile is masked for my row
                unsigned ballot = __ballot_sync(0xffffffffu, (unsigned)(mcur[k] - wrow0) < 32u);
                while (ballot != 0) {
                    const int src = __ffs(ballot) - 1;
                    ballot &= ballot - 1;
                    if (__shfl_sync(0xffffffffu, mcur[k], src) == brow) mb[k] |= 1u << src;
                }
                // which 8-column groups hold a masked entry for any row of this warp (usually none or one of the 4)
                wor[k] = __reduce_or_sync(0xffffffffu, mb[k]);
            }
        };
        bool alive = true;
        // ---------------- sweep 1: running (max, sum) over the group's tiles ----------------
        const int first1 = grp;  // the group's first sweep-1 iteration
        load_mask(first1 < nA ? first1 : n_iter, mnext);
        for (int i = first1; alive && i < nA; i += 2) {
            const int n0 = tile_n0(i);
            mask_bits(i + 2 < nA ? i + 2 : n_iter);
            const int sb = s_buf(i);
            if (!warp_wait(kBarSFull + grp, (i >> 1) & 1)) { alive = false; break; }  // warp-uniform: tcgen05.ld is collective
            tc_fence_after();
#pragma unroll
            for (int k = 0; k < 2; k++) {
                const int nv = min(BN, d.N - n0) - ch * 64 - k * 32;  // live columns among these 32
                float v[32];
                tmem_ld_32x32(tS + sb * 128 + ch * 64 + k * 32 + lane_sel, v);
                if (k == 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[kBarSEmpty + sb]);  // the tile is in registers: this S accumulator is free again
                }
                if (nv <= 0) continue;
                if (nv < 32 || dump != nullptr) {  // ragged last tile, or the score dump of the tests
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        float sc = ((mb[k] >> j) & 1u) ? kMasked : v[j];
                        if (dump != nullptr && row_live && j < nv) dump[(int64_t)brow * d.N + n0 + ch * 64 + k * 32 + j] = sc;
                        v[j] = j < nv ? sc : -INFINITY;
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
        const int cg = warp >> 2;  // sweep 2: this warp's 32 columns of every tile
        auto load_mask2 = [&](int i) -> int32_t {
            if (i >= n_iter) return -1;
            const int n0 = tile_n0(i);
            const int idx = cg * 32 + lane;
            return idx < min(BN, d.N - n0) ? __ldg(&maskc[n0 + idx]) : -1;
        };
        int32_t m2next = load_mask2(nA);  // fetched before the exchange below, used after it
        if (alive && nA > 0) {
            // the four partials of a row (two groups x two column halves) meet in shared memory; the wait is an mbarrier
            // (bounded), not a named barrier
            float2* xch = reinterpret_cast<float2*>(smem + LY::kXch);
            xch[slot * 128 + my_row] = make_float2(run_m, run_l);
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarXch]);  // used once per launch: one arrival per softmax warp
            alive = warp_wait(kBarXch, 0);
            if (alive) {
                float2 pr[kColGroups];
                float nm = -INFINITY;
#pragma unroll
                for (int k = 0; k < kColGroups; k++) {
                    pr[k] = xch[k * 128 + my_row];
                    nm = fmaxf(nm, pr[k].x);
                }
                float l = 0.f;
                if (nm > -INFINITY) {
#pragma unroll
                    for (int k = 0; k < kColGroups; k++) l += pr[k].y * exp2f_fast(pr[k].x - nm);  // an empty partial has sum 0 and max -inf
                }
                if (row_live) {
                    if (mode == 1) {  // hand the partial over to the sweep-2 launch
                        if (slot == 0) reinterpret_cast<float2*>(L.part)[(grow0 + my_row) * kMaxSplit + split_h] = make_float2(nm, l);
                    } else {
                        const float pos2 = pos_mine * kLog2e;
                        const float nm2 = fmaxf(nm, pos2);
                        lse2 = nm2 + __log2f(l * exp2f_fast(nm - nm2) + exp2f_fast(pos2 - nm2));
                        if (slot == 0) L.lse[grow0 + my_row] = lse2 * 0.6931471805599453f;
                        my_loss = (lse2 - pos2) * 0.6931471805599453f;
                    }
                }
            }
        }
        // ---------------- sweep 2: probabilities, all 16 warps on every tile ----------------
        // There is one score accumulator now (the gradient accumulators fill tensor memory), so the tile is spread over all
        // warps: each copies its 32 x 32 piece to registers and hands the accumulator back at once.  Warp w: rows 32*(w & 3)
        // ... + 31, columns 32*(w >> 2) ... + 31.
        for (int i = nA; alive && i < n_iter; i++) {
            const int t = i - nA, pb = t & 1;
            const int32_t mcur = m2next;
            m2next = load_mask2(i + 1);
            uint32_t mbits = 0u;  // bit j = column cg*32 + j of this tile is masked for my row
            {
                unsigned ballot = __ballot_sync(0xffffffffu, (unsigned)(mcur - wrow0) < 32u);
                while (ballot != 0) {
                    const int src = __ffs(ballot) - 1;
                    ballot &= ballot - 1;
                    if (__shfl_sync(0xffffffffu, mcur, src) == brow) mbits |= 1u << src;
                }
            }
            const uint32_t wbits = __reduce_or_sync(0xffffffffu, mbits);
            if (!warp_wait(kBarSFull + 2, t & 1)) break;
            tc_fence_after();
            float v[32];
            tmem_ld_32x32(tS + cg * 32 + lane_sel, v);
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarSEmpty + 2]);  // the tile is in registers: the S accumulator is free again
#pragma unroll
            for (int j = 0; j < 32; j++) v[j] = exp2f_fast(fmaf(v[j], kLog2e, -lse2));
            // Masked entries were overwritten in place by the reference: no gradient reaches them.  Nothing else needs
            // zeroing: a column past the chunk's last negative meets an all-zero row of K in dQ and is clipped from dK by
            // the tensor map, and a row past the block's last query has an all-zero row of Q (out-of-range rows of both
            // tiles are zero-filled by the loads) whose dQ is never stored; exp2 of their zero scores is finite.
#pragma unroll
            for (int q = 0; q < 4; q++) {
                if ((wbits >> (q * 8)) & 0xffu) {  // warp-uniform
#pragma unroll
                    for (int j = 8 * q; j < 8 * q + 8; j++) v[j] = ((mbits >> j) & 1u) ? 0.f : v[j];
                }
            }
            // the gradient MMAs that read this P buffer two tiles ago must be done
            if (!warp_wait(kBarPEmpty + pb, ((t >> 1) & 1) ^ 1)) break;
            unsigned char* sPb = sP + pb * LY::kPBytes;
#pragma unroll
            for (int q = 0; q < 4; q++) {  // 8 halves = one 16-byte chunk
                uint4 pk;
                pk.x = pack_half2(v[8 * q + 0], v[8 * q + 1]);
                pk.y = pack_half2(v[8 * q + 2], v[8 * q + 3]);
                pk.z = pack_half2(v[8 * q + 4], v[8 * q + 5]);
                pk.w = pack_half2(v[8 * q + 6], v[8 * q + 7]);
                *reinterpret_cast<uint4*>(sPb + swz_chunk_offset(my_row, cg * 32 + q * 8)) = pk;
            }
            fence_proxy_async_smem();  // P was written with ordinary stores; the MMA reads it through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&bars[kBarPFull + pb]);
        }
        // the loss of this block's rows, off the path between the sweeps
        if (alive && mode != 1 && slot == 0 && (mode == 0 || split_h == 0)) add_row_loss(my_loss);
    } else {
        // ================================ drain warps (16-19) ================================
        // columns of dK that are reduced into global memory: full 32-column slabs, then a narrow one
        int full_slabs = d.D / 32, tail = ((d.D % 32) + 3) & ~3;
        if (tail == 32) {
            full_slabs++;
            tail = 0;
        }
        const int n_slabs = full_slabs + (tail > 0 ? 1 : 0);
        bool ok = true;
        for (int t = 0; t < nB; t++) {
            const int n0 = tile_n0(nA + t);
            if (!warp_wait(kBarDkFull + (t & 1), (t >> 1) & 1)) { ok = false; break; }
            tc_fence_after();
            // Each 32 x 32 slab of the accumulator goes through a per-warp staging buffer in shared memory (128-byte rows,
            // 16-byte chunks XOR-swizzled by row: conflict-free stores, and the layout a SWIZZLE_128B tensor map expects) and
            // from there to global dK as ONE TMA reduce-add per slab: the load/store units only see the shared-memory
            // stores, rows past the chunk's last negative are clipped by the tensor map, and the accumulator is handed
            // back as soon as its last slab is in registers.  Two staging buffers alternate, so a slab is written while
            // the TMA engine still reads the previous one.
            // Only real columns travel: D / 32 full slabs, then one narrow slab (its own tensor map, dense rows of `tail`
            // floats) for the remainder rounded up to 4 -- with D = 100 that is 100 columns instead of the padded 128; the
            // reductions into L2 are what bounds this sweep.
            unsigned char* scr0 = smem + LY::kDrain + (warp - kDrainWarp0) * 8192;
#pragma unroll 1
            for (int cb = 0; cb < n_slabs; cb++) {
                float v[32];
                tmem_ld_32x32(tdK + (t & 1) * 128 + lane_sel + cb * 32, v);  // warp-collective
                if (cb == n_slabs - 1) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars[kBarDkEmpty + (t & 1)]);
                }
                unsigned char* scr = scr0 + (cb & 1) * 4096;
                if (lane == 0) bulk_wait_group_read<1>();  // the reduction that last used this buffer (two slabs ago) has read it
                __syncwarp();
                const bool narrow = cb == full_slabs;
                if (!narrow) {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *reinterpret_cast<float4*>(scr + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if (q * 4 < tail) *reinterpret_cast<float4*>(scr + lane * (tail * 4) + q * 16) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_reduce_add_3d(narrow ? &tmDKt : &tmDK, cb * 32, n0 + (warp - kDrainWarp0) * 32, zc, scr);
                    bulk_commit_group();
                }
            }
        }
        if (lane == 0) bulk_wait_group<0>();  // all of this warp's reductions have landed before the CTA can exit
        __syncwarp();
        if (ok && nB > 0 && warp_wait(kBarDqFull, 0)) {
            // dQ leaves the same way as dK: 32 x 32 slabs through the staging buffers, one TMA operation per slab -- a plain
            // store when this CTA owns the block's rows, a reduce-add when the block's tiles are shared (dQ is then the sum
            // over the sharing CTAs and was cleared by the host side).  Rows past the chunk's last query are clipped by the
            // tensor map, columns past D (rounded up to 4) are not written: nobody reads them.
            tc_fence_after();
            unsigned char* scr0 = smem + LY::kDrain + (warp - kDrainWarp0) * 8192;
#pragma unroll 1
            for (int cb = 0; cb < n_slabs; cb++) {
                float v[32];
                tmem_ld_32x32(tdQ + lane_sel + cb * 32, v);
                unsigned char* scr = scr0 + (cb & 1) * 4096;
                if (lane == 0) bulk_wait_group_read<1>();
                __syncwarp();
                const bool narrow = cb == full_slabs;
                if (!narrow) {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *reinterpret_cast<float4*>(scr + lane * 128 + ((q ^ (lane & 7)) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        if (q * 4 < tail) *reinterpret_cast<float4*>(scr + lane * (tail * 4) + q * 16) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                }
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const CUtensorMap* map = narrow ? &tmDQt : &tmDQ;
                    const int y = row0 + (warp - kDrainWarp0) * 32;
                    if (nsplit == 1) tma_store_3d(map, cb * 32, y, zc, scr);
                    else tma_reduce_add_3d(map, cb * 32, y, zc, scr);
                    bulk_commit_group();
                }
            }
            if (lane == 0) bulk_wait_group<0>();
            __syncwarp();
        }
    }
    // ---- common exit: every role ends here, normally or after an abort; then tensor memory is released ----------
    tc_fence_before();
    __syncthreads();
    if (warp == kMmaWarp) {
        if (*s_abort && lane == 0) {
            // a wait ran out somewhere: give copies / MMAs still in flight a bounded chance to land before the SM's
            // shared and tensor memory are handed to the next CTA
            for (int k = 0; k < kStagesK; k++) mbar_wait(&bars[kBarKFull + k], 0, 1u << 14);
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

// How many CTAs share one (side, chunk, row block), for a set of `items` blocks that does not fill the GPU: dealing each
// block's tiles to 2, 4 or 8 CTAs (sweep 1 and sweep 2 then run as two launches) fills the machine.  Splitting adds per-CTA
// set-up (Q load, barriers, tensor memory) and a second launch, so the largest split that still fits one round is used.
int choose_nsplit(int items, int tiles) {
    if (const char* e = getenv("GE2_F16_NSPLIT")) {
        const int v = atoi(e);
        if ((v == 1 || v == 2 || v == 4 || v == 8) && v <= tiles) return v;
    }
    int best = 1;
    for (int ns = 2; ns <= kMaxSplit && ns <= tiles; ns *= 2)
        if (items * ns <= kNumSMs) best = ns;
    return best;
}

// dK [S*C][N][ld floats] as a 3-D tensor for the reduce-add stores: box = 32 floats x 32 rows with the 128-byte swizzle, or
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

template <int DP>
int launch(const LpKernelArgs& a, cudaStream_t stream) {
    if (a.L.Qh == nullptr || a.L.Kh == nullptr) return GE2_ERR_WORKSPACE;
    CUtensorMap tmQ, tmK;
    int rc = make_map(&tmQ, a.L.Qh, DP, a.L.npc, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    rc = make_map(&tmK, a.L.Kh, DP, a.d.N, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    CUtensorMap tmDK;
    rc = make_map_f32_slab(&tmDK, a.L.dK, DP, a.d.N, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    CUtensorMap tmDKt = tmDK;  // narrow slab for the last D % 32 columns (rounded up to 4), when there are any
    const int tail_cols = ((a.d.D % 32) + 3) & ~3;
    if (tail_cols > 0 && tail_cols < 32) {
        rc = make_map_f32_slab(&tmDKt, a.L.dK, DP, a.d.N, a.L.S * a.d.C, tail_cols);
        if (rc != GE2_OK) return rc;
    }
    // dQ [S*C chunks][rows per chunk][ld floats]: the same slab shapes, for the stores / reductions of the query gradients
    CUtensorMap tmDQ, tmDQt;
    rc = make_map_f32_slab(&tmDQ, a.L.dQ, DP, a.L.npc, a.L.S * a.d.C);
    if (rc != GE2_OK) return rc;
    tmDQt = tmDQ;
    if (tail_cols > 0 && tail_cols < 32) {
        rc = make_map_f32_slab(&tmDQt, a.L.dQ, DP, a.L.npc, a.L.S * a.d.C, tail_cols);
        if (rc != GE2_OK) return rc;
    }
    const int smem = Layout<DP>::kDynamic;
    GE2_CUDA_TRY(cudaFuncSetAttribute(lp_scores_f16_kernel<DP>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    const int row_blocks = ceil_div(a.L.npc, BM);
    const int items = row_blocks * a.d.C * a.L.S, tiles = ceil_div(a.d.N, BN);
    // One CTA per item, one CTA per SM.  Whole rounds of kNumSMs items run unsplit in one launch; the items left over
    // would occupy a few SMs for a full round of their own, so their tiles are dealt to 2, 4 or 8 CTAs each (sweep 1 and sweep 2
    // then run as two launches, meeting in the per-row partials) and the machine is filled once more for a fraction of a round.
    int whole = (items / kNumSMs) * kNumSMs, rest = items - whole;
    if (getenv("GE2_F16_NSPLIT") != nullptr) whole = 0, rest = items;  // development switch: one split factor for everything
    const int nsplit = rest > 0 ? choose_nsplit(rest, tiles) : 1;
    if (nsplit > 1) {
        // dQ of a split item is the sum over its CTAs: those rows start from zero (dK next to it is zeroed by the caller).
        // Items are numbered in row order, so the rows of items [whole, items) are one contiguous range.  Cleared first, so
        // that nothing but the kernels themselves sits between the launches below.
        const int64_t first_row = (int64_t)(whole / (row_blocks * a.d.C)) * a.L.Bp + (int64_t)((whole / row_blocks) % a.d.C) * a.L.npc +
                                  (int64_t)(whole % row_blocks) * BM;
        const int64_t end_row = (int64_t)a.L.S * a.L.Bp;
        GE2_CUDA_TRY(cudaMemsetAsync(a.L.dQ + first_row * DP, 0, (size_t)(end_row - first_row) * DP * sizeof(float), stream));
    }
    if (whole > 0) {
        lp_scores_f16_kernel<DP><<<(unsigned)whole, kThreads, smem, stream>>>(tmQ, tmK, tmDK, tmDKt, tmDQ, tmDQt, a, 0, 1, 0);
        GE2_LAUNCH_CHECK();
    }
    if (rest > 0) {
        if (nsplit == 1) {
            lp_scores_f16_kernel<DP><<<(unsigned)rest, kThreads, smem, stream>>>(tmQ, tmK, tmDK, tmDKt, tmDQ, tmDQt, a, 0, 1, whole);
            GE2_LAUNCH_CHECK();
        } else {
            lp_scores_f16_kernel<DP><<<(unsigned)(rest * nsplit), kThreads, smem, stream>>>(tmQ, tmK, tmDK, tmDKt, tmDQ, tmDQt, a, 1, nsplit, whole);
            GE2_LAUNCH_CHECK();
            lp_scores_f16_kernel<DP><<<(unsigned)(rest * nsplit), kThreads, smem, stream>>>(tmQ, tmK, tmDK, tmDKt, tmDQ, tmDQt, a, 2, nsplit, whole);
            GE2_LAUNCH_CHECK();
        }
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
