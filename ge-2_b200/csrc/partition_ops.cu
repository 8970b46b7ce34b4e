// Partition-buffer kernels: the per-state edge list (bucket gather + slot remap + shuffle in one pass) and the partition
// swap between supersteps as receiver-side pulls over peer memory behind a device-side barrier.
//
// Follows, in the reference project (paths relative to gege/src/cpp/src):
//   state rebuild   storage/graph_storage.cpp:938-1240 (updateInMemorySubGraph_: which buckets are resident, copy of their edges,
//                   arithmetic remap :270-303) and data/dataloader.cpp:524-633 (setActiveEdges: concatenation of the state's
//                   buckets, randperm, index_select) -- host loops, OpenMP and a full upload there, one kernel here;
//   swap            storage/storage.cpp:576-689 (MemPartitionBufferStorage::performNextSwap, peer-relay branch :599-652: every slot
//                   of the next state is copied from the device and slot that hold the partition now, between thread barriers).
#include <algorithm>

#include "common.cuh"

namespace ge2 {
namespace {

__device__ __forceinline__ uint64_t mix64(uint64_t x) {  // splitmix64 finaliser
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// A permutation of [0, n): four Feistel rounds over the smallest even number of bits that covers n, walked until the value
// falls below n (a bijection of [0, 2^bits) restricted to its cycle through [0, n)).  On average fewer than four walks.
__device__ __forceinline__ uint64_t feistel_perm(uint64_t j, uint64_t n, int half_bits, uint64_t key) {
    const uint64_t mask = (1ull << half_bits) - 1ull;
    uint64_t x = j;
    do {
        uint64_t l = x >> half_bits, r = x & mask;
#pragma unroll
        for (int round = 0; round < 4; round++) {
            const uint64_t f = mix64(key + (uint64_t)round * 0xD1342543DE82EF95ull + r) & mask;
            const uint64_t nl = r;
            r = l ^ f;
            l = nl;
        }
        x = (l << half_bits) | r;
    } while (x >= n);
    return x;
}

constexpr int kMaxBuckets = 64;
struct BucketList {
    int64_t begin[kMaxBuckets];   // first row of the bucket in the bucket-sorted edge list
    int64_t prefix[kMaxBuckets];  // rows of the state's buckets before this one
    int32_t count;
};

template <int COLS>
__global__ void __launch_bounds__(256) build_state_edges_kernel(const int64_t* __restrict__ edges, BucketList bl, int64_t total,
                                                                const int64_t* __restrict__ part_to_slot, int num_partitions,
                                                                int64_t partition_size, int half_bits, uint64_t key,
                                                                int64_t* __restrict__ out, int32_t* status) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < total; j += stride) {
        const int64_t p = (int64_t)feistel_perm((uint64_t)j, (uint64_t)total, half_bits, key);  // row of the concatenated buckets
        int b = 0;
#pragma unroll 1
        for (int k = 1; k < bl.count; k++) b = p >= bl.prefix[k] ? k : b;  // prefix is ascending
        const int64_t* row = edges + (bl.begin[b] + (p - bl.prefix[b])) * COLS;
        int64_t v[COLS];
#pragma unroll
        for (int c = 0; c < COLS; c++) v[c] = __ldg(row + c);
#pragma unroll
        for (int c = 0; c < COLS; c += COLS - 1) {  // first and last column: node ids -> buffer-local ids
            const int64_t id = v[c];
            const int64_t part = id / partition_size;  // ids are non-negative: same as the reference's floor of a double division
            int64_t slot = -1;
            if (id >= 0 && part < num_partitions) slot = __ldg(&part_to_slot[part]);
            if (slot < 0) {
                or_status(status, GE2_STATUS_BAD_INDEX);
                v[c] = -1;
            } else {
                v[c] = slot * partition_size + (id - part * partition_size);
            }
        }
#pragma unroll
        for (int c = 0; c < COLS; c++) out[j * COLS + c] = v[c];
    }
}

// ---- swap ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void st_release_sys(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr int kMaxRanks = 16;
struct FlagRows {
    unsigned long long* row[kMaxRanks];  // this process's mapping of every rank's flag row (`world` slots + one verdict word)
};

// One warp: announce "my training of the superstep that ends here is complete" (epoch) in my slot of every rank's flag
// row, wait -- lane p polls rank p, bounded by a time budget -- until every rank has announced the same, and publish one
// verdict for the swap (epoch = go, 0 = a rank never arrived).
__global__ void __launch_bounds__(32) swap_arrive_kernel(FlagRows flags, int world, int rank, unsigned long long epoch,
                                                         unsigned long long budget_ns, int32_t* status) {
    const int lane = threadIdx.x;
    int ok = 1;
    if (lane < world) {
        st_release_sys(flags.row[lane] + rank, epoch);
        const unsigned long long* mine = flags.row[rank] + lane;
        const unsigned long long t0 = timer_ns();
        ok = 0;
        for (uint32_t i = 0; i < (1u << 26); i++) {  // bounded twice: by the time budget and by an iteration count
            if (ld_acquire_sys(mine) >= epoch) {
                ok = 1;
                break;
            }
            if ((i & 15u) == 15u && timer_ns() - t0 > budget_ns) break;
            __nanosleep(i < 64 ? 20 : 400);
        }
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    if (lane == 0) {
        flags.row[rank][world] = all_ok ? epoch : 0ull;
        if (!all_ok) or_status(status, GE2_STATUS_PEER_TIMEOUT);
    }
}

constexpr int kMaxPulls = 32;
struct PullList {
    const float4* src[kMaxPulls];  // slab in the holder's buffer or home array (a peer mapping or local memory)
    float4* dst[kMaxPulls];        // slab in this rank's next buffer or home array
    int32_t count;
};

// Copies every slab of the list -- unless the verdict of the barrier before it says that a rank never arrived, in which
// case nothing is touched.  Plain 16-byte peer loads; no multicast object is involved.  The list is cut into pieces of
// kPullPiece bytes dealt round-robin over slabs and CTAs, so every CTA works on local and remote slabs alike; a warp
// instruction covers 512 contiguous bytes and every thread keeps eight loads in flight.
constexpr int kPullThreads = 256, kPullInFlight = 8;
constexpr int64_t kPullPieceVec4 = (int64_t)kPullThreads * kPullInFlight;  // 32 KB
__global__ void __launch_bounds__(kPullThreads) swap_pull_kernel(PullList pulls, int64_t slab_vec4, const unsigned long long* __restrict__ verdict,
                                                                 unsigned long long epoch) {
    if (verdict != nullptr && *verdict != epoch) return;
    const int64_t per_slab = (slab_vec4 + kPullPieceVec4 - 1) / kPullPieceVec4;
    const int64_t total = per_slab * pulls.count;
    for (int64_t q = blockIdx.x; q < total; q += gridDim.x) {
        const int slab = (int)(q % pulls.count);
        const int64_t base = (q / pulls.count) * kPullPieceVec4 + threadIdx.x;
        const float4* __restrict__ s = pulls.src[slab];
        float4* __restrict__ d = pulls.dst[slab];
        float4 v[kPullInFlight];
#pragma unroll
        for (int k = 0; k < kPullInFlight; k++)
            if (base + k * kPullThreads < slab_vec4) v[k] = __ldcv(s + base + k * kPullThreads);
#pragma unroll
        for (int k = 0; k < kPullInFlight; k++)
            if (base + k * kPullThreads < slab_vec4) d[base + k * kPullThreads] = v[k];
    }
}

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" int ge2_build_state_edges(const int64_t* edges_sorted, int32_t cols, const int64_t* bucket_begin_host, const int64_t* bucket_len_host,
                                     int32_t num_buckets, const int64_t* partition_to_slot, int32_t num_partitions, int64_t partition_size,
                                     uint64_t seed, int64_t* out_edges, int64_t* out_total_host, int32_t* status, ge2_stream_t stream_) {
    if ((cols != 2 && cols != 3) || num_buckets < 0 || num_buckets > kMaxBuckets || num_partitions <= 0 || partition_size <= 0)
        return GE2_ERR_INVALID_ARGUMENT;
    if (num_buckets > 0 && (bucket_begin_host == nullptr || bucket_len_host == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    BucketList bl;
    bl.count = num_buckets;
    int64_t total = 0;
    for (int k = 0; k < num_buckets; k++) {
        if (bucket_begin_host[k] < 0 || bucket_len_host[k] < 0) return GE2_ERR_INVALID_ARGUMENT;
        bl.begin[k] = bucket_begin_host[k];
        bl.prefix[k] = total;
        total += bucket_len_host[k];
    }
    for (int k = num_buckets; k < kMaxBuckets; k++) bl.begin[k] = 0, bl.prefix[k] = INT64_MAX;
    if (out_total_host != nullptr) *out_total_host = total;
    if (total == 0) return GE2_OK;
    if (edges_sorted == nullptr || partition_to_slot == nullptr || out_edges == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    int bits = 2;
    while (bits < 62 && (1ll << bits) < total) bits++;
    if (bits & 1) bits++;
    const uint64_t key = seed * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;
    const int grid = stream_grid(total, 256);
    cudaStream_t stream = as_stream(stream_);
    if (cols == 3)
        build_state_edges_kernel<3><<<grid, 256, 0, stream>>>(edges_sorted, bl, total, partition_to_slot, num_partitions, partition_size, bits / 2, key,
                                                              out_edges, status);
    else
        build_state_edges_kernel<2><<<grid, 256, 0, stream>>>(edges_sorted, bl, total, partition_to_slot, num_partitions, partition_size, bits / 2, key,
                                                              out_edges, status);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_swap_begin(const ge2_swap_desc* desc, ge2_stream_t stream_) {
    if (desc == nullptr || desc->world < 1 || desc->world > kMaxRanks || desc->rank < 0 || desc->rank >= desc->world) return GE2_ERR_INVALID_ARGUMENT;
    if (desc->num_pulls < 0 || desc->num_pulls > kMaxPulls || desc->slab_bytes < 0 || (desc->slab_bytes & 15) != 0) return GE2_ERR_INVALID_ARGUMENT;
    if (desc->num_pulls > 0 && (desc->pull_src == nullptr || desc->pull_dst == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = as_stream(stream_);
    const unsigned long long* verdict = nullptr;
    if (desc->world > 1) {
        if (desc->flag_rows == nullptr || desc->status == nullptr || desc->epoch == 0) return GE2_ERR_INVALID_ARGUMENT;
        FlagRows fr;
        for (int r = 0; r < kMaxRanks; r++) fr.row[r] = r < desc->world ? reinterpret_cast<unsigned long long*>(desc->flag_rows[r]) : nullptr;
        for (int r = 0; r < desc->world; r++)
            if (fr.row[r] == nullptr) return GE2_ERR_INVALID_ARGUMENT;
        const unsigned long long budget_ns = (desc->wait_budget_us == 0 ? 4000000ull : (unsigned long long)desc->wait_budget_us) * 1000ull;
        swap_arrive_kernel<<<1, 32, 0, stream>>>(fr, desc->world, desc->rank, desc->epoch, budget_ns, desc->status);
        GE2_LAUNCH_CHECK();
        verdict = fr.row[desc->rank] + desc->world;
    }
    if (desc->num_pulls == 0 || desc->slab_bytes == 0) return GE2_OK;
    PullList pl;
    pl.count = desc->num_pulls;
    for (int k = 0; k < kMaxPulls; k++) {
        pl.src[k] = k < desc->num_pulls ? reinterpret_cast<const float4*>(desc->pull_src[k]) : nullptr;
        pl.dst[k] = k < desc->num_pulls ? reinterpret_cast<float4*>(desc->pull_dst[k]) : nullptr;
    }
    for (int k = 0; k < desc->num_pulls; k++)
        if (pl.src[k] == nullptr || pl.dst[k] == nullptr || (((uintptr_t)pl.src[k] | (uintptr_t)pl.dst[k]) & 15) != 0) return GE2_ERR_INVALID_ARGUMENT;
    const int64_t v4 = desc->slab_bytes / 16;
    // the copy engine of this GPU is its SMs: every SM full of copy warps, pieces of all slabs dealt over them
    const int64_t pieces = ceil_div<int64_t>(v4, kPullPieceVec4) * desc->num_pulls;
    const int grid = (int)std::min<int64_t>(pieces, (int64_t)kNumSMs * 6);
    swap_pull_kernel<<<grid, kPullThreads, 0, stream>>>(pl, v4, verdict, desc->epoch);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_swap_wait(ge2_stream_t swap_stream_, ge2_stream_t compute_stream_) {
    // the pulls were enqueued on swap_stream: make compute_stream wait for them (no host synchronisation)
    cudaStream_t ss = as_stream(swap_stream_), cs = as_stream(compute_stream_);
    if (ss == cs) return GE2_OK;
    cudaEvent_t ev;
    GE2_CUDA_TRY(cudaEventCreateWithFlags(&ev, cudaEventDisableTiming));
    cudaError_t e = cudaEventRecord(ev, ss);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, ev, 0);
    cudaEventDestroy(ev);
    GE2_CUDA_TRY(e);
    return GE2_OK;
}
