// Bitmap unique-map for sm_100a: distinct ids in ascending order + rank of every input id, no host round trip.
//
// Stands in for the bitmap backend of the reference's map_tensors_unique_inverse_cuda
// (cuda/src/common/unique_map_cuda.cu:771-882 of the reference project: memset, mark, popcount, CUB scan,
// extract, inverse, two stream syncs and four scalar read-backs).  Here:
//   memset(control words + bitset)                       one cudaMemsetAsync (they are adjacent in the workspace)
//   mark_kernel        ids -> bits                       n threads, 64-bit atomicOr (red) into an L2-resident bitset
//   scan_extract_kernel popcount + exclusive scan + emit  one pass over the words; tiles chained by a
//                                                        decoupled look-back (ticketed, bounded spin)
//   inverse_kernel     rank of every input id            n threads; also hands the status word to the caller
// The scan and the inverse kernel are launched with programmatic dependent launch behind their predecessors.
// The bitset (domain/8 bytes) and the per-word offsets (domain/16 bytes) stay in the 126 MB L2 for every
// configuration of interest (12.5 M-node domain: 1.6 MB + 0.8 MB), so HBM traffic is the ids in and the two
// outputs: 16 n + 8 U bytes.
#include "common.cuh"

namespace ge2 {
namespace {

constexpr int kScanThreads = 256;
constexpr int kWordsPerThread = 4;
constexpr int kTileWords = kScanThreads * kWordsPerThread;  // 1024 words = 65536 ids per tile
constexpr uint32_t kFlagAggregate = 1u << 30;               // tile state: local sum published
constexpr uint32_t kFlagPrefix = 2u << 30;                  // tile state: inclusive prefix published
constexpr uint32_t kValueMask = (1u << 30) - 1;
constexpr int kSpinLimit = 1 << 20;                          // look-back poll budget before giving up

struct UniqueWorkspace {
    uint32_t* tile_state;       // [num_tiles]   } control words: cleared together with the bitset by one memset
    uint32_t* ticket;           // [1]           }
    int32_t* status;            // [1]           } GE2_STATUS_* bits of this call
    unsigned long long* words;  // [num_words]
    int32_t* word_offsets;      // [num_words]
};

constexpr size_t align256c(size_t x) { return (x + 255) & ~(size_t)255; }
// control words (tile states, ticket, status, one spare), bitset, per-word offsets
constexpr size_t unique_ws_bytes(int64_t domain) {
    const int64_t nw = (domain + 63) >> 6;
    const int64_t tiles = (nw + 1023) / 1024;
    return align256c((size_t)(tiles + 4) * 4) + align256c((size_t)nw * 8) + align256c((size_t)nw * 4);
}

__host__ __device__ inline int64_t num_words_of(int64_t domain) { return (domain + 63) >> 6; }

__global__ void __launch_bounds__(256) mark_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t domain,
                                                   unsigned long long* __restrict__ words, int32_t* __restrict__ status) {
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    bool bad = false;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t key = ids[i];
        if (key < 0 || key >= domain) {
            bad = true;
            continue;
        }
        atomicOr(&words[key >> 6], 1ull << (key & 63));
    }
    if (bad) atomicOr(status, GE2_STATUS_ID_OUT_OF_RANGE);
}

// One tile = 1024 consecutive words.  Tiles are handed out by an atomic ticket so a tile only ever waits for tiles
// that have already started (forward progress without co-residency assumptions); the wait is bounded anyway.
__global__ void __launch_bounds__(kScanThreads) scan_extract_kernel(const unsigned long long* __restrict__ words, int64_t num_words,
                                                                    int32_t* __restrict__ word_offsets, uint32_t* tile_state,
                                                                    uint32_t* ticket, int num_tiles, int64_t* __restrict__ out_unique,
                                                                    int64_t out_capacity, int32_t* __restrict__ out_count,
                                                                    int32_t* __restrict__ status) {
    __shared__ uint32_t s_warp_sums[kScanThreads / 32];
    __shared__ uint32_t s_tile;
    __shared__ uint32_t s_prefix;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    griddep_wait();  // the bitset comes from the marking kernel

    for (;;) {
        if (tid == 0) s_tile = atomicAdd(ticket, 1u);
        __syncthreads();
        const uint32_t tile = s_tile;
        if (tile >= (uint32_t)num_tiles) return;

        // each thread owns 4 consecutive words (one 32-byte load)
        const int64_t w0 = (int64_t)tile * kTileWords + (int64_t)tid * kWordsPerThread;
        unsigned long long w[kWordsPerThread];
        uint32_t cnt[kWordsPerThread];
        uint32_t local = 0;
#pragma unroll
        for (int k = 0; k < kWordsPerThread; k++) {
            w[k] = (w0 + k < num_words) ? words[w0 + k] : 0ull;
            cnt[k] = __popcll(w[k]);
            local += cnt[k];
        }
        // block exclusive scan of `local`
        uint32_t incl = local;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += v;
        }
        if (lane == 31) s_warp_sums[warp] = incl;
        __syncthreads();
        uint32_t warp_base = 0, tile_total = 0;
#pragma unroll
        for (int k = 0; k < kScanThreads / 32; k++) {
            uint32_t v = s_warp_sums[k];
            if (k < warp) warp_base += v;
            tile_total += v;
        }
        const uint32_t excl_in_tile = warp_base + incl - local;

        // decoupled look-back, done by warp 0 lane 0 (the chain is short: one predecessor in the common case)
        if (tid == 0) {
            uint32_t prefix = 0;
            if (tile == 0) {
                __threadfence();
                atomicExch(&tile_state[0], kFlagPrefix | tile_total);
            } else {
                atomicExch(&tile_state[tile], kFlagAggregate | tile_total);
                int64_t look = (int64_t)tile - 1;
                int spins = 0;
                bool failed = false;
                while (look >= 0) {
                    uint32_t st = *((volatile uint32_t*)&tile_state[look]);
                    uint32_t flag = st & ~kValueMask;
                    if (flag == kFlagPrefix) {
                        prefix += st & kValueMask;
                        break;
                    } else if (flag == kFlagAggregate) {
                        prefix += st & kValueMask;
                        look--;
                    } else if (++spins > kSpinLimit) {
                        failed = true;
                        break;
                    }
                }
                if (failed) atomicOr(status, GE2_STATUS_SCAN_TIMEOUT);
                __threadfence();
                atomicExch(&tile_state[tile], kFlagPrefix | ((prefix + tile_total) & kValueMask));
            }
            s_prefix = prefix;
            if (tile == (uint32_t)num_tiles - 1) out_count[0] = (int32_t)(prefix + tile_total);
        }
        __syncthreads();
        uint32_t out = s_prefix + excl_in_tile;
#pragma unroll
        for (int k = 0; k < kWordsPerThread; k++) {
            if (w0 + k < num_words) {
                word_offsets[w0 + k] = (int32_t)out;
                unsigned long long bits = w[k];
                const int64_t base = (w0 + k) << 6;
                uint32_t o = out;
                while (bits != 0ull) {
                    int b = __ffsll((long long)bits) - 1;
                    if ((int64_t)o < out_capacity) out_unique[o] = base + b;
                    o++;
                    bits &= bits - 1ull;
                }
                out += cnt[k];
            }
        }
        __syncthreads();  // s_tile / s_prefix / s_warp_sums are reused by the next ticket
    }
}

__global__ void __launch_bounds__(256) inverse_kernel(const int64_t* __restrict__ ids, int64_t n, int64_t domain,
                                                      const unsigned long long* __restrict__ words,
                                                      const int32_t* __restrict__ word_offsets, int64_t* __restrict__ inverse,
                                                      const int32_t* __restrict__ status, int32_t* __restrict__ out_status) {
    griddep_wait();  // offsets and the count come from the scan kernel
    if (blockIdx.x == 0 && threadIdx.x == 0) *out_status = *status;  // the marking and scan kernels are over: the word is final
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        int64_t key = ids[i];
        if (key < 0 || key >= domain) {
            inverse[i] = -1;
            continue;
        }
        const int64_t wi = key >> 6;
        const int bit = (int)(key & 63);
        const unsigned long long bits = __ldg(&words[wi]);
        const unsigned long long lower = (bit == 0) ? 0ull : (bits & ((1ull << bit) - 1ull));
        inverse[i] = (int64_t)__ldg(&word_offsets[wi]) + (int64_t)__popcll(lower);
    }
}

__global__ void pack_ids_kernel(const int64_t* p0, const int64_t* p1, const int64_t* p2, const int64_t* p3, int64_t l0, int64_t l1,
                                int64_t l2, int64_t l3, int64_t s0, int64_t s1, int64_t s2, int64_t s3, int64_t* __restrict__ out) {
    const int64_t total = l0 + l1 + l2 + l3;
    int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t v;
        if (i < l0) v = p0[i * s0];
        else if (i < l0 + l1) v = p1[(i - l0) * s1];
        else if (i < l0 + l1 + l2) v = p2[(i - l0 - l1) * s2];
        else v = p3[(i - l0 - l1 - l2) * s3];
        out[i] = v;
    }
}

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" size_t ge2_unique_workspace_bytes(int64_t domain) {
    if (domain <= 0) return 0;
    return unique_ws_bytes(domain);
}

extern "C" int ge2_unique_bitmap(const int64_t* ids, int64_t n, int64_t domain, void* workspace, size_t workspace_bytes,
                                 int64_t* out_unique, int64_t* out_inverse, int32_t* out_count, ge2_stream_t stream_) {
    if (n < 0 || domain <= 0 || out_count == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if (n > 0 && (ids == nullptr || out_unique == nullptr || out_inverse == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    if (n > (int64_t)kValueMask) return GE2_ERR_UNSUPPORTED;  // the reference stops at INT32_MAX ids (unique_map_cuda.cu:784); the packed tile state here holds 30 bits
    cudaStream_t stream = as_stream(stream_);
    if (n == 0) {
        GE2_CUDA_TRY(cudaMemsetAsync(out_count, 0, 2 * sizeof(int32_t), stream));
        return GE2_OK;
    }
    const int64_t nw = num_words_of(domain);
    if (nw > (int64_t)kValueMask) return GE2_ERR_UNSUPPORTED;
    const int64_t tiles = ceil_div<int64_t>(nw, kTileWords);
    if (workspace == nullptr || ((uintptr_t)workspace & 255) != 0 || workspace_bytes < ge2_unique_workspace_bytes(domain))
        return GE2_ERR_WORKSPACE;

    char* p = (char*)workspace;
    UniqueWorkspace ws;
    ws.tile_state = (uint32_t*)p;
    ws.ticket = ws.tile_state + tiles;
    ws.status = (int32_t*)(ws.tile_state + tiles + 1);
    const size_t ctl_bytes = align256c((size_t)(tiles + 4) * 4);
    p += ctl_bytes;
    ws.words = (unsigned long long*)p;
    p += align256c((size_t)nw * 8);
    ws.word_offsets = (int32_t*)p;

    // control words and bitset are adjacent: one memset; out_count needs none (the scan's last tile writes the count, the
    // inverse kernel the status)
    GE2_CUDA_TRY(cudaMemsetAsync(ws.tile_state, 0, ctl_bytes + (size_t)nw * 8, stream));

    mark_kernel<<<stream_grid(n, 256), 256, 0, stream>>>(ids, n, domain, ws.words, ws.status);
    GE2_LAUNCH_CHECK();
    const int64_t cap = n < domain ? n : domain;
    const int scan_grid = (int)(tiles < (int64_t)kNumSMs * 4 ? tiles : (int64_t)kNumSMs * 4);
    GE2_CUDA_TRY(launch_after(scan_extract_kernel, dim3((unsigned)scan_grid), dim3(kScanThreads), 0, stream, (const unsigned long long*)ws.words, nw,
                              ws.word_offsets, ws.tile_state, ws.ticket, (int)tiles, out_unique, cap, out_count, ws.status));
    GE2_CUDA_TRY(launch_after(inverse_kernel, dim3((unsigned)stream_grid(n, 256)), dim3(256), 0, stream, ids, n, domain,
                              (const unsigned long long*)ws.words, (const int32_t*)ws.word_offsets, out_inverse, (const int32_t*)ws.status,
                              out_count + 1));
    return GE2_OK;
}

extern "C" int ge2_pack_ids(const int64_t* const parts[4], const int64_t lens[4], const int64_t strides[4], int64_t* out,
                            ge2_stream_t stream_) {
    if (parts == nullptr || lens == nullptr || out == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    int64_t total = 0;
    for (int k = 0; k < 4; k++) {
        if (lens[k] < 0 || (lens[k] > 0 && parts[k] == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
        total += lens[k];
    }
    if (total == 0) return GE2_OK;
    int64_t s[4];
    for (int k = 0; k < 4; k++) s[k] = (strides != nullptr && strides[k] > 0) ? strides[k] : 1;
    pack_ids_kernel<<<stream_grid(total, 256), 256, 0, as_stream(stream_)>>>(parts[0], parts[1], parts[2], parts[3], lens[0], lens[1],
                                                                           lens[2], lens[3], s[0], s[1], s[2], s[3], out);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Allocation-free variant of the unique-map.
//
// Some callers of this library run where cudaMalloc is off limits: inside a runtime that owns all device memory and
// hands none out after start-up, in a plugin that is only ever given its input and output buffers, or on a hot path
// whose latency budget has no room for an allocator call.  For them the scratch of the unique-map (bitset, per-word
// offsets, scan tile states) lives in the array below, which is part of the library image: every GPU that loads the
// library holds these bytes until the process exits.  The size fixes the largest id domain the entry point accepts.
// ---------------------------------------------------------------------------------------------------------------
namespace ge2 {
namespace {

constexpr int64_t kStaticMaxDomain = GE2_UNIQUE_STATIC_MAX_DOMAIN;
constexpr size_t kStaticBytes = unique_ws_bytes(kStaticMaxDomain);

static __device__ __align__(256) unsigned char g_unique_static_scratch[kStaticBytes];

constexpr int kMaxDevices = 64;
void* g_static_scratch_addr[kMaxDevices] = {};  // device address of the array, per device, resolved on first use

}  // namespace
}  // namespace ge2

extern "C" int ge2_unique_bitmap_static(const int64_t* ids, int64_t n, int64_t domain, int64_t* out_unique, int64_t* out_inverse,
                                        int32_t* out_count, ge2_stream_t stream) {
    if (domain <= 0 || n < 0) return GE2_ERR_INVALID_ARGUMENT;
    if (domain > kStaticMaxDomain) return GE2_ERR_UNSUPPORTED;  // the built-in scratch is sized for GE2_UNIQUE_STATIC_MAX_DOMAIN ids
    int device = -1;
    GE2_CUDA_TRY(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return GE2_ERR_UNSUPPORTED;
    void* scratch = g_static_scratch_addr[device];
    if (scratch == nullptr) {
        // In host code the array's name is only a handle; the address a kernel can use has to be asked for, once per device,
        // with that device current (it is: cudaGetDevice above).  Not a stream operation, but do it before any stream capture.
        GE2_CUDA_TRY(cudaGetSymbolAddress(&scratch, g_unique_static_scratch));
        if (scratch == nullptr) return GE2_ERR_CUDA;
        g_static_scratch_addr[device] = scratch;
    }
    // Same kernels as ge2_unique_bitmap, which clears the parts of the scratch that must start at zero on every call.
    return ge2_unique_bitmap(ids, n, domain, scratch, kStaticBytes, out_unique, out_inverse, out_count, stream);
}
