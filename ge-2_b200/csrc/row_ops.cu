// Row-wise bandwidth kernels: gather / scatter-add of embedding rows, sparse Adagrad (batch-local and fused with the
// scatter into the resident table), dense Adagrad for the relation tables, partition-slot remap of edge endpoints,
// slab copies and the on-device negative sampler.  All are HBM-bound: each touched float is read once and written
// once, rows are contiguous (D*4 bytes), accesses are 16-byte vectors when D % 4 == 0 (8-byte for even D).
//
// Floating-point updates use explicit round-to-nearest intrinsics so no multiply-add contraction happens: the result
// is bit-identical to evaluating the reference's chain of element-wise ATen ops (cpp/src/data/batch.cpp:264-266,
// cpp/src/nn/optim.cpp:130-137 of the reference project) one IEEE operation at a time.
#include "common.cuh"

namespace ge2 {
namespace {

constexpr float kAdagradEps = 1e-10f;  // literal in cpp/src/data/batch.cpp:266 of the reference project

template <int V>
struct Vec;
template <>
struct Vec<4> {
    using type = float4;
};
template <>
struct Vec<2> {
    using type = float2;
};
template <>
struct Vec<1> {
    using type = float;
};

template <int V>
__device__ __forceinline__ void to_arr(const typename Vec<V>::type& v, float (&a)[V]);
template <>
__device__ __forceinline__ void to_arr<4>(const float4& v, float (&a)[4]) {
    a[0] = v.x; a[1] = v.y; a[2] = v.z; a[3] = v.w;
}
template <>
__device__ __forceinline__ void to_arr<2>(const float2& v, float (&a)[2]) {
    a[0] = v.x; a[1] = v.y;
}
template <>
__device__ __forceinline__ void to_arr<1>(const float& v, float (&a)[1]) {
    a[0] = v;
}
template <int V>
__device__ __forceinline__ typename Vec<V>::type from_arr(const float (&a)[V]);
template <>
__device__ __forceinline__ float4 from_arr<4>(const float (&a)[4]) {
    return make_float4(a[0], a[1], a[2], a[3]);
}
template <>
__device__ __forceinline__ float2 from_arr<2>(const float (&a)[2]) {
    return make_float2(a[0], a[1]);
}
template <>
__device__ __forceinline__ float from_arr<1>(const float (&a)[1]) {
    return a[0];
}

__device__ __forceinline__ int64_t live_rows(int64_t rows, const int32_t* rows_dev) {
    if (rows_dev == nullptr) return rows;
    int64_t r = (int64_t)__ldg(rows_dev);
    if (r < 0) r = 0;
    return r < rows ? r : rows;
}

// state += g*g ; delta = -lr * g / (sqrt(state) + eps)
__device__ __forceinline__ void adagrad_elem(float g, float& state, float& delta, float& upd, float neg_lr) {
    upd = __fmul_rn(g, g);
    state = __fadd_rn(state, upd);
    const float den = __fadd_rn(__fsqrt_rn(state), kAdagradEps);
    delta = __fmul_rn(neg_lr, __fdiv_rn(g, den));
}

template <int V>
__global__ void __launch_bounds__(256) sparse_adagrad_kernel(const float* __restrict__ grad, float* __restrict__ state, float* out_delta,
                                                             float* __restrict__ out_upd, int64_t rows, const int32_t* rows_dev, int vec_per_row,
                                                             float neg_lr) {
    using VT = typename Vec<V>::type;
    const int64_t total = live_rows(rows, rows_dev) * vec_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        float g[V], s[V], d[V], u[V];
        to_arr<V>(reinterpret_cast<const VT*>(grad)[i], g);
        to_arr<V>(reinterpret_cast<const VT*>(state)[i], s);
#pragma unroll
        for (int k = 0; k < V; k++) adagrad_elem(g[k], s[k], d[k], u[k], neg_lr);
        reinterpret_cast<VT*>(state)[i] = from_arr<V>(s);
        if (out_upd != nullptr) reinterpret_cast<VT*>(out_upd)[i] = from_arr<V>(u);
        reinterpret_cast<VT*>(out_delta)[i] = from_arr<V>(d);
    }
}

template <int V, bool kAdd>
__global__ void __launch_bounds__(256) index_rows_kernel(float* __restrict__ table, int64_t table_rows, const int64_t* __restrict__ ids,
                                                         int64_t n, const int32_t* n_dev, int vec_per_row, float* __restrict__ dense,
                                                         int32_t* status) {
    using VT = typename Vec<V>::type;
    const int64_t total = live_rows(n, n_dev) * vec_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t l = i / vec_per_row;
        const int c = (int)(i - l * vec_per_row);
        const int64_t row = __ldg(&ids[l]);
        if (row < 0 || row >= table_rows) {
            or_status(status, GE2_STATUS_BAD_INDEX);
            if (!kAdd) {  // a row outside the table reads as zeros
                float z[V];
#pragma unroll
                for (int k = 0; k < V; k++) z[k] = 0.f;
                reinterpret_cast<VT*>(dense)[i] = from_arr<V>(z);
            }
            continue;
        }
        VT* trow = reinterpret_cast<VT*>(table) + row * vec_per_row + c;
        if (kAdd) {
            float a[V], b[V];
            to_arr<V>(*trow, a);
            to_arr<V>(reinterpret_cast<const VT*>(dense)[i], b);
#pragma unroll
            for (int k = 0; k < V; k++) a[k] = __fadd_rn(a[k], b[k]);
            *trow = from_arr<V>(a);
        } else {
            reinterpret_cast<VT*>(dense)[i] = *trow;
        }
    }
}

// Fused accumulateGradients + indexAdd(embeddings) + indexAdd(state): one read-modify-write of the touched rows.
template <int V>
__global__ void __launch_bounds__(256) adagrad_scatter_kernel(float* __restrict__ table, float* __restrict__ state, int64_t table_rows,
                                                              const int64_t* __restrict__ unique_ids, int64_t U, const int32_t* U_dev,
                                                              float* __restrict__ node_grad, int vec_per_row, float neg_lr, int clear_grad,
                                                              int32_t* status) {
    using VT = typename Vec<V>::type;
    griddep_wait();  // the gradient rows come from the kernel before this one
    const int64_t total = live_rows(U, U_dev) * vec_per_row;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t l = i / vec_per_row;
        const int c = (int)(i - l * vec_per_row);
        const int64_t row = __ldg(&unique_ids[l]);
        if (row < 0 || row >= table_rows) {
            or_status(status, GE2_STATUS_BAD_INDEX);
            continue;
        }
        const int64_t off = row * vec_per_row + c;
        float g[V], s[V], e[V], d[V], u[V];
        to_arr<V>(reinterpret_cast<const VT*>(node_grad)[i], g);
        to_arr<V>(reinterpret_cast<const VT*>(state)[off], s);
        to_arr<V>(reinterpret_cast<const VT*>(table)[off], e);
#pragma unroll
        for (int k = 0; k < V; k++) {
            adagrad_elem(g[k], s[k], d[k], u[k], neg_lr);
            e[k] = __fadd_rn(e[k], d[k]);
        }
        reinterpret_cast<VT*>(state)[off] = from_arr<V>(s);
        reinterpret_cast<VT*>(table)[off] = from_arr<V>(e);
        if (clear_grad) {
            float z[V];
#pragma unroll
            for (int k = 0; k < V; k++) z[k] = 0.f;
            reinterpret_cast<VT*>(node_grad)[i] = from_arr<V>(z);
        }
    }
}

__global__ void __launch_bounds__(256) dense_adagrad_kernel(float* __restrict__ param, float* __restrict__ sum, float* __restrict__ grad,
                                                            int64_t numel, float neg_lr, float eps, float grad_scale, int clear_grad) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride) {
        float g = grad[i];
        if (grad_scale != 1.0f) g = __fmul_rn(g, grad_scale);
        const float s = __fadd_rn(sum[i], __fmul_rn(g, g));
        const float den = __fadd_rn(__fsqrt_rn(s), eps);
        sum[i] = s;
        param[i] = __fadd_rn(param[i], __fmul_rn(neg_lr, __fdiv_rn(g, den)));
        if (clear_grad) grad[i] = 0.f;
    }
}

// ---- dense Adagrad fused with the relation-gradient all-reduce over peer memory -------------------------------------
// Every rank keeps its relation gradients in a buffer its peers can read: two halves used by alternate steps, then one
// 8-byte arrival flag per rank, one 8-byte verdict word and one 8-byte wait-time counter.  Two launches per rank and step:
//   peer_arrive_kernel (one warp): announce "my gradients of step t are complete" by writing t + 1 into my slot of every
//     peer's flag row, then wait -- lane p polls peer p, bounded by a time budget -- until every peer has announced the
//     same, and publish ONE verdict for the step in this rank's verdict word (t + 1 = go, 0 = a peer never arrived);
//   dense_adagrad_peers_kernel: every block reads that verdict, so all of them either run the optimizer step on the sum
//     of the ranks' gradients (read straight from the peers over NVLink, 16 bytes at a time) and clear the half the step
//     after next will accumulate into, or all of them leave the tables and the buffer untouched.
// Why one barrier is enough: a rank announces step t + 1 only when its step-t launches are over, so whoever gets past
// the wait of step t + 1 knows that nobody reads the half of step t any more.
__device__ __forceinline__ void st_release_sys_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_sys_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

constexpr int kMaxPeers = 16;
struct PeerBuffers {
    float* buf[kMaxPeers];  // this process's mapping of every rank's gradient buffer, own rank included
};

__global__ void __launch_bounds__(32) peer_arrive_kernel(PeerBuffers peers, int world, int rank, int64_t numel,
                                                         const unsigned long long* __restrict__ step_dev, unsigned long long budget_ns,
                                                         int32_t* status) {
    const unsigned long long epoch = *step_dev + 1ull;
    const int64_t flags_off = 2 * numel;  // in floats; numel is even, so the flags are 8-byte aligned
    const int lane = threadIdx.x;
    int ok = 1;
    const unsigned long long t_enter = global_timer_ns();
    if (lane < world) {
        st_release_sys_u64(reinterpret_cast<unsigned long long*>(peers.buf[lane] + flags_off) + rank, epoch);
        const unsigned long long* mine = reinterpret_cast<const unsigned long long*>(peers.buf[rank] + flags_off) + lane;
        const unsigned long long t0 = global_timer_ns();
        ok = 0;
        // bounded twice: by the time budget and by an iteration count (should the timer not advance)
        for (uint32_t i = 0; i < (1u << 26); i++) {
            if (ld_acquire_sys_u64(mine) >= epoch) {
                ok = 1;
                break;
            }
            if ((i & 15u) == 15u && global_timer_ns() - t0 > budget_ns) break;
            __nanosleep(i < 64 ? 20 : 400);
        }
    }
    const bool all_ok = __all_sync(0xffffffffu, ok);
    const unsigned waited = __reduce_max_sync(0xffffffffu, lane < world ? (unsigned)min(global_timer_ns() - t_enter, 0xffffffffull) : 0u);
    if (lane == 0) {
        unsigned long long* verdict = reinterpret_cast<unsigned long long*>(peers.buf[rank] + flags_off) + world;
        *verdict = all_ok ? epoch : 0ull;
        verdict[1] += waited;  // diagnostic: nanoseconds this rank has spent in this kernel waiting for the slowest rank
        if (!all_ok) or_status(status, GE2_STATUS_PEER_TIMEOUT);
    }
}

template <int V>
__global__ void __launch_bounds__(256) dense_adagrad_peers_kernel(float* __restrict__ param, float* __restrict__ sum, PeerBuffers peers, int world,
                                                                  int rank, int64_t numel, const unsigned long long* __restrict__ step_dev,
                                                                  float neg_lr, float eps, float grad_scale) {
    using VT = typename Vec<V>::type;
    const unsigned long long epoch = *step_dev + 1ull;
    const int64_t flags_off = 2 * numel;
    // the one verdict of this step, written by the launch before this one on the same stream
    if (*(reinterpret_cast<const unsigned long long*>(peers.buf[rank] + flags_off) + world) != epoch) return;
    const int64_t cur = (int64_t)((epoch - 1ull) & 1ull) * numel;  // half holding this step's gradients
    const int64_t other = numel - cur;                            // half to clear for the step after next
    const int64_t nv = numel / V;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nv; i += stride) {
        float g[V], t[V], sm[V], pr[V], z[V];
#pragma unroll
        for (int k = 0; k < V; k++) g[k] = 0.f, z[k] = 0.f;
        for (int p = 0; p < world; p++) {  // volatile-style load: never a stale cached copy of peer memory
            to_arr<V>(__ldcv(reinterpret_cast<const VT*>(peers.buf[p] + cur) + i), t);
#pragma unroll
            for (int k = 0; k < V; k++) g[k] += t[k];
        }
        to_arr<V>(reinterpret_cast<const VT*>(sum)[i], sm);
        to_arr<V>(reinterpret_cast<const VT*>(param)[i], pr);
#pragma unroll
        for (int k = 0; k < V; k++) {
            const float gk = __fmul_rn(g[k], grad_scale);
            sm[k] = __fadd_rn(sm[k], __fmul_rn(gk, gk));
            const float den = __fadd_rn(__fsqrt_rn(sm[k]), eps);
            pr[k] = __fadd_rn(pr[k], __fmul_rn(neg_lr, __fdiv_rn(gk, den)));
        }
        reinterpret_cast<VT*>(sum)[i] = from_arr<V>(sm);
        reinterpret_cast<VT*>(param)[i] = from_arr<V>(pr);
        reinterpret_cast<VT*>(peers.buf[rank] + other)[i] = from_arr<V>(z);
    }
}

__global__ void __launch_bounds__(256) remap_edges_kernel(const int64_t* __restrict__ edges, int64_t n, int cols,
                                                          const int64_t* __restrict__ part_to_slot, int num_partitions,
                                                          int64_t partition_size, int64_t* __restrict__ out, int32_t* status) {
    const int64_t total = n * cols;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int c = (int)(i % cols);
        int64_t v = edges[i];
        if (c == 0 || c == cols - 1) {
            const int64_t part = v / partition_size;  // ids are non-negative: same as the reference's floor of a double division
            int64_t slot = -1;
            if (v >= 0 && part < num_partitions) slot = __ldg(&part_to_slot[part]);
            if (slot < 0) {
                or_status(status, GE2_STATUS_BAD_INDEX);
                v = -1;
            } else {
                v = slot * partition_size + (v - part * partition_size);
            }
        }
        out[i] = v;
    }
}

struct SlabMoves {
    int32_t src[16];
    int32_t dst[16];
    int32_t count;
};

__global__ void __launch_bounds__(256) copy_slabs_kernel(const float4* __restrict__ src, float4* __restrict__ dst, SlabMoves moves,
                                                         int64_t slab_vec4) {
    const int m = blockIdx.y;
    const float4* s = src + (int64_t)moves.src[m] * slab_vec4;
    float4* d = dst + (int64_t)moves.dst[m] * slab_vec4;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < slab_vec4; i += stride) d[i] = s[i];
}

__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

__global__ void __launch_bounds__(256) sample_negatives_kernel(const int64_t* __restrict__ src_ids, const int64_t* __restrict__ dst_ids,
                                                               int64_t edge_stride, int B, int C, int N, int n_deg, int64_t domain,
                                                               int want_src, uint64_t key, int64_t* __restrict__ packed,
                                                               int64_t* __restrict__ deg_rows, const uint64_t* __restrict__ step_dev,
                                                               int64_t num_batches, const int64_t* __restrict__ rel_ids,
                                                               int64_t* __restrict__ out_rel, const int64_t* __restrict__ num_batches_dev) {
    // graph-replay form: the batch index lives on the device, so the same launch serves every batch of the epoch
    if (step_dev != nullptr) {
        const uint64_t step = *step_dev;
        if (num_batches_dev != nullptr) {  // ... and so does the length of the resident edge list
            num_batches = *num_batches_dev;
            if (num_batches < 1) num_batches = 1;
        }
        const int64_t off = (int64_t)(step % (uint64_t)num_batches) * B * edge_stride;
        src_ids += off;
        dst_ids += off;
        if (rel_ids != nullptr) rel_ids += off;
        key += step * 0x9E3779B97F4A7C15ull;
    }
    const int64_t CN = (int64_t)C * N;
    const int64_t total = 2 * (int64_t)B + CN;
    int64_t* out_src_neg = packed + 2 * (int64_t)B;
    int64_t* out_dst_neg = out_src_neg + (want_src ? CN : 0);
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        if (i < B) {
            packed[i] = src_ids[i * edge_stride];
            if (out_rel != nullptr) out_rel[i] = rel_ids[i * edge_stride];
        } else if (i < 2 * (int64_t)B) {
            packed[i] = dst_ids[(i - B) * edge_stride];
        } else {
            const int64_t e = i - 2 * (int64_t)B;
            const int c = (int)(e / N);
            const int j = (int)(e - (int64_t)c * N);
            const uint64_t r = splitmix64(key ^ splitmix64((uint64_t)e));
            if (j < n_deg) {
                const int64_t row = (int64_t)__umul64hi(r, (uint64_t)B);
                if (deg_rows != nullptr) deg_rows[(int64_t)c * n_deg + j] = row;
                out_dst_neg[e] = dst_ids[row * edge_stride];
                if (want_src) out_src_neg[e] = src_ids[row * edge_stride];
            } else {
                const int64_t id = (int64_t)__umul64hi(r, (uint64_t)domain);
                out_dst_neg[e] = id;
                if (want_src) out_src_neg[e] = id;
            }
        }
    }
}

inline int vec_width(int D, const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
    uintptr_t bits = (uintptr_t)a | (uintptr_t)b | (uintptr_t)c | (uintptr_t)d;
    if (D % 4 == 0 && (bits & 15) == 0) return 4;
    if (D % 2 == 0 && (bits & 7) == 0) return 2;
    return 1;
}

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" int ge2_sparse_adagrad(const float* grad, float* state_local, float* out_delta, float* out_state_update, int64_t rows,
                                  const int32_t* rows_dev, int32_t D, float lr, ge2_stream_t stream_) {
    if (rows < 0 || D <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (rows == 0) return GE2_OK;
    if (grad == nullptr || state_local == nullptr || out_delta == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = as_stream(stream_);
    const int V = vec_width(D, grad, state_local, out_delta, out_state_update);
    const int grid = stream_grid(rows * (D / V), 256);
    if (V == 4) sparse_adagrad_kernel<4><<<grid, 256, 0, stream>>>(grad, state_local, out_delta, out_state_update, rows, rows_dev, D / 4, -lr);
    else if (V == 2) sparse_adagrad_kernel<2><<<grid, 256, 0, stream>>>(grad, state_local, out_delta, out_state_update, rows, rows_dev, D / 2, -lr);
    else sparse_adagrad_kernel<1><<<grid, 256, 0, stream>>>(grad, state_local, out_delta, out_state_update, rows, rows_dev, D, -lr);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

template <bool kAdd>
static int index_rows(float* table, int64_t table_rows, const int64_t* ids, int64_t n, const int32_t* n_dev, int32_t D, float* dense,
                      int32_t* status, ge2_stream_t stream_) {
    if (n < 0 || D <= 0 || table_rows < 0) return GE2_ERR_INVALID_ARGUMENT;
    if (n == 0) return GE2_OK;
    if (table == nullptr || ids == nullptr || dense == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = as_stream(stream_);
    const int V = vec_width(D, table, dense);
    const int grid = stream_grid(n * (D / V), 256);
    if (V == 4) index_rows_kernel<4, kAdd><<<grid, 256, 0, stream>>>(table, table_rows, ids, n, n_dev, D / 4, dense, status);
    else if (V == 2) index_rows_kernel<2, kAdd><<<grid, 256, 0, stream>>>(table, table_rows, ids, n, n_dev, D / 2, dense, status);
    else index_rows_kernel<1, kAdd><<<grid, 256, 0, stream>>>(table, table_rows, ids, n, n_dev, D, dense, status);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_index_read(const float* table, int64_t table_rows, const int64_t* ids, int64_t n, const int32_t* n_dev, int32_t D,
                              float* out, int32_t* status, ge2_stream_t stream) {
    return index_rows<false>(const_cast<float*>(table), table_rows, ids, n, n_dev, D, out, status, stream);
}

extern "C" int ge2_index_add(float* table, int64_t table_rows, const int64_t* ids, int64_t n, const int32_t* n_dev, int32_t D,
                             const float* values, int32_t* status, ge2_stream_t stream) {
    return index_rows<true>(table, table_rows, ids, n, n_dev, D, const_cast<float*>(values), status, stream);
}

extern "C" int ge2_adagrad_scatter(float* table, float* state, int64_t table_rows, const int64_t* unique_ids, int64_t U,
                                   const int32_t* U_dev, float* node_grad, int32_t D, float lr, int32_t clear_grad, int32_t* status,
                                   ge2_stream_t stream_) {
    if (U < 0 || D <= 0 || table_rows < 0) return GE2_ERR_INVALID_ARGUMENT;
    if (U == 0) return GE2_OK;
    if (table == nullptr || state == nullptr || unique_ids == nullptr || node_grad == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    cudaStream_t stream = as_stream(stream_);
    const int V = vec_width(D, table, state, node_grad);
    const int grid = stream_grid(U * (D / V), 256);
    const dim3 g((unsigned)grid), b(256);
    if (V == 4) GE2_CUDA_TRY(launch_after(adagrad_scatter_kernel<4>, g, b, 0, stream, table, state, table_rows, unique_ids, U, U_dev, node_grad, D / 4, -lr, clear_grad, status));
    else if (V == 2) GE2_CUDA_TRY(launch_after(adagrad_scatter_kernel<2>, g, b, 0, stream, table, state, table_rows, unique_ids, U, U_dev, node_grad, D / 2, -lr, clear_grad, status));
    else GE2_CUDA_TRY(launch_after(adagrad_scatter_kernel<1>, g, b, 0, stream, table, state, table_rows, unique_ids, U, U_dev, node_grad, D, -lr, clear_grad, status));
    return GE2_OK;
}

extern "C" int ge2_dense_adagrad(float* param, float* sum_state, float* grad, int64_t numel, float lr, float eps, float grad_scale,
                                 int32_t clear_grad, ge2_stream_t stream_) {
    if (numel < 0) return GE2_ERR_INVALID_ARGUMENT;
    if (numel == 0) return GE2_OK;
    if (param == nullptr || sum_state == nullptr || grad == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    dense_adagrad_kernel<<<stream_grid(numel, 256), 256, 0, as_stream(stream_)>>>(param, sum_state, grad, numel, -lr, eps, grad_scale, clear_grad);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_dense_adagrad_peers(float* param, float* sum_state, float* const* peer_bufs, int32_t world, int32_t rank, int64_t numel,
                                       const uint64_t* step_dev, float lr, float eps, float grad_scale, uint32_t wait_budget_us, int32_t* status,
                                       ge2_stream_t stream_) {
    if (numel <= 0 || (numel & 1) || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) return GE2_ERR_INVALID_ARGUMENT;
    if (param == nullptr || sum_state == nullptr || peer_bufs == nullptr || step_dev == nullptr || status == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    PeerBuffers pb;
    for (int p = 0; p < kMaxPeers; p++) pb.buf[p] = p < world ? peer_bufs[p] : nullptr;
    for (int p = 0; p < world; p++)
        if (pb.buf[p] == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    const unsigned long long budget_ns = (wait_budget_us == 0 ? 4000000ull : (unsigned long long)wait_budget_us) * 1000ull;
    cudaStream_t stream = as_stream(stream_);
    const unsigned long long* step = reinterpret_cast<const unsigned long long*>(step_dev);
    peer_arrive_kernel<<<1, 32, 0, stream>>>(pb, world, rank, numel, step, budget_ns, status);
    GE2_LAUNCH_CHECK();
    uintptr_t bits = (uintptr_t)param | (uintptr_t)sum_state;
    for (int p = 0; p < world; p++) bits |= (uintptr_t)pb.buf[p];
    if (numel % 4 == 0 && (bits & 15) == 0)
        dense_adagrad_peers_kernel<4><<<stream_grid(numel / 4, 256), 256, 0, stream>>>(param, sum_state, pb, world, rank, numel, step, -lr, eps, grad_scale);
    else
        dense_adagrad_peers_kernel<1><<<stream_grid(numel, 256), 256, 0, stream>>>(param, sum_state, pb, world, rank, numel, step, -lr, eps, grad_scale);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_enable_peer_access(int32_t peer_device) {
    int dev = 0;
    GE2_CUDA_TRY(cudaGetDevice(&dev));
    if (peer_device == dev) return GE2_OK;
    int can = 0;
    GE2_CUDA_TRY(cudaDeviceCanAccessPeer(&can, dev, peer_device));
    if (!can) return GE2_ERR_INVALID_ARGUMENT;
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return GE2_OK;
    }
    GE2_CUDA_TRY(e);
    return GE2_OK;
}

extern "C" int ge2_sample_negatives(const int64_t* src_ids, const int64_t* dst_ids, int64_t edge_stride, int32_t B, int32_t C, int32_t N,
                                    int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed, uint64_t batch_index,
                                    int64_t* out_packed_ids, int64_t* out_deg_rows, ge2_stream_t stream_) {
    if (B <= 0 || C <= 0 || N <= 0 || n_deg < 0 || n_deg > N || domain <= 0 || edge_stride <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (src_ids == nullptr || dst_ids == nullptr || out_packed_ids == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if (n_deg > 0 && out_deg_rows == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    const int64_t total = 2 * (int64_t)B + (int64_t)C * N;
    const uint64_t key = seed * 0xD1342543DE82EF95ull + batch_index * 0x9E3779B97F4A7C15ull + 0x632BE59BD9B4E019ull;
    sample_negatives_kernel<<<stream_grid(total, 256), 256, 0, as_stream(stream_)>>>(src_ids, dst_ids, edge_stride, B, C, N, n_deg, domain,
                                                                                   want_src_negs, key, out_packed_ids, out_deg_rows, nullptr, 1,
                                                                                   nullptr, nullptr, nullptr);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

static int sample_batch_impl(const int64_t* edges, int32_t cols, int64_t num_batches, const int64_t* num_batches_dev, const uint64_t* step_dev,
                             int32_t B, int32_t C, int32_t N, int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed,
                             int64_t* out_packed_ids, int64_t* out_deg_rows, int64_t* out_rel_ids, ge2_stream_t stream_) {
    if (B <= 0 || C <= 0 || N <= 0 || n_deg < 0 || n_deg > N || domain <= 0 || num_batches <= 0 || (cols != 2 && cols != 3))
        return GE2_ERR_INVALID_ARGUMENT;
    if (edges == nullptr || step_dev == nullptr || out_packed_ids == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if ((n_deg > 0 && out_deg_rows == nullptr) || (cols == 3 && out_rel_ids == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    const int64_t total = 2 * (int64_t)B + (int64_t)C * N;
    const uint64_t key = seed * 0xD1342543DE82EF95ull + 0x632BE59BD9B4E019ull;
    sample_negatives_kernel<<<stream_grid(total, 256), 256, 0, as_stream(stream_)>>>(
        edges, edges + cols - 1, cols, B, C, N, n_deg, domain, want_src_negs, key, out_packed_ids, out_deg_rows, step_dev, num_batches,
        cols == 3 ? edges + 1 : nullptr, cols == 3 ? out_rel_ids : nullptr, num_batches_dev);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_sample_batch(const int64_t* edges, int32_t cols, int64_t num_batches, const uint64_t* step_dev, int32_t B, int32_t C,
                                int32_t N, int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed, int64_t* out_packed_ids,
                                int64_t* out_deg_rows, int64_t* out_rel_ids, ge2_stream_t stream) {
    return sample_batch_impl(edges, cols, num_batches, nullptr, step_dev, B, C, N, n_deg, domain, want_src_negs, seed, out_packed_ids,
                             out_deg_rows, out_rel_ids, stream);
}

extern "C" int ge2_sample_batch_dev(const int64_t* edges, int32_t cols, const int64_t* num_batches_dev, const uint64_t* step_dev, int32_t B,
                                    int32_t C, int32_t N, int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed,
                                    int64_t* out_packed_ids, int64_t* out_deg_rows, int64_t* out_rel_ids, ge2_stream_t stream) {
    if (num_batches_dev == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    return sample_batch_impl(edges, cols, 1, num_batches_dev, step_dev, B, C, N, n_deg, domain, want_src_negs, seed, out_packed_ids,
                             out_deg_rows, out_rel_ids, stream);
}

__global__ void advance_step_kernel(uint64_t* step, int n) {
    if ((int)threadIdx.x < n) step[threadIdx.x] += 1;
}

extern "C" int ge2_advance_step(uint64_t* step_dev, int32_t n, ge2_stream_t stream_) {
    if (step_dev == nullptr || n < 1 || n > 32) return GE2_ERR_INVALID_ARGUMENT;
    advance_step_kernel<<<1, 32, 0, as_stream(stream_)>>>(step_dev, n);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_remap_edges_to_slots(const int64_t* edges, int64_t n, int32_t cols, const int64_t* partition_to_slot,
                                        int32_t num_partitions, int64_t partition_size, int64_t* out, int32_t* status,
                                        ge2_stream_t stream_) {
    if (n < 0 || (cols != 2 && cols != 3) || num_partitions <= 0 || partition_size <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (n == 0) return GE2_OK;
    if (edges == nullptr || partition_to_slot == nullptr || out == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    remap_edges_kernel<<<stream_grid(n * cols, 256), 256, 0, as_stream(stream_)>>>(edges, n, cols, partition_to_slot, num_partitions,
                                                                                 partition_size, out, status);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}

extern "C" int ge2_copy_slabs(const float* src, float* dst, const int32_t* moves_host, int32_t num_moves, int64_t slab_floats,
                              ge2_stream_t stream_) {
    if (num_moves < 0 || num_moves > 16 || slab_floats < 0) return GE2_ERR_INVALID_ARGUMENT;
    if (num_moves == 0 || slab_floats == 0) return GE2_OK;
    if (src == nullptr || dst == nullptr || moves_host == nullptr) return GE2_ERR_INVALID_ARGUMENT;
    if ((slab_floats & 3) != 0 || (((uintptr_t)src | (uintptr_t)dst) & 15) != 0) return GE2_ERR_UNSUPPORTED;
    SlabMoves mv;
    mv.count = num_moves;
    for (int k = 0; k < num_moves; k++) {
        mv.src[k] = moves_host[2 * k];
        mv.dst[k] = moves_host[2 * k + 1];
        if (mv.src[k] < 0 || mv.dst[k] < 0) return GE2_ERR_INVALID_ARGUMENT;
    }
    const int64_t v4 = slab_floats / 4;
    dim3 grid((unsigned)stream_grid(v4, 256 * 4, 8), (unsigned)num_moves);
    copy_slabs_kernel<<<grid, 256, 0, as_stream(stream_)>>>(reinterpret_cast<const float4*>(src), reinterpret_cast<float4*>(dst), mv, v4);
    GE2_LAUNCH_CHECK();
    return GE2_OK;
}
