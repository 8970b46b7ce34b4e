// Link-prediction evaluation: the rank of every test edge among ALL candidate nodes, both corruption sides, with the
// reference's filter semantics (a filtered score is replaced by -1e9 before the comparison).
//
// Follows, in the reference project (paths relative to gege/src/cpp/src):
//   scores   nn/decoders/edge/decoder_methods.cpp:597-659 (node_corrupt_forward: relation-adjusted source against the
//            destination and against every negative; the inverse relation applied to the destination against the sources),
//            relation operators nn/decoders/edge/relation_operators.cpp:3-31
//   filter   data/samplers/negative.cpp:421-575 (pairs (edge row, negative column) whose score becomes -1e9);
//            filtered evaluation uses one chunk holding every node (negative.cpp:585-589)
//   ranks    reporting/reporting.cpp:52-54: rank = #(negative score >= positive score) + 1
//
// The [B x nodes] score matrix is never stored: a CTA keeps 64 query rows in shared memory, streams tiles of 64 node rows
// and counts.  Every score -- the positive's, a tile entry's, a filter pair's -- is the same chain
// acc = fma(q[d], e[d], acc), d ascending, so that "the candidate is the positive's own node" compares equal and the
// correction for a filter pair undoes exactly what the tile pass counted.  fp32 on the CUDA cores: ranks are integers
// decided by comparisons of nearly equal scores, which 11-bit operands would flip.
#include "common.cuh"

namespace ge2 {
namespace {

constexpr int kTileQ = 64, kTileN = 64, kChunk = 32, kEvalThreads = 256;
constexpr int kMaxD = 128;

struct EvalArgs {
    ge2_eval_desc d;
    float* Q;                     // [S][Bp][D] relation-adjusted query rows
    float* pos;                   // [S][Bp]
    unsigned long long* hash;     // open-addressing set of filter pairs already applied (keys are pair + 1, 0 = empty)
    int64_t hash_slots;           // power of two
    int64_t Bp;
    int S;
};

__device__ __forceinline__ const float* node_row(const ge2_eval_desc& d, int64_t col) {
    const int64_t id = d.neg_ids != nullptr ? d.neg_ids[col] : col;
    if (id < 0 || id >= d.num_nodes) return nullptr;
    return d.node_emb + id * d.emb_stride;
}

// One thread per (side, edge): the query row, the positive score, rank = 1.
__global__ void __launch_bounds__(128) eval_prep_kernel(EvalArgs a) {
    const ge2_eval_desc& d = a.d;
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w >= (int64_t)a.S * a.Bp) return;
    const int s = (int)(w / a.Bp);
    const int64_t i = w - (int64_t)s * a.Bp;
    float* q = a.Q + w * d.D;
    const int D = d.D, h = D / 2;
    bool ok = i < d.B;
    int64_t sid = 0, did = 0, rid = 0;
    if (ok) {
        sid = d.src_ids[i * d.edge_stride];
        did = d.dst_ids[i * d.edge_stride];
        ok = sid >= 0 && sid < d.num_nodes && did >= 0 && did < d.num_nodes;
        if (d.has_relations) {
            rid = d.rel_ids[i * d.rel_stride];
            ok = ok && rid >= 0 && rid < d.R;
        }
        if (!ok) or_status(d.status, GE2_STATUS_BAD_INDEX);
    }
    if (!ok) {
        for (int k = 0; k < D; k++) q[k] = 0.f;
        a.pos[w] = 0.f;
        if (i < d.B) (s == 0 ? d.dst_ranks : d.src_ranks)[i] = 0;  // no rank for a row with bad ids
        return;
    }
    const float* ea = d.node_emb + (s == 0 ? sid : did) * d.emb_stride;  // the endpoint the relation is applied to
    const float* eb = d.node_emb + (s == 0 ? did : sid) * d.emb_stride;  // the endpoint it is compared with
    const float* r = d.has_relations ? (s == 0 ? d.rel : d.inv_rel) + rid * D : nullptr;
    float acc = 0.f;
    for (int k = 0; k < D; k++) {
        float v;
        if (r == nullptr) {
            v = ea[k];
        } else if (d.decoder == GE2_DECODER_DISTMULT) {
            v = __fmul_rn(ea[k], r[k]);
        } else {  // complex product, columns [0, h) real and [h, D) imaginary; separate roundings as the reference's tensor ops
            const int kp = k < h ? k + h : k - h;
            v = k < h ? __fsub_rn(__fmul_rn(ea[k], r[k]), __fmul_rn(ea[kp], r[kp]))
                      : __fadd_rn(__fmul_rn(ea[kp], r[k]), __fmul_rn(ea[k], r[kp]));
        }
        q[k] = v;
        acc = __fmaf_rn(v, eb[k], acc);
    }
    a.pos[w] = acc;
    (s == 0 ? d.dst_ranks : d.src_ranks)[i] = 1;
    float* out = s == 0 ? d.pos_scores : d.inv_pos_scores;
    if (out != nullptr) out[i] = acc;
}

// grid: x = query tiles, y = shares of the node tiles, z = side.  256 threads as 16 x 16, each 4 query rows x 4 nodes.
__global__ void __launch_bounds__(kEvalThreads) eval_count_kernel(EvalArgs a, int64_t num_cols) {
    __shared__ float Qt[kMaxD][kTileQ];            // the CTA's query rows, transposed: Qt[d][row]
    __shared__ float Et[kChunk][kTileN + 4];       // a chunk of the node tile, transposed: Et[d][node]
    __shared__ float pos_s[kTileQ];
    const ge2_eval_desc& d = a.d;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int s = blockIdx.z, D = d.D;
    const int64_t q0 = (int64_t)blockIdx.x * kTileQ;
    const float* Q = a.Q + ((int64_t)s * a.Bp + q0) * D;
    for (int k = tid; k < kTileQ * D; k += kEvalThreads) {
        const int row = k / D, c = k - row * D;
        Qt[c][row] = Q[k];  // rows past B were written as zeros by the prep kernel (Bp is a multiple of the tile)
    }
    if (tid < kTileQ) pos_s[tid] = a.pos[(int64_t)s * a.Bp + q0 + tid];
    __syncthreads();
    float pos[4];
#pragma unroll
    for (int i = 0; i < 4; i++) pos[i] = pos_s[ty * 4 + i];
    unsigned cnt[4] = {0u, 0u, 0u, 0u};
    const int64_t tiles = ceil_div<int64_t>(num_cols, kTileN);
    for (int64_t t = blockIdx.y; t < tiles; t += gridDim.y) {
        const int64_t n0 = t * kTileN;
        float acc[4][4];
#pragma unroll
        for (int i = 0; i < 4; i++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
        for (int c0 = 0; c0 < D; c0 += kChunk) {
            // 64 nodes x 32 columns: a thread loads 8 consecutive columns of one node row (two 16-byte pieces when aligned)
            {
                const int node = tid >> 2, cc = (tid & 3) * 8;
                const int64_t col = n0 + node;
                const float* row = col < num_cols ? node_row(d, col) : nullptr;
#pragma unroll
                for (int k = 0; k < 8; k++) {
                    const int c = c0 + cc + k;
                    Et[cc + k][node] = (row != nullptr && c < D) ? __ldg(row + c) : 0.f;
                }
            }
            __syncthreads();
            const int kmax = D - c0 < kChunk ? D - c0 : kChunk;
            for (int k = 0; k < kmax; k++) {
                const float4 qa = *reinterpret_cast<const float4*>(&Qt[c0 + k][ty * 4]);
                const float4 eb = *reinterpret_cast<const float4*>(&Et[k][tx * 4]);
                const float qv[4] = {qa.x, qa.y, qa.z, qa.w}, ev[4] = {eb.x, eb.y, eb.z, eb.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = __fmaf_rn(qv[i], ev[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t col = n0 + tx * 4 + j;
            if (col >= num_cols) continue;
            // a candidate id outside the table scores 0 (its row was read as zeros); the prep of the filter flags it
#pragma unroll
            for (int i = 0; i < 4; i++) cnt[i] += acc[i][j] >= pos[i] ? 1u : 0u;
        }
    }
    // the 16 threads that share ty sit in one half-warp
#pragma unroll
    for (int i = 0; i < 4; i++) {
        unsigned v = cnt[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        const int64_t row = q0 + ty * 4 + i;
        if (tx == 0 && v != 0u && row < d.B) {
            int64_t* ranks = s == 0 ? d.dst_ranks : d.src_ranks;
            if (ranks[row] != 0) atomicAdd(reinterpret_cast<unsigned long long*>(ranks + row), (unsigned long long)v);
        }
    }
}

// One thread per filter pair (edge row, candidate column): the first thread to enter the pair into the set undoes what the
// count pass did for it and counts the replacement score -1e9 instead (duplicates of a pair change nothing, like index_put_).
__global__ void __launch_bounds__(256) eval_filter_kernel(EvalArgs a, int s, const int64_t* __restrict__ pairs, int64_t n_pairs, int64_t num_cols) {
    const ge2_eval_desc& d = a.d;
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= n_pairs) return;
    const int64_t i = pairs[2 * p], col = pairs[2 * p + 1];
    if (i < 0 || i >= d.B || col < 0 || col >= num_cols) {
        or_status(d.status, GE2_STATUS_BAD_INDEX);
        return;
    }
    int64_t* ranks = s == 0 ? d.dst_ranks : d.src_ranks;
    if (ranks[i] == 0) return;  // row with bad ids
    const unsigned long long key = ((unsigned long long)s << 62) + (unsigned long long)i * (unsigned long long)num_cols + (unsigned long long)col + 1ull;
    unsigned long long slot = (key * 0x9E3779B97F4A7C15ull) >> 20;
    bool first = false, placed = false;
    for (int64_t probe = 0; probe < a.hash_slots; probe++) {
        slot &= (unsigned long long)(a.hash_slots - 1);
        const unsigned long long old = atomicCAS(&a.hash[slot], 0ull, key);
        if (old == 0ull) {
            first = placed = true;
            break;
        }
        if (old == key) {
            placed = true;
            break;
        }
        slot++;
    }
    if (!placed) or_status(d.status, GE2_STATUS_FILTER_COLLISION);  // cannot happen: the set has twice as many slots as pairs
    if (!first) return;
    const float* q = a.Q + ((int64_t)s * a.Bp + i) * d.D;
    const float* e = node_row(d, col);
    float acc = 0.f;
    if (e != nullptr)
        for (int k = 0; k < d.D; k++) acc = __fmaf_rn(q[k], __ldg(e + k), acc);
    const float pos = a.pos[(int64_t)s * a.Bp + i];
    long long delta = 0;
    if (acc >= pos) delta -= 1;
    if (-1e9f >= pos) delta += 1;
    if (delta != 0) atomicAdd(reinterpret_cast<unsigned long long*>(ranks + i), (unsigned long long)delta);
}

int64_t hash_slots_for(int64_t pairs) {
    int64_t s = 64;
    while (s < 2 * pairs) s <<= 1;
    return s;
}

size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

int sides_of(const ge2_eval_desc* d) { return (d->has_relations && d->use_inverse) ? 2 : 1; }

}  // namespace
}  // namespace ge2

using namespace ge2;

extern "C" size_t ge2_eval_workspace_bytes(const ge2_eval_desc* d) {
    if (d == nullptr || d->B <= 0 || d->D <= 0) return 0;
    const int S = sides_of(d);
    const int64_t Bp = round_up<int64_t>(d->B, kTileQ);
    const int64_t pairs = (d->dst_filter_n > 0 ? d->dst_filter_n : 0) + (d->src_filter_n > 0 ? d->src_filter_n : 0);
    return align256((size_t)S * Bp * d->D * 4) + align256((size_t)S * Bp * 4) + align256((size_t)hash_slots_for(pairs) * 8);
}

extern "C" int ge2_eval_ranks(const ge2_eval_desc* d, ge2_stream_t stream_) {
    if (d == nullptr || d->B <= 0 || d->num_nodes <= 0 || d->D <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (d->D > kMaxD) return GE2_ERR_UNSUPPORTED;
    if (d->decoder != GE2_DECODER_DISTMULT && d->decoder != GE2_DECODER_COMPLEX) return GE2_ERR_INVALID_ARGUMENT;
    if (d->decoder == GE2_DECODER_COMPLEX && d->has_relations && (d->D & 1)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->node_emb == nullptr || d->src_ids == nullptr || d->dst_ids == nullptr || d->dst_ranks == nullptr || d->edge_stride <= 0 ||
        d->emb_stride < d->D)
        return GE2_ERR_INVALID_ARGUMENT;
    if (d->has_relations && (d->rel_ids == nullptr || d->rel == nullptr || d->R <= 0 || d->rel_stride <= 0)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->use_inverse && !d->has_relations) return GE2_ERR_INVALID_ARGUMENT;
    const int S = sides_of(d);
    if (S == 2 && (d->inv_rel == nullptr || d->src_ranks == nullptr)) return GE2_ERR_INVALID_ARGUMENT;
    if (d->dst_filter_n < 0 || d->src_filter_n < 0 || (d->dst_filter_n > 0 && d->dst_filter == nullptr) ||
        (d->src_filter_n > 0 && (d->src_filter == nullptr || S != 2)))
        return GE2_ERR_INVALID_ARGUMENT;
    const int64_t num_cols = d->neg_ids != nullptr ? d->num_negs : d->num_nodes;
    if (num_cols <= 0) return GE2_ERR_INVALID_ARGUMENT;
    if (d->workspace == nullptr || ((uintptr_t)d->workspace & 255) != 0 || d->workspace_bytes < ge2_eval_workspace_bytes(d)) return GE2_ERR_WORKSPACE;

    cudaStream_t stream = as_stream(stream_);
    EvalArgs a;
    a.d = *d;
    a.S = S;
    a.Bp = round_up<int64_t>(d->B, kTileQ);
    char* p = (char*)d->workspace;
    a.Q = (float*)p;
    p += align256((size_t)S * a.Bp * d->D * 4);
    a.pos = (float*)p;
    p += align256((size_t)S * a.Bp * 4);
    a.hash = (unsigned long long*)p;
    a.hash_slots = hash_slots_for(d->dst_filter_n + d->src_filter_n);
    if (d->dst_filter_n + d->src_filter_n > 0) GE2_CUDA_TRY(cudaMemsetAsync(a.hash, 0, (size_t)a.hash_slots * 8, stream));

    eval_prep_kernel<<<(unsigned)ceil_div<int64_t>((int64_t)S * a.Bp, 128), 128, 0, stream>>>(a);
    GE2_LAUNCH_CHECK();
    const int64_t q_tiles = a.Bp / kTileQ, n_tiles = ceil_div<int64_t>(num_cols, kTileN);
    int64_t shares = ceil_div<int64_t>((int64_t)kNumSMs * 4, q_tiles * S);  // about four CTAs per SM over the whole grid
    if (shares > n_tiles) shares = n_tiles;
    if (shares > 65535) shares = 65535;
    if (q_tiles > 0x7fffffffLL) return GE2_ERR_UNSUPPORTED;
    dim3 grid((unsigned)q_tiles, (unsigned)shares, (unsigned)S);
    eval_count_kernel<<<grid, kEvalThreads, 0, stream>>>(a, num_cols);
    GE2_LAUNCH_CHECK();
    if (d->dst_filter_n > 0) {
        eval_filter_kernel<<<(unsigned)ceil_div<int64_t>(d->dst_filter_n, 256), 256, 0, stream>>>(a, 0, d->dst_filter, d->dst_filter_n, num_cols);
        GE2_LAUNCH_CHECK();
    }
    if (d->src_filter_n > 0) {
        eval_filter_kernel<<<(unsigned)ceil_div<int64_t>(d->src_filter_n, 256), 256, 0, stream>>>(a, 1, d->src_filter, d->src_filter_n, num_cols);
        GE2_LAUNCH_CHECK();
    }
    return GE2_OK;
}
