/*
 * ge2_b200 -- C ABI of the B200 (sm_100a) per-batch embedding-training path.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as void*, a cudaStream_t)
 * and returns an int status (GE2_OK == 0).  Nothing here allocates, synchronises the stream or touches the
 * host except where a function says so; scratch memory is passed in by the caller and sized by the matching
 * *_workspace_bytes function.  Counts that only exist on the device (the number of unique ids of a batch)
 * stay on the device: consumers take a pointer to them.
 *
 * Each declaration names the interface of the reference project (paths relative to gege/src/) that it
 * stands in for.
 */
#ifndef GE2_B200_H_
#define GE2_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define GE2_API __attribute__((visibility("default")))
#else
#define GE2_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes ------------------------------------------------------------------------------- */
#define GE2_OK 0
#define GE2_ERR_INVALID_ARGUMENT 1 /* null pointer, negative size, unsupported shape               */
#define GE2_ERR_CUDA 2             /* a CUDA runtime call failed; ge2_last_cuda_error() has the code */
#define GE2_ERR_WORKSPACE 3        /* workspace pointer null / too small / misaligned               */
#define GE2_ERR_UNSUPPORTED 4      /* valid request outside what the kernels cover (e.g. D > 128)   */
#define GE2_ERR_NO_DEVICE 5        /* no CUDA device, or not compute capability 10.x               */

/* Bits of the device-side status word (int32) kernels OR into when the data itself is bad. */
#define GE2_STATUS_ID_OUT_OF_RANGE 1  /* unique-map: id < 0 or >= domain (reference: fallback to sort backend) */
#define GE2_STATUS_SCAN_TIMEOUT 2     /* unique-map: a scan tile gave up waiting for its predecessor        */
#define GE2_STATUS_FILTER_COLLISION 4 /* lp step: two filter pairs name the same (chunk, column)            */
#define GE2_STATUS_BAD_INDEX 8        /* lp step / scatter: a local id or relation id out of bounds         */
#define GE2_STATUS_PIPE_TIMEOUT 16    /* lp step (tensor path): a bounded mbarrier wait ran out             */
#define GE2_STATUS_PEER_TIMEOUT 32    /* peer-reduced dense step: a rank did not announce its gradients in time */

typedef void *ge2_stream_t; /* cudaStream_t */

GE2_API const char *ge2_version(void);
GE2_API int ge2_last_cuda_error(void);            /* cudaError_t of the last failing runtime call on this thread */
GE2_API const char *ge2_status_string(int status);
/* GE2_OK when device `device` exists and is compute capability 10.x; selects nothing. */
GE2_API int ge2_check_device(int device);

/* =====================================================================================================
 * (1) unique-map -- replaces map_tensors_unique_inverse_cuda, bitmap backend
 *     (cuda/src/common/unique_map_cuda.cu:771-882; declared cpp/include/common/unique_map_cuda.h:22-24),
 *     the kernel behind map_tensors (cpp/include/common/util.h:100-101, cpp/src/common/util.cpp:311-387).
 *
 * ids[n] int64 in [0, domain).  out_unique receives the distinct ids in ASCENDING order (capacity
 * min(n, domain) entries), out_inverse[n] the rank of ids[i] inside out_unique, out_count[0] the number of
 * distinct ids and out_count[1] a GE2_STATUS_* word (0 when clean).  Bit-exact with the reference's output.
 * No host synchronisation: the count is left on the device (the reference reads it back twice per call).
 * ===================================================================================================== */
GE2_API size_t ge2_unique_workspace_bytes(int64_t domain);
GE2_API int ge2_unique_bitmap(const int64_t *ids, int64_t n, int64_t domain, void *workspace, size_t workspace_bytes,
                      int64_t *out_unique, int64_t *out_inverse, int32_t *out_count, ge2_stream_t stream);

/* Unique-map for callers that cannot allocate device memory -- a host runtime that owns the whole GPU heap and hands
 * out none of it after start-up, a plugin that only ever receives its input and output buffers, a latency-bound loop
 * that may not call an allocator.  No counterpart in the reference project.  Same results as ge2_unique_bitmap, but
 * the scratch is a fixed array inside the library (about 0.8 MB on every GPU that loads it, held until the process
 * exits), so the id domain is limited to GE2_UNIQUE_STATIC_MAX_DOMAIN; a larger domain returns GE2_ERR_UNSUPPORTED.
 * The call makes no cudaMalloc/cudaFree and uses no allocating library routine.  The first call on each device looks
 * up the array's device address; make that first call outside any stream capture.  All calls share the one array,
 * which keeps the previous call's contents (the parts that must start at zero are cleared by every call): two calls
 * whose kernels can overlap on the GPU -- different streams without an ordering between them -- race. */
#define GE2_UNIQUE_STATIC_MAX_DOMAIN 4194304
GE2_API int ge2_unique_bitmap_static(const int64_t *ids, int64_t n, int64_t domain, int64_t *out_unique, int64_t *out_inverse,
                                     int32_t *out_count, ge2_stream_t stream);

/* Packs up to four id vectors into one contiguous buffer, the job of pack_ids_into_cached_buffer
 * (cpp/src/common/util.cpp:113-159).  Any part may be NULL with length 0. */
GE2_API int ge2_pack_ids(const int64_t *const parts[4], const int64_t lens[4], const int64_t strides[4], int64_t *out,
                 ge2_stream_t stream);

/* =====================================================================================================
 * (2) link-prediction training step: forward scores, softmax cross-entropy, backward
 *     replaces, for CORRUPT_NODE + RNS + SOFTMAX_CE(SUM):
 *       Model::forward_lp / Model::train_batch up to loss.backward()   cpp/src/nn/model.cpp:318-397
 *       mod_node_corrupt_forward                                        cpp/src/nn/decoders/edge/decoder_methods.cpp:724-806,933-946,1089-1097
 *       DotCompare::operator() + pad_and_reshape                        cpp/src/nn/decoders/edge/comparators.cpp:62-75,128-138
 *       HadamardOperator / ComplexHadamardOperator                      cpp/src/nn/decoders/edge/relation_operators.cpp:3-31
 *       apply_score_filter                                              cpp/src/data/samplers/negative.cpp:570-575
 *       SoftmaxCrossEntropy::operator()                                 cpp/src/nn/loss.cpp:46-63
 * ===================================================================================================== */
#define GE2_DECODER_DISTMULT 0 /* Hadamard relation operator; with has_relations == 0 this is the "Dot" decoder */
#define GE2_DECODER_COMPLEX 1  /* complex Hadamard: first D/2 columns real, remaining D - D/2 imaginary         */

/* ge2_lp_desc.flags: the caller guarantees node_grad is all zero on entry (e.g. ge2_adagrad_scatter with clear_grad
 * consumed the previous batch's gradients), so the step skips its own memset of U * D floats */
#define GE2_LP_NODE_GRAD_IS_ZERO 1

#define GE2_PRECISION_FP32 0 /* CUDA-core FFMA contraction, fp32 throughout (1e-4 relative parity)      */
#define GE2_PRECISION_F16 1  /* tcgen05 kind::f16 tiles (fp16 operands, 11-bit significand like TF32), fp32
                                accumulate in TMEM, fp32 everywhere else (1e-2 relative parity)         */

typedef struct ge2_lp_desc {
    int32_t decoder;       /* GE2_DECODER_*                                                       */
    int32_t has_relations; /* 1: edges carry a relation id; 0: relation-free graph                */
    int32_t use_inverse;   /* 1: also corrupt sources with inverse_relation_embeddings (needs has_relations) */
    int32_t precision;     /* GE2_PRECISION_*                                                     */
    int32_t B;             /* edges in the batch                                                  */
    int32_t C;             /* num_chunks                                                          */
    int32_t N;             /* negatives per chunk                                                 */
    int32_t D;             /* embedding dimension (<= 128)                                        */
    int32_t R;             /* rows of the relation tables                                         */
    int32_t phases;        /* 0 = whole step; else bit mask 1 = gather/prepare, 2 = scores, 4 = scatter/loss: lets a
                              benchmark time one phase on the workspace a full step left behind             */
    int64_t U;             /* rows of node_grad (and of node_emb when row_index == NULL)          */

    /* node embeddings: batch-local [U, D] when row_index == NULL (Batch::node_embeddings_), else a resident
     * table of which row row_index[l] is local node l (skips the indexRead copy). Row stride emb_stride floats. */
    const float *node_emb;
    const int64_t *row_index;
    int64_t emb_stride;

    /* batch edges in local ids; element i of the endpoint columns is at ptr[i * edge_stride], of the relation column
     * at rel_ids[i * rel_stride] (3/3 for the reference's interleaved [B,3] edges_, 2 for [B,2], 1 for separate
     * columns such as slices of the unique-map's inverse). rel_ids may be NULL when !has_relations. */
    const int64_t *src_ids;
    const int64_t *rel_ids;
    const int64_t *dst_ids;
    int64_t edge_stride;
    int64_t rel_stride;

    const int64_t *dst_negs; /* [C, N] local ids (Batch::dst_neg_indices_mapping_)                 */
    const int64_t *src_negs; /* [C, N] local ids, needed when use_inverse                           */

    /* score filter, either form (both may be NULL):
     *  - filter pairs [F, 2] (row, column), Batch::dst_neg_filter_ / src_neg_filter_; at most one row per
     *    (chunk, column), which is what deg_negative_local_filter produces;
     *  - or the degree-sample plan itself: deg_sample_rows[C, n_deg] = batch row each of the first n_deg negatives
     *    of a chunk was drawn from (the filter is derived on the device, no nonzero()/host count). */
    const int64_t *dst_filter;
    int64_t dst_filter_n;
    const int64_t *src_filter;
    int64_t src_filter_n;
    const int64_t *deg_sample_rows;
    int32_t n_deg;
    int32_t flags;        /* GE2_LP_* bits */

    const float *rel;     /* [R, D] relation_embeddings                                           */
    const float *inv_rel; /* [R, D] inverse_relation_embeddings                                   */

    /* outputs */
    float *node_grad;    /* [U, D]  d loss / d node_emb, overwritten (zeroed first unless GE2_LP_NODE_GRAD_IS_ZERO) */
    float *rel_grad;     /* [R, D]  accumulated into (+=), like autograd's .grad                   */
    float *inv_rel_grad; /* [R, D]  accumulated into (+=)                                          */
    float *loss;         /* [1]     overwritten                                                    */
    /* optional outputs for inspection (NULL to skip): the four score tensors forward_lp returns.
     * pos: [C*ceil(B/C)], neg: [C*ceil(B/C), N] (padded rows included, masked entries = -1e9).
     * Writing neg scores costs a [B,N] round trip the training path otherwise never makes. */
    float *pos_scores;
    float *neg_scores;
    float *inv_pos_scores;
    float *inv_neg_scores;

    int32_t *status;      /* device int32, GE2_STATUS_* bits are OR-ed in; may be NULL             */
    void *workspace;      /* ge2_lp_workspace_bytes() bytes, 256-byte aligned                      */
    size_t workspace_bytes;
} ge2_lp_desc;

GE2_API int ge2_lp_workspace_bytes(const ge2_lp_desc *desc, size_t *bytes);
GE2_API int ge2_lp_step(const ge2_lp_desc *desc, ge2_stream_t stream);

/* =====================================================================================================
 * (3) optimizer updates
 * ===================================================================================================== */
/* Batch::accumulateGradients (cpp/src/data/batch.cpp:229-286, math :264-266) on batch-local tensors:
 * upd = g*g; state += upd (in place); delta = -lr * g / (sqrt(state) + 1e-10).  rows may come from the device
 * (rows_dev != NULL: min(*rows_dev, rows) rows are processed).  delta may alias grad. */
GE2_API int ge2_sparse_adagrad(const float *grad, float *state_local, float *out_delta, float *out_state_update, int64_t rows,
                       const int32_t *rows_dev, int32_t D, float lr, ge2_stream_t stream);

/* Storage::indexRead / indexAdd for device tables (cpp/include/storage/storage.h:49-51;
 * InMemory: cpp/src/storage/storage.cpp:1173-1259; MemPartitionBuffer: cpp/src/storage/buffer.cpp:973-1045,1221-1228).
 * ids must be distinct for index_add (the reference relies on that too, buffer.cpp:619).  An id outside [0, table_rows) sets
 * GE2_STATUS_BAD_INDEX in *status (may be NULL); index_read writes a zero row for it, index_add skips it. */
GE2_API int ge2_index_read(const float *table, int64_t table_rows, const int64_t *ids, int64_t n, const int32_t *n_dev, int32_t D,
                   float *out, int32_t *status, ge2_stream_t stream);
GE2_API int ge2_index_add(float *table, int64_t table_rows, const int64_t *ids, int64_t n, const int32_t *n_dev, int32_t D,
                  const float *values, int32_t *status, ge2_stream_t stream);

/* The fused form of accumulateGradients + updateEmbeddings (cpp/src/data/dataloader.cpp:1381-1395,
 * cpp/src/storage/graph_storage.cpp:539-546,603-614): for every unique node l < U,
 *   row = unique_ids[l]; state[row] += g*g; table[row] += -lr * g / (sqrt(state[row]) + 1e-10)
 * with g = node_grad[l].  One read-modify-write pass over the touched rows, no temporaries.
 * clear_grad != 0 also zeroes node_grad rows after use (saves the next batch's memset). */
GE2_API int ge2_adagrad_scatter(float *table, float *state, int64_t table_rows, const int64_t *unique_ids, int64_t U,
                        const int32_t *U_dev, float *node_grad, int32_t D, float lr, int32_t clear_grad, int32_t *status,
                        ge2_stream_t stream);

/* AdagradOptimizer::step on a dense table (cpp/src/nn/optim.cpp:109-143; weight_decay = lr_decay = 0):
 * sum += g*g; param += -lr * g / (sqrt(sum) + eps).  grad_scale multiplies g first (1/num_gpus in
 * Model::all_reduce, cpp/src/nn/model.cpp:188-192); clear_grad != 0 zeroes grad afterwards (clear_grad_all). */
GE2_API int ge2_dense_adagrad(float *param, float *sum_state, float *grad, int64_t numel, float lr, float eps, float grad_scale,
                      int32_t clear_grad, ge2_stream_t stream);

/* Model::all_reduce + the dense optimizer step of every replica (cpp/src/nn/model.cpp:174-204, cpp/src/nn/optim.cpp:109-143):
 * the sum over ranks is read straight from the peers' gradient buffers over NVLink instead of going through a collective
 * call.  peer_bufs[r] (host array of `world` device pointers) is this process's mapping of rank r's buffer, own rank
 * included; every buffer holds 2 * numel floats (two halves, used by alternate steps: the step whose counter *step_dev is
 * t accumulates its gradients into half t & 1) followed by `world` 8-byte arrival flags, one 8-byte verdict word and one 8-byte counter (the nanoseconds the
 * announcing kernel has spent waiting for the slowest rank, summed over the steps: a diagnostic), all
 * zero at start; numel must be even.  Two launches: a one-warp kernel announces step t to every peer, waits for all
 * peers' announcements -- at most wait_budget_us microseconds (0 = 4 s) -- and writes one verdict for the step; the update
 * kernel then either applies Adagrad to param / sum_state with g = grad_scale * sum over ranks and clears half (t + 1) & 1
 * of its own buffer, or -- a peer never arrived -- changes nothing at all: GE2_STATUS_PEER_TIMEOUT is set in *status and
 * param, sum_state and the buffer are left bit for bit as they were.  After a timeout the replicas can no longer be
 * assumed equal (the peers may have gone on with this rank's gradients): treat it as fatal for the run.
 * Every rank launches it once per step, on devices that can access each other (ge2_enable_peer_access); a rank that has
 * no batch in a step (lanes of a superstep have unequal batch counts; the reference zero-fills their gradients,
 * model.cpp:182-187) launches only this: its half is still zero, so it contributes zeros and keeps its replica in step. */
GE2_API int ge2_dense_adagrad_peers(float *param, float *sum_state, float *const *peer_bufs, int32_t world, int32_t rank, int64_t numel,
                            const uint64_t *step_dev, float lr, float eps, float grad_scale, uint32_t wait_budget_us, int32_t *status,
                            ge2_stream_t stream);

/* cudaDeviceEnablePeerAccess from the current device to peer_device (no-op when already enabled or the same device):
 * what the relay path does before its peer copies (cpp/src/storage/storage.cpp:599-652 copies between device buffers). */
GE2_API int ge2_enable_peer_access(int32_t peer_device);

/* =====================================================================================================
 * producer side kept on the device so a training step needs no host round trip
 * ===================================================================================================== */
/* Shared chunked negatives of NegativeSamplingBase::getNodeCorruptNegatives (cpp/src/data/samplers/negative.cpp:938-1119;
 * plan :104-134, materialise :136-169): per chunk n_deg rows drawn uniformly from the batch (their dst / src ids are
 * the degree-proportional negatives) followed by N - n_deg ids uniform over [0, domain).  The same picks serve both
 * corruption sides.  Counter-based generator keyed by (seed, batch_index): reproducible, not the reference's Philox stream.
 * Also packs ids = [src(B), dst(B), src_negs(C*N) if wanted, dst_negs(C*N)] for the unique-map
 * (order of cpp/src/data/dataloader.cpp:1128-1137).  out_deg_rows[C, n_deg] feeds ge2_lp_desc.deg_sample_rows. */
GE2_API int ge2_sample_negatives(const int64_t *src_ids, const int64_t *dst_ids, int64_t edge_stride, int32_t B, int32_t C, int32_t N,
                         int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed, uint64_t batch_index,
                         int64_t *out_packed_ids, int64_t *out_deg_rows, ge2_stream_t stream);

/* The same producer in a form a captured CUDA graph can replay for every batch of an epoch: the batch is batch number
 * (*step_dev % num_batches) of the resident, already shuffled edge list edges[num_batches * B, cols] (the reference slices
 * its shuffled active edges the same way, cpp/src/data/dataloader.cpp:671-689), the generator is keyed by (seed, *step_dev),
 * and the batch's relation column is copied to out_rel_ids[B] (cols == 3) so that no later kernel needs the edge pointer.
 * ge2_advance_step increments n consecutive device-side counters (one launch at the end of the step; a pipelined host
 * keeps {t, t + 1} so that batch t + 1 can be sampled while batch t is still training). */
GE2_API int ge2_sample_batch(const int64_t *edges, int32_t cols, int64_t num_batches, const uint64_t *step_dev, int32_t B, int32_t C,
                             int32_t N, int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed, int64_t *out_packed_ids,
                             int64_t *out_deg_rows, int64_t *out_rel_ids, ge2_stream_t stream);
/* The same with the number of batches read from device memory (*num_batches_dev >= 1): a partition-buffer state replaces the
 * resident edge list by one of another length (ge2_build_state_edges) without the captured launch changing. */
GE2_API int ge2_sample_batch_dev(const int64_t *edges, int32_t cols, const int64_t *num_batches_dev, const uint64_t *step_dev, int32_t B,
                                 int32_t C, int32_t N, int32_t n_deg, int64_t domain, int32_t want_src_negs, uint64_t seed,
                                 int64_t *out_packed_ids, int64_t *out_deg_rows, int64_t *out_rel_ids, ge2_stream_t stream);
GE2_API int ge2_advance_step(uint64_t *step_dev, int32_t n, ge2_stream_t stream);

/* GraphModelStorage::mapEdgesWithPartitionSlots_ (cpp/src/storage/graph_storage.cpp:270-303):
 * id -> slot[id / partition_size] * partition_size + id % partition_size on the first and last column of
 * edges[n, cols] (int64, in place or out of place).  A non-resident partition sets GE2_STATUS_BAD_INDEX. */
GE2_API int ge2_remap_edges_to_slots(const int64_t *edges, int64_t n, int32_t cols, const int64_t *partition_to_slot,
                             int32_t num_partitions, int64_t partition_size, int64_t *out, int32_t *status,
                             ge2_stream_t stream);

/* The edge list of one partition-buffer state, ready to train on, in ONE pass over the state's edges:
 * GraphModelStorage::updateInMemorySubGraph_ (cpp/src/storage/graph_storage.cpp:938-1240: copy of the resident buckets' edges,
 * arithmetic remap :270-303) + DataLoader::setActiveEdges (cpp/src/data/dataloader.cpp:524-633: concatenation, randperm,
 * index_select) -- CPU loops, OpenMP and an upload of the whole state in the reference.
 * edges_sorted[E, cols] int64 (device) is the training edge list sorted by bucket (src partition * P + dst partition), global
 * node ids, as the preprocessor writes it (python/tools/preprocess/converters/partitioners/torch_partitioner.py:12-31);
 * bucket_begin_host / bucket_len_host[num_buckets] (HOST arrays, <= 64 entries) name the buckets of the state in the order they
 * are concatenated; partition_to_slot[num_partitions] (device) is the buffer slot of every resident partition (-1 otherwise).
 * out_edges[total, cols] receives row perm(j) of the concatenation at position j, first and last column remapped to
 * slot * partition_size + id % partition_size; perm is a fixed function of (seed, total): four Feistel rounds with cycle
 * walking (a uniform shuffle is all the reference asks of its randperm; this one needs no sort and no scratch).
 * *out_total_host = total (host, written before the launch).  An endpoint whose partition is not resident sets
 * GE2_STATUS_BAD_INDEX and becomes -1. */
GE2_API int ge2_build_state_edges(const int64_t *edges_sorted, int32_t cols, const int64_t *bucket_begin_host,
                                  const int64_t *bucket_len_host, int32_t num_buckets, const int64_t *partition_to_slot,
                                  int32_t num_partitions, int64_t partition_size, uint64_t seed, int64_t *out_edges,
                                  int64_t *out_total_host, int32_t *status, ge2_stream_t stream);

/* MemPartitionBufferStorage::performNextSwap(int32_t device_idx) (cpp/include/storage/storage.h:157-187,
 * cpp/src/storage/storage.cpp:576-689), peer-relay branch :599-652, as receiver-side pulls behind a device-side barrier:
 * no host synchronisation, no cudaDeviceSynchronize, no staging through the host.
 * Every rank keeps TWO active buffers and alternates between them from superstep to superstep, so a swap only reads the
 * buffers of the superstep that ended and only writes the buffers of the one that begins: one barrier per swap is enough
 * (everybody has finished training before anybody pulls; by the time these source buffers are written again, in the swap
 * after next, every rank has announced the end of another superstep, which it does after its own pulls).
 *   flag_rows[r]  (host array of `world` device pointers) this process's mapping of rank r's flag row: world + 1 8-byte words,
 *                 all zero at start; needed when world > 1
 *   epoch         1, 2, 3, ... the number of this swap (the same on every rank)
 *   pull_src/dst  (host arrays of num_pulls <= 32 device pointers) slabs of slab_bytes bytes (a multiple of 16): sources are
 *                 peer mappings or local memory (a partition's slot in its holder's current buffer, or its home slab),
 *                 destinations this rank's memory (a slot of its next buffer, or a home slab for a partition nobody keeps)
 * ge2_swap_begin enqueues on `stream`: a one-warp kernel that announces `epoch` to every rank and waits for all of them, at
 * most wait_budget_us microseconds (0 = 4 s), then one copy kernel for all slabs (plain 16-byte peer loads) that does nothing
 * when the wait ran out (GE2_STATUS_PEER_TIMEOUT in *status; buffers untouched).  ge2_swap_wait makes compute_stream wait for
 * what ge2_swap_begin enqueued on swap_stream (an event; nothing blocks the host), so the pulls can run beside the tail of the
 * superstep's other work. */
typedef struct ge2_swap_desc {
    int32_t world, rank;
    void *const *flag_rows;
    uint64_t epoch;
    uint32_t wait_budget_us;
    int32_t num_pulls;
    const void *const *pull_src;
    void *const *pull_dst;
    int64_t slab_bytes;
    int32_t *status;
} ge2_swap_desc;
GE2_API int ge2_swap_begin(const ge2_swap_desc *desc, ge2_stream_t stream);
GE2_API int ge2_swap_wait(ge2_stream_t swap_stream, ge2_stream_t compute_stream);

/* Slab copies of MemPartitionBufferStorage::performNextSwap's relay branch that stay on one device
 * (cpp/src/storage/storage.cpp:626-652, src_dev == device_idx): moves[k] = {src_slot, dst_slot}; copies whole
 * partition slabs src[src_slot] -> dst[dst_slot] in one launch.  Slabs that cross devices are pulled by ge2_swap_begin
 * (or travel by NCCL send/recv issued by the host layer when the processes cannot map each other's memory). */
GE2_API int ge2_copy_slabs(const float *src, float *dst, const int32_t *moves_host, int32_t num_moves, int64_t slab_floats,
                   ge2_stream_t stream);

/* =====================================================================================================
 * Link-prediction evaluation: ranks of a batch of test edges against candidate nodes, both corruption sides.
 * Reference: node_corrupt_forward (cpp/src/nn/decoders/edge/decoder_methods.cpp:597-659) -> apply_score_filter
 * (cpp/src/data/samplers/negative.cpp:570-575; filter pairs from compute_filter_corruption, :421-568) ->
 * LinkPredictionReporter::computeRanks (cpp/src/reporting/reporting.cpp:52-54): rank = #(negative score >= positive score) + 1,
 * a filtered score counting as -1e9.  Candidates are all rows [0, num_nodes) of node_emb (the filtered evaluation of the
 * reference: one chunk with every node, negative.cpp:585-589) or, with neg_ids != NULL, the num_negs rows it lists (one shared
 * chunk); filter pairs are (edge row, candidate column), duplicates allowed.  Edge ids are rows of node_emb.  fp32 throughout;
 * every score is the chain acc = fma(q[d], e[d], acc) with d ascending.  The [B, candidates] score matrix is never stored.
 * src_ranks / src_filter are used when has_relations && use_inverse (the inverse relation applied to the destination,
 * compared with candidate sources).  A row with an id out of range sets GE2_STATUS_BAD_INDEX and gets rank 0.
 * ===================================================================================================== */
typedef struct ge2_eval_desc {
    int32_t decoder;       /* GE2_DECODER_* */
    int32_t has_relations;
    int32_t use_inverse;
    int32_t D;             /* <= 128 */
    int64_t B;             /* test edges */
    int64_t num_nodes;     /* rows of node_emb */
    int64_t R;
    const float *node_emb; /* [num_nodes, D], row stride emb_stride floats */
    int64_t emb_stride;
    const int64_t *src_ids, *rel_ids, *dst_ids; /* element i at ptr[i * edge_stride] (rel_ids: i * rel_stride) */
    int64_t edge_stride, rel_stride;
    const float *rel, *inv_rel;                 /* [R, D] */
    const int64_t *neg_ids;                     /* NULL: every node is a candidate; else [num_negs] rows of node_emb */
    int64_t num_negs;
    const int64_t *dst_filter; /* [F, 2] (edge row, candidate column) */
    int64_t dst_filter_n;
    const int64_t *src_filter;
    int64_t src_filter_n;
    int64_t *dst_ranks;    /* [B] out */
    int64_t *src_ranks;    /* [B] out (two-sided evaluation) */
    float *pos_scores;     /* [B] out, optional */
    float *inv_pos_scores; /* [B] out, optional */
    int32_t *status;       /* device int32, GE2_STATUS_* bits OR-ed in; may be NULL */
    void *workspace;       /* 256-byte aligned, ge2_eval_workspace_bytes(desc) bytes */
    size_t workspace_bytes;
} ge2_eval_desc;
GE2_API size_t ge2_eval_workspace_bytes(const ge2_eval_desc *desc);
GE2_API int ge2_eval_ranks(const ge2_eval_desc *desc, ge2_stream_t stream);

/* =====================================================================================================
 * Selected-negative scoring (the DNS / GAN / tournament samplers of the reference): a query row is scored against the few
 * negatives chosen for it.  chunked [chunks, rows_per_chunk, D] (relation-adjusted, padded query rows), negatives
 * [chunks, num_negs, D], selected [chunks, rows_per_chunk * num_selected] int64 columns of the row's own chunk, all dense
 * fp32 / int64 device arrays; D <= 128.
 *
 * ge2_selected_neg_scores replaces selected_neg_scores_cuda_forward (cuda/src/nn/decoders/edge/distmult_selected_neg_cuda.cu:
 * 204-268): out_scores [chunks * rows_per_chunk, num_selected]; kind DOT is the dot product, L2 is sqrt(max(|q - n|^2, 1e-8)).
 * ge2_selected_neg_scores_backward replaces selected_neg_scores_cuda_backward (same file :270-362): grad_out as out_scores;
 * grad_chunked [chunks, rows_per_chunk, D] is written, grad_negatives [chunks, num_negs, D] is zeroed and accumulated.
 * A selected column outside [0, num_negs) scores 0, contributes no gradient and sets GE2_STATUS_BAD_INDEX in *status (may be
 * NULL); the reference reads out of bounds there.
 *
 * ge2_tournament_select replaces distmult_tiled_tournament_selected_scores (cpp/src/nn/decoders/edge/
 * distmult_selected_neg_cuda.cpp:46-121): the num_negs negatives of a chunk form num_selected groups of num_negs / num_selected
 * consecutive ones (num_negs must divide evenly, else GE2_ERR_INVALID_ARGUMENT); per row and group the negative with the highest
 * selector score is kept (the first of equal ones; a NaN score never wins).  out_idx [chunks, rows_per_chunk * num_selected] is its
 * column in the chunk, out_scores [chunks * rows_per_chunk, num_selected] its score by the score_* tensors (NULL: the
 * selector's, which is also what equal pointers mean).  The reference's groups_per_tile only sizes its temporary score
 * matrix; no score matrix is stored here.  chunks <= 65535.
 * ===================================================================================================== */
#define GE2_SELECTED_DOT 1 /* the values of the reference's SelectedNegScoreKind */
#define GE2_SELECTED_L2 2
GE2_API int ge2_selected_neg_scores(int kind, const float *chunked, const float *negatives, const int64_t *selected, int64_t chunks,
                                    int64_t rows_per_chunk, int64_t num_negs, int64_t num_selected, int D, float *out_scores,
                                    int32_t *status, ge2_stream_t stream);
GE2_API int ge2_selected_neg_scores_backward(int kind, const float *grad_out, const float *chunked, const float *negatives,
                                             const int64_t *selected, int64_t chunks, int64_t rows_per_chunk, int64_t num_negs,
                                             int64_t num_selected, int D, float *grad_chunked, float *grad_negatives, int32_t *status,
                                             ge2_stream_t stream);
GE2_API int ge2_tournament_select(const float *selector_chunked, const float *selector_negatives, const float *score_chunked,
                                  const float *score_negatives, int64_t chunks, int64_t rows_per_chunk, int64_t num_negs,
                                  int64_t num_selected, int D, float *out_scores, int64_t *out_idx, ge2_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* GE2_B200_H_ */
