// Host layer: the reference project's C++ interface for the per-batch path (same names, argument meaning and error
// behaviour), implemented on top of the C ABI in include/ge2_b200.h.  libtorch tensors appear only here, as device
// memory; every arithmetic step is a kernel of libge2_b200.so.  There is no CPU path: CPU tensors are rejected.
//
// Mirrors (paths relative to gege/src/cpp/ of the reference project):
//   map_tensors                         include/common/util.h:100-101
//   map_tensors_unique_inverse_cuda     include/common/unique_map_cuda.h:22-24
//   Batch, Batch::accumulateGradients   include/data/batch.h:13-79
//   Model::train_batch / step / clear_grad / all_reduce hook   include/nn/model.h:37-59
//   Storage::indexRead / indexAdd       include/storage/storage.h:49-51
//   MemPartitionBufferStorage (performNextSwap, hasSwap, getNextAdmit/Evict, getPartitionToBufferSlotMap, indexRead/indexAdd
//     with device_idx)                  include/storage/storage.h:113-187
//   Model::broadcast / all_reduce       include/nn/model.h:59, src/nn/model.cpp:174-204,454-478
//   DataLoader::getBatch / updateEmbeddings   src/data/dataloader.cpp:1069-1291,1354-1395
//   selected_neg_scores (autograd), selected_neg_scores_cuda_forward / _backward, distmult_tiled_tournament_selected_scores
//                                       include/nn/decoders/edge/distmult_selected_neg_cuda.h:5-29
#pragma once
#include <torch/torch.h>

#include <array>
#include <memory>
#include <stdexcept>
#include <string>
#include <tuple>
#include <vector>

namespace ge2host {

// the reference throws GegeRuntimeException (include/common/exception.h:7-37); same name, same base class
struct GegeRuntimeException : public std::runtime_error {
    explicit GegeRuntimeException(const std::string& msg) : std::runtime_error(msg) {}
};

using Indices = torch::Tensor;

std::tuple<torch::Tensor, torch::Tensor> map_tensors_unique_inverse_cuda(torch::Tensor all_ids, bool sorted, int64_t value_domain_size = -1);

std::tuple<torch::Tensor, std::vector<torch::Tensor>> map_tensors(std::vector<torch::Tensor> unmapped_tensors, bool sorted = true,
                                                                  int64_t value_domain_size = -1);

// The reference's selected-negative operators (include/nn/decoders/edge/distmult_selected_neg_cuda.h:5-29): same names,
// arguments and shapes.  fp32 CUDA tensors, D <= 128.  A selected column outside its chunk scores 0, gets no gradient and is
// recorded in a per-device status word that selected_neg_status() returns and clears (the reference reads out of bounds).
enum class SelectedNegScoreKind : int64_t { NONE = 0, DOT = 1, L2 = 2 };

torch::Tensor selected_neg_scores_cuda_forward(torch::Tensor chunked_adjusted_embeddings, torch::Tensor negative_embeddings,
                                               torch::Tensor selected_neg_indices, int64_t score_kind);
std::tuple<torch::Tensor, torch::Tensor> selected_neg_scores_cuda_backward(torch::Tensor grad_out, torch::Tensor chunked_adjusted_embeddings,
                                                                           torch::Tensor negative_embeddings, torch::Tensor selected_neg_indices,
                                                                           int64_t score_kind);
// differentiable in the first two arguments
torch::Tensor selected_neg_scores(torch::Tensor chunked_adjusted_embeddings, torch::Tensor negative_embeddings, torch::Tensor selected_neg_indices,
                                  SelectedNegScoreKind score_kind);
// (scores [chunks * rows, selected], columns [chunks, rows * selected]); the scores are differentiable in the score_* tensors,
// the selector's only choose.  groups_per_tile is accepted and ignored: no score tile is stored.
std::tuple<torch::Tensor, torch::Tensor> distmult_tiled_tournament_selected_scores(torch::Tensor selector_chunked_embeddings,
                                                                                    torch::Tensor selector_negative_embeddings,
                                                                                    torch::Tensor score_chunked_embeddings,
                                                                                    torch::Tensor score_negative_embeddings,
                                                                                    int64_t selected_negatives_num, int64_t groups_per_tile);
int32_t selected_neg_status(torch::Device device);

class Batch {
   public:
    Indices unique_node_indices_;         // global node ids of the batch's unique nodes (ascending)
    torch::Tensor node_embeddings_;       // [U, D] gathered embeddings
    torch::Tensor node_gradients_;        // [U, D] gradients; after accumulateGradients the embedding update
    torch::Tensor node_embeddings_state_; // [U, D] gathered Adagrad state
    torch::Tensor node_state_update_;     // [U, D] state update
    Indices src_neg_indices_mapping_;     // [C, N] local ids
    Indices dst_neg_indices_mapping_;     // [C, N] local ids
    torch::Tensor edges_;                 // [B, 2|3] local ids (src[, rel], dst)
    torch::Tensor src_neg_filter_;        // [F, 2] (row, col)
    torch::Tensor dst_neg_filter_;
    torch::Tensor deg_sample_rows_;       // [C, n_deg] batch row each degree-based negative was drawn from; when set, the
                                          // local filter of both sides is derived from it on the device (no nonzero())
    torch::Tensor loss_;                  // scalar on the device, written by train_batch

    void accumulateGradients(float learning_rate);
    void clear();
};

enum class DecoderType { DISTMULT, COMPLEX };

// The slice of the reference's Model that the training step touches: a DistMult / ComplEx edge decoder with its relation
// tables, softmax cross-entropy with SUM reduction, a dense Adagrad optimizer for the relation tables.
class Model : public std::enable_shared_from_this<Model> {
   public:
    Model(DecoderType type, int64_t num_relations, int64_t dim, bool use_inverse_relations, float dense_lr, float sparse_lr,
          torch::Device device, const std::string& precision = "fp32");

    void train_batch(std::shared_ptr<Batch> batch, bool call_step = true);  // forward, loss, backward, [dense step], accumulateGradients
    void step();        // AdagradOptimizer::step on the relation tables
    void clear_grad();  // zero the relation gradients
    // Model::all_reduce minus the collective: the caller sums the gradient tensors across replicas (NCCL), then calls this
    // with 1 / #replicas, which divides, steps and clears -- same arithmetic as model.cpp:174-204 of the reference.
    void step_after_all_reduce(float grad_scale);

    // Replicas on several GPUs of this process (Model::broadcast, model.cpp:454-478): device_models_[i] lives on devices[i],
    // device_models_[0] being this model.  Afterwards every replica accumulates its relation gradients into a buffer its
    // peers can read, and all_reduce() -- called once per batch round after every replica's train_batch(batch, false) --
    // averages the gradients over the replicas, steps every replica's relation tables and clears the gradients
    // (Model::all_reduce + step_all, model.cpp:174-204) as ONE launch pair per device and no collective call:
    // ge2_dense_adagrad_peers.  A replica that trained no batch in the round contributes zeros, as in the reference.
    void broadcast(std::vector<torch::Device> devices);
    void all_reduce();
    void check_status();  // throws when a device-side status word is set (peer timeout, bad index, ...)
    std::vector<std::shared_ptr<Model>> device_models_;

    torch::Tensor relations_, inverse_relations_;            // [R, D]
    torch::Tensor relations_grad_, inverse_relations_grad_;  // [R, D] accumulated like autograd's .grad
    torch::Tensor relations_state_, inverse_relations_state_;
    DecoderType type_;
    bool use_inverse_relations_;
    float dense_lr_, sparse_lr_;
    int precision_;

   private:
    void point_at_half(int half);
    torch::Tensor workspace_, status_;
    torch::Tensor rel_both_, state_both_;  // [S, R, D]: the two tables (and their states) back to back
    torch::Tensor grad_buf_;               // replicated form: two halves of S*R*D floats, arrival flags, verdict, wait counter
    torch::Tensor step_dev_;               // replicated form: device-side round counter
    std::vector<float*> peer_ptrs_;        // every replica's grad_buf_
    int64_t round_ = 0;
    int replica_ = 0;
};

// InMemory storage on the device (storage.cpp:1173-1259 of the reference)
class InMemory {
   public:
    explicit InMemory(torch::Tensor data) : data_(std::move(data)) {}
    torch::Tensor indexRead(Indices indices);
    void indexAdd(Indices indices, torch::Tensor values);
    // An index outside the table is skipped on the device (rows read as zero) and recorded in a status word; the reference's
    // index ops throw at once, here the word is read where the caller synchronises anyway: throws GegeRuntimeException.
    void checkStatus();
    torch::Tensor data_;

   private:
    torch::Tensor status_;
};

// Partition buffer over the GPUs of this process: every partition has a home slab on device p % G; a device's active set of
// four partitions sits in one of its two buffers [4 * partition_size, dim1]; performNextSwap(device_idx) -- called by every
// device thread (or by one thread for every device in turn: nothing blocks the host) -- pulls the next state's partitions
// from wherever they are into the device's other buffer behind a device-side barrier (ge2_swap_begin).  The counterpart of
// the reference's MemPartitionBufferStorage with its peer relay (storage.cpp:359-757); unlike it, nothing is staged through
// the host when G * 4 < num_partitions.
class MemPartitionBufferStorage {
   public:
    MemPartitionBufferStorage(int64_t dim0_size, int64_t dim1_size, int32_t num_partitions, std::vector<torch::Device> devices);

    void load(torch::Tensor values);   // [dim0_size, dim1_size] on any device: the rows of partition p go to its home slab
    torch::Tensor unload();            // every resident partition goes home; returns the whole table on the CPU
    // buffer_states[k * G + g] = the partitions (up to four, int64) device g holds in superstep k (buffer.cpp:1134-1146)
    void setBufferOrdering(std::vector<torch::Tensor> buffer_states);
    bool hasSwap(int32_t device_idx = 0);
    void performNextSwap(int32_t device_idx);
    std::vector<int> getNextAdmit(int32_t device_idx = 0);
    std::vector<int> getNextEvict(int32_t device_idx = 0);
    torch::Tensor getPartitionToBufferSlotMap(int32_t device_idx = 0);  // [num_partitions] int64 on the CPU, -1 = not resident
    torch::Tensor indexRead(Indices indices, int32_t device_idx);      // buffer-local row ids
    void indexAdd(Indices indices, torch::Tensor values, int32_t device_idx);
    torch::Tensor activeBuffer(int32_t device_idx);                    // [4 * partition_size, dim1] view of the current buffer
    int64_t getPartitionSize(int32_t = 0) { return partition_size_; }
    int64_t getNumInMemory(int32_t = 0) { return 4 * partition_size_; }
    void checkStatus();

   private:
    struct Pull {
        bool src_home, dst_home;
        int src_dev;
        int64_t src_index, dst_index;
    };
    struct Plan {
        std::vector<std::vector<int64_t>> slots;  // per device: partition in each of the four slots, -1 = empty
        std::vector<std::vector<Pull>> pulls;     // per device
    };
    Plan make_plan(const std::vector<std::vector<int64_t>>& current, const std::vector<std::vector<int64_t>>& next_states);
    void run_plan(const Plan& plan, int32_t device_idx);

    int64_t dim0_, dim1_, partition_size_;
    int32_t num_partitions_;
    std::vector<torch::Device> devices_;
    std::vector<torch::Tensor> home_, flags_, status_;
    std::vector<std::array<torch::Tensor, 2>> bufs_;
    std::vector<uint64_t> epoch_;
    std::vector<size_t> next_;   // per device: index of the next plan
    std::vector<Plan> plans_;    // one per superstep, then the flush
    std::vector<std::vector<int64_t>> resident_;  // slots before plans_[0]
};

// The reference's per-batch loader calls for a device-resident edge list (DataLoader::getBatch -> edgeSample + loadGPUParameters,
// dataloader.cpp:1069-1291,1354-1379; DataLoader::updateEmbeddings, :1381-1395), unfused: sample, map_tensors, gather.
class DataLoader {
   public:
    DataLoader(torch::Tensor edges, std::shared_ptr<InMemory> node_embeddings, std::shared_ptr<InMemory> node_embeddings_state, int64_t batch_size,
               int32_t num_chunks, int32_t negatives_per_chunk, float degree_fraction, bool inverse_edges, uint64_t seed);
    std::shared_ptr<Batch> getBatch();                  // batch number batch_id_++ of the edge list (wraps around)
    void updateEmbeddings(std::shared_ptr<Batch> batch);  // indexAdd of the embedding and state updates
    int64_t batch_id_ = 0;

   private:
    torch::Tensor edges_, packed_, deg_rows_, rel_ids_, step_dev_;
    std::shared_ptr<InMemory> emb_, state_;
    int64_t B_;
    int32_t C_, N_, n_deg_;
    bool want_src_;
    uint64_t seed_;
};

}  // namespace ge2host
