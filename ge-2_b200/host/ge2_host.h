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
#pragma once
#include <torch/torch.h>

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
    torch::Tensor loss_;                  // scalar on the device, written by train_batch

    void accumulateGradients(float learning_rate);
    void clear();
};

enum class DecoderType { DISTMULT, COMPLEX };

// The slice of the reference's Model that the training step touches: a DistMult / ComplEx edge decoder with its relation
// tables, softmax cross-entropy with SUM reduction, a dense Adagrad optimizer for the relation tables.
class Model {
   public:
    Model(DecoderType type, int64_t num_relations, int64_t dim, bool use_inverse_relations, float dense_lr, float sparse_lr,
          torch::Device device, const std::string& precision = "fp32");

    void train_batch(std::shared_ptr<Batch> batch, bool call_step = true);  // forward, loss, backward, [dense step], accumulateGradients
    void step();        // AdagradOptimizer::step on the relation tables
    void clear_grad();  // zero the relation gradients
    // Model::all_reduce minus the collective: the caller sums the gradient tensors across replicas (NCCL), then calls this
    // with 1 / #replicas, which divides, steps and clears -- same arithmetic as model.cpp:174-204 of the reference.
    void step_after_all_reduce(float grad_scale);

    torch::Tensor relations_, inverse_relations_;            // [R, D]
    torch::Tensor relations_grad_, inverse_relations_grad_;  // [R, D] accumulated like autograd's .grad
    torch::Tensor relations_state_, inverse_relations_state_;
    DecoderType type_;
    bool use_inverse_relations_;
    float dense_lr_, sparse_lr_;
    int precision_;

   private:
    torch::Tensor workspace_, status_;
};

// InMemory storage on the device (storage.cpp:1173-1259 of the reference)
class InMemory {
   public:
    explicit InMemory(torch::Tensor data) : data_(std::move(data)) {}
    torch::Tensor indexRead(Indices indices);
    void indexAdd(Indices indices, torch::Tensor values);
    torch::Tensor data_;
};

}  // namespace ge2host
