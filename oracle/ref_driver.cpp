// TEST INFRASTRUCTURE ONLY -- never part of the product path.
//
// Python-callable driver around the UNMODIFIED reference sources (compiled where they lie by
// oracle/Makefile, CPU-only build, outputs into oracle/_ref/).  It replays the per-batch sequence of
// the reference's Model::train_batch (gege/src/cpp/src/nn/model.cpp:362-404) with the reference's own
// functions: mod_node_corrupt_forward (decoder_methods.cpp:724), apply_score_filter (negative.cpp:570),
// SoftmaxCrossEntropy (loss.cpp:46), AdagradOptimizer::step (optim.cpp:109), Batch::accumulateGradients
// (batch.cpp:229); plus map_tensors (util.cpp:311) and deg_negative_local_filter (negative.cpp:215).
// Used to pin the numpy restatement (oracle/ge2_oracle.py), to generate tests/golden fixtures and as the
// timed CPU reference arm of bench.py.  Nothing here is a copy of reference code: it only calls it.
//
// The same file builds twice: CPU-only as gege_ref, and with -DGEGE_CUDA beside the reference's CUDA sources as
// gege_ref_cuda, where RefModel takes a device string, its tensors live on that GPU, and the reference's
// map_tensors_unique_inverse_cuda (unique_map_cuda.cu:1002-1023) is exported for the bit-exact unique-map tests.
#include <torch/extension.h>

#include <cstdlib>

#include "common/util.h"
#ifdef GEGE_CUDA
#include "common/unique_map_cuda.h"
#include "nn/decoders/edge/distmult_selected_neg_cuda.h"
#endif
#include "data/batch.h"
#include "data/samplers/negative.h"
#include "nn/decoders/edge/complex.h"
#include "nn/decoders/edge/decoder_methods.h"
#include "nn/decoders/edge/distmult.h"
#include "nn/loss.h"
#include "nn/optim.h"

namespace {

struct RefModel {
    std::shared_ptr<EdgeDecoder> decoder;
    std::shared_ptr<SoftmaxCrossEntropy> loss;
    std::shared_ptr<AdagradOptimizer> dense_opt;
    float sparse_lr;

    RefModel(const std::string &decoder_type, int64_t num_relations, int64_t dim, bool inverse, double dense_lr, double sparse_lr_,
             const std::string &device = "cpu") {
        setenv("GEGE_CSR_DEBUG", "0", 1);
        setenv("GEGE_STAGE_DEBUG", "0", 1);
        setenv("GEGE_CSR_GATHER", "0", 1);
        auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(torch::Device(device));
        if (decoder_type == "DISTMULT") {
            decoder = std::make_shared<DistMult>((int)num_relations, (int)dim, opts, inverse, EdgeDecoderMethod::CORRUPT_NODE);
        } else if (decoder_type == "COMPLEX") {
            decoder = std::make_shared<ComplEx>((int)num_relations, (int)dim, opts, inverse, EdgeDecoderMethod::CORRUPT_NODE);
        } else {
            throw std::runtime_error("decoder_type must be DISTMULT or COMPLEX");
        }
        auto lopts = std::make_shared<LossOptions>();
        lopts->loss_reduction = LossReduction::SUM;
        loss = std::make_shared<SoftmaxCrossEntropy>(lopts);

        torch::OrderedDict<std::string, torch::Tensor> params;
        params.insert("relation_embeddings", decoder->relations_);
        if (decoder->inverse_relations_.defined()) params.insert("inverse_relation_embeddings", decoder->inverse_relations_);
        auto aopts = std::make_shared<AdagradOptions>();
        aopts->learning_rate = (float)dense_lr;
        aopts->eps = 1e-10f;
        aopts->init_value = 0;
        aopts->lr_decay = 0;
        aopts->weight_decay = 0;
        dense_opt = std::make_shared<AdagradOptimizer>(params, aopts);
        sparse_lr = (float)sparse_lr_;
    }

    void set_relations(torch::Tensor rel, torch::Tensor inv_rel) {
        torch::NoGradGuard ng;
        decoder->relations_.copy_(rel);
        if (decoder->inverse_relations_.defined() && inv_rel.defined()) decoder->inverse_relations_.copy_(inv_rel);
    }
    void set_relation_state(torch::Tensor st, torch::Tensor inv_st) {
        torch::NoGradGuard ng;
        dense_opt->state_dict_["relation_embeddings"]["sum"].copy_(st);
        if (decoder->inverse_relations_.defined() && inv_st.defined()) dense_opt->state_dict_["inverse_relation_embeddings"]["sum"].copy_(inv_st);
    }
    std::vector<torch::Tensor> get_relations() {
        std::vector<torch::Tensor> out{decoder->relations_.detach().clone(), dense_opt->state_dict_["relation_embeddings"]["sum"].clone()};
        if (decoder->inverse_relations_.defined()) {
            out.push_back(decoder->inverse_relations_.detach().clone());
            out.push_back(dense_opt->state_dict_["inverse_relation_embeddings"]["sum"].clone());
        }
        return out;
    }

    // One reference training step on batch-local tensors.  edges: [B,2|3] int64 local ids; emb/state: [U,D].
    // Returns a dict of every intermediate the parity tests look at.
    std::map<std::string, torch::Tensor> train_batch(torch::Tensor edges, torch::Tensor node_embeddings, torch::Tensor node_state,
                                                     torch::Tensor dst_negs, c10::optional<torch::Tensor> src_negs_o,
                                                     c10::optional<torch::Tensor> dst_filter_o, c10::optional<torch::Tensor> src_filter_o,
                                                     bool call_step, bool want_scores) {
        torch::Tensor src_negs = src_negs_o.has_value() ? *src_negs_o : torch::Tensor();
        torch::Tensor dst_filter = dst_filter_o.has_value() ? *dst_filter_o : torch::Tensor();
        torch::Tensor src_filter = src_filter_o.has_value() ? *src_filter_o : torch::Tensor();

        auto batch = std::make_shared<Batch>(true);
        batch->edges_ = edges;
        batch->node_embeddings_ = node_embeddings.clone();
        batch->node_embeddings_state_ = node_state.clone();
        batch->dst_neg_indices_mapping_ = dst_negs;
        batch->src_neg_indices_mapping_ = src_negs;
        batch->dst_neg_filter_ = dst_filter;
        batch->src_neg_filter_ = src_filter;
        batch->unique_node_indices_ = torch::arange(node_embeddings.size(0), torch::TensorOptions().dtype(torch::kInt64).device(node_embeddings.device()));

        if (call_step) dense_opt->clear_grad();              // model.cpp:363-365
        batch->node_embeddings_.requires_grad_();            // model.cpp:367-369

        auto scores = mod_node_corrupt_forward(NegativeSamplingMethod::RNS, 1.0f, nullptr, decoder, batch->edges_, batch->node_embeddings_,
                                               batch->dst_neg_indices_mapping_, batch->src_neg_indices_mapping_, torch::Tensor());  // model.cpp:336
        torch::Tensor pos = std::get<0>(scores), neg = std::get<1>(scores), ipos = std::get<2>(scores), ineg = std::get<3>(scores);
        if (neg.defined()) neg = apply_score_filter(neg, batch->dst_neg_filter_);    // model.cpp:351
        if (ineg.defined()) ineg = apply_score_filter(ineg, batch->src_neg_filter_);  // model.cpp:355

        torch::Tensor l;
        if (ineg.defined()) {
            torch::Tensor rhs = (*loss)(pos, neg, true);
            torch::Tensor lhs = (*loss)(ipos, ineg, true);
            l = lhs + rhs;  // model.cpp:383-386
        } else {
            l = (*loss)(pos, neg, true);
        }
        l.backward();  // model.cpp:397

        std::map<std::string, torch::Tensor> out;
        out["loss"] = l.detach().clone();
        if (want_scores) {
            out["pos_scores"] = pos.detach().clone();
            out["neg_scores"] = neg.detach().clone();
            if (ineg.defined()) {
                out["inv_pos_scores"] = ipos.detach().clone();
                out["inv_neg_scores"] = ineg.detach().clone();
            }
        }
        out["node_grad"] = batch->node_embeddings_.grad().clone();
        if (decoder->relations_.grad().defined()) out["rel_grad"] = decoder->relations_.grad().clone();
        if (decoder->inverse_relations_.defined() && decoder->inverse_relations_.grad().defined())
            out["inv_rel_grad"] = decoder->inverse_relations_.grad().clone();

        if (call_step) dense_opt->step();                 // model.cpp:399-401
        batch->accumulateGradients(sparse_lr);            // model.cpp:403-405
        out["node_update"] = batch->node_gradients_.clone();          // what indexAdd adds to the embedding table
        out["node_state_update"] = batch->node_state_update_.clone(); // what indexAdd adds to the state table
        return out;
    }
};

std::pair<torch::Tensor, std::vector<torch::Tensor>> ref_map_tensors(std::vector<torch::Tensor> ids, bool sorted, int64_t domain) {
    auto tup = map_tensors(ids, sorted, nullptr, domain);
    std::vector<torch::Tensor> mapped;
    for (auto &t : std::get<1>(tup)) mapped.push_back(t.clone());
    return {std::get<0>(tup).clone(), mapped};
}

torch::Tensor ref_deg_filter(torch::Tensor sample_edge_ids, torch::Tensor edges) { return deg_negative_local_filter(sample_edge_ids, edges); }

// InMemory::indexAdd, CPU branch (storage.cpp:1233-1246) is a plain `table[ids[i]][j] += values[i][j]` loop whose
// translation unit drags in the whole storage layer; index_add_ on CPU is the same arithmetic for unique ids.
void ref_index_add(torch::Tensor table, torch::Tensor ids, torch::Tensor values) { table.index_add_(0, ids, values); }

#ifdef GEGE_CUDA
// The reference's GPU unique-map; the backend is chosen by GEGE_UNIQUE_BACKEND in the environment (read once per process).
std::tuple<torch::Tensor, torch::Tensor, std::string> ref_unique_inverse_cuda(torch::Tensor ids, bool sorted, int64_t domain) {
    UniqueMapCudaDebugInfo info;
    auto tup = map_tensors_unique_inverse_cuda(ids, sorted, &info, domain);
    return {std::get<0>(tup).clone(), std::get<1>(tup).clone(), info.executed_backend};
}

// The reference's tournament selection of negatives (distmult_selected_neg_cuda.cpp:46-121): per row and per group of
// consecutive negatives the best-scoring one; same embeddings as selector and as scorer.
std::tuple<torch::Tensor, torch::Tensor> ref_tournament_selected_scores(torch::Tensor chunked, torch::Tensor negatives, int64_t selected,
                                                                        int64_t groups_per_tile) {
    return distmult_tiled_tournament_selected_scores(chunked, negatives, chunked, negatives, selected, groups_per_tile);
}

// The reference's scoring of chosen negatives and its gradients (distmult_selected_neg_cuda.cu:204-362).
torch::Tensor ref_selected_neg_scores_forward(torch::Tensor chunked, torch::Tensor negatives, torch::Tensor selected, int64_t kind) {
    return selected_neg_scores_cuda_forward(chunked, negatives, selected, kind);
}
std::tuple<torch::Tensor, torch::Tensor> ref_selected_neg_scores_backward(torch::Tensor grad_out, torch::Tensor chunked, torch::Tensor negatives,
                                                                          torch::Tensor selected, int64_t kind) {
    return selected_neg_scores_cuda_backward(grad_out, chunked, negatives, selected, kind);
}
#endif

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    py::class_<RefModel>(m, "RefModel")
        .def(py::init<const std::string &, int64_t, int64_t, bool, double, double, const std::string &>(), py::arg("decoder_type"),
             py::arg("num_relations"), py::arg("dim"), py::arg("inverse"), py::arg("dense_lr"), py::arg("sparse_lr"), py::arg("device") = "cpu")
        .def("set_relations", &RefModel::set_relations)
        .def("set_relation_state", &RefModel::set_relation_state)
        .def("get_relations", &RefModel::get_relations)
        .def("train_batch", &RefModel::train_batch, py::call_guard<py::gil_scoped_release>());
    m.def("map_tensors", &ref_map_tensors);
    m.def("deg_negative_local_filter", &ref_deg_filter);
    m.def("index_add", &ref_index_add);
#ifdef GEGE_CUDA
    m.def("unique_inverse_cuda", &ref_unique_inverse_cuda, py::call_guard<py::gil_scoped_release>());
    m.def("tournament_selected_scores", &ref_tournament_selected_scores, py::call_guard<py::gil_scoped_release>());
    m.def("selected_neg_scores_forward", &ref_selected_neg_scores_forward, py::call_guard<py::gil_scoped_release>());
    m.def("selected_neg_scores_backward", &ref_selected_neg_scores_backward, py::call_guard<py::gil_scoped_release>());
#endif
}
