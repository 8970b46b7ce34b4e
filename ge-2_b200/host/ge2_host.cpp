#include "ge2_host.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <cuda_runtime_api.h>

#include <algorithm>
#include <map>

#include "ge2_b200.h"

namespace ge2host {
namespace {

void check(int rc, const char* what) {
    if (rc != GE2_OK) {
        std::string msg = std::string(what) + ": " + ge2_status_string(rc);
        if (rc == GE2_ERR_CUDA) msg += " (cudaError " + std::to_string(ge2_last_cuda_error()) + ")";
        throw GegeRuntimeException(msg);
    }
}

void require_cuda(const torch::Tensor& t, const char* what) {
    if (!t.defined() || !t.is_cuda()) throw GegeRuntimeException(std::string(what) + " must be a CUDA tensor: this build has no CPU path");
}

ge2_stream_t current_stream(const torch::Tensor& t) { return (ge2_stream_t)at::cuda::getCurrentCUDAStream(t.device().index()).stream(); }

}  // namespace

std::tuple<torch::Tensor, torch::Tensor> map_tensors_unique_inverse_cuda(torch::Tensor all_ids, bool /*sorted*/, int64_t value_domain_size) {
    require_cuda(all_ids, "all_ids");
    TORCH_CHECK(all_ids.scalar_type() == torch::kInt64, "bitmap unique supports int64 tensors");
    TORCH_CHECK(all_ids.dim() == 1, "bitmap unique expects a 1D tensor");
    const int64_t n = all_ids.numel();
    if (n == 0) return {torch::empty({0}, all_ids.options()), torch::empty({0}, all_ids.options())};
    if (value_domain_size <= 0) throw GegeRuntimeException("bitmap unique needs the value domain size (number of nodes resident on the device)");
    c10::cuda::CUDAGuard guard(all_ids.device());
    all_ids = all_ids.contiguous();
    // per-thread workspace cache, like the reference's thread_local bitmap workspace (unique_map_cuda.cu:118-122)
    thread_local torch::Tensor ws, count;
    const size_t need = ge2_unique_workspace_bytes(value_domain_size);
    if (!ws.defined() || ws.device() != all_ids.device() || (size_t)ws.numel() < need)
        ws = torch::empty({(int64_t)need}, all_ids.options().dtype(torch::kUInt8));
    if (!count.defined() || count.device() != all_ids.device()) count = torch::empty({2}, all_ids.options().dtype(torch::kInt32));
    auto unique = torch::empty({std::min(n, value_domain_size)}, all_ids.options());
    auto inverse = torch::empty({n}, all_ids.options());
    check(ge2_unique_bitmap(all_ids.data_ptr<int64_t>(), n, value_domain_size, ws.data_ptr(), (size_t)ws.numel(), unique.data_ptr<int64_t>(),
                            inverse.data_ptr<int64_t>(), count.data_ptr<int32_t>(), current_stream(all_ids)),
          "ge2_unique_bitmap");
    // an exactly sized result needs the count on the host: one read-back (the reference makes four)
    auto h = count.cpu();
    const int32_t u = h[0].item<int32_t>(), status = h[1].item<int32_t>();
    if (status & GE2_STATUS_ID_OUT_OF_RANGE) {
        // the reference falls back to its sort backend here (unique_map_cuda.cu:841-844); same result through torch's device sort
        auto tup = at::_unique2(all_ids, /*sorted=*/true, /*return_inverse=*/true);
        return {std::get<0>(tup), std::get<1>(tup)};
    }
    if (status != 0) throw GegeRuntimeException("unique-map failed on the device (status " + std::to_string(status) + ")");
    return {unique.narrow(0, 0, u), inverse};
}

std::tuple<torch::Tensor, std::vector<torch::Tensor>> map_tensors(std::vector<torch::Tensor> unmapped_tensors, bool sorted, int64_t value_domain_size) {
    if (unmapped_tensors.empty()) throw GegeRuntimeException("Input tensors must not be empty");
    for (const auto& t : unmapped_tensors) {
        if (t.sizes().size() > 1) throw GegeRuntimeException("Input tensors must be 1D");
        require_cuda(t, "map_tensors input");
        if (t.scalar_type() != torch::kInt64 || t.device() != unmapped_tensors.front().device())
            throw GegeRuntimeException("Input tensors must share dtype and device");
    }
    // pack_ids_into_cached_buffer (util.cpp:113-159): one launch gathers up to four strided vectors
    int64_t total = 0;
    for (const auto& t : unmapped_tensors) total += t.numel();
    auto all_ids = torch::empty({total}, unmapped_tensors.front().options());
    c10::cuda::CUDAGuard guard(all_ids.device());
    int64_t off = 0;
    for (size_t base = 0; base < unmapped_tensors.size(); base += 4) {
        const int64_t* parts[4] = {nullptr, nullptr, nullptr, nullptr};
        int64_t lens[4] = {0, 0, 0, 0}, strides[4] = {1, 1, 1, 1};
        int64_t chunk = 0;
        for (size_t k = 0; k < 4 && base + k < unmapped_tensors.size(); k++) {
            const auto& t = unmapped_tensors[base + k];
            parts[k] = t.numel() ? t.data_ptr<int64_t>() : nullptr;
            lens[k] = t.numel();
            strides[k] = t.numel() ? t.stride(0) : 1;
            chunk += t.numel();
        }
        if (chunk > 0) check(ge2_pack_ids(parts, lens, strides, all_ids.data_ptr<int64_t>() + off, current_stream(all_ids)), "ge2_pack_ids");
        off += chunk;
    }
    auto tup = map_tensors_unique_inverse_cuda(all_ids, sorted, value_domain_size);
    std::vector<torch::Tensor> mapped;
    off = 0;
    for (const auto& t : unmapped_tensors) {
        mapped.emplace_back(std::get<1>(tup).narrow(0, off, t.size(0)));
        off += t.size(0);
    }
    return {std::get<0>(tup), mapped};
}

// ---------------------------------------------------------------------------------------------------------------------------
// selected-negative operators
// ---------------------------------------------------------------------------------------------------------------------------
namespace {

torch::Tensor& selected_status_word(const torch::Device& device) {
    thread_local std::map<int, torch::Tensor> words;
    auto& w = words[device.index()];
    if (!w.defined()) w = torch::zeros({1}, torch::dtype(torch::kInt32).device(device));
    return w;
}

struct SelectedShapes {
    int64_t chunks, rows, negs, selected;
    int D;
};

SelectedShapes selected_shapes(const torch::Tensor& chunked, const torch::Tensor& negatives, const torch::Tensor& selected, int64_t score_kind) {
    require_cuda(chunked, "chunked_adjusted_embeddings");
    require_cuda(negatives, "negative_embeddings");
    require_cuda(selected, "selected_neg_indices");
    TORCH_CHECK(chunked.dim() == 3, "chunked_adjusted_embeddings must be rank 3");
    TORCH_CHECK(negatives.dim() == 3, "negative_embeddings must be rank 3");
    TORCH_CHECK(selected.dim() == 2, "selected_neg_indices must be rank 2");
    TORCH_CHECK(chunked.size(0) == negatives.size(0), "chunk and negative chunk counts must match");
    TORCH_CHECK(chunked.size(0) == selected.size(0), "chunk and selected index chunk counts must match");
    TORCH_CHECK(chunked.size(2) == negatives.size(2), "embedding dimensions must match");
    TORCH_CHECK(selected.scalar_type() == torch::kInt64, "selected_neg_indices must be int64");
    TORCH_CHECK(chunked.scalar_type() == torch::kFloat32 && negatives.scalar_type() == torch::kFloat32, "embeddings must be float32");
    TORCH_CHECK(score_kind == GE2_SELECTED_DOT || score_kind == GE2_SELECTED_L2, "score_kind must be DOT or L2");
    SelectedShapes s;
    s.chunks = chunked.size(0);
    s.rows = chunked.size(1);
    s.negs = negatives.size(1);
    s.D = (int)chunked.size(2);
    s.selected = selected.size(1) / std::max<int64_t>(s.rows, 1);
    TORCH_CHECK(selected.size(1) == s.rows * s.selected, "selected_neg_indices width must be num_per_chunk * selected_negatives_num");
    return s;
}

class SelectedNegScores : public torch::autograd::Function<SelectedNegScores> {
   public:
    static torch::autograd::variable_list forward(torch::autograd::AutogradContext* ctx, torch::Tensor chunked, torch::Tensor negatives,
                                                  torch::Tensor selected, int64_t score_kind) {
        auto out = selected_neg_scores_cuda_forward(chunked, negatives, selected, score_kind);
        ctx->save_for_backward({chunked, negatives, selected});
        ctx->saved_data["score_kind"] = score_kind;
        return {out};
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grad_outs) {
        auto saved = ctx->get_saved_variables();
        auto grads = selected_neg_scores_cuda_backward(grad_outs[0], saved[0], saved[1], saved[2], ctx->saved_data["score_kind"].toInt());
        return {std::get<0>(grads), std::get<1>(grads), torch::Tensor(), torch::Tensor()};
    }
};

// the tournament's scores as a function of the scorer's tensors: forward is the selection kernel's output, backward the chosen
// pairs' dot-product gradient (what autograd derives for the reference's bmm -> gather)
class TournamentScores : public torch::autograd::Function<TournamentScores> {
   public:
    static torch::autograd::variable_list forward(torch::autograd::AutogradContext* ctx, torch::Tensor score_chunked, torch::Tensor score_negatives,
                                                  torch::Tensor selector_chunked, torch::Tensor selector_negatives, int64_t selected_num) {
        const int64_t chunks = score_chunked.size(0), rows = score_chunked.size(1), negs = score_negatives.size(1);
        auto scores = torch::empty({chunks * rows, selected_num}, score_chunked.options());
        auto columns = torch::empty({chunks, rows * selected_num}, score_chunked.options().dtype(torch::kInt64));
        check(ge2_tournament_select(selector_chunked.data_ptr<float>(), selector_negatives.data_ptr<float>(), score_chunked.data_ptr<float>(),
                                    score_negatives.data_ptr<float>(), chunks, rows, negs, selected_num, (int)score_chunked.size(2),
                                    scores.data_ptr<float>(), columns.data_ptr<int64_t>(), current_stream(score_chunked)),
              "ge2_tournament_select");
        ctx->save_for_backward({score_chunked, score_negatives, columns});
        ctx->mark_non_differentiable({columns});
        return {scores, columns};
    }
    static torch::autograd::variable_list backward(torch::autograd::AutogradContext* ctx, torch::autograd::variable_list grad_outs) {
        auto saved = ctx->get_saved_variables();
        auto grads = selected_neg_scores_cuda_backward(grad_outs[0], saved[0], saved[1], saved[2], GE2_SELECTED_DOT);
        return {std::get<0>(grads), std::get<1>(grads), torch::Tensor(), torch::Tensor(), torch::Tensor()};
    }
};

}  // namespace

torch::Tensor selected_neg_scores_cuda_forward(torch::Tensor chunked_adjusted_embeddings, torch::Tensor negative_embeddings,
                                               torch::Tensor selected_neg_indices, int64_t score_kind) {
    const SelectedShapes s = selected_shapes(chunked_adjusted_embeddings, negative_embeddings, selected_neg_indices, score_kind);
    c10::cuda::CUDAGuard guard(chunked_adjusted_embeddings.device());
    auto chunked = chunked_adjusted_embeddings.contiguous(), negatives = negative_embeddings.contiguous(), selected = selected_neg_indices.contiguous();
    auto out = torch::empty({s.chunks * s.rows, s.selected}, chunked.options());
    check(ge2_selected_neg_scores((int)score_kind, chunked.data_ptr<float>(), negatives.data_ptr<float>(), selected.data_ptr<int64_t>(), s.chunks,
                                  s.rows, s.negs, s.selected, s.D, out.data_ptr<float>(), selected_status_word(chunked.device()).data_ptr<int32_t>(),
                                  current_stream(chunked)),
          "ge2_selected_neg_scores");
    return out;
}

std::tuple<torch::Tensor, torch::Tensor> selected_neg_scores_cuda_backward(torch::Tensor grad_out, torch::Tensor chunked_adjusted_embeddings,
                                                                           torch::Tensor negative_embeddings, torch::Tensor selected_neg_indices,
                                                                           int64_t score_kind) {
    const SelectedShapes s = selected_shapes(chunked_adjusted_embeddings, negative_embeddings, selected_neg_indices, score_kind);
    require_cuda(grad_out, "grad_out");
    TORCH_CHECK(grad_out.dim() == 2, "grad_out must be rank 2");
    TORCH_CHECK(grad_out.size(0) == s.chunks * s.rows, "grad_out leading dimension must equal chunk_num * num_per_chunk");
    TORCH_CHECK(grad_out.size(1) == s.selected, "selected_neg_indices width must be num_per_chunk * selected_negatives_num");
    c10::cuda::CUDAGuard guard(chunked_adjusted_embeddings.device());
    auto grad = grad_out.contiguous().to(torch::kFloat32);
    auto chunked = chunked_adjusted_embeddings.contiguous(), negatives = negative_embeddings.contiguous(), selected = selected_neg_indices.contiguous();
    auto grad_chunked = torch::empty_like(chunked), grad_negatives = torch::empty_like(negatives);  // the call zeroes grad_negatives
    check(ge2_selected_neg_scores_backward((int)score_kind, grad.data_ptr<float>(), chunked.data_ptr<float>(), negatives.data_ptr<float>(),
                                           selected.data_ptr<int64_t>(), s.chunks, s.rows, s.negs, s.selected, s.D, grad_chunked.data_ptr<float>(),
                                           grad_negatives.data_ptr<float>(), selected_status_word(chunked.device()).data_ptr<int32_t>(),
                                           current_stream(chunked)),
          "ge2_selected_neg_scores_backward");
    return {grad_chunked, grad_negatives};
}

torch::Tensor selected_neg_scores(torch::Tensor chunked_adjusted_embeddings, torch::Tensor negative_embeddings, torch::Tensor selected_neg_indices,
                                  SelectedNegScoreKind score_kind) {
    return SelectedNegScores::apply(chunked_adjusted_embeddings, negative_embeddings, selected_neg_indices, static_cast<int64_t>(score_kind))[0];
}

std::tuple<torch::Tensor, torch::Tensor> distmult_tiled_tournament_selected_scores(torch::Tensor selector_chunked_embeddings,
                                                                                    torch::Tensor selector_negative_embeddings,
                                                                                    torch::Tensor score_chunked_embeddings,
                                                                                    torch::Tensor score_negative_embeddings,
                                                                                    int64_t selected_negatives_num, int64_t /*groups_per_tile*/) {
    for (const auto* t : {&selector_chunked_embeddings, &selector_negative_embeddings, &score_chunked_embeddings, &score_negative_embeddings}) {
        require_cuda(*t, "tournament embeddings");
        TORCH_CHECK(t->dim() == 3, "tournament embeddings must be rank 3");
        TORCH_CHECK(t->scalar_type() == torch::kFloat32, "embeddings must be float32");
    }
    TORCH_CHECK(selector_chunked_embeddings.sizes() == score_chunked_embeddings.sizes(), "selector and score chunked embeddings must match");
    TORCH_CHECK(selector_negative_embeddings.sizes() == score_negative_embeddings.sizes(), "selector and score negative embeddings must match");
    TORCH_CHECK(selector_chunked_embeddings.size(0) == selector_negative_embeddings.size(0), "chunk counts must match");
    TORCH_CHECK(selector_chunked_embeddings.size(2) == selector_negative_embeddings.size(2), "embedding dimensions must match");
    TORCH_CHECK(selected_negatives_num > 0, "selected_negatives_num must be positive");
    TORCH_CHECK(score_negative_embeddings.size(1) % selected_negatives_num == 0, "negatives_num must be divisible by selected_negatives_num");
    c10::cuda::CUDAGuard guard(score_chunked_embeddings.device());
    auto out = TournamentScores::apply(score_chunked_embeddings.contiguous(), score_negative_embeddings.contiguous(),
                                       selector_chunked_embeddings.detach().contiguous(), selector_negative_embeddings.detach().contiguous(),
                                       selected_negatives_num);
    return {out[0], out[1]};
}

int32_t selected_neg_status(torch::Device device) {
    auto& w = selected_status_word(device);
    const int32_t v = w.cpu().item<int32_t>();
    w.zero_();
    return v;
}

void Batch::accumulateGradients(float learning_rate) {
    if (!node_gradients_.defined()) return;
    require_cuda(node_gradients_, "node_gradients_");
    c10::cuda::CUDAGuard guard(node_gradients_.device());
    node_gradients_ = node_gradients_.contiguous();
    node_embeddings_state_ = node_embeddings_state_.contiguous();
    node_state_update_ = torch::empty_like(node_gradients_);
    // state += g*g; node_gradients_ <- -lr * g / (sqrt(state) + 1e-10)   (batch.cpp:264-266 of the reference)
    check(ge2_sparse_adagrad(node_gradients_.data_ptr<float>(), node_embeddings_state_.data_ptr<float>(), node_gradients_.data_ptr<float>(),
                             node_state_update_.data_ptr<float>(), node_gradients_.size(0), nullptr, (int32_t)node_gradients_.size(1),
                             learning_rate, current_stream(node_gradients_)),
          "ge2_sparse_adagrad");
    node_embeddings_state_ = torch::Tensor();  // batch.cpp:275
}

void Batch::clear() { *this = Batch(); }

Model::Model(DecoderType type, int64_t num_relations, int64_t dim, bool use_inverse_relations, float dense_lr, float sparse_lr, torch::Device device,
             const std::string& precision)
    : type_(type), use_inverse_relations_(use_inverse_relations), dense_lr_(dense_lr), sparse_lr_(sparse_lr) {
    if (!device.is_cuda()) throw GegeRuntimeException("Model needs a CUDA device: this build has no CPU path");
    if (precision == "fp32") precision_ = GE2_PRECISION_FP32;
    else if (precision == "f16") precision_ = GE2_PRECISION_F16;
    else throw GegeRuntimeException("precision must be fp32 or f16");
    auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(device);
    auto init = [&]() {  // distmult.cpp:18 (ones) / complex.cpp:18-20 (real part one, imaginary part zero)
        auto t = type == DecoderType::DISTMULT ? torch::ones({num_relations, dim}, opts) : torch::zeros({num_relations, dim}, opts);
        if (type == DecoderType::COMPLEX) t.narrow(1, 0, dim / 2).fill_(1);
        return t;
    };
    // both tables (and their states, and their gradients) back to back: one launch serves them, and the replicated form
    // exchanges them as one buffer
    const int64_t S = use_inverse_relations ? 2 : 1;
    rel_both_ = torch::empty({S, num_relations, dim}, opts);
    state_both_ = torch::zeros({S, num_relations, dim}, opts);
    grad_buf_ = torch::zeros({S * num_relations * dim}, opts);
    for (int64_t k = 0; k < S; k++) rel_both_[k].copy_(init());
    relations_ = rel_both_[0];
    relations_state_ = state_both_[0];
    if (use_inverse_relations) {
        inverse_relations_ = rel_both_[1];
        inverse_relations_state_ = state_both_[1];
    }
    point_at_half(0);
    status_ = torch::zeros({1}, opts.dtype(torch::kInt32));
}

void Model::point_at_half(int half) {
    const int64_t S = rel_both_.size(0), numel = rel_both_.numel();
    auto g = grad_buf_.narrow(0, half * numel, numel).view({S, rel_both_.size(1), rel_both_.size(2)});
    relations_grad_ = g[0];
    if (S == 2) inverse_relations_grad_ = g[1];
}

void Model::broadcast(std::vector<torch::Device> devices) {
    if (devices.empty() || devices[0] != relations_.device()) throw GegeRuntimeException("broadcast: the first device must be this model's");
    if (!device_models_.empty()) throw GegeRuntimeException("broadcast: already replicated");
    const int G = (int)devices.size();
    if (G > 16) throw GegeRuntimeException("broadcast: at most 16 devices");
    const int64_t numel = rel_both_.numel();
    if (numel % 2) throw GegeRuntimeException("broadcast: the relation tables must hold an even number of floats");
    device_models_.push_back(shared_from_this());
    for (int i = 1; i < G; i++) {
        auto m = std::make_shared<Model>(type_, relations_.size(0), relations_.size(1), use_inverse_relations_, dense_lr_, sparse_lr_, devices[i],
                                         precision_ == GE2_PRECISION_F16 ? "f16" : "fp32");
        m->rel_both_.copy_(rel_both_);
        m->state_both_.copy_(state_both_);
        device_models_.push_back(m);
    }
    for (int i = 0; i < G; i++) {
        c10::cuda::CUDAGuard guard(devices[i]);
        for (int j = 0; j < G; j++)
            if (j != i) check(ge2_enable_peer_access(devices[j].index()), "ge2_enable_peer_access");
        auto& m = *device_models_[i];
        auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(devices[i]);
        m.grad_buf_ = torch::zeros({2 * numel + 2 * G + 8}, opts);  // two halves, G flags, verdict, wait counter (8-byte words)
        m.step_dev_ = torch::zeros({1}, opts.dtype(torch::kInt64));
        m.replica_ = i;
        m.round_ = 0;
        m.point_at_half(0);
    }
    std::vector<float*> ptrs;
    for (auto& m : device_models_) ptrs.push_back(m->grad_buf_.data_ptr<float>());
    for (auto& m : device_models_) {
        m->peer_ptrs_ = ptrs;
        if (m.get() != this) m->device_models_ = device_models_;
    }
    for (auto& dv : devices) {
        c10::cuda::CUDAGuard guard(dv);
        check(cudaDeviceSynchronize() == cudaSuccess ? GE2_OK : GE2_ERR_CUDA, "cudaDeviceSynchronize");
    }
}

void Model::all_reduce() {
    if (device_models_.empty()) throw GegeRuntimeException("all_reduce: call broadcast first");
    const int G = (int)device_models_.size();
    const int64_t numel = rel_both_.numel();
    for (int i = 0; i < G; i++) {
        auto& m = *device_models_[i];
        c10::cuda::CUDAGuard guard(m.relations_.device());
        auto stream = current_stream(m.relations_);
        // sum over the replicas' halves (read over peer memory), divide by G, Adagrad on both tables, clear the other half
        check(ge2_dense_adagrad_peers(m.rel_both_.data_ptr<float>(), m.state_both_.data_ptr<float>(), m.peer_ptrs_.data(), G, i, numel,
                                      reinterpret_cast<const uint64_t*>(m.step_dev_.data_ptr<int64_t>()), m.dense_lr_, 1e-10f, 1.0f / G, 0,
                                      m.status_.data_ptr<int32_t>(), stream),
              "ge2_dense_adagrad_peers");
        check(ge2_advance_step(reinterpret_cast<uint64_t*>(m.step_dev_.data_ptr<int64_t>()), 1, stream), "ge2_advance_step");
        m.round_ += 1;
        m.point_at_half((int)(m.round_ & 1));
    }
}

void Model::check_status() {
    std::vector<std::shared_ptr<Model>> all = device_models_;
    if (all.empty()) {
        const int32_t word = status_.cpu().item<int32_t>();
        if (word) throw GegeRuntimeException("device status " + std::to_string(word));
        return;
    }
    for (auto& m : all) {
        const int32_t word = m->status_.cpu().item<int32_t>();
        if (word) throw GegeRuntimeException("device status " + std::to_string(word) + " on replica " + std::to_string(m->replica_));
    }
}

void Model::clear_grad() {
    if (!device_models_.empty()) return;  // replicated form: all_reduce clears the half the round after next accumulates into
    relations_grad_.zero_();
    if (inverse_relations_grad_.defined()) inverse_relations_grad_.zero_();
}

void Model::step() { step_after_all_reduce(1.0f); }

void Model::step_after_all_reduce(float grad_scale) {
    c10::cuda::CUDAGuard guard(relations_.device());
    // relation and inverse-relation tables, states and gradients sit back to back: one launch
    check(ge2_dense_adagrad(rel_both_.data_ptr<float>(), state_both_.data_ptr<float>(), relations_grad_.data_ptr<float>(), rel_both_.numel(),
                            dense_lr_, 1e-10f, grad_scale, 0, current_stream(relations_)),
          "ge2_dense_adagrad");
}

void Model::train_batch(std::shared_ptr<Batch> batch, bool call_step) {
    if (call_step) clear_grad();  // model.cpp:363-365
    require_cuda(batch->node_embeddings_, "node_embeddings_");
    require_cuda(batch->edges_, "edges_");
    c10::cuda::CUDAGuard guard(batch->node_embeddings_.device());
    const int cols = (int)batch->edges_.size(1);
    if (cols != 2 && cols != 3) throw GegeRuntimeException("Edge list must be a 3 or 2 column tensor");  // decoder_methods.cpp:739
    auto edges = batch->edges_.contiguous();
    auto emb = batch->node_embeddings_.contiguous();
    auto dst_negs = batch->dst_neg_indices_mapping_.contiguous();
    torch::Tensor src_negs, dst_filter, src_filter;
    ge2_lp_desc d{};
    d.decoder = type_ == DecoderType::COMPLEX ? GE2_DECODER_COMPLEX : GE2_DECODER_DISTMULT;
    d.precision = precision_;
    d.has_relations = cols == 3;
    d.use_inverse = d.has_relations && use_inverse_relations_;
    d.B = (int32_t)edges.size(0);
    d.C = (int32_t)dst_negs.size(0);
    d.N = (int32_t)dst_negs.size(1);
    d.D = (int32_t)emb.size(1);
    d.R = (int32_t)relations_.size(0);
    d.U = emb.size(0);
    d.node_emb = emb.data_ptr<float>();
    d.emb_stride = d.D;
    const int64_t* e = edges.data_ptr<int64_t>();
    d.src_ids = e;
    d.dst_ids = e + cols - 1;
    d.rel_ids = cols == 3 ? e + 1 : nullptr;
    d.edge_stride = d.rel_stride = cols;
    d.dst_negs = dst_negs.data_ptr<int64_t>();
    if (d.use_inverse) {
        src_negs = batch->src_neg_indices_mapping_.contiguous();
        d.src_negs = src_negs.data_ptr<int64_t>();
    }
    torch::Tensor deg_rows;
    if (batch->deg_sample_rows_.defined() && batch->deg_sample_rows_.numel() > 0) {
        deg_rows = batch->deg_sample_rows_.contiguous();
        d.deg_sample_rows = deg_rows.data_ptr<int64_t>();
        d.n_deg = (int32_t)deg_rows.size(1);
    } else if (batch->dst_neg_filter_.defined() && batch->dst_neg_filter_.size(0) > 0) {
        dst_filter = batch->dst_neg_filter_.contiguous();
        d.dst_filter = dst_filter.data_ptr<int64_t>();
        d.dst_filter_n = dst_filter.size(0);
    }
    if (!deg_rows.defined() && d.use_inverse && batch->src_neg_filter_.defined() && batch->src_neg_filter_.size(0) > 0) {
        src_filter = batch->src_neg_filter_.contiguous();
        d.src_filter = src_filter.data_ptr<int64_t>();
        d.src_filter_n = src_filter.size(0);
    }
    d.rel = relations_.data_ptr<float>();
    d.rel_grad = relations_grad_.data_ptr<float>();
    if (d.use_inverse) {
        d.inv_rel = inverse_relations_.data_ptr<float>();
        d.inv_rel_grad = inverse_relations_grad_.data_ptr<float>();
    }
    batch->node_gradients_ = torch::empty_like(emb);
    batch->loss_ = torch::empty({1}, emb.options());
    d.node_grad = batch->node_gradients_.data_ptr<float>();
    d.loss = batch->loss_.data_ptr<float>();
    d.status = status_.data_ptr<int32_t>();
    size_t ws = 0;
    check(ge2_lp_workspace_bytes(&d, &ws), "ge2_lp_workspace_bytes");
    if (!workspace_.defined() || (size_t)workspace_.numel() < ws) workspace_ = torch::empty({(int64_t)ws}, emb.options().dtype(torch::kUInt8));
    d.workspace = workspace_.data_ptr();
    d.workspace_bytes = (size_t)workspace_.numel();
    check(ge2_lp_step(&d, current_stream(emb)), "ge2_lp_step");
    if (call_step) step();                                            // model.cpp:399-401
    if (batch->node_embeddings_.defined()) batch->accumulateGradients(sparse_lr_);  // model.cpp:403-405
}

torch::Tensor InMemory::indexRead(Indices indices) {
    if (indices.sizes().size() != 1) throw std::runtime_error("");  // storage.cpp:1174-1177
    require_cuda(data_, "storage data");
    c10::cuda::CUDAGuard guard(data_.device());
    indices = indices.to(data_.device()).contiguous();
    auto out = torch::empty({indices.size(0), data_.size(1)}, data_.options());
    if (!status_.defined()) status_ = torch::zeros({1}, data_.options().dtype(torch::kInt32));
    check(ge2_index_read(data_.data_ptr<float>(), data_.size(0), indices.data_ptr<int64_t>(), indices.size(0), nullptr, (int32_t)data_.size(1),
                         out.data_ptr<float>(), status_.data_ptr<int32_t>(), current_stream(data_)),
          "ge2_index_read");
    return out;
}

void InMemory::checkStatus() {
    if (!status_.defined()) return;
    const int32_t word = status_.cpu().item<int32_t>();
    if (word) {
        status_.zero_();
        throw GegeRuntimeException("storage index out of range (device status " + std::to_string(word) + ")");
    }
}

void InMemory::indexAdd(Indices indices, torch::Tensor values) {
    if (!values.defined() || indices.sizes().size() != 1 || indices.size(0) != values.size(0) || data_.size(1) != values.size(1))
        throw std::runtime_error("");  // storage.cpp:1187-1190
    require_cuda(values, "values");
    c10::cuda::CUDAGuard guard(data_.device());
    indices = indices.contiguous();
    values = values.contiguous();
    if (!status_.defined()) status_ = torch::zeros({1}, data_.options().dtype(torch::kInt32));
    check(ge2_index_add(data_.data_ptr<float>(), data_.size(0), indices.data_ptr<int64_t>(), indices.size(0), nullptr, (int32_t)data_.size(1),
                        values.data_ptr<float>(), status_.data_ptr<int32_t>(), current_stream(data_)),
          "ge2_index_add");
}

// ---------------------------------------------------------------------------------------------------------------------
// MemPartitionBufferStorage
// ---------------------------------------------------------------------------------------------------------------------
namespace {
constexpr int kCapacity = 4;  // buffer_capacity of the reference's relay (buffer.cpp:950,1106)
}

MemPartitionBufferStorage::MemPartitionBufferStorage(int64_t dim0_size, int64_t dim1_size, int32_t num_partitions, std::vector<torch::Device> devices)
    : dim0_(dim0_size), dim1_(dim1_size), num_partitions_(num_partitions), devices_(std::move(devices)) {
    if (devices_.empty() || devices_.size() > 16) throw GegeRuntimeException("MemPartitionBufferStorage needs 1 to 16 CUDA devices");
    if (num_partitions <= 0 || dim0_size <= 0 || dim1_size <= 0) throw GegeRuntimeException("MemPartitionBufferStorage: bad sizes");
    partition_size_ = (dim0_ + num_partitions_ - 1) / num_partitions_;  // ceil, storage.cpp:368
    if ((partition_size_ * dim1_ * 4) % 16) throw GegeRuntimeException("MemPartitionBufferStorage: a slab must be a multiple of 16 bytes");
    const int G = (int)devices_.size();
    for (int g = 0; g < G; g++) {
        if (!devices_[g].is_cuda()) throw GegeRuntimeException("MemPartitionBufferStorage: CUDA devices only");
        c10::cuda::CUDAGuard guard(devices_[g]);
        for (int j = 0; j < G; j++)
            if (j != g) check(ge2_enable_peer_access(devices_[j].index()), "ge2_enable_peer_access");
        auto opts = torch::TensorOptions().dtype(torch::kFloat32).device(devices_[g]);
        const int64_t n_home = (num_partitions_ - g + G - 1) / G;  // partitions p with p % G == g
        home_.push_back(torch::zeros({std::max<int64_t>(n_home, 1) * partition_size_, dim1_}, opts));
        bufs_.push_back({torch::zeros({kCapacity * partition_size_, dim1_}, opts), torch::zeros({kCapacity * partition_size_, dim1_}, opts)});
        flags_.push_back(torch::zeros({G + 1}, opts.dtype(torch::kInt64)));
        status_.push_back(torch::zeros({1}, opts.dtype(torch::kInt32)));
    }
    epoch_.assign(G, 0);
    next_.assign(G, 0);
    resident_.assign(G, std::vector<int64_t>(kCapacity, -1));
}

void MemPartitionBufferStorage::load(torch::Tensor values) {
    if (values.dim() != 2 || values.size(0) != dim0_ || values.size(1) != dim1_) throw GegeRuntimeException("load: expected the whole [dim0, dim1] table");
    const int G = (int)devices_.size();
    for (int p = 0; p < num_partitions_; p++) {
        const int64_t begin = p * partition_size_, rows = std::min(partition_size_, dim0_ - begin);
        if (rows <= 0) continue;
        home_[p % G].narrow(0, (p / G) * partition_size_, rows).copy_(values.narrow(0, begin, rows));
    }
}

MemPartitionBufferStorage::Plan MemPartitionBufferStorage::make_plan(const std::vector<std::vector<int64_t>>& current,
                                                                     const std::vector<std::vector<int64_t>>& next_states) {
    // every device's next buffer is filled slot by slot (the state's partitions in ascending order) from wherever each
    // partition is now -- a slot of some device's current buffer (the relay copy of storage.cpp:626-652) or its home slab --
    // and a resident partition that nobody keeps is pulled by its home device
    const int G = (int)devices_.size();
    std::map<int64_t, std::pair<int, int>> in_buffer;
    for (int g = 0; g < G; g++)
        for (int k = 0; k < kCapacity; k++)
            if (current[g][k] >= 0) in_buffer[current[g][k]] = {g, k};
    Plan plan;
    plan.slots.assign(G, std::vector<int64_t>(kCapacity, -1));
    plan.pulls.assign(G, {});
    std::map<int64_t, int> claimed;
    for (int g = 0; g < G; g++) {
        std::vector<int64_t> st = next_states[g];
        std::sort(st.begin(), st.end());
        if ((int)st.size() > kCapacity || std::adjacent_find(st.begin(), st.end()) != st.end())
            throw GegeRuntimeException("a state holds at most 4 distinct partitions");
        for (size_t k = 0; k < st.size(); k++) {
            const int64_t p = st[k];
            if (p < 0 || p >= num_partitions_) throw GegeRuntimeException("partition id out of range");
            if (claimed.count(p)) throw GegeRuntimeException("the states of a superstep must be disjoint");
            claimed[p] = g;
            plan.slots[g][k] = p;
            auto it = in_buffer.find(p);
            if (it != in_buffer.end()) plan.pulls[g].push_back({false, false, it->second.first, it->second.second, (int64_t)k});
            else plan.pulls[g].push_back({true, false, (int)(p % G), p / G, (int64_t)k});
        }
    }
    for (auto& kv : in_buffer)
        if (!claimed.count(kv.first)) plan.pulls[kv.first % G].push_back({false, true, kv.second.first, kv.second.second, kv.first / G});
    return plan;
}

void MemPartitionBufferStorage::setBufferOrdering(std::vector<torch::Tensor> buffer_states) {
    const int G = (int)devices_.size();
    if (buffer_states.size() % G) throw GegeRuntimeException("setBufferOrdering: the number of states must be a multiple of the device count");
    plans_.clear();
    auto cur = resident_;
    for (auto& n : next_)
        if (n != 0) throw GegeRuntimeException("setBufferOrdering: swaps already in progress");
    for (size_t k = 0; k < buffer_states.size() / G; k++) {
        std::vector<std::vector<int64_t>> st(G);
        for (int g = 0; g < G; g++) {
            auto t = buffer_states[k * G + g].to(torch::kCPU).to(torch::kInt64).contiguous();
            st[g].assign(t.data_ptr<int64_t>(), t.data_ptr<int64_t>() + t.numel());
        }
        plans_.push_back(make_plan(cur, st));
        cur = plans_.back().slots;
    }
    plans_.push_back(make_plan(cur, std::vector<std::vector<int64_t>>(G)));  // the flush: everything goes home
}

bool MemPartitionBufferStorage::hasSwap(int32_t device_idx) { return next_.at(device_idx) + 1 < plans_.size(); }

void MemPartitionBufferStorage::run_plan(const Plan& plan, int32_t g) {
    const int G = (int)devices_.size();
    c10::cuda::CUDAGuard guard(devices_[g]);
    // after its n-th swap a device's active buffer is buffer n & 1, so the sources of swap n are the devices' buffers
    // (n - 1) & 1 wherever their host threads are; the device-side barrier makes the data ready
    const int old = (int)(next_[g] & 1), nw = old ^ 1;
    const int64_t slab_bytes = partition_size_ * dim1_ * 4;
    std::vector<const void*> src;
    std::vector<void*> dst;
    for (const auto& pl : plan.pulls[g]) {
        const char* s = pl.src_home ? (const char*)home_[pl.src_dev].data_ptr<float>() : (const char*)bufs_[pl.src_dev][old].data_ptr<float>();
        char* d = pl.dst_home ? (char*)home_[g].data_ptr<float>() : (char*)bufs_[g][nw].data_ptr<float>();
        src.push_back(s + pl.src_index * slab_bytes);
        dst.push_back(d + pl.dst_index * slab_bytes);
    }
    std::vector<void*> rows;
    for (int j = 0; j < G; j++) rows.push_back(flags_[j].data_ptr<int64_t>());
    ge2_swap_desc d{};
    d.world = G;
    d.rank = g;
    d.flag_rows = rows.data();
    d.epoch = ++epoch_[g];
    d.wait_budget_us = 0;
    d.num_pulls = (int32_t)src.size();
    d.pull_src = src.data();
    d.pull_dst = dst.data();
    d.slab_bytes = slab_bytes;
    d.status = status_[g].data_ptr<int32_t>();
    check(ge2_swap_begin(&d, (ge2_stream_t)at::cuda::getCurrentCUDAStream(devices_[g].index()).stream()), "ge2_swap_begin");
}

void MemPartitionBufferStorage::performNextSwap(int32_t device_idx) {
    if (!hasSwap(device_idx)) throw GegeRuntimeException("performNextSwap: no swap left");
    run_plan(plans_[next_[device_idx]], device_idx);
    next_[device_idx] += 1;
}

std::vector<int> MemPartitionBufferStorage::getNextAdmit(int32_t g) {
    std::vector<int> out;
    if (next_.at(g) >= plans_.size()) return out;
    const auto& cur = next_[g] == 0 ? resident_[g] : plans_[next_[g] - 1].slots[g];
    for (auto p : plans_[next_[g]].slots[g])
        if (p >= 0 && std::find(cur.begin(), cur.end(), p) == cur.end()) out.push_back((int)p);
    return out;
}

std::vector<int> MemPartitionBufferStorage::getNextEvict(int32_t g) {
    std::vector<int> out;
    if (next_.at(g) >= plans_.size()) return out;
    const auto& cur = next_[g] == 0 ? resident_[g] : plans_[next_[g] - 1].slots[g];
    const auto& nxt = plans_[next_[g]].slots[g];
    for (auto p : cur)
        if (p >= 0 && std::find(nxt.begin(), nxt.end(), p) == nxt.end()) out.push_back((int)p);
    return out;
}

torch::Tensor MemPartitionBufferStorage::getPartitionToBufferSlotMap(int32_t g) {
    auto map = torch::full({num_partitions_}, -1, torch::kInt64);
    const auto& cur = next_.at(g) == 0 ? resident_[g] : plans_[next_[g] - 1].slots[g];
    for (int k = 0; k < kCapacity; k++)
        if (cur[k] >= 0) map[cur[k]] = k;
    return map;
}

torch::Tensor MemPartitionBufferStorage::activeBuffer(int32_t g) {
    return bufs_.at(g)[next_[g] & 1];
}

torch::Tensor MemPartitionBufferStorage::indexRead(Indices indices, int32_t device_idx) { return InMemory(activeBuffer(device_idx)).indexRead(indices); }

void MemPartitionBufferStorage::indexAdd(Indices indices, torch::Tensor values, int32_t device_idx) {
    InMemory(activeBuffer(device_idx)).indexAdd(indices, values);
}

torch::Tensor MemPartitionBufferStorage::unload() {
    const int G = (int)devices_.size();
    if (!plans_.empty()) {
        for (int g = 0; g < G; g++) {
            if (next_[g] + 1 != plans_.size()) throw GegeRuntimeException("unload: supersteps left");
        }
        const bool odd = next_[0] & 1;
        for (int g = 0; g < G; g++) run_plan(plans_.back(), g);
        if (odd)  // the next ordering starts from buffer 0 again: nothing is resident, only the numbering restarts
            for (int g = 0; g < G; g++) std::swap(bufs_[g][0], bufs_[g][1]);
        for (int g = 0; g < G; g++) next_[g] = 0;
        plans_.clear();
        resident_.assign(G, std::vector<int64_t>(kCapacity, -1));
    }
    checkStatus();
    auto out = torch::empty({dim0_, dim1_}, torch::kFloat32);
    for (int p = 0; p < num_partitions_; p++) {
        const int64_t begin = p * partition_size_, rows = std::min(partition_size_, dim0_ - begin);
        if (rows <= 0) continue;
        out.narrow(0, begin, rows).copy_(home_[p % G].narrow(0, (p / G) * partition_size_, rows));
    }
    return out;
}

void MemPartitionBufferStorage::checkStatus() {
    for (size_t g = 0; g < devices_.size(); g++) {
        c10::cuda::CUDAGuard guard(devices_[g]);
        const int32_t word = status_[g].cpu().item<int32_t>();  // synchronises the device's current stream
        if (word) throw GegeRuntimeException("partition swap failed on device " + std::to_string(g) + " (status " + std::to_string(word) + ")");
    }
}

// ---------------------------------------------------------------------------------------------------------------------
// DataLoader
// ---------------------------------------------------------------------------------------------------------------------
DataLoader::DataLoader(torch::Tensor edges, std::shared_ptr<InMemory> node_embeddings, std::shared_ptr<InMemory> node_embeddings_state,
                       int64_t batch_size, int32_t num_chunks, int32_t negatives_per_chunk, float degree_fraction, bool inverse_edges, uint64_t seed)
    : edges_(edges.contiguous()), emb_(std::move(node_embeddings)), state_(std::move(node_embeddings_state)), B_(batch_size), C_(num_chunks),
      N_(negatives_per_chunk), seed_(seed) {
    require_cuda(edges_, "edges");
    if (edges_.dim() != 2 || (edges_.size(1) != 2 && edges_.size(1) != 3) || edges_.scalar_type() != torch::kInt64)
        throw GegeRuntimeException("edges must be an int64 [n, 2|3] tensor");
    if (edges_.size(0) < B_) throw GegeRuntimeException("fewer edges than one batch");
    n_deg_ = (int32_t)(N_ * degree_fraction);                       // negative.cpp:608
    want_src_ = edges_.size(1) == 3 && inverse_edges;                // dataloader.cpp:1321
    const int64_t n_ids = 2 * B_ + (want_src_ ? 2 : 1) * (int64_t)C_ * N_;
    packed_ = torch::empty({n_ids}, edges_.options());
    deg_rows_ = torch::empty({C_, std::max(n_deg_, 1)}, edges_.options());
}

std::shared_ptr<Batch> DataLoader::getBatch() {
    c10::cuda::CUDAGuard guard(edges_.device());
    const int64_t cols = edges_.size(1), nb = edges_.size(0) / B_, b = batch_id_ % nb;
    const int64_t domain = emb_->data_.size(0);
    auto slice = edges_.narrow(0, b * B_, B_);
    const int64_t* e = slice.data_ptr<int64_t>();
    check(ge2_sample_negatives(e, e + cols - 1, cols, (int32_t)B_, C_, N_, n_deg_, domain, want_src_ ? 1 : 0, seed_, (uint64_t)batch_id_,
                               packed_.data_ptr<int64_t>(), n_deg_ > 0 ? deg_rows_.data_ptr<int64_t>() : nullptr, current_stream(edges_)),
          "ge2_sample_negatives");
    batch_id_ += 1;
    auto tup = map_tensors_unique_inverse_cuda(packed_, true, domain);
    auto batch = std::make_shared<Batch>();
    batch->unique_node_indices_ = std::get<0>(tup);
    const auto& inv = std::get<1>(tup);
    const int64_t CN = (int64_t)C_ * N_;
    auto src_l = inv.narrow(0, 0, B_), dst_l = inv.narrow(0, B_, B_);
    batch->edges_ = cols == 3 ? torch::stack({src_l, slice.select(1, 1), dst_l}, 1) : torch::stack({src_l, dst_l}, 1);
    int64_t off = 2 * B_;
    if (want_src_) {
        batch->src_neg_indices_mapping_ = inv.narrow(0, off, CN).view({C_, N_});
        off += CN;
    }
    batch->dst_neg_indices_mapping_ = inv.narrow(0, off, CN).view({C_, N_});
    if (n_deg_ > 0) batch->deg_sample_rows_ = deg_rows_.narrow(1, 0, n_deg_).clone();
    batch->node_embeddings_ = emb_->indexRead(batch->unique_node_indices_);            // loadGPUParameters, dataloader.cpp:1354-1379
    batch->node_embeddings_state_ = state_->indexRead(batch->unique_node_indices_);
    return batch;
}

void DataLoader::updateEmbeddings(std::shared_ptr<Batch> batch) {
    emb_->indexAdd(batch->unique_node_indices_, batch->node_gradients_);       // dataloader.cpp:1381-1395
    state_->indexAdd(batch->unique_node_indices_, batch->node_state_update_);
}

}  // namespace ge2host
