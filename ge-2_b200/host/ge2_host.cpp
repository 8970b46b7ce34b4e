#include "ge2_host.h"

#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>

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
    relations_ = init();
    relations_grad_ = torch::zeros_like(relations_);
    relations_state_ = torch::zeros_like(relations_);
    if (use_inverse_relations) {
        inverse_relations_ = init();
        inverse_relations_grad_ = torch::zeros_like(relations_);
        inverse_relations_state_ = torch::zeros_like(relations_);
    }
    status_ = torch::zeros({1}, opts.dtype(torch::kInt32));
}

void Model::clear_grad() {
    relations_grad_.zero_();
    if (inverse_relations_grad_.defined()) inverse_relations_grad_.zero_();
}

void Model::step() { step_after_all_reduce(1.0f); }

void Model::step_after_all_reduce(float grad_scale) {
    c10::cuda::CUDAGuard guard(relations_.device());
    check(ge2_dense_adagrad(relations_.data_ptr<float>(), relations_state_.data_ptr<float>(), relations_grad_.data_ptr<float>(), relations_.numel(),
                            dense_lr_, 1e-10f, grad_scale, 0, current_stream(relations_)),
          "ge2_dense_adagrad");
    if (inverse_relations_.defined())
        check(ge2_dense_adagrad(inverse_relations_.data_ptr<float>(), inverse_relations_state_.data_ptr<float>(),
                                inverse_relations_grad_.data_ptr<float>(), inverse_relations_.numel(), dense_lr_, 1e-10f, grad_scale, 0,
                                current_stream(relations_)),
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
    if (batch->dst_neg_filter_.defined() && batch->dst_neg_filter_.size(0) > 0) {
        dst_filter = batch->dst_neg_filter_.contiguous();
        d.dst_filter = dst_filter.data_ptr<int64_t>();
        d.dst_filter_n = dst_filter.size(0);
    }
    if (d.use_inverse && batch->src_neg_filter_.defined() && batch->src_neg_filter_.size(0) > 0) {
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
    check(ge2_index_read(data_.data_ptr<float>(), data_.size(0), indices.data_ptr<int64_t>(), indices.size(0), nullptr, (int32_t)data_.size(1),
                         out.data_ptr<float>(), nullptr, current_stream(data_)),
          "ge2_index_read");
    return out;
}

void InMemory::indexAdd(Indices indices, torch::Tensor values) {
    if (!values.defined() || indices.sizes().size() != 1 || indices.size(0) != values.size(0) || data_.size(1) != values.size(1))
        throw std::runtime_error("");  // storage.cpp:1187-1190
    require_cuda(values, "values");
    c10::cuda::CUDAGuard guard(data_.device());
    indices = indices.contiguous();
    values = values.contiguous();
    check(ge2_index_add(data_.data_ptr<float>(), data_.size(0), indices.data_ptr<int64_t>(), indices.size(0), nullptr, (int32_t)data_.size(1),
                        values.data_ptr<float>(), nullptr, current_stream(data_)),
          "ge2_index_add");
}

}  // namespace ge2host
