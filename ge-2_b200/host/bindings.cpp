// Python binding of the host layer (module ge2_host), used by the tests; same class and member names as the reference's
// own pybind modules (python_bindings/ of the reference project) for the members that exist here.
#include <torch/extension.h>

#include "ge2_host.h"

using namespace ge2host;

PYBIND11_MODULE(ge2_host, m) {
    py::register_exception<GegeRuntimeException>(m, "GegeRuntimeException");
    m.def("map_tensors", &map_tensors, py::arg("unmapped_tensors"), py::arg("sorted") = true, py::arg("value_domain_size") = -1);
    m.def("map_tensors_unique_inverse_cuda", &map_tensors_unique_inverse_cuda, py::arg("all_ids"), py::arg("sorted") = true,
          py::arg("value_domain_size") = -1);
    py::enum_<SelectedNegScoreKind>(m, "SelectedNegScoreKind")
        .value("NONE", SelectedNegScoreKind::NONE)
        .value("DOT", SelectedNegScoreKind::DOT)
        .value("L2", SelectedNegScoreKind::L2);
    m.def("selected_neg_scores", &selected_neg_scores);
    m.def("selected_neg_scores_cuda_forward", &selected_neg_scores_cuda_forward);
    m.def("selected_neg_scores_cuda_backward", &selected_neg_scores_cuda_backward);
    m.def("distmult_tiled_tournament_selected_scores", &distmult_tiled_tournament_selected_scores);
    m.def("selected_neg_status", &selected_neg_status);
    py::class_<Batch, std::shared_ptr<Batch>>(m, "Batch")
        .def(py::init<>())
        .def_readwrite("unique_node_indices", &Batch::unique_node_indices_)
        .def_readwrite("node_embeddings", &Batch::node_embeddings_)
        .def_readwrite("node_gradients", &Batch::node_gradients_)
        .def_readwrite("node_embeddings_state", &Batch::node_embeddings_state_)
        .def_readwrite("node_state_update", &Batch::node_state_update_)
        .def_readwrite("src_neg_indices_mapping", &Batch::src_neg_indices_mapping_)
        .def_readwrite("dst_neg_indices_mapping", &Batch::dst_neg_indices_mapping_)
        .def_readwrite("edges", &Batch::edges_)
        .def_readwrite("src_neg_filter", &Batch::src_neg_filter_)
        .def_readwrite("dst_neg_filter", &Batch::dst_neg_filter_)
        .def_readwrite("deg_sample_rows", &Batch::deg_sample_rows_)
        .def_readwrite("loss", &Batch::loss_)
        .def("accumulateGradients", &Batch::accumulateGradients)
        .def("clear", &Batch::clear);
    py::enum_<DecoderType>(m, "DecoderType").value("DISTMULT", DecoderType::DISTMULT).value("COMPLEX", DecoderType::COMPLEX);
    py::class_<Model, std::shared_ptr<Model>>(m, "Model")
        .def(py::init<DecoderType, int64_t, int64_t, bool, float, float, torch::Device, const std::string&>(), py::arg("type"),
             py::arg("num_relations"), py::arg("dim"), py::arg("use_inverse_relations"), py::arg("dense_lr"), py::arg("sparse_lr"),
             py::arg("device"), py::arg("precision") = "fp32")
        .def("train_batch", &Model::train_batch, py::arg("batch"), py::arg("call_step") = true)
        .def("step", &Model::step)
        .def("clear_grad", &Model::clear_grad)
        .def("step_after_all_reduce", &Model::step_after_all_reduce)
        .def("broadcast", &Model::broadcast)
        .def("all_reduce", &Model::all_reduce)
        .def("check_status", &Model::check_status)
        .def_readonly("device_models", &Model::device_models_)
        // the tables are views of one allocation (both tables back to back): assignment copies into them
        .def_property("relations", [](Model& m) { return m.relations_; }, [](Model& m, torch::Tensor v) { m.relations_.copy_(v); })
        .def_property("inverse_relations", [](Model& m) { return m.inverse_relations_; }, [](Model& m, torch::Tensor v) { m.inverse_relations_.copy_(v); })
        .def_property("relations_state", [](Model& m) { return m.relations_state_; }, [](Model& m, torch::Tensor v) { m.relations_state_.copy_(v); })
        .def_property("inverse_relations_state", [](Model& m) { return m.inverse_relations_state_; },
                      [](Model& m, torch::Tensor v) { m.inverse_relations_state_.copy_(v); })
        .def_readonly("relations_grad", &Model::relations_grad_)
        .def_readonly("inverse_relations_grad", &Model::inverse_relations_grad_);
    py::class_<MemPartitionBufferStorage, std::shared_ptr<MemPartitionBufferStorage>>(m, "MemPartitionBufferStorage")
        .def(py::init<int64_t, int64_t, int32_t, std::vector<torch::Device>>(), py::arg("dim0_size"), py::arg("dim1_size"), py::arg("num_partitions"),
             py::arg("devices"))
        .def("load", &MemPartitionBufferStorage::load)
        .def("unload", &MemPartitionBufferStorage::unload)
        .def("setBufferOrdering", &MemPartitionBufferStorage::setBufferOrdering)
        .def("hasSwap", &MemPartitionBufferStorage::hasSwap, py::arg("device_idx") = 0)
        .def("performNextSwap", &MemPartitionBufferStorage::performNextSwap)
        .def("getNextAdmit", &MemPartitionBufferStorage::getNextAdmit, py::arg("device_idx") = 0)
        .def("getNextEvict", &MemPartitionBufferStorage::getNextEvict, py::arg("device_idx") = 0)
        .def("getPartitionToBufferSlotMap", &MemPartitionBufferStorage::getPartitionToBufferSlotMap, py::arg("device_idx") = 0)
        .def("indexRead", &MemPartitionBufferStorage::indexRead)
        .def("indexAdd", &MemPartitionBufferStorage::indexAdd)
        .def("activeBuffer", &MemPartitionBufferStorage::activeBuffer)
        .def("getPartitionSize", &MemPartitionBufferStorage::getPartitionSize, py::arg("device_idx") = 0)
        .def("getNumInMemory", &MemPartitionBufferStorage::getNumInMemory, py::arg("device_idx") = 0)
        .def("checkStatus", &MemPartitionBufferStorage::checkStatus);
    py::class_<DataLoader, std::shared_ptr<DataLoader>>(m, "DataLoader")
        .def(py::init<torch::Tensor, std::shared_ptr<InMemory>, std::shared_ptr<InMemory>, int64_t, int32_t, int32_t, float, bool, uint64_t>(),
             py::arg("edges"), py::arg("node_embeddings"), py::arg("node_embeddings_state"), py::arg("batch_size"), py::arg("num_chunks"),
             py::arg("negatives_per_chunk"), py::arg("degree_fraction"), py::arg("inverse_edges"), py::arg("seed"))
        .def("getBatch", &DataLoader::getBatch)
        .def("updateEmbeddings", &DataLoader::updateEmbeddings)
        .def_readwrite("batch_id", &DataLoader::batch_id_);
    py::class_<InMemory, std::shared_ptr<InMemory>>(m, "InMemory")
        .def(py::init<torch::Tensor>())
        .def("indexRead", &InMemory::indexRead)
        .def("indexAdd", &InMemory::indexAdd)
        .def("checkStatus", &InMemory::checkStatus)
        .def_readwrite("data", &InMemory::data_);
}
