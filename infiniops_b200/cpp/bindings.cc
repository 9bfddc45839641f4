// pybind11 module `infini.ops`: the Python face of the operators.
//
// Mirrors what the reference generates per operator (scripts/generate_wrappers.py:612-998): a
// snake_case function taking the operator's arguments positionally plus keyword-only `stream`
// (an integer `cudaStream_t`, 0 = default stream) and `implementation_index` (None = first active
// slot); and a PascalCase class built from the same arguments whose instances are called with
// them again, with static `active_implementation_indices(device)` and `clear_cache()`.
// Tensors are any Python objects with `data_ptr()`, `shape`, `dtype`, `device.type/.index` and
// `stride()` (src/pybind11_utils.h:248-266); `bool` travels as uint8.  Functions return None;
// outputs are caller-allocated.
#include "binding_utils.h"

void RegisterMoeBindings(pybind11::module_& m);
void RegisterSiblingBindings(pybind11::module_& m);

PYBIND11_MODULE(ops, m) {
  m.doc() = "B200 (sm_100a) W4A16 linear and MoE operators behind the infini.ops interface";

  // ---- gptq_marlin_repack ---------------------------------------------------------------------
  m.def("gptq_marlin_repack",
        [](py::object w, py::object perm, int64_t k, int64_t n, int64_t bits, bool a8, py::object out, std::uintptr_t stream,
           py::object impl) {
          GptqMarlinRepack::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(w), ToTensor(perm), k, n, bits, a8,
                                 ToTensor(out));
        },
        py::arg("b_q_weight"), py::arg("perm"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"),
        py::arg("is_a_8bit"), py::arg("out"), KW);
  {
    using D = Descriptor<GptqMarlinRepack>;
    auto cls = py::class_<D>(m, "GptqMarlinRepack");
    cls.def(py::init([](py::object w, py::object perm, int64_t k, int64_t n, int64_t bits, bool a8, py::object out,
                        py::object impl) {
              return D{GptqMarlinRepack::Make(MakeConfig(impl), ToTensor(w), ToTensor(perm), k, n, bits, a8, ToTensor(out))};
            }),
            py::arg("b_q_weight"), py::arg("perm"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"),
            py::arg("is_a_8bit"), py::arg("out"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object w, py::object perm, int64_t k, int64_t n, int64_t bits, bool a8, py::object out,
                std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(w), ToTensor(perm), k, n, bits, a8, ToTensor(out));
             },
             py::arg("b_q_weight"), py::arg("perm"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"),
             py::arg("is_a_8bit"), py::arg("out"), py::kw_only(), py::arg("stream") = 0);
    AddStatics<GptqMarlinRepack>(cls);
  }

  // ---- awq_marlin_repack ----------------------------------------------------------------------
  m.def("awq_marlin_repack",
        [](py::object w, int64_t k, int64_t n, int64_t bits, bool a8, py::object out, std::uintptr_t stream, py::object impl) {
          AwqMarlinRepack::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(w), k, n, bits, a8, ToTensor(out));
        },
        py::arg("b_q_weight"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"), py::arg("is_a_8bit"),
        py::arg("out"), KW);
  {
    using D = Descriptor<AwqMarlinRepack>;
    auto cls = py::class_<D>(m, "AwqMarlinRepack");
    cls.def(py::init([](py::object w, int64_t k, int64_t n, int64_t bits, bool a8, py::object out, py::object impl) {
              return D{AwqMarlinRepack::Make(MakeConfig(impl), ToTensor(w), k, n, bits, a8, ToTensor(out))};
            }),
            py::arg("b_q_weight"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"), py::arg("is_a_8bit"),
            py::arg("out"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object w, int64_t k, int64_t n, int64_t bits, bool a8, py::object out, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(w), k, n, bits, a8, ToTensor(out));
             },
             py::arg("b_q_weight"), py::arg("size_k"), py::arg("size_n"), py::arg("num_bits"), py::arg("is_a_8bit"),
             py::arg("out"), py::kw_only(), py::arg("stream") = 0);
    AddStatics<AwqMarlinRepack>(cls);
  }

  // ---- topk_softmax ---------------------------------------------------------------------------
  m.def("topk_softmax",
        [](py::object gate, py::object bias, py::object pad, bool renorm, py::object w, py::object idx, py::object tei,
           std::uintptr_t stream, py::object impl) {
          TopkSoftmax::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm,
                            ToTensor(w), ToTensor(idx), ToTensor(tei));
        },
        py::arg("gating_output"), py::arg("bias"), py::arg("is_padding"), py::arg("renormalize"),
        py::arg("topk_weights"), py::arg("topk_indices"), py::arg("token_expert_indices"), KW);
  {
    using D = Descriptor<TopkSoftmax>;
    auto cls = py::class_<D>(m, "TopkSoftmax");
    cls.def(py::init([](py::object gate, py::object bias, py::object pad, bool renorm, py::object w, py::object idx,
                        py::object tei, py::object impl) {
              return D{TopkSoftmax::Make(MakeConfig(impl), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm,
                                         ToTensor(w), ToTensor(idx), ToTensor(tei))};
            }),
            py::arg("gating_output"), py::arg("bias"), py::arg("is_padding"), py::arg("renormalize"),
            py::arg("topk_weights"), py::arg("topk_indices"), py::arg("token_expert_indices"), py::kw_only(),
            py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object gate, py::object bias, py::object pad, bool renorm, py::object w, py::object idx,
                py::object tei, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm, ToTensor(w),
                       ToTensor(idx), ToTensor(tei));
             },
             py::arg("gating_output"), py::arg("bias"), py::arg("is_padding"), py::arg("renormalize"),
             py::arg("topk_weights"), py::arg("topk_indices"), py::arg("token_expert_indices"), py::kw_only(),
             py::arg("stream") = 0);
    AddStatics<TopkSoftmax>(cls);
  }

  // ---- grouped_topk ---------------------------------------------------------------------------
  m.def("grouped_topk",
        [](py::object scores, py::object bias, int64_t groups, int64_t topk_group, int64_t topk, bool renorm, double scale,
           int64_t scoring, py::object values, py::object idx, std::uintptr_t stream, py::object impl) {
          GroupedTopk::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(scores), ToTensor(bias), groups, topk_group, topk,
                            renorm, scale, scoring, ToTensor(values), ToTensor(idx));
        },
        py::arg("scores"), py::arg("bias"), py::arg("num_expert_group"), py::arg("topk_group"), py::arg("topk"),
        py::arg("renormalize"), py::arg("routed_scaling_factor"), py::arg("scoring_func"), py::arg("topk_values"),
        py::arg("topk_indices"), KW);
  {
    using D = Descriptor<GroupedTopk>;
    auto cls = py::class_<D>(m, "GroupedTopk");
    cls.def(py::init([](py::object scores, py::object bias, int64_t groups, int64_t topk_group, int64_t topk, bool renorm,
                        double scale, int64_t scoring, py::object values, py::object idx, py::object impl) {
              return D{GroupedTopk::Make(MakeConfig(impl), ToTensor(scores), ToTensor(bias), groups, topk_group, topk, renorm,
                                         scale, scoring, ToTensor(values), ToTensor(idx))};
            }),
            py::arg("scores"), py::arg("bias"), py::arg("num_expert_group"), py::arg("topk_group"), py::arg("topk"),
            py::arg("renormalize"), py::arg("routed_scaling_factor"), py::arg("scoring_func"), py::arg("topk_values"),
            py::arg("topk_indices"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object scores, py::object bias, int64_t groups, int64_t topk_group, int64_t topk, bool renorm,
                double scale, int64_t scoring, py::object values, py::object idx, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(scores), ToTensor(bias), groups, topk_group, topk, renorm, scale, scoring,
                       ToTensor(values), ToTensor(idx));
             },
             py::arg("scores"), py::arg("bias"), py::arg("num_expert_group"), py::arg("topk_group"), py::arg("topk"),
             py::arg("renormalize"), py::arg("routed_scaling_factor"), py::arg("scoring_func"), py::arg("topk_values"),
             py::arg("topk_indices"), py::kw_only(), py::arg("stream") = 0);
    AddStatics<GroupedTopk>(cls);
  }

  // the remaining operators are registered in bindings_moe.cc
  RegisterMoeBindings(m);
  RegisterSiblingBindings(m);
}
