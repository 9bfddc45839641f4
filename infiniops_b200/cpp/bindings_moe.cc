// Second half of the `infini.ops` bindings: token sort, activation, combine and the two GEMMs.
#include "binding_utils.h"

void RegisterMoeBindings(py::module_& m) {
  // ---- moe_align_block_size -------------------------------------------------------------------
  m.def("moe_align_block_size",
        [](py::object ids, py::object emap, int64_t experts, int64_t block, py::object sorted, py::object eids,
           py::object npost, std::uintptr_t stream, py::object impl) {
          MoeAlignBlockSize::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(ids), ToOptional(emap), experts, block,
                                  ToTensor(sorted), ToTensor(eids), ToTensor(npost));
        },
        py::arg("topk_ids"), py::arg("expert_map"), py::arg("num_experts"), py::arg("block_size"),
        py::arg("sorted_token_ids"), py::arg("experts_ids"), py::arg("num_tokens_post_pad"), KW);
  {
    using D = Descriptor<MoeAlignBlockSize>;
    auto cls = py::class_<D>(m, "MoeAlignBlockSize");
    cls.def(py::init([](py::object ids, py::object emap, int64_t experts, int64_t block, py::object sorted, py::object eids,
                        py::object npost, py::object impl) {
              return D{MoeAlignBlockSize::Make(MakeConfig(impl), ToTensor(ids), ToOptional(emap), experts, block,
                                               ToTensor(sorted), ToTensor(eids), ToTensor(npost))};
            }),
            py::arg("topk_ids"), py::arg("expert_map"), py::arg("num_experts"), py::arg("block_size"),
            py::arg("sorted_token_ids"), py::arg("experts_ids"), py::arg("num_tokens_post_pad"), py::kw_only(),
            py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object ids, py::object emap, int64_t experts, int64_t block, py::object sorted, py::object eids,
                py::object npost, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(ids), ToOptional(emap), experts, block, ToTensor(sorted), ToTensor(eids),
                       ToTensor(npost));
             },
             py::arg("topk_ids"), py::arg("expert_map"), py::arg("num_experts"), py::arg("block_size"),
             py::arg("sorted_token_ids"), py::arg("experts_ids"), py::arg("num_tokens_post_pad"), py::kw_only(),
             py::arg("stream") = 0);
    AddStatics<MoeAlignBlockSize>(cls);
  }

  // ---- silu_and_mul ---------------------------------------------------------------------------
  m.def("silu_and_mul",
        [](py::object input, py::object out, std::uintptr_t stream, py::object impl) {
          SiluAndMul::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(input), ToTensor(out));
        },
        py::arg("input"), py::arg("out"), KW);
  {
    using D = Descriptor<SiluAndMul>;
    auto cls = py::class_<D>(m, "SiluAndMul");
    cls.def(py::init([](py::object input, py::object out, py::object impl) {
              return D{SiluAndMul::Make(MakeConfig(impl), ToTensor(input), ToTensor(out))};
            }),
            py::arg("input"), py::arg("out"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object input, py::object out, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(input), ToTensor(out));
             },
             py::arg("input"), py::arg("out"), py::kw_only(), py::arg("stream") = 0);
    AddStatics<SiluAndMul>(cls);
  }

  // ---- moe_sum (two overloads: plain, and with routing masks) -----------------------------------
  m.def("moe_sum",
        [](py::object input, py::object output, std::uintptr_t stream, py::object impl) {
          MoeSum::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(input), std::optional<Tensor>{},
                       std::optional<Tensor>{}, ToTensor(output));
        },
        py::arg("input"), py::arg("output"), KW);
  m.def("moe_sum",
        [](py::object input, py::object ids, py::object emap, py::object output, std::uintptr_t stream, py::object impl) {
          MoeSum::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(input), ToOptional(ids), ToOptional(emap),
                       ToTensor(output));
        },
        py::arg("input"), py::arg("topk_ids"), py::arg("expert_map"), py::arg("output"), KW);
  {
    using D = Descriptor<MoeSum>;
    auto cls = py::class_<D>(m, "MoeSum");
    cls.def(py::init([](py::object input, py::object output, py::object impl) {
              return D{MoeSum::Make(MakeConfig(impl), ToTensor(input), std::optional<Tensor>{}, std::optional<Tensor>{},
                                    ToTensor(output))};
            }),
            py::arg("input"), py::arg("output"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def(py::init([](py::object input, py::object ids, py::object emap, py::object output, py::object impl) {
               return D{MoeSum::Make(MakeConfig(impl), ToTensor(input), ToOptional(ids), ToOptional(emap), ToTensor(output))};
             }),
             py::arg("input"), py::arg("topk_ids"), py::arg("expert_map"), py::arg("output"), py::kw_only(),
             py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object input, py::object output, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(input), std::optional<Tensor>{}, std::optional<Tensor>{},
                       ToTensor(output));
             },
             py::arg("input"), py::arg("output"), py::kw_only(), py::arg("stream") = 0)
        .def("__call__",
             [](D& d, py::object input, py::object ids, py::object emap, py::object output, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(input), ToOptional(ids), ToOptional(emap), ToTensor(output));
             },
             py::arg("input"), py::arg("topk_ids"), py::arg("expert_map"), py::arg("output"), py::kw_only(),
             py::arg("stream") = 0);
    AddStatics<MoeSum>(cls);
  }

  // ---- marlin_gemm (dense) --------------------------------------------------------------------
  m.def("marlin_gemm",
        [](py::object a, py::object w, py::object bias, py::object scales, py::object a_scales, py::object global_scale,
           py::object zeros, py::object g_idx, py::object perm, py::object workspace, int64_t b_type_id, int64_t size_m,
           int64_t size_n, int64_t size_k, bool is_k_full, bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float,
           py::object out, std::uintptr_t stream, py::object impl) {
          MarlinGemm::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(a), ToTensor(w), ToOptional(bias), ToTensor(scales),
                           ToOptional(a_scales), ToOptional(global_scale), ToOptional(zeros), ToOptional(g_idx),
                           ToOptional(perm), ToTensor(workspace), b_type_id, size_m, size_n, size_k, is_k_full,
                           use_atomic_add, use_fp32_reduce, is_zp_float, ToTensor(out));
        },
        py::arg("a"), py::arg("b_q_weight"), py::arg("b_bias"), py::arg("b_scales"), py::arg("a_scales"),
        py::arg("global_scale"), py::arg("b_zeros"), py::arg("g_idx"), py::arg("perm"), py::arg("workspace"),
        py::arg("b_type_id"), py::arg("size_m"), py::arg("size_n"), py::arg("size_k"), py::arg("is_k_full"),
        py::arg("use_atomic_add"), py::arg("use_fp32_reduce"), py::arg("is_zp_float"), py::arg("out"), KW);
  {
    using D = Descriptor<MarlinGemm>;
    auto cls = py::class_<D>(m, "MarlinGemm");
    cls.def(py::init([](py::object a, py::object w, py::object bias, py::object scales, py::object a_scales,
                        py::object global_scale, py::object zeros, py::object g_idx, py::object perm, py::object workspace,
                        int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k, bool is_k_full,
                        bool use_atomic_add, bool use_fp32_reduce, bool is_zp_float, py::object out, py::object impl) {
              return D{MarlinGemm::Make(MakeConfig(impl), ToTensor(a), ToTensor(w), ToOptional(bias), ToTensor(scales),
                                        ToOptional(a_scales), ToOptional(global_scale), ToOptional(zeros), ToOptional(g_idx),
                                        ToOptional(perm), ToTensor(workspace), b_type_id, size_m, size_n, size_k, is_k_full,
                                        use_atomic_add, use_fp32_reduce, is_zp_float, ToTensor(out))};
            }),
            py::arg("a"), py::arg("b_q_weight"), py::arg("b_bias"), py::arg("b_scales"), py::arg("a_scales"),
            py::arg("global_scale"), py::arg("b_zeros"), py::arg("g_idx"), py::arg("perm"), py::arg("workspace"),
            py::arg("b_type_id"), py::arg("size_m"), py::arg("size_n"), py::arg("size_k"), py::arg("is_k_full"),
            py::arg("use_atomic_add"), py::arg("use_fp32_reduce"), py::arg("is_zp_float"), py::arg("out"), py::kw_only(),
            py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object a, py::object w, py::object bias, py::object scales, py::object a_scales,
                py::object global_scale, py::object zeros, py::object g_idx, py::object perm, py::object workspace,
                int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k, bool is_k_full, bool use_atomic_add,
                bool use_fp32_reduce, bool is_zp_float, py::object out, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(a), ToTensor(w), ToOptional(bias), ToTensor(scales), ToOptional(a_scales),
                       ToOptional(global_scale), ToOptional(zeros), ToOptional(g_idx), ToOptional(perm), ToTensor(workspace),
                       b_type_id, size_m, size_n, size_k, is_k_full, use_atomic_add, use_fp32_reduce, is_zp_float,
                       ToTensor(out));
             },
             py::arg("a"), py::arg("b_q_weight"), py::arg("b_bias"), py::arg("b_scales"), py::arg("a_scales"),
             py::arg("global_scale"), py::arg("b_zeros"), py::arg("g_idx"), py::arg("perm"), py::arg("workspace"),
             py::arg("b_type_id"), py::arg("size_m"), py::arg("size_n"), py::arg("size_k"), py::arg("is_k_full"),
             py::arg("use_atomic_add"), py::arg("use_fp32_reduce"), py::arg("is_zp_float"), py::arg("out"), py::kw_only(),
             py::arg("stream") = 0);
    AddStatics<MarlinGemm>(cls);
  }

  void RegisterMoeGemmBinding(py::module_&);
  RegisterMoeGemmBinding(m);
}
