// `infini.ops` bindings of the sibling MoE operators: topk_sigmoid, moe_wna16_gemm,
// get_cutlass_moe_mm_data (same conventions as bindings.cc).
#include "binding_utils.h"

void RegisterSiblingBindings(py::module_& m) {
  // ---- topk_sigmoid -----------------------------------------------------------------------------
  m.def("topk_sigmoid",
        [](py::object gate, py::object bias, py::object pad, bool renorm, double scale, py::object w, py::object ids,
           py::object tei, std::uintptr_t stream, py::object impl) {
          TopkSigmoid::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm,
                            scale, ToTensor(w), ToTensor(ids), ToTensor(tei));
        },
        py::arg("gating_output"), py::arg("e_score_correction_bias"), py::arg("is_padding"), py::arg("renormalize"),
        py::arg("routed_scaling_factor"), py::arg("topk_weights"), py::arg("topk_ids"), py::arg("token_expert_indices"),
        KW);
  {
    using D = Descriptor<TopkSigmoid>;
    auto cls = py::class_<D>(m, "TopkSigmoid");
    cls.def(py::init([](py::object gate, py::object bias, py::object pad, bool renorm, double scale, py::object w,
                        py::object ids, py::object tei, py::object impl) {
              return D{TopkSigmoid::Make(MakeConfig(impl), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm, scale,
                                         ToTensor(w), ToTensor(ids), ToTensor(tei))};
            }),
            py::arg("gating_output"), py::arg("e_score_correction_bias"), py::arg("is_padding"), py::arg("renormalize"),
            py::arg("routed_scaling_factor"), py::arg("topk_weights"), py::arg("topk_ids"),
            py::arg("token_expert_indices"), py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object gate, py::object bias, py::object pad, bool renorm, double scale, py::object w,
                py::object ids, py::object tei, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(gate), ToOptional(bias), ToOptional(pad), renorm, scale, ToTensor(w),
                       ToTensor(ids), ToTensor(tei));
             },
             py::arg("gating_output"), py::arg("e_score_correction_bias"), py::arg("is_padding"), py::arg("renormalize"),
             py::arg("routed_scaling_factor"), py::arg("topk_weights"), py::arg("topk_ids"),
             py::arg("token_expert_indices"), py::kw_only(), py::arg("stream") = 0);
    AddStatics<TopkSigmoid>(cls);
  }

  // ---- moe_wna16_gemm ---------------------------------------------------------------------------
  m.def("moe_wna16_gemm",
        [](py::object x, py::object qw, py::object s, py::object qz, py::object tw, py::object sorted, py::object eids,
           py::object npost, int64_t top_k, int64_t bm, int64_t bn, int64_t bk, int64_t bit, py::object out,
           std::uintptr_t stream, py::object impl) {
          MoeWna16Gemm::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(x), ToTensor(qw), ToTensor(s), ToOptional(qz),
                             ToOptional(tw), ToTensor(sorted), ToTensor(eids), ToTensor(npost), top_k, bm, bn, bk, bit,
                             ToTensor(out));
        },
        py::arg("input"), py::arg("b_qweight"), py::arg("b_scales"), py::arg("b_qzeros"), py::arg("topk_weights"),
        py::arg("sorted_token_ids"), py::arg("expert_ids"), py::arg("num_tokens_post_pad"), py::arg("top_k"),
        py::arg("block_size_m"), py::arg("block_size_n"), py::arg("block_size_k"), py::arg("bit"), py::arg("output"), KW);
  {
    using D = Descriptor<MoeWna16Gemm>;
    auto cls = py::class_<D>(m, "MoeWna16Gemm");
    cls.def(py::init([](py::object x, py::object qw, py::object s, py::object qz, py::object tw, py::object sorted,
                        py::object eids, py::object npost, int64_t top_k, int64_t bm, int64_t bn, int64_t bk, int64_t bit,
                        py::object out, py::object impl) {
              return D{MoeWna16Gemm::Make(MakeConfig(impl), ToTensor(x), ToTensor(qw), ToTensor(s), ToOptional(qz),
                                          ToOptional(tw), ToTensor(sorted), ToTensor(eids), ToTensor(npost), top_k, bm, bn,
                                          bk, bit, ToTensor(out))};
            }),
            py::arg("input"), py::arg("b_qweight"), py::arg("b_scales"), py::arg("b_qzeros"), py::arg("topk_weights"),
            py::arg("sorted_token_ids"), py::arg("expert_ids"), py::arg("num_tokens_post_pad"), py::arg("top_k"),
            py::arg("block_size_m"), py::arg("block_size_n"), py::arg("block_size_k"), py::arg("bit"), py::arg("output"),
            py::kw_only(), py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object x, py::object qw, py::object s, py::object qz, py::object tw, py::object sorted,
                py::object eids, py::object npost, int64_t top_k, int64_t bm, int64_t bn, int64_t bk, int64_t bit,
                py::object out, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(x), ToTensor(qw), ToTensor(s), ToOptional(qz), ToOptional(tw),
                       ToTensor(sorted), ToTensor(eids), ToTensor(npost), top_k, bm, bn, bk, bit, ToTensor(out));
             },
             py::arg("input"), py::arg("b_qweight"), py::arg("b_scales"), py::arg("b_qzeros"), py::arg("topk_weights"),
             py::arg("sorted_token_ids"), py::arg("expert_ids"), py::arg("num_tokens_post_pad"), py::arg("top_k"),
             py::arg("block_size_m"), py::arg("block_size_n"), py::arg("block_size_k"), py::arg("bit"), py::arg("output"),
             py::kw_only(), py::arg("stream") = 0);
    AddStatics<MoeWna16Gemm>(cls);
  }

  // ---- get_cutlass_moe_mm_data ---------------------------------------------------------------------
  // Two positional forms, as in the reference: with `is_gated` after `k`, and without it (gated).
  // The form with the flag is registered first: a tensor never converts to its `bool` slot in the
  // first (no-conversion) overload pass, so the shorter call falls through to the second form.
  m.def("get_cutlass_moe_mm_data",
        [](py::object ids, int64_t experts, int64_t n, int64_t k, bool is_gated, py::object offsets, py::object ps1,
           py::object ps2, py::object in_perm, py::object out_perm, py::object blockscale, std::uintptr_t stream,
           py::object impl) {
          GetCutlassMoeMmData::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(ids), experts, n, k, is_gated,
                                    ToTensor(offsets), ToTensor(ps1), ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm),
                                    ToOptional(blockscale));
        },
        py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("is_gated").noconvert(),
        py::arg("expert_offsets"), py::arg("problem_sizes1"), py::arg("problem_sizes2"), py::arg("input_permutation"),
        py::arg("output_permutation"), py::arg("blockscale_offsets") = py::none(), KW);
  m.def("get_cutlass_moe_mm_data",
        [](py::object ids, int64_t experts, int64_t n, int64_t k, py::object offsets, py::object ps1, py::object ps2,
           py::object in_perm, py::object out_perm, py::object blockscale, std::uintptr_t stream, py::object impl) {
          GetCutlassMoeMmData::Call(MakeHandle(stream), MakeConfig(impl), ToTensor(ids), experts, n, k, true,
                                    ToTensor(offsets), ToTensor(ps1), ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm),
                                    ToOptional(blockscale));
        },
        py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("expert_offsets"),
        py::arg("problem_sizes1"), py::arg("problem_sizes2"), py::arg("input_permutation"), py::arg("output_permutation"),
        py::arg("blockscale_offsets") = py::none(), KW);
  {
    using D = Descriptor<GetCutlassMoeMmData>;
    auto cls = py::class_<D>(m, "GetCutlassMoeMmData");
    cls.def(py::init([](py::object ids, int64_t experts, int64_t n, int64_t k, bool is_gated, py::object offsets,
                        py::object ps1, py::object ps2, py::object in_perm, py::object out_perm, py::object blockscale,
                        py::object impl) {
              return D{GetCutlassMoeMmData::Make(MakeConfig(impl), ToTensor(ids), experts, n, k, is_gated, ToTensor(offsets),
                                                 ToTensor(ps1), ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm),
                                                 ToOptional(blockscale))};
            }),
            py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("is_gated").noconvert(),
            py::arg("expert_offsets"), py::arg("problem_sizes1"), py::arg("problem_sizes2"), py::arg("input_permutation"),
            py::arg("output_permutation"), py::arg("blockscale_offsets") = py::none(), py::kw_only(),
            py::arg("implementation_index") = py::none())
        .def(py::init([](py::object ids, int64_t experts, int64_t n, int64_t k, py::object offsets, py::object ps1,
                         py::object ps2, py::object in_perm, py::object out_perm, py::object blockscale, py::object impl) {
               return D{GetCutlassMoeMmData::Make(MakeConfig(impl), ToTensor(ids), experts, n, k, true, ToTensor(offsets),
                                                  ToTensor(ps1), ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm),
                                                  ToOptional(blockscale))};
             }),
             py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("expert_offsets"),
             py::arg("problem_sizes1"), py::arg("problem_sizes2"), py::arg("input_permutation"),
             py::arg("output_permutation"), py::arg("blockscale_offsets") = py::none(), py::kw_only(),
             py::arg("implementation_index") = py::none())
        .def("__call__",
             [](D& d, py::object ids, int64_t experts, int64_t n, int64_t k, bool is_gated, py::object offsets,
                py::object ps1, py::object ps2, py::object in_perm, py::object out_perm, py::object blockscale,
                std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(ids), experts, n, k, is_gated, ToTensor(offsets), ToTensor(ps1),
                       ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm), ToOptional(blockscale));
             },
             py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("is_gated").noconvert(),
             py::arg("expert_offsets"), py::arg("problem_sizes1"), py::arg("problem_sizes2"),
             py::arg("input_permutation"), py::arg("output_permutation"), py::arg("blockscale_offsets") = py::none(),
             py::kw_only(), py::arg("stream") = 0)
        .def("__call__",
             [](D& d, py::object ids, int64_t experts, int64_t n, int64_t k, py::object offsets, py::object ps1,
                py::object ps2, py::object in_perm, py::object out_perm, py::object blockscale, std::uintptr_t stream) {
               (*d.op)(MakeHandle(stream), ToTensor(ids), experts, n, k, true, ToTensor(offsets), ToTensor(ps1),
                       ToTensor(ps2), ToTensor(in_perm), ToTensor(out_perm), ToOptional(blockscale));
             },
             py::arg("topk_ids"), py::arg("num_experts"), py::arg("n"), py::arg("k"), py::arg("expert_offsets"),
             py::arg("problem_sizes1"), py::arg("problem_sizes2"), py::arg("input_permutation"),
             py::arg("output_permutation"), py::arg("blockscale_offsets") = py::none(), py::kw_only(),
             py::arg("stream") = 0);
    AddStatics<GetCutlassMoeMmData>(cls);
  }
}
