// `infini.ops.moe_wna16_marlin_gemm` / `MoeWna16MarlinGemm` (29 arguments, order of
// src/base/moe_wna16_marlin_gemm.h:18-34 of the reference).
#include "binding_utils.h"

namespace {

struct MoeArgs {
  py::object a, w, bias, scales, a_scales, global_scale, zeros, g_idx, perm, workspace, sorted, expert_ids, npost,
      topk_weights;
  int64_t block, top_k;
  bool mul;
  int64_t b_type_id, size_m, size_n, size_k;
  bool is_full_k, use_atomic_add, use_fp32_reduce, is_zp_float;
  int64_t thread_k, thread_n, blocks_per_sm;
  py::object out;
};

template <typename F>
auto Expand(const MoeArgs& x, F&& f) {
  return f(ToTensor(x.a), ToTensor(x.w), ToOptional(x.bias), ToTensor(x.scales), ToOptional(x.a_scales),
           ToOptional(x.global_scale), ToOptional(x.zeros), ToOptional(x.g_idx), ToOptional(x.perm), ToTensor(x.workspace),
           ToTensor(x.sorted), ToTensor(x.expert_ids), ToTensor(x.npost), ToTensor(x.topk_weights), x.block, x.top_k, x.mul,
           x.b_type_id, x.size_m, x.size_n, x.size_k, x.is_full_k, x.use_atomic_add, x.use_fp32_reduce, x.is_zp_float,
           x.thread_k, x.thread_n, x.blocks_per_sm, ToTensor(x.out));
}

#define MOE_PARAMS                                                                                                     \
  py::object a, py::object w, py::object bias, py::object scales, py::object a_scales, py::object global_scale,         \
      py::object zeros, py::object g_idx, py::object perm, py::object workspace, py::object sorted,                     \
      py::object expert_ids, py::object npost, py::object topk_weights, int64_t block, int64_t top_k, bool mul,         \
      int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k, bool is_full_k, bool use_atomic_add,           \
      bool use_fp32_reduce, bool is_zp_float, int64_t thread_k, int64_t thread_n, int64_t blocks_per_sm, py::object out
#define MOE_PACK                                                                                                       \
  MoeArgs {                                                                                                            \
    a, w, bias, scales, a_scales, global_scale, zeros, g_idx, perm, workspace, sorted, expert_ids, npost, topk_weights, \
        block, top_k, mul, b_type_id, size_m, size_n, size_k, is_full_k, use_atomic_add, use_fp32_reduce, is_zp_float,  \
        thread_k, thread_n, blocks_per_sm, out                                                                          \
  }
#define MOE_NAMES                                                                                                      \
  py::arg("a"), py::arg("b_q_weight"), py::arg("b_bias_or_none"), py::arg("b_scales"), py::arg("a_scales"),            \
      py::arg("global_scale"), py::arg("b_zeros_or_none"), py::arg("g_idx_or_none"), py::arg("perm_or_none"),          \
      py::arg("workspace"), py::arg("sorted_token_ids"), py::arg("expert_ids"), py::arg("num_tokens_past_padded"),      \
      py::arg("topk_weights"), py::arg("moe_block_size"), py::arg("top_k"), py::arg("mul_topk_weights"),               \
      py::arg("b_type_id"), py::arg("size_m"), py::arg("size_n"), py::arg("size_k"), py::arg("is_full_k"),             \
      py::arg("use_atomic_add"), py::arg("use_fp32_reduce"), py::arg("is_zp_float"), py::arg("thread_k"),              \
      py::arg("thread_n"), py::arg("blocks_per_sm"), py::arg("out")

}  // namespace

void RegisterMoeGemmBinding(py::module_& m) {
  m.def("moe_wna16_marlin_gemm",
        [](MOE_PARAMS, std::uintptr_t stream, py::object impl) {
          const Handle handle = MakeHandle(stream);
          const Config config = MakeConfig(impl);
          Expand(MOE_PACK, [&](auto&&... args) { MoeWna16MarlinGemm::Call(handle, config, args...); });
        },
        MOE_NAMES, KW);
  using D = Descriptor<MoeWna16MarlinGemm>;
  auto cls = py::class_<D>(m, "MoeWna16MarlinGemm");
  cls.def(py::init([](MOE_PARAMS, py::object impl) {
            const Config config = MakeConfig(impl);
            return Expand(MOE_PACK, [&](auto&&... args) { return D{MoeWna16MarlinGemm::Make(config, args...)}; });
          }),
          MOE_NAMES, py::kw_only(), py::arg("implementation_index") = py::none())
      .def("__call__",
           [](D& d, MOE_PARAMS, std::uintptr_t stream) {
             const Handle handle = MakeHandle(stream);
             Expand(MOE_PACK, [&](auto&&... args) { (*d.op)(handle, args...); });
           },
           MOE_NAMES, py::kw_only(), py::arg("stream") = 0);
  AddStatics<MoeWna16MarlinGemm>(cls);
}
