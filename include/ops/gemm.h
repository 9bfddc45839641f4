// NVIDIA slot-0 implementations of the dense and the routed W4A16 GEMM.
//
// The `workspace` tensor of the operator signature (vLLM's lock array) is accepted and left
// untouched: this kernel's split-K needs more room (fp32 partials) than that array has, so its
// scratch comes from the Handle's workspace or, failing that, from the library's per-thread
// buffer.  `use_atomic_add`, `use_fp32_reduce`, `thread_k`, `thread_n`, `blocks_per_sm` are tuning
// hints of the upstream kernel; they are validated for consistency and otherwise ignored (the
// reduction here is always fp32 and deterministic).
#ifndef INFINI_OPS_IMPL_GEMM_H_
#define INFINI_OPS_IMPL_GEMM_H_

#include "base/marlin_gemm.h"
#include "base/moe_wna16_marlin_gemm.h"
#include "ops/common.h"

namespace infini::ops {

namespace impl {
inline void RequireFourBit(int64_t b_type_id, const char* op) {
  if (b_type_id != qtype::kUint4B8 && b_type_id != qtype::kUint4 && b_type_id != qtype::kUint8B128 &&
      b_type_id != qtype::kUint8 && b_type_id != qtype::kFloat8E4M3Fn) {
    std::fprintf(stderr,
                 "`%s`: only the weight types uint4b8, uint4, uint8b128, uint8 and float8_e4m3fn are implemented in this build\n",
                 op);
    std::fflush(stderr);
    std::abort();
  }
}
}  // namespace impl

template <>
class Operator<MarlinGemm, Device::Type::kNvidia, 0> : public MarlinGemm {
 public:
  using MarlinGemm::MarlinGemm;

  std::size_t workspace_size_in_bytes() const override {
    // (activation order keeps a column-permuted copy of `a` in the scratch as well)
    const auto& perm = optionals_[5];
    return perm && perm->numel() != 0 ? infiniops_b200_marlin_gemm_act_order_scratch_bytes(size_m_, size_n_, size_k_)
                                      : infiniops_b200_marlin_gemm_scratch_bytes(size_m_, size_n_, size_k_);
  }

  void operator()(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias, const Tensor b_scales,
                  std::optional<Tensor> a_scales, std::optional<Tensor> global_scale, std::optional<Tensor> b_zeros,
                  std::optional<Tensor> g_idx, std::optional<Tensor> perm, const Tensor workspace,
                  const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                  const bool is_k_full, const bool use_atomic_add, const bool use_fp32_reduce, const bool is_zp_float,
                  Tensor out) const override {
    const Tensor tensors[5] = {a, b_q_weight, b_scales, workspace, out};
    const std::optional<Tensor> optionals[6] = {b_bias, a_scales, global_scale, b_zeros, g_idx, perm};
    ValidateCallMetadata(tensors, optionals, b_type_id, size_m, size_n, size_k, is_k_full, use_atomic_add,
                         use_fp32_reduce, is_zp_float);
    impl::DeviceGuard guard(device_index_);
    std::size_t scratch_bytes = 0;
    void* scratch = impl::PickScratch(workspace_, workspace_size_in_bytes_, workspace_size_in_bytes(), 0, stream_, scratch_bytes);
    iob_gemm_problem problem{};
    problem.a = a.data();
    problem.b_q_weight = static_cast<const int32_t*>(b_q_weight.data());
    problem.b_bias = impl::DataOrNull(b_bias);
    problem.b_scales = b_scales.data();
    problem.b_zeros = static_cast<const int32_t*>(impl::DataOrNull(b_zeros));
    problem.out = out.data();
    problem.size_m = size_m;
    problem.size_n = size_n;
    problem.size_k = size_k;
    problem.num_groups = static_cast<int64_t>(b_scales.size(0));
    problem.scale_layout = scale_layout();
    if (perm && perm->numel() != 0) {
      problem.g_idx = static_cast<const int32_t*>(g_idx->data());
      problem.perm = static_cast<const int32_t*>(perm->data());
    }
    impl::Require(infiniops_b200_marlin_gemm_placed(&problem, impl::TypeCode(a.dtype()), b_type_id, nullptr, scratch,
                                                    scratch_bytes, stream_),
                  kName);
  }

 protected:
  // 0: `b_scales` / `b_zeros` in plain column order; the provider slot reads vLLM's Marlin layouts.
  virtual int scale_layout() const { return 0; }
};

template <>
class Operator<MarlinGemm, Device::Type::kNvidia, kProviderSlot> : public Operator<MarlinGemm, Device::Type::kNvidia, 0> {
 public:
  using Operator<MarlinGemm, Device::Type::kNvidia, 0>::Operator;

 protected:
  int scale_layout() const override { return 1; }
};

template <>
class Operator<MoeWna16MarlinGemm, Device::Type::kNvidia, 0> : public MoeWna16MarlinGemm {
 public:
  using MoeWna16MarlinGemm::MoeWna16MarlinGemm;

  std::size_t workspace_size_in_bytes() const override {
    return infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(size_m_, top_k_, size_n_, size_k_,
                                                              static_cast<int64_t>(tensors_[1].size(0)),
                                                              moe_block_size_);
  }

  void operator()(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias_or_none, const Tensor b_scales,
                  std::optional<Tensor> a_scales, std::optional<Tensor> global_scale,
                  std::optional<Tensor> b_zeros_or_none, std::optional<Tensor> g_idx_or_none,
                  std::optional<Tensor> perm_or_none, const Tensor workspace, const Tensor sorted_token_ids,
                  const Tensor expert_ids, const Tensor num_tokens_past_padded, const Tensor topk_weights,
                  const int64_t moe_block_size, const int64_t top_k, const bool mul_topk_weights,
                  const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                  const bool is_full_k, const bool use_atomic_add, const bool use_fp32_reduce, const bool is_zp_float,
                  const int64_t thread_k, const int64_t thread_n, const int64_t blocks_per_sm,
                  Tensor out) const override {
    const Tensor tensors[9] = {a, b_q_weight, b_scales, workspace, sorted_token_ids, expert_ids,
                               num_tokens_past_padded, topk_weights, out};
    const std::optional<Tensor> optionals[6] = {b_bias_or_none, a_scales, global_scale, b_zeros_or_none,
                                                g_idx_or_none, perm_or_none};
    ValidateCallMetadata(tensors, optionals, moe_block_size, top_k, mul_topk_weights, b_type_id, size_m, size_n,
                         size_k, is_full_k, use_atomic_add, use_fp32_reduce, is_zp_float, thread_k, thread_n,
                         blocks_per_sm);
    // Parts of the upstream contract this build does not implement: refuse them loudly.
    impl::RequireFourBit(b_type_id, kName);
    INFINI_OPS_CHECK(a.dtype() != DataType::kInt8 && !a_scales && !global_scale,
                     "`MoeWna16MarlinGemm` int8 activations and global scales are not implemented");
    INFINI_OPS_CHECK(!is_zp_float, "`MoeWna16MarlinGemm` float zero points are not implemented");
    impl::DeviceGuard guard(device_index_);
    std::size_t scratch_bytes = 0;
    void* scratch = impl::PickScratch(workspace_, workspace_size_in_bytes_, workspace_size_in_bytes(), 0, stream_, scratch_bytes);
    iob_routed_options options{};
    options.scale_layout = scale_layout();
    if (g_idx_or_none && g_idx_or_none->numel() != 0) {
      // activation order: per-expert row order of the weights, and the (sorted) group of every row
      INFINI_OPS_CHECK(g_idx_or_none->IsContiguous() && perm_or_none->IsContiguous(),
                       "`MoeWna16MarlinGemm` requires contiguous `g_idx_or_none` and `perm_or_none`");
      options.g_idx = static_cast<const int32_t*>(g_idx_or_none->data());
      options.perm = static_cast<const int32_t*>(perm_or_none->data());
    }
    impl::Require(
        infiniops_b200_moe_wna16_marlin_gemm_ex(
            a.data(), impl::TypeCode(a.dtype()), static_cast<const int32_t*>(b_q_weight.data()),
            impl::DataOrNull(b_bias_or_none), b_scales.data(),
            static_cast<const int32_t*>(impl::DataOrNull(b_zeros_or_none)),
            static_cast<const int32_t*>(sorted_token_ids.data()), static_cast<const int32_t*>(expert_ids.data()),
            static_cast<const int32_t*>(num_tokens_past_padded.data()), // (16-bit routing weights are only accepted when they are not applied: they are never read then)
            mul_topk_weights ? static_cast<const float*>(topk_weights.data()) : nullptr, moe_block_size, top_k, mul_topk_weights ? 1 : 0, b_type_id, size_m, size_n, size_k,
            static_cast<int64_t>(b_scales.size(1)), static_cast<int64_t>(b_q_weight.size(0)),
            static_cast<int64_t>(sorted_token_ids.numel()), out.data(), &options, scratch, scratch_bytes, stream_),
        kName);
  }

 protected:
  virtual int scale_layout() const { return 0; }
};

template <>
class Operator<MoeWna16MarlinGemm, Device::Type::kNvidia, kProviderSlot>
    : public Operator<MoeWna16MarlinGemm, Device::Type::kNvidia, 0> {
 public:
  using Operator<MoeWna16MarlinGemm, Device::Type::kNvidia, 0>::Operator;

 protected:
  int scale_layout() const override { return 1; }
};

}  // namespace infini::ops

#endif
