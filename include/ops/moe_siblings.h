// NVIDIA slot-0 implementations of the sibling MoE operators: topk_sigmoid, moe_wna16_gemm (plain
// weight layout) and get_cutlass_moe_mm_data.
#ifndef INFINI_OPS_IMPL_MOE_SIBLINGS_H_
#define INFINI_OPS_IMPL_MOE_SIBLINGS_H_

#include "base/get_cutlass_moe_mm_data.h"
#include "base/moe_wna16_gemm.h"
#include "base/topk_sigmoid.h"
#include "ops/common.h"

namespace infini::ops {

template <>
class Operator<TopkSigmoid, Device::Type::kNvidia, 0> : public TopkSigmoid {
 public:
  using TopkSigmoid::TopkSigmoid;

  void operator()(const Tensor gating_output, std::optional<Tensor> e_score_correction_bias,
                  std::optional<Tensor> is_padding, const bool renormalize, const double routed_scaling_factor,
                  Tensor topk_weights, Tensor topk_ids, Tensor token_expert_indices) const override {
    ValidateCallMetadata(gating_output, e_score_correction_bias, is_padding, renormalize, routed_scaling_factor,
                         topk_weights, topk_ids, token_expert_indices);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_topk_sigmoid(
                      gating_output.data(), impl::TypeCode(input_dtype_),
                      static_cast<const float*>(impl::DataOrNull(e_score_correction_bias)),
                      static_cast<const uint8_t*>(impl::DataOrNull(is_padding)), renormalize ? 1 : 0,
                      routed_scaling_factor, static_cast<float*>(topk_weights.data()), topk_ids.data(),
                      impl::TypeCode(index_dtype_), static_cast<int32_t*>(token_expert_indices.data()),
                      static_cast<int64_t>(num_tokens_), static_cast<int64_t>(num_experts_), static_cast<int64_t>(topk_),
                      stream_),
                  kName);
  }
};

template <>
class Operator<MoeWna16Gemm, Device::Type::kNvidia, 0> : public MoeWna16Gemm {
 public:
  using MoeWna16Gemm::MoeWna16Gemm;

  // `block_size_n` and `block_size_k` are tiling hints of the upstream kernel: validated, not used.
  void operator()(const Tensor input, const Tensor b_qweight, const Tensor b_scales, std::optional<Tensor> b_qzeros,
                  std::optional<Tensor> topk_weights, const Tensor sorted_token_ids, const Tensor expert_ids,
                  const Tensor num_tokens_post_pad, const int64_t top_k, const int64_t block_size_m,
                  const int64_t block_size_n, const int64_t block_size_k, const int64_t bit,
                  Tensor output) const override {
    ValidateCallMetadata(input, b_qweight, b_scales, b_qzeros, topk_weights, sorted_token_ids, expert_ids,
                         num_tokens_post_pad, top_k, block_size_m, block_size_n, block_size_k, bit, output);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_moe_wna16_gemm(
                      input.data(), impl::TypeCode(dtype_), static_cast<const uint8_t*>(b_qweight.data()), b_scales.data(),
                      static_cast<const uint8_t*>(impl::DataOrNull(b_qzeros)),
                      static_cast<const float*>(impl::DataOrNull(topk_weights)),
                      static_cast<const int32_t*>(sorted_token_ids.data()), static_cast<const int32_t*>(expert_ids.data()),
                      static_cast<const int32_t*>(num_tokens_post_pad.data()),
                      static_cast<int64_t>(sorted_token_ids_size_), static_cast<int64_t>(expert_ids_size_), top_k,
                      block_size_m, bit, static_cast<int64_t>(m_), static_cast<int64_t>(n_), static_cast<int64_t>(k_),
                      static_cast<int64_t>(num_groups_), static_cast<int64_t>(num_experts_), output.data(), stream_),
                  kName);
  }
};

template <>
class Operator<GetCutlassMoeMmData, Device::Type::kNvidia, 0> : public GetCutlassMoeMmData {
 public:
  using GetCutlassMoeMmData::GetCutlassMoeMmData;
  using GetCutlassMoeMmData::operator();

  void operator()(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k, const bool is_gated,
                  Tensor expert_offsets, Tensor problem_sizes1, Tensor problem_sizes2, Tensor input_permutation,
                  Tensor output_permutation, std::optional<Tensor> blockscale_offsets = std::nullopt) const override {
    ValidateCallMetadata(topk_ids, num_experts, n, k, is_gated, expert_offsets, problem_sizes1, problem_sizes2,
                         input_permutation, output_permutation, blockscale_offsets);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_get_cutlass_moe_mm_data(
                      static_cast<const int32_t*>(topk_ids.data()), static_cast<int64_t>(numel_),
                      static_cast<int64_t>(topk_), num_experts, n, k, is_gated ? 1 : 0,
                      static_cast<int32_t*>(expert_offsets.data()), static_cast<int32_t*>(problem_sizes1.data()),
                      static_cast<int32_t*>(problem_sizes2.data()), static_cast<int32_t*>(input_permutation.data()),
                      static_cast<int32_t*>(output_permutation.data()),
                      blockscale_offsets ? static_cast<int32_t*>(blockscale_offsets->data()) : nullptr, stream_),
                  kName);
  }
};

}  // namespace infini::ops

#endif
