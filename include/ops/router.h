// NVIDIA slot-0 implementations of the two routers.
#ifndef INFINI_OPS_IMPL_ROUTER_H_
#define INFINI_OPS_IMPL_ROUTER_H_

#include "base/grouped_topk.h"
#include "base/topk_softmax.h"
#include "ops/common.h"

namespace infini::ops {

template <>
class Operator<TopkSoftmax, Device::Type::kNvidia, 0> : public TopkSoftmax {
 public:
  using TopkSoftmax::TopkSoftmax;

  void operator()(const Tensor gating_output, std::optional<Tensor> bias, std::optional<Tensor> is_padding,
                  const bool renormalize, Tensor topk_weights, Tensor topk_indices,
                  Tensor token_expert_indices) const override {
    ValidateCallMetadata(gating_output, bias, is_padding, renormalize, topk_weights, topk_indices,
                         token_expert_indices);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_topk_softmax(
                      gating_output.data(), impl::TypeCode(input_dtype_), static_cast<const float*>(impl::DataOrNull(bias)),
                      static_cast<const uint8_t*>(impl::DataOrNull(is_padding)), renormalize ? 1 : 0,
                      static_cast<float*>(topk_weights.data()), topk_indices.data(), impl::TypeCode(index_dtype_),
                      static_cast<int32_t*>(token_expert_indices.data()), static_cast<int64_t>(num_tokens_),
                      static_cast<int64_t>(num_experts_), static_cast<int64_t>(topk_), stream_),
                  kName);
  }
};

template <>
class Operator<GroupedTopk, Device::Type::kNvidia, 0> : public GroupedTopk {
 public:
  using GroupedTopk::GroupedTopk;

  void operator()(const Tensor scores, const Tensor bias, const int64_t num_expert_group, const int64_t topk_group,
                  const int64_t topk, const bool renormalize, const double routed_scaling_factor,
                  const int64_t scoring_func, Tensor topk_values, Tensor topk_indices) const override {
    ValidateCallMetadata(scores, bias, num_expert_group, topk_group, topk, renormalize, routed_scaling_factor,
                         scoring_func, topk_values, topk_indices);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_grouped_topk(scores.data(), impl::TypeCode(scores_dtype_), bias.data(),
                                              impl::TypeCode(bias_dtype_), static_cast<int64_t>(num_tokens_),
                                              static_cast<int64_t>(num_experts_), num_expert_group, topk_group, topk,
                                              renormalize ? 1 : 0, routed_scaling_factor,
                                              static_cast<int>(scoring_func), static_cast<float*>(topk_values.data()),
                                              static_cast<int32_t*>(topk_indices.data()), stream_),
                  kName);
  }
};

}  // namespace infini::ops

#endif
