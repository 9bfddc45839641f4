// Descriptor of `grouped_topk` (src/base/grouped_topk.h:14-159 of the reference).
#ifndef INFINI_OPS_BASE_GROUPED_TOPK_H_
#define INFINI_OPS_BASE_GROUPED_TOPK_H_

#include <cstdint>
#include <limits>

#include "operator.h"

namespace infini::ops {

class GroupedTopk : public Operator<GroupedTopk> {
 public:
  static constexpr const char* kName = "GroupedTopk";

  GroupedTopk(const Tensor scores, const Tensor bias, const int64_t num_expert_group, const int64_t topk_group,
              const int64_t topk, const bool renormalize, const double routed_scaling_factor,
              const int64_t scoring_func, Tensor topk_values, Tensor topk_indices)
      : num_tokens_{scores.ndim() == 2 ? scores.size(0) : 0}, num_experts_{scores.ndim() == 2 ? scores.size(1) : 0},
        num_expert_group_{num_expert_group}, topk_group_{topk_group}, topk_{topk}, renormalize_{renormalize},
        routed_scaling_factor_{routed_scaling_factor}, scoring_func_{scoring_func}, scores_dtype_{scores.dtype()},
        bias_dtype_{bias.dtype()}, device_index_{scores.device().index()}, scores_{scores}, bias_{bias},
        topk_values_{topk_values}, topk_indices_{topk_indices} {
    constexpr auto kMax = static_cast<Tensor::Size>(std::numeric_limits<int32_t>::max());
    const auto is_float = [](DataType t) {
      return t == DataType::kFloat16 || t == DataType::kBFloat16 || t == DataType::kFloat32;
    };
    INFINI_OPS_CHECK(scores.ndim() == 2, "`GroupedTopk` requires 2D `scores`");
    INFINI_OPS_CHECK(is_float(scores_dtype_), "`GroupedTopk` supports float16, bfloat16, and float32 `scores`");
    INFINI_OPS_CHECK(scores.IsContiguous(), "`GroupedTopk` requires contiguous `scores`");
    INFINI_OPS_CHECK(num_tokens_ <= kMax && num_experts_ <= kMax, "`GroupedTopk` dimensions must fit int32 indexing");
    INFINI_OPS_CHECK(bias.ndim() == 1 && bias.numel() == num_experts_,
                     "`GroupedTopk` requires `bias` shape `[num_experts]`");
    INFINI_OPS_CHECK(is_float(bias_dtype_), "`GroupedTopk` supports float16, bfloat16, and float32 `bias`");
    INFINI_OPS_CHECK(bias.IsContiguous(), "`GroupedTopk` requires contiguous `bias`");
    INFINI_OPS_CHECK(num_expert_group_ > 0 && num_expert_group_ <= 32,
                     "`GroupedTopk` requires `num_expert_group` in `[1, 32]`");
    INFINI_OPS_CHECK(topk_group_ > 0 && topk_group_ <= num_expert_group_,
                     "`GroupedTopk` requires `topk_group` in `[1, num_expert_group]`");
    INFINI_OPS_CHECK(num_experts_ > 0 && num_experts_ % static_cast<Tensor::Size>(num_expert_group_) == 0,
                     "`GroupedTopk` requires experts divisible by `num_expert_group`");
    INFINI_OPS_CHECK(num_experts_ / static_cast<Tensor::Size>(num_expert_group_) >= 2,
                     "`GroupedTopk` requires at least two experts per group");
    INFINI_OPS_CHECK(topk_ > 0 && topk_ <= 32 &&
                         topk_ <= topk_group_ * static_cast<int64_t>(num_experts_ / num_expert_group_),
                     "`GroupedTopk` requires `topk` in the selected-group capacity");
    INFINI_OPS_CHECK(scoring_func_ == 0 || scoring_func_ == 1,
                     "`GroupedTopk` requires `scoring_func` 0 (none) or 1 (sigmoid)");
    const Tensor::Shape output_shape{num_tokens_, static_cast<Tensor::Size>(topk_)};
    INFINI_OPS_CHECK(topk_values.shape() == output_shape && topk_indices.shape() == output_shape,
                     "`GroupedTopk` outputs must have shape `[num_tokens, topk]`");
    INFINI_OPS_CHECK(topk_values.dtype() == DataType::kFloat32, "`GroupedTopk` requires float32 `topk_values`");
    INFINI_OPS_CHECK(topk_indices.dtype() == DataType::kInt32, "`GroupedTopk` requires int32 `topk_indices`");
    INFINI_OPS_CHECK(topk_values.IsContiguous() && topk_indices.IsContiguous(),
                     "`GroupedTopk` requires contiguous outputs");
    INFINI_OPS_CHECK(SameDevice(bias, scores) && SameDevice(topk_values, scores) && SameDevice(topk_indices, scores),
                     "`GroupedTopk` requires all tensors on the same device");
  }

  virtual void operator()(const Tensor scores, const Tensor bias, const int64_t num_expert_group,
                          const int64_t topk_group, const int64_t topk, const bool renormalize,
                          const double routed_scaling_factor, const int64_t scoring_func, Tensor topk_values,
                          Tensor topk_indices) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor scores, const Tensor bias, const int64_t num_expert_group,
                            const int64_t topk_group, const int64_t topk, const bool renormalize,
                            const double routed_scaling_factor, const int64_t scoring_func, Tensor topk_values,
                            Tensor topk_indices) const {
    INFINI_OPS_CHECK(num_expert_group == num_expert_group_ && topk_group == topk_group_ && topk == topk_ &&
                         renormalize == renormalize_ && routed_scaling_factor == routed_scaling_factor_ &&
                         scoring_func == scoring_func_,
                     "`GroupedTopk` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(scores_, scores) && SameMetadata(bias_, bias) &&
                         SameMetadata(topk_values_, topk_values) && SameMetadata(topk_indices_, topk_indices),
                     "`GroupedTopk` call metadata must match descriptor");
  }

  Tensor::Size num_tokens_, num_experts_;
  int64_t num_expert_group_, topk_group_, topk_;
  bool renormalize_;
  double routed_scaling_factor_;
  int64_t scoring_func_;
  DataType scores_dtype_, bias_dtype_;
  int device_index_;
  Tensor scores_, bias_, topk_values_, topk_indices_;
};

}  // namespace infini::ops

#endif
