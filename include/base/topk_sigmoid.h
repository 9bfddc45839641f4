// Descriptor of `topk_sigmoid` (src/base/topk_sigmoid.h:15-185 of the reference).
#ifndef INFINI_OPS_BASE_TOPK_SIGMOID_H_
#define INFINI_OPS_BASE_TOPK_SIGMOID_H_

#include <cmath>
#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class TopkSigmoid : public Operator<TopkSigmoid> {
 public:
  static constexpr const char* kName = "TopkSigmoid";

  TopkSigmoid(const Tensor gating_output, std::optional<Tensor> e_score_correction_bias, std::optional<Tensor> is_padding,
              const bool renormalize, const double routed_scaling_factor, Tensor topk_weights, Tensor topk_ids,
              Tensor token_expert_indices)
      : num_tokens_{gating_output.ndim() == 2 ? gating_output.size(0) : 0},
        num_experts_{gating_output.ndim() == 2 ? gating_output.size(1) : 0},
        topk_{topk_weights.ndim() == 2 ? topk_weights.size(1) : 0}, input_dtype_{gating_output.dtype()},
        index_dtype_{topk_ids.dtype()}, renormalize_{renormalize}, routed_scaling_factor_{routed_scaling_factor},
        device_index_{gating_output.device().index()}, gating_output_{gating_output}, bias_{e_score_correction_bias},
        is_padding_{is_padding}, topk_weights_{topk_weights}, topk_ids_{topk_ids},
        token_expert_indices_{token_expert_indices} {
    constexpr auto kMax = static_cast<Tensor::Size>(std::numeric_limits<int32_t>::max());
    INFINI_OPS_CHECK(gating_output.ndim() == 2, "`TopkSigmoid` requires 2D `gating_output`");
    INFINI_OPS_CHECK(input_dtype_ == DataType::kFloat32 || input_dtype_ == DataType::kFloat16 ||
                         input_dtype_ == DataType::kBFloat16,
                     "`TopkSigmoid` supports float32, float16, and bfloat16 input");
    INFINI_OPS_CHECK(gating_output.IsContiguous(), "`TopkSigmoid` requires contiguous `gating_output`");
    INFINI_OPS_CHECK(num_experts_ > 0 && topk_ > 0 && topk_ <= num_experts_,
                     "`TopkSigmoid` requires `topk` in `[1, num_experts]`");
    INFINI_OPS_CHECK(std::isfinite(routed_scaling_factor_), "`TopkSigmoid` requires a finite `routed_scaling_factor`");
    INFINI_OPS_CHECK(num_tokens_ <= kMax && num_experts_ <= kMax && num_tokens_ <= kMax / topk_,
                     "`TopkSigmoid` output indices must fit int32 indexing");
    const Tensor::Shape output_shape{num_tokens_, topk_};
    INFINI_OPS_CHECK(topk_weights.shape() == output_shape && topk_ids.shape() == output_shape &&
                         token_expert_indices.shape() == output_shape,
                     "`TopkSigmoid` outputs must have shape `[num_tokens, topk]`");
    INFINI_OPS_CHECK(topk_weights.dtype() == DataType::kFloat32, "`TopkSigmoid` requires float32 `topk_weights`");
    INFINI_OPS_CHECK(index_dtype_ == DataType::kInt32 || index_dtype_ == DataType::kUInt32 ||
                         index_dtype_ == DataType::kInt64,
                     "`TopkSigmoid` requires int32, uint32, or int64 `topk_ids`");
    INFINI_OPS_CHECK(token_expert_indices.dtype() == DataType::kInt32,
                     "`TopkSigmoid` requires int32 `token_expert_indices`");
    INFINI_OPS_CHECK(topk_weights.IsContiguous() && topk_ids.IsContiguous() && token_expert_indices.IsContiguous(),
                     "`TopkSigmoid` requires contiguous outputs");
    INFINI_OPS_CHECK(SameDevice(topk_weights, gating_output) && SameDevice(topk_ids, gating_output) &&
                         SameDevice(token_expert_indices, gating_output),
                     "`TopkSigmoid` requires all tensors on the same device");
    if (bias_) {
      INFINI_OPS_CHECK(bias_->ndim() == 1 && bias_->numel() == num_experts_,
                       "`TopkSigmoid` requires `e_score_correction_bias` shape `[num_experts]`");
      INFINI_OPS_CHECK(bias_->dtype() == DataType::kFloat32 && bias_->IsContiguous(),
                       "`TopkSigmoid` requires contiguous float32 `e_score_correction_bias`");
      INFINI_OPS_CHECK(SameDevice(*bias_, gating_output),
                       "`TopkSigmoid` requires `e_score_correction_bias` on the input device");
    }
    if (is_padding) {
      INFINI_OPS_CHECK(is_padding->ndim() == 1 && is_padding->numel() == num_tokens_,
                       "`TopkSigmoid` requires `is_padding` shape `[num_tokens]`");
      INFINI_OPS_CHECK(is_padding->dtype() == DataType::kUInt8 && is_padding->IsContiguous(),
                       "`TopkSigmoid` requires contiguous bool `is_padding`");
      INFINI_OPS_CHECK(SameDevice(*is_padding, gating_output), "`TopkSigmoid` requires `is_padding` on the input device");
    }
  }

  virtual void operator()(const Tensor gating_output, std::optional<Tensor> e_score_correction_bias,
                          std::optional<Tensor> is_padding, const bool renormalize, const double routed_scaling_factor,
                          Tensor topk_weights, Tensor topk_ids, Tensor token_expert_indices) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor gating_output, std::optional<Tensor> e_score_correction_bias,
                            std::optional<Tensor> is_padding, const bool renormalize,
                            const double routed_scaling_factor, Tensor topk_weights, Tensor topk_ids,
                            Tensor token_expert_indices) const {
    INFINI_OPS_CHECK(renormalize == renormalize_ && routed_scaling_factor == routed_scaling_factor_,
                     "`TopkSigmoid` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(gating_output_, gating_output) && SameMetadata(bias_, e_score_correction_bias) &&
                         SameMetadata(is_padding_, is_padding) && SameMetadata(topk_weights_, topk_weights) &&
                         SameMetadata(topk_ids_, topk_ids) && SameMetadata(token_expert_indices_, token_expert_indices),
                     "`TopkSigmoid` call metadata must match descriptor");
  }

  Tensor::Size num_tokens_, num_experts_, topk_;
  DataType input_dtype_, index_dtype_;
  bool renormalize_;
  double routed_scaling_factor_;
  int device_index_;
  Tensor gating_output_;
  std::optional<Tensor> bias_, is_padding_;
  Tensor topk_weights_, topk_ids_, token_expert_indices_;
};

}  // namespace infini::ops

#endif
