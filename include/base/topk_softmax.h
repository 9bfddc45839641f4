// Descriptor of `topk_softmax` (src/base/topk_softmax.h:15-167 of the reference).
#ifndef INFINI_OPS_BASE_TOPK_SOFTMAX_H_
#define INFINI_OPS_BASE_TOPK_SOFTMAX_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class TopkSoftmax : public Operator<TopkSoftmax> {
 public:
  static constexpr const char* kName = "TopkSoftmax";

  TopkSoftmax(const Tensor gating_output, std::optional<Tensor> bias, std::optional<Tensor> is_padding,
              const bool renormalize, Tensor topk_weights, Tensor topk_indices, Tensor token_expert_indices)
      : num_tokens_{gating_output.ndim() == 2 ? gating_output.size(0) : 0},
        num_experts_{gating_output.ndim() == 2 ? gating_output.size(1) : 0},
        topk_{topk_weights.ndim() == 2 ? topk_weights.size(1) : 0}, input_dtype_{gating_output.dtype()},
        index_dtype_{topk_indices.dtype()}, renormalize_{renormalize}, device_index_{gating_output.device().index()},
        gating_output_{gating_output}, bias_{bias}, is_padding_{is_padding}, topk_weights_{topk_weights},
        topk_indices_{topk_indices}, token_expert_indices_{token_expert_indices} {
    constexpr auto kMax = static_cast<Tensor::Size>(std::numeric_limits<int32_t>::max());
    INFINI_OPS_CHECK(gating_output.ndim() == 2, "`TopkSoftmax` requires 2D `gating_output`");
    INFINI_OPS_CHECK(input_dtype_ == DataType::kFloat32 || input_dtype_ == DataType::kFloat16 ||
                         input_dtype_ == DataType::kBFloat16,
                     "`TopkSoftmax` supports float32, float16, and bfloat16 input");
    INFINI_OPS_CHECK(gating_output.IsContiguous(), "`TopkSoftmax` requires contiguous `gating_output`");
    INFINI_OPS_CHECK(num_experts_ > 0 && topk_ > 0 && topk_ <= num_experts_,
                     "`TopkSoftmax` requires `topk` in `[1, num_experts]`");
    INFINI_OPS_CHECK(num_tokens_ <= kMax && num_experts_ <= kMax && num_tokens_ <= kMax / topk_,
                     "`TopkSoftmax` output indices must fit int32 indexing");
    const Tensor::Shape output_shape{num_tokens_, topk_};
    INFINI_OPS_CHECK(topk_weights.shape() == output_shape && topk_indices.shape() == output_shape &&
                         token_expert_indices.shape() == output_shape,
                     "`TopkSoftmax` outputs must have shape `[num_tokens, topk]`");
    INFINI_OPS_CHECK(topk_weights.dtype() == DataType::kFloat32, "`TopkSoftmax` requires float32 `topk_weights`");
    INFINI_OPS_CHECK(index_dtype_ == DataType::kInt32 || index_dtype_ == DataType::kUInt32 ||
                         index_dtype_ == DataType::kInt64,
                     "`TopkSoftmax` requires int32, uint32, or int64 `topk_indices`");
    INFINI_OPS_CHECK(token_expert_indices.dtype() == DataType::kInt32,
                     "`TopkSoftmax` requires int32 `token_expert_indices`");
    INFINI_OPS_CHECK(topk_weights.IsContiguous() && topk_indices.IsContiguous() && token_expert_indices.IsContiguous(),
                     "`TopkSoftmax` requires contiguous outputs");
    INFINI_OPS_CHECK(SameDevice(topk_weights, gating_output) && SameDevice(topk_indices, gating_output) &&
                         SameDevice(token_expert_indices, gating_output),
                     "`TopkSoftmax` requires all tensors on the same device");
    if (bias) {
      INFINI_OPS_CHECK(bias->ndim() == 1 && bias->numel() == num_experts_,
                       "`TopkSoftmax` requires `bias` shape `[num_experts]`");
      INFINI_OPS_CHECK(bias->dtype() == DataType::kFloat32 && bias->IsContiguous(),
                       "`TopkSoftmax` requires contiguous float32 `bias`");
      INFINI_OPS_CHECK(SameDevice(*bias, gating_output), "`TopkSoftmax` requires `bias` on the input device");
    }
    if (is_padding) {
      INFINI_OPS_CHECK(is_padding->ndim() == 1 && is_padding->numel() == num_tokens_,
                       "`TopkSoftmax` requires `is_padding` shape `[num_tokens]`");
      INFINI_OPS_CHECK(is_padding->dtype() == DataType::kUInt8 && is_padding->IsContiguous(),
                       "`TopkSoftmax` requires contiguous bool `is_padding`");
      INFINI_OPS_CHECK(SameDevice(*is_padding, gating_output),
                       "`TopkSoftmax` requires `is_padding` on the input device");
    }
  }

  virtual void operator()(const Tensor gating_output, std::optional<Tensor> bias, std::optional<Tensor> is_padding,
                          const bool renormalize, Tensor topk_weights, Tensor topk_indices,
                          Tensor token_expert_indices) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor gating_output, std::optional<Tensor> bias, std::optional<Tensor> is_padding,
                            const bool renormalize, Tensor topk_weights, Tensor topk_indices,
                            Tensor token_expert_indices) const {
    INFINI_OPS_CHECK(renormalize == renormalize_, "`TopkSoftmax` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(gating_output_, gating_output) && SameMetadata(bias_, bias) &&
                         SameMetadata(is_padding_, is_padding) && SameMetadata(topk_weights_, topk_weights) &&
                         SameMetadata(topk_indices_, topk_indices) &&
                         SameMetadata(token_expert_indices_, token_expert_indices),
                     "`TopkSoftmax` call metadata must match descriptor");
  }

  Tensor::Size num_tokens_, num_experts_, topk_;
  DataType input_dtype_, index_dtype_;
  bool renormalize_;
  int device_index_;
  Tensor gating_output_;
  std::optional<Tensor> bias_, is_padding_;
  Tensor topk_weights_, topk_indices_, token_expert_indices_;
};

}  // namespace infini::ops

#endif
