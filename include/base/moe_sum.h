// Descriptor of `moe_sum` (src/base/moe_sum.h:14-208 of the reference).
#ifndef INFINI_OPS_BASE_MOE_SUM_H_
#define INFINI_OPS_BASE_MOE_SUM_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class MoeSum : public Operator<MoeSum> {
 public:
  static constexpr const char* kName = "MoeSum";

  MoeSum(const Tensor input, Tensor output) : MoeSum{input, std::nullopt, std::nullopt, output} {}

  MoeSum(const Tensor input, std::optional<Tensor> topk_ids, std::optional<Tensor> expert_map, Tensor output)
      : input_{input}, topk_ids_{topk_ids}, expert_map_{expert_map}, output_{output},
        num_tokens_{input.ndim() == 3 ? input.size(0) : 0}, topk_{input.ndim() == 3 ? input.size(1) : 0},
        hidden_size_{input.ndim() == 3 ? input.size(2) : 0}, dtype_{input.dtype()},
        device_index_{input.device().index()} {
    INFINI_OPS_CHECK(input.ndim() == 3 && output.ndim() == 2,
                     "`MoeSum` requires `[num_tokens, topk, hidden_size]` input and `[num_tokens, hidden_size]` output");
    INFINI_OPS_CHECK(output.size(0) == num_tokens_ && output.size(1) == hidden_size_,
                     "`MoeSum` output shape is incompatible with the input");
    INFINI_OPS_CHECK(topk_ > 0, "`MoeSum` requires at least one top-k slot");
    INFINI_OPS_CHECK(dtype_ == DataType::kFloat32 || dtype_ == DataType::kFloat16 || dtype_ == DataType::kBFloat16,
                     "`MoeSum` supports float32, float16, and bfloat16 inputs");
    INFINI_OPS_CHECK(output.dtype() == dtype_, "`MoeSum` input and output dtypes must match");
    INFINI_OPS_CHECK(output.IsContiguous(), "`MoeSum` requires contiguous output");
    INFINI_OPS_CHECK(num_tokens_ <= static_cast<Tensor::Size>(std::numeric_limits<int>::max()),
                     "`MoeSum` token count exceeds the CUDA grid limit");
    INFINI_OPS_CHECK(NonNegative(input), "`MoeSum` input requires non-negative strides with signed offsets");
    INFINI_OPS_CHECK(SameDevice(output, input), "`MoeSum` input and output must be on the same device");
    INFINI_OPS_CHECK(!expert_map || topk_ids, "`MoeSum` expert_map requires topk_ids");
    if (topk_ids) {
      INFINI_OPS_CHECK(topk_ids->ndim() == 2 && topk_ids->size(0) == num_tokens_ && topk_ids->size(1) == topk_,
                       "`MoeSum` topk_ids must have shape `[num_tokens, topk]`");
      INFINI_OPS_CHECK(topk_ids->dtype() == DataType::kInt32 || topk_ids->dtype() == DataType::kInt64,
                       "`MoeSum` topk_ids must have int32 or int64 dtype");
      INFINI_OPS_CHECK(SameDevice(*topk_ids, input), "`MoeSum` topk_ids must be on the input device");
      INFINI_OPS_CHECK(NonNegative(*topk_ids), "`MoeSum` topk_ids requires non-negative strides with signed offsets");
    }
    if (expert_map) {
      INFINI_OPS_CHECK(expert_map->ndim() == 1 && expert_map->dtype() == DataType::kInt32,
                       "`MoeSum` expert_map must be a 1D int32 tensor");
      INFINI_OPS_CHECK(SameDevice(*expert_map, input), "`MoeSum` expert_map must be on the input device");
      INFINI_OPS_CHECK(NonNegative(*expert_map), "`MoeSum` expert_map requires non-negative strides with signed offsets");
    }
  }

  void operator()(const Tensor input, Tensor output) const { (*this)(input, std::nullopt, std::nullopt, output); }

  virtual void operator()(const Tensor input, std::optional<Tensor> topk_ids, std::optional<Tensor> expert_map,
                          Tensor output) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor input, std::optional<Tensor> topk_ids, std::optional<Tensor> expert_map,
                            const Tensor output) const {
    INFINI_OPS_CHECK(SameMetadata(input_, input) && SameMetadata(topk_ids_, topk_ids) &&
                         SameMetadata(expert_map_, expert_map) && SameMetadata(output_, output),
                     "`MoeSum` call metadata must match descriptor");
  }

  static bool NonNegative(const Tensor& t) {
    for (auto s : t.strides()) {
      if (s < 0) return false;
    }
    return true;
  }

  Tensor input_;
  std::optional<Tensor> topk_ids_, expert_map_;
  Tensor output_;
  Tensor::Size num_tokens_, topk_, hidden_size_;
  DataType dtype_;
  int device_index_;
};

}  // namespace infini::ops

#endif
