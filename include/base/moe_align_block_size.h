// Descriptor of `moe_align_block_size` (src/base/moe_align_block_size.h:16-177 of the reference).
#ifndef INFINI_OPS_BASE_MOE_ALIGN_BLOCK_SIZE_H_
#define INFINI_OPS_BASE_MOE_ALIGN_BLOCK_SIZE_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class MoeAlignBlockSize : public Operator<MoeAlignBlockSize> {
 public:
  static constexpr const char* kName = "MoeAlignBlockSize";

  MoeAlignBlockSize(const Tensor topk_ids, const std::optional<Tensor> expert_map, const int64_t num_experts,
                    const int64_t block_size, Tensor sorted_token_ids, Tensor experts_ids, Tensor num_tokens_post_pad)
      : topk_ids_{topk_ids}, expert_map_{expert_map}, sorted_token_ids_{sorted_token_ids}, experts_ids_{experts_ids},
        num_tokens_post_pad_{num_tokens_post_pad}, numel_{topk_ids.numel()}, num_experts_{num_experts},
        block_size_{block_size}, sorted_size_{sorted_token_ids.numel()}, experts_size_{experts_ids.numel()},
        device_index_{topk_ids.device().index()} {
    constexpr auto kMax = static_cast<Tensor::Size>(std::numeric_limits<int32_t>::max());
    INFINI_OPS_CHECK(topk_ids.ndim() == 2, "`MoeAlignBlockSize` requires 2D `topk_ids`");
    INFINI_OPS_CHECK(topk_ids.dtype() == DataType::kInt32, "`MoeAlignBlockSize` currently requires int32 `topk_ids`");
    INFINI_OPS_CHECK(topk_ids.IsContiguous(), "`MoeAlignBlockSize` requires contiguous `topk_ids`");
    INFINI_OPS_CHECK(num_experts_ > 0 && num_experts_ < 1024, "`MoeAlignBlockSize` requires `num_experts` in [1, 1023]");
    INFINI_OPS_CHECK(block_size_ > 0, "`MoeAlignBlockSize` requires a positive `block_size`");
    INFINI_OPS_CHECK(block_size_ <= std::numeric_limits<int32_t>::max() && numel_ <= kMax,
                     "`MoeAlignBlockSize` requires int32-addressable token indices");
    INFINI_OPS_CHECK(SameDevice(sorted_token_ids, topk_ids) && SameDevice(experts_ids, topk_ids) &&
                         SameDevice(num_tokens_post_pad, topk_ids),
                     "`MoeAlignBlockSize` requires all tensors on the same device");
    INFINI_OPS_CHECK(sorted_token_ids.ndim() == 1 && experts_ids.ndim() == 1 && num_tokens_post_pad.ndim() == 1 &&
                         num_tokens_post_pad.numel() == 1,
                     "`MoeAlignBlockSize` requires 1D output tensors");
    INFINI_OPS_CHECK(sorted_token_ids.dtype() == DataType::kInt32 && experts_ids.dtype() == DataType::kInt32 &&
                         num_tokens_post_pad.dtype() == DataType::kInt32,
                     "`MoeAlignBlockSize` requires int32 output tensors");
    INFINI_OPS_CHECK(sorted_token_ids.IsContiguous() && experts_ids.IsContiguous() && num_tokens_post_pad.IsContiguous(),
                     "`MoeAlignBlockSize` requires contiguous output tensors");
    const auto experts = static_cast<Tensor::Size>(num_experts_), block = static_cast<Tensor::Size>(block_size_);
    auto need_sorted = numel_ + experts * (block - 1);
    if (numel_ < experts && numel_ * block < need_sorted) need_sorted = numel_ * block;
    const auto need_blocks = (need_sorted + block - 1) / block;
    INFINI_OPS_CHECK(need_sorted <= kMax, "`MoeAlignBlockSize` requires int32-addressable padded indices");
    INFINI_OPS_CHECK(sorted_size_ >= need_sorted && experts_size_ >= need_blocks,
                     "`MoeAlignBlockSize` output tensors are too small");
    if (expert_map) {
      INFINI_OPS_CHECK(expert_map->ndim() == 1 && expert_map->numel() == experts,
                       "`MoeAlignBlockSize` requires `expert_map` shape [`num_experts`]");
      INFINI_OPS_CHECK(expert_map->dtype() == DataType::kInt32,
                       "`MoeAlignBlockSize` currently requires int32 `expert_map`");
      INFINI_OPS_CHECK(expert_map->IsContiguous(), "`MoeAlignBlockSize` requires contiguous `expert_map`");
      INFINI_OPS_CHECK(SameDevice(*expert_map, topk_ids), "`MoeAlignBlockSize` requires `expert_map` on the input device");
    }
  }

  void operator()(const Tensor topk_ids, const std::optional<Tensor> expert_map, const int64_t num_experts,
                  const int64_t block_size, Tensor sorted_token_ids, Tensor experts_ids,
                  Tensor num_tokens_post_pad) const {
    INFINI_OPS_CHECK(num_experts == num_experts_ && block_size == block_size_,
                     "`MoeAlignBlockSize` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(topk_ids_, topk_ids) && SameMetadata(expert_map_, expert_map) &&
                         SameMetadata(sorted_token_ids_, sorted_token_ids) && SameMetadata(experts_ids_, experts_ids) &&
                         SameMetadata(num_tokens_post_pad_, num_tokens_post_pad),
                     "`MoeAlignBlockSize` tensor metadata differs from its descriptor");
    Run(topk_ids, expert_map, num_experts, block_size, sorted_token_ids, experts_ids, num_tokens_post_pad);
  }

 protected:
  virtual void Run(const Tensor topk_ids, const std::optional<Tensor> expert_map, const int64_t num_experts,
                   const int64_t block_size, Tensor sorted_token_ids, Tensor experts_ids,
                   Tensor num_tokens_post_pad) const = 0;

  Tensor topk_ids_;
  std::optional<Tensor> expert_map_;
  Tensor sorted_token_ids_, experts_ids_, num_tokens_post_pad_;
  Tensor::Size numel_;
  int64_t num_experts_, block_size_;
  Tensor::Size sorted_size_, experts_size_;
  int device_index_;
};

}  // namespace infini::ops

#endif
