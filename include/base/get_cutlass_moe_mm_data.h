// Descriptor of `get_cutlass_moe_mm_data` (src/base/get_cutlass_moe_mm_data.h:14-224 of the reference).
#ifndef INFINI_OPS_BASE_GET_CUTLASS_MOE_MM_DATA_H_
#define INFINI_OPS_BASE_GET_CUTLASS_MOE_MM_DATA_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class GetCutlassMoeMmData : public Operator<GetCutlassMoeMmData> {
 public:
  static constexpr const char* kName = "GetCutlassMoeMmData";

  GetCutlassMoeMmData(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k,
                      Tensor expert_offsets, Tensor problem_sizes1, Tensor problem_sizes2, Tensor input_permutation,
                      Tensor output_permutation, std::optional<Tensor> blockscale_offsets = std::nullopt)
      : GetCutlassMoeMmData{topk_ids, num_experts, n, k, true, expert_offsets, problem_sizes1, problem_sizes2,
                            input_permutation, output_permutation, blockscale_offsets} {}

  GetCutlassMoeMmData(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k,
                      const bool is_gated, Tensor expert_offsets, Tensor problem_sizes1, Tensor problem_sizes2,
                      Tensor input_permutation, Tensor output_permutation,
                      std::optional<Tensor> blockscale_offsets = std::nullopt)
      : topk_ids_{topk_ids}, expert_offsets_{expert_offsets}, problem_sizes1_{problem_sizes1},
        problem_sizes2_{problem_sizes2}, input_permutation_{input_permutation}, output_permutation_{output_permutation},
        blockscale_offsets_{blockscale_offsets}, num_experts_{num_experts}, n_{n}, k_{k}, is_gated_{is_gated},
        numel_{topk_ids.numel()}, topk_{topk_ids.ndim() == 2 ? topk_ids.size(1) : 0},
        device_index_{topk_ids.device().index()} {
    constexpr int64_t kMax = std::numeric_limits<int32_t>::max();
    INFINI_OPS_CHECK(topk_ids.ndim() == 2, "`GetCutlassMoeMmData` requires 2D `topk_ids`");
    INFINI_OPS_CHECK(topk_ids.dtype() == DataType::kInt32, "`GetCutlassMoeMmData` requires int32 `topk_ids`");
    INFINI_OPS_CHECK(topk_ids.IsContiguous(), "`GetCutlassMoeMmData` requires contiguous `topk_ids`");
    INFINI_OPS_CHECK(numel_ > 0 && topk_ > 0, "`GetCutlassMoeMmData` requires non-empty `topk_ids`");
    INFINI_OPS_CHECK(num_experts_ > 0 && num_experts_ <= kMax / 3,
                     "`GetCutlassMoeMmData` requires indexable int32 `num_experts`");
    INFINI_OPS_CHECK(n_ > 0 && n_ <= (is_gated_ ? kMax / 2 : kMax) && k_ > 0 && k_ <= kMax,
                     "`GetCutlassMoeMmData` requires positive int32 GEMM dimensions");
    INFINI_OPS_CHECK(static_cast<int64_t>(numel_) <= kMax,
                     "`GetCutlassMoeMmData` requires int32-addressable routing indices");
    if (blockscale_offsets) {
      INFINI_OPS_CHECK(num_experts_ * 127 <= kMax && static_cast<int64_t>(numel_) <= kMax - num_experts_ * 127,
                       "`GetCutlassMoeMmData` blockscale offsets must fit int32");
    }
    const auto same = [&](const Tensor& t) { return SameDevice(t, topk_ids); };
    INFINI_OPS_CHECK(same(expert_offsets) && same(problem_sizes1) && same(problem_sizes2) && same(input_permutation) &&
                         same(output_permutation) && (!blockscale_offsets || same(*blockscale_offsets)),
                     "`GetCutlassMoeMmData` requires all tensors on the same device");
    const auto experts = static_cast<Tensor::Size>(num_experts_);
    INFINI_OPS_CHECK(expert_offsets.ndim() == 1 && expert_offsets.numel() == experts + 1,
                     "`GetCutlassMoeMmData` requires `expert_offsets` shape [`num_experts + 1`]");
    INFINI_OPS_CHECK(problem_sizes1.ndim() == 2 && problem_sizes1.size(0) == experts && problem_sizes1.size(1) == 3 &&
                         problem_sizes2.ndim() == 2 && problem_sizes2.shape() == problem_sizes1.shape(),
                     "`GetCutlassMoeMmData` requires problem sizes shape [`num_experts`, 3]");
    INFINI_OPS_CHECK(input_permutation.ndim() == 1 && input_permutation.numel() == numel_ &&
                         output_permutation.ndim() == 1 && output_permutation.numel() == numel_,
                     "`GetCutlassMoeMmData` requires permutation shape [`topk_ids.numel()`]");
    INFINI_OPS_CHECK(!blockscale_offsets || (blockscale_offsets->ndim() == 1 && blockscale_offsets->numel() == experts + 1),
                     "`GetCutlassMoeMmData` requires `blockscale_offsets` shape [`num_experts + 1`]");
    const auto plain = [](const Tensor& t) { return t.dtype() == DataType::kInt32 && t.IsContiguous(); };
    INFINI_OPS_CHECK(plain(expert_offsets) && plain(problem_sizes1) && plain(problem_sizes2) && plain(input_permutation) &&
                         plain(output_permutation) && (!blockscale_offsets || plain(*blockscale_offsets)),
                     "`GetCutlassMoeMmData` requires contiguous int32 outputs");
  }

  void operator()(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k,
                  Tensor expert_offsets, Tensor problem_sizes1, Tensor problem_sizes2, Tensor input_permutation,
                  Tensor output_permutation, std::optional<Tensor> blockscale_offsets = std::nullopt) const {
    (*this)(topk_ids, num_experts, n, k, true, expert_offsets, problem_sizes1, problem_sizes2, input_permutation,
            output_permutation, blockscale_offsets);
  }

  virtual void operator()(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k,
                          const bool is_gated, Tensor expert_offsets, Tensor problem_sizes1, Tensor problem_sizes2,
                          Tensor input_permutation, Tensor output_permutation,
                          std::optional<Tensor> blockscale_offsets = std::nullopt) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor topk_ids, const int64_t num_experts, const int64_t n, const int64_t k,
                            const bool is_gated, const Tensor expert_offsets, const Tensor problem_sizes1,
                            const Tensor problem_sizes2, const Tensor input_permutation, const Tensor output_permutation,
                            const std::optional<Tensor> blockscale_offsets) const {
    INFINI_OPS_CHECK(num_experts == num_experts_ && n == n_ && k == k_ && is_gated == is_gated_,
                     "`GetCutlassMoeMmData` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(topk_ids_, topk_ids) && SameMetadata(expert_offsets_, expert_offsets) &&
                         SameMetadata(problem_sizes1_, problem_sizes1) && SameMetadata(problem_sizes2_, problem_sizes2) &&
                         SameMetadata(input_permutation_, input_permutation) &&
                         SameMetadata(output_permutation_, output_permutation) &&
                         SameMetadata(blockscale_offsets_, blockscale_offsets),
                     "`GetCutlassMoeMmData` tensor metadata differs from its descriptor");
  }

  Tensor topk_ids_, expert_offsets_, problem_sizes1_, problem_sizes2_, input_permutation_, output_permutation_;
  std::optional<Tensor> blockscale_offsets_;
  int64_t num_experts_, n_, k_;
  bool is_gated_;
  Tensor::Size numel_, topk_;
  int device_index_;
};

}  // namespace infini::ops

#endif
