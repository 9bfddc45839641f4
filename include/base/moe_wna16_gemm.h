// Descriptor of `moe_wna16_gemm` (src/base/moe_wna16_gemm.h:16-226 of the reference).
#ifndef INFINI_OPS_BASE_MOE_WNA16_GEMM_H_
#define INFINI_OPS_BASE_MOE_WNA16_GEMM_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

class MoeWna16Gemm : public Operator<MoeWna16Gemm> {
 public:
  static constexpr const char* kName = "MoeWna16Gemm";

  MoeWna16Gemm(const Tensor input, const Tensor b_qweight, const Tensor b_scales, std::optional<Tensor> b_qzeros,
               std::optional<Tensor> topk_weights, const Tensor sorted_token_ids, const Tensor expert_ids,
               const Tensor num_tokens_post_pad, const int64_t top_k, const int64_t block_size_m,
               const int64_t block_size_n, const int64_t block_size_k, const int64_t bit, Tensor output)
      : num_experts_{b_qweight.ndim() == 3 ? b_qweight.size(0) : 0}, m_{input.ndim() == 2 ? input.size(0) : 0},
        n_{b_qweight.ndim() == 3 ? b_qweight.size(1) : 0}, k_{input.ndim() == 2 ? input.size(1) : 0},
        num_groups_{b_scales.ndim() == 3 ? b_scales.size(2) : 0},
        group_size_{num_groups_ > 0 && k_ % num_groups_ == 0 ? k_ / num_groups_ : 0},
        sorted_token_ids_size_{sorted_token_ids.numel()}, expert_ids_size_{expert_ids.numel()}, top_k_{top_k},
        block_size_m_{block_size_m}, block_size_n_{block_size_n}, block_size_k_{block_size_k}, bit_{bit},
        dtype_{input.dtype()}, has_qzeros_{b_qzeros.has_value()}, has_topk_weights_{topk_weights.has_value()},
        device_{input.device()}, device_index_{input.device().index()} {
    INFINI_OPS_CHECK(dtype_ == DataType::kFloat16 || dtype_ == DataType::kBFloat16,
                     "`MoeWna16Gemm` supports float16 and bfloat16 inputs");
    INFINI_OPS_CHECK(bit_ == 4 || bit_ == 8, "`MoeWna16Gemm` requires 4-bit or 8-bit weights");
    INFINI_OPS_CHECK(m_ > 0 && n_ > 0 && k_ > 0 && num_experts_ > 0 && top_k_ > 0,
                     "`MoeWna16Gemm` requires positive dimensions");
    INFINI_OPS_CHECK(num_groups_ > 0 && group_size_ > 0, "`MoeWna16Gemm` requires an integral quantization group size");
    const auto per_byte = static_cast<Tensor::Size>(8 / bit_), per_word = static_cast<Tensor::Size>(32 / bit_);
    INFINI_OPS_CHECK(k_ % per_byte == 0 && n_ % per_word == 0 && group_size_ % per_word == 0,
                     "`MoeWna16Gemm` packed dimensions are incompatible with `bit`");
    INFINI_OPS_CHECK(block_size_m_ > 0 && block_size_m_ <= 64 && block_size_n_ > 0 && block_size_n_ <= 1024 &&
                         block_size_k_ > 0 && block_size_k_ <= static_cast<int64_t>(k_) &&
                         block_size_k_ % static_cast<int64_t>(group_size_) == 0 &&
                         static_cast<int64_t>(k_) % block_size_k_ == 0 &&
                         block_size_n_ % static_cast<int64_t>(per_word) == 0 &&
                         (block_size_k_ / static_cast<int64_t>(per_word)) % 4 == 0,
                     "`MoeWna16Gemm` received unsupported block sizes");
    const auto groups_per_block = block_size_k_ / static_cast<int64_t>(group_size_);
    INFINI_OPS_CHECK(groups_per_block == 1 || groups_per_block == 2 || groups_per_block == 4 || groups_per_block == 8,
                     "`MoeWna16Gemm` requires 1, 2, 4, or 8 groups per K block");
    constexpr Tensor::Size kMaxU16 = std::numeric_limits<uint16_t>::max(), kMaxU32 = std::numeric_limits<uint32_t>::max();
    INFINI_OPS_CHECK(num_experts_ <= kMaxU16 && group_size_ <= kMaxU16 && top_k_ <= static_cast<int64_t>(kMaxU16) &&
                         m_ <= kMaxU32 && n_ <= kMaxU32 && k_ <= kMaxU32,
                     "`MoeWna16Gemm` dimensions exceed CUDA kernel limits");
    auto effective = sorted_token_ids_size_;
    if (m_ <= static_cast<Tensor::Size>(block_size_m_)) {
      const auto limit = m_ * static_cast<Tensor::Size>(block_size_m_ * top_k_);
      if (effective > limit) effective = limit;
    }
    const auto blocks = (effective + block_size_m_ - 1) / block_size_m_;
    INFINI_OPS_CHECK(sorted_token_ids_size_ > 0 && expert_ids_size_ >= blocks,
                     "`MoeWna16Gemm` routing metadata is too small");
    ValidateCallMetadata(input, b_qweight, b_scales, b_qzeros, topk_weights, sorted_token_ids, expert_ids,
                         num_tokens_post_pad, top_k_, block_size_m_, block_size_n_, block_size_k_, bit_, output);
  }

  virtual void operator()(const Tensor input, const Tensor b_qweight, const Tensor b_scales,
                          std::optional<Tensor> b_qzeros, std::optional<Tensor> topk_weights,
                          const Tensor sorted_token_ids, const Tensor expert_ids, const Tensor num_tokens_post_pad,
                          const int64_t top_k, const int64_t block_size_m, const int64_t block_size_n,
                          const int64_t block_size_k, const int64_t bit, Tensor output) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor input, const Tensor b_qweight, const Tensor b_scales,
                            std::optional<Tensor> b_qzeros, std::optional<Tensor> topk_weights,
                            const Tensor sorted_token_ids, const Tensor expert_ids, const Tensor num_tokens_post_pad,
                            const int64_t top_k, const int64_t block_size_m, const int64_t block_size_n,
                            const int64_t block_size_k, const int64_t bit, const Tensor output) const {
    INFINI_OPS_CHECK(top_k == top_k_ && block_size_m == block_size_m_ && block_size_n == block_size_n_ &&
                         block_size_k == block_size_k_ && bit == bit_,
                     "`MoeWna16Gemm` attributes changed after descriptor creation");
    const auto here = [&](const Tensor& t) { return t.device() == device_; };
    const auto per_byte = static_cast<Tensor::Size>(8 / bit_);
    const bool matches =
        input.ndim() == 2 && input.size(0) == m_ && input.size(1) == k_ && input.dtype() == dtype_ &&
        input.IsContiguous() && here(input) && b_qweight.ndim() == 3 && b_qweight.size(0) == num_experts_ &&
        b_qweight.size(1) == n_ && b_qweight.size(2) == k_ / per_byte && b_qweight.dtype() == DataType::kUInt8 &&
        b_qweight.IsContiguous() && here(b_qweight) && b_scales.ndim() == 3 && b_scales.size(0) == num_experts_ &&
        b_scales.size(1) == n_ && b_scales.size(2) == num_groups_ && b_scales.dtype() == dtype_ &&
        b_scales.IsContiguous() && here(b_scales) && sorted_token_ids.ndim() == 1 &&
        sorted_token_ids.numel() == sorted_token_ids_size_ && sorted_token_ids.dtype() == DataType::kInt32 &&
        sorted_token_ids.IsContiguous() && here(sorted_token_ids) && expert_ids.ndim() == 1 &&
        expert_ids.numel() == expert_ids_size_ && expert_ids.dtype() == DataType::kInt32 && expert_ids.IsContiguous() &&
        here(expert_ids) && num_tokens_post_pad.ndim() == 1 && num_tokens_post_pad.numel() == 1 &&
        num_tokens_post_pad.dtype() == DataType::kInt32 && num_tokens_post_pad.IsContiguous() &&
        here(num_tokens_post_pad) && output.ndim() == 3 && output.size(0) == m_ &&
        output.size(1) == static_cast<Tensor::Size>(top_k_) && output.size(2) == n_ && output.dtype() == dtype_ &&
        output.IsContiguous() && here(output) && b_qzeros.has_value() == has_qzeros_ &&
        topk_weights.has_value() == has_topk_weights_;
    INFINI_OPS_CHECK(matches, "`MoeWna16Gemm` call metadata must match descriptor");
    if (b_qzeros) {
      INFINI_OPS_CHECK(b_qzeros->ndim() == 3 && b_qzeros->size(0) == num_experts_ && b_qzeros->size(1) == n_ / per_byte &&
                           b_qzeros->size(2) == num_groups_ && b_qzeros->dtype() == DataType::kUInt8 &&
                           b_qzeros->IsContiguous() && here(*b_qzeros),
                       "`MoeWna16Gemm` zero-point metadata must match descriptor");
    }
    if (topk_weights) {
      INFINI_OPS_CHECK(topk_weights->ndim() == 2 && topk_weights->size(0) == m_ &&
                           topk_weights->size(1) == static_cast<Tensor::Size>(top_k_) &&
                           topk_weights->dtype() == DataType::kFloat32 && topk_weights->IsContiguous() &&
                           here(*topk_weights),
                       "`MoeWna16Gemm` top-k weight metadata must match descriptor");
    }
  }

  Tensor::Size num_experts_, m_, n_, k_, num_groups_, group_size_, sorted_token_ids_size_, expert_ids_size_;
  int64_t top_k_, block_size_m_, block_size_n_, block_size_k_, bit_;
  DataType dtype_;
  bool has_qzeros_, has_topk_weights_;
  Device device_;
  int device_index_;
};

}  // namespace infini::ops

#endif
