// Descriptor of `gptq_marlin_repack` (src/base/gptq_marlin_repack.h:14-125 of the reference).
#ifndef INFINI_OPS_BASE_GPTQ_MARLIN_REPACK_H_
#define INFINI_OPS_BASE_GPTQ_MARLIN_REPACK_H_

#include <cstdint>
#include <limits>

#include "operator.h"

namespace infini::ops {

class GptqMarlinRepack : public Operator<GptqMarlinRepack> {
 public:
  static constexpr const char* kName = "GptqMarlinRepack";

  GptqMarlinRepack(const Tensor b_q_weight, const Tensor perm, const int64_t size_k, const int64_t size_n,
                   const int64_t num_bits, const bool is_a_8bit, Tensor out)
      : b_q_weight_{b_q_weight}, perm_{perm}, out_{out}, size_k_{size_k}, size_n_{size_n}, num_bits_{num_bits},
        pack_factor_{num_bits == 4 ? 8 : num_bits == 8 ? 4 : 0}, is_a_8bit_{is_a_8bit},
        has_perm_{perm.numel() != 0}, device_index_{b_q_weight.device().index()} {
    INFINI_OPS_CHECK(num_bits_ == 4 || num_bits_ == 8, "`GptqMarlinRepack` requires `num_bits` to be 4 or 8");
    INFINI_OPS_CHECK(size_k_ > 0 && size_n_ > 0 && size_k_ % 16 == 0 && size_n_ % 64 == 0,
                     "`GptqMarlinRepack` requires positive `size_k` divisible by 16 and `size_n` divisible by 64");
    INFINI_OPS_CHECK(!is_a_8bit_ || size_k_ % 32 == 0,
                     "`GptqMarlinRepack` requires `size_k` divisible by 32 for A8 layouts");
    INFINI_OPS_CHECK(size_k_ <= std::numeric_limits<int>::max() && size_n_ <= std::numeric_limits<int>::max(),
                     "`GptqMarlinRepack` dimensions exceed CUDA kernel limits");
    INFINI_OPS_CHECK(b_q_weight.ndim() == 2 && b_q_weight.size(0) == static_cast<Tensor::Size>(size_k_ / pack_factor_) &&
                         b_q_weight.size(1) == static_cast<Tensor::Size>(size_n_),
                     "`GptqMarlinRepack` requires `b_q_weight` shape [`size_k / pack_factor`, `size_n`]");
    INFINI_OPS_CHECK(b_q_weight.dtype() == DataType::kInt32 && b_q_weight.IsContiguous(),
                     "`GptqMarlinRepack` requires contiguous int32 `b_q_weight`");
    INFINI_OPS_CHECK(perm.ndim() == 1 && (!has_perm_ || perm.numel() == static_cast<Tensor::Size>(size_k_)),
                     "`GptqMarlinRepack` requires empty `perm` or shape [`size_k`]");
    INFINI_OPS_CHECK(perm.dtype() == DataType::kInt32 && perm.IsContiguous(),
                     "`GptqMarlinRepack` requires contiguous int32 `perm`");
    INFINI_OPS_CHECK(!is_a_8bit_ || !has_perm_, "`GptqMarlinRepack` does not support `perm` for A8 layouts");
    const Tensor::Shape expected{static_cast<Tensor::Size>(size_k_ / 16),
                                 static_cast<Tensor::Size>(size_n_ * 16 / pack_factor_)};
    INFINI_OPS_CHECK(out.shape() == expected, "`GptqMarlinRepack` output shape is incorrect");
    INFINI_OPS_CHECK(out.dtype() == DataType::kInt32 && out.IsContiguous(),
                     "`GptqMarlinRepack` requires contiguous int32 output");
    INFINI_OPS_CHECK(SameDevice(perm, b_q_weight) && SameDevice(out, b_q_weight),
                     "`GptqMarlinRepack` requires all tensors on the same device");
  }

  virtual void operator()(const Tensor b_q_weight, const Tensor perm, const int64_t size_k, const int64_t size_n,
                          const int64_t num_bits, const bool is_a_8bit, Tensor out) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor b_q_weight, const Tensor perm, const int64_t size_k, const int64_t size_n,
                            const int64_t num_bits, const bool is_a_8bit, const Tensor out) const {
    INFINI_OPS_CHECK(size_k == size_k_ && size_n == size_n_ && num_bits == num_bits_ && is_a_8bit == is_a_8bit_,
                     "`GptqMarlinRepack` attributes changed after descriptor creation");
    INFINI_OPS_CHECK(SameMetadata(b_q_weight_, b_q_weight) && SameMetadata(perm_, perm) && SameMetadata(out_, out),
                     "`GptqMarlinRepack` tensor metadata differs from its descriptor");
  }

  Tensor b_q_weight_, perm_, out_;
  int64_t size_k_, size_n_, num_bits_, pack_factor_;
  bool is_a_8bit_, has_perm_;
  int device_index_;
};

}  // namespace infini::ops

#endif
