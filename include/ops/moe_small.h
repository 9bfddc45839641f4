// NVIDIA slot-0 implementations of moe_align_block_size, silu_and_mul and moe_sum.
#ifndef INFINI_OPS_IMPL_MOE_SMALL_H_
#define INFINI_OPS_IMPL_MOE_SMALL_H_

#include "base/moe_align_block_size.h"
#include "base/moe_sum.h"
#include "base/silu_and_mul.h"
#include "ops/common.h"

namespace infini::ops {

template <>
class Operator<MoeAlignBlockSize, Device::Type::kNvidia, 0> : public MoeAlignBlockSize {
 public:
  using MoeAlignBlockSize::MoeAlignBlockSize;

  std::size_t workspace_size_in_bytes() const override {
    return infiniops_b200_moe_align_block_size_scratch_bytes(static_cast<int64_t>(numel_), num_experts_);
  }

 protected:
  void Run(const Tensor topk_ids, const std::optional<Tensor> expert_map, const int64_t num_experts,
           const int64_t block_size, Tensor sorted_token_ids, Tensor experts_ids,
           Tensor num_tokens_post_pad) const override {
    impl::DeviceGuard guard(device_index_);
    std::size_t scratch_bytes = 0;
    void* scratch = impl::PickScratch(workspace_, workspace_size_in_bytes_, workspace_size_in_bytes(), 1, stream_, scratch_bytes);
    impl::Require(infiniops_b200_moe_align_block_size(
                      static_cast<const int32_t*>(topk_ids.data()),
                      static_cast<const int32_t*>(impl::DataOrNull(expert_map)), static_cast<int64_t>(numel_),
                      num_experts, block_size, static_cast<int32_t*>(sorted_token_ids.data()),
                      static_cast<int64_t>(sorted_size_), static_cast<int32_t*>(experts_ids.data()),
                      static_cast<int64_t>(experts_size_), static_cast<int32_t*>(num_tokens_post_pad.data()), scratch,
                      scratch_bytes, stream_),
                  kName);
  }
};

template <>
class Operator<SiluAndMul, Device::Type::kNvidia, 0> : public SiluAndMul {
 public:
  using SiluAndMul::SiluAndMul;

  void operator()(const Tensor input, Tensor out) const override {
    INFINI_OPS_CHECK(SameMetadata(input_, input) && SameMetadata(out_, out),
                     "`SiluAndMul` call metadata must match descriptor");
    impl::DeviceGuard guard(device_index_);
    int64_t shape[8], in_strides[8], out_strides[8];
    const int ndim = static_cast<int>(out.ndim());
    for (int d = 0; d < ndim; ++d) {
      shape[d] = static_cast<int64_t>(out.size(d));
      in_strides[d] = input.stride(d);
      out_strides[d] = out.stride(d);
    }
    impl::Require(infiniops_b200_silu_and_mul(input.data(), out.data(), impl::TypeCode(dtype_), ndim, shape,
                                              in_strides, out_strides, stream_),
                  kName);
  }
};

template <>
class Operator<MoeSum, Device::Type::kNvidia, 0> : public MoeSum {
 public:
  using MoeSum::MoeSum;
  using MoeSum::operator();

  void operator()(const Tensor input, std::optional<Tensor> topk_ids, std::optional<Tensor> expert_map,
                  Tensor output) const override {
    ValidateCallMetadata(input, topk_ids, expert_map, output);
    impl::DeviceGuard guard(device_index_);
    impl::Require(
        infiniops_b200_moe_sum(input.data(), impl::TypeCode(dtype_), static_cast<int64_t>(num_tokens_),
                               static_cast<int64_t>(topk_), static_cast<int64_t>(hidden_size_), input.stride(0),
                               input.stride(1), input.stride(2), impl::DataOrNull(topk_ids),
                               topk_ids ? impl::TypeCode(topk_ids->dtype()) : IOB_I32,
                               topk_ids ? topk_ids->stride(0) : 0, topk_ids ? topk_ids->stride(1) : 0,
                               static_cast<const int32_t*>(impl::DataOrNull(expert_map)),
                               expert_map ? static_cast<int64_t>(expert_map->numel()) : 0,
                               expert_map ? expert_map->stride(0) : 0, output.data(), stream_),
        kName);
  }
};

}  // namespace infini::ops

#endif
