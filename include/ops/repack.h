// NVIDIA slot-0 implementations of the two repack operators.
#ifndef INFINI_OPS_IMPL_REPACK_H_
#define INFINI_OPS_IMPL_REPACK_H_

#include "base/awq_marlin_repack.h"
#include "base/gptq_marlin_repack.h"
#include "ops/common.h"

namespace infini::ops {

template <>
class Operator<GptqMarlinRepack, Device::Type::kNvidia, 0> : public GptqMarlinRepack {
 public:
  using GptqMarlinRepack::GptqMarlinRepack;

  void operator()(const Tensor b_q_weight, const Tensor perm, const int64_t size_k, const int64_t size_n,
                  const int64_t num_bits, const bool is_a_8bit, Tensor out) const override {
    ValidateCallMetadata(b_q_weight, perm, size_k, size_n, num_bits, is_a_8bit, out);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_gptq_marlin_repack(
                      static_cast<const int32_t*>(b_q_weight.data()),
                      has_perm_ ? static_cast<const int32_t*>(perm.data()) : nullptr, size_k, size_n,
                      static_cast<int>(num_bits), is_a_8bit ? 1 : 0, static_cast<int32_t*>(out.data()), stream_),
                  kName);
  }
};

template <>
class Operator<AwqMarlinRepack, Device::Type::kNvidia, 0> : public AwqMarlinRepack {
 public:
  using AwqMarlinRepack::AwqMarlinRepack;

  void operator()(const Tensor b_q_weight, const int64_t size_k, const int64_t size_n, const int64_t num_bits,
                  const bool is_a_8bit, Tensor out) const override {
    ValidateCallMetadata(b_q_weight, size_k, size_n, num_bits, is_a_8bit, out);
    impl::DeviceGuard guard(device_index_);
    impl::Require(infiniops_b200_awq_marlin_repack(static_cast<const int32_t*>(b_q_weight.data()), size_k, size_n,
                                                   static_cast<int>(num_bits), is_a_8bit ? 1 : 0,
                                                   static_cast<int32_t*>(out.data()), stream_),
                  kName);
  }
};

}  // namespace infini::ops

#endif
