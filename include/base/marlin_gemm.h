// Descriptor of the dense `marlin_gemm`.
//
// The reference has no dense Marlin GEMM operator.  Following its own alignment rule for new
// operators (docs/operator-api-alignment.md:13-24,88-102: mirror the upstream wrapper, inputs
// then attributes then outputs), the argument set is vLLM's public `marlin_gemm` wrapper with
// the output moved last -- i.e. the MoE form (src/base/moe_wna16_marlin_gemm.h:18-34) without the
// routing arguments.
#ifndef INFINI_OPS_BASE_MARLIN_GEMM_H_
#define INFINI_OPS_BASE_MARLIN_GEMM_H_

#include <cstdint>
#include <optional>

#include "base/moe_wna16_marlin_gemm.h"
#include "operator.h"

namespace infini::ops {

class MarlinGemm : public Operator<MarlinGemm> {
 public:
  static constexpr const char* kName = "MarlinGemm";

  MarlinGemm(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias, const Tensor b_scales,
             std::optional<Tensor> a_scales, std::optional<Tensor> global_scale, std::optional<Tensor> b_zeros,
             std::optional<Tensor> g_idx, std::optional<Tensor> perm, const Tensor workspace, const int64_t b_type_id,
             const int64_t size_m, const int64_t size_n, const int64_t size_k, const bool is_k_full,
             const bool use_atomic_add, const bool use_fp32_reduce, const bool is_zp_float, Tensor out)
      : tensors_{a, b_q_weight, b_scales, workspace, out},
        optionals_{b_bias, a_scales, global_scale, b_zeros, g_idx, perm}, b_type_id_{b_type_id}, size_m_{size_m},
        size_n_{size_n}, size_k_{size_k}, is_k_full_{is_k_full}, use_atomic_add_{use_atomic_add},
        use_fp32_reduce_{use_fp32_reduce}, is_zp_float_{is_zp_float}, device_index_{a.device().index()} {
    INFINI_OPS_CHECK(a.ndim() == 2 && static_cast<int64_t>(a.size(0)) == size_m_ &&
                         static_cast<int64_t>(a.size(1)) == size_k_,
                     "`MarlinGemm` `a` shape must match `size_m` and `size_k`");
    INFINI_OPS_CHECK((a.dtype() == DataType::kFloat16 || a.dtype() == DataType::kBFloat16) && a.IsContiguous(),
                     "`MarlinGemm` requires contiguous float16 or bfloat16 `a`");
    INFINI_OPS_CHECK(size_m_ > 0 && size_n_ > 0 && size_k_ > 0 && size_k_ % 16 == 0 && size_n_ % 64 == 0,
                     "`MarlinGemm` received unsupported dimensions");
    const bool has_zp = b_zeros.has_value();
    INFINI_OPS_CHECK((b_type_id_ == qtype::kUint4B8 || b_type_id_ == qtype::kUint4 || b_type_id_ == qtype::kUint8B128 ||
                      b_type_id_ == qtype::kUint8 || b_type_id_ == qtype::kFloat8E4M3Fn) &&
                         has_zp == (b_type_id_ == qtype::kUint4 || b_type_id_ == qtype::kUint8) && !is_zp_float_,
                     "`MarlinGemm` received an unsupported quantization configuration");
    const int64_t pack = (b_type_id_ == qtype::kUint8B128 || b_type_id_ == qtype::kUint8 || b_type_id_ == qtype::kFloat8E4M3Fn) ? 4 : 8;  // weights per 32-bit word
    INFINI_OPS_CHECK(b_q_weight.ndim() == 2 && static_cast<int64_t>(b_q_weight.size(0)) == size_k_ / 16 &&
                         static_cast<int64_t>(b_q_weight.size(1)) == size_n_ * 16 / pack &&
                         b_q_weight.dtype() == DataType::kInt32 && b_q_weight.IsContiguous(),
                     "`MarlinGemm` received invalid packed weights");
    INFINI_OPS_CHECK(b_scales.ndim() == 2 && b_scales.size(0) > 0 && static_cast<int64_t>(b_scales.size(1)) == size_n_ &&
                         size_k_ % static_cast<int64_t>(b_scales.size(0)) == 0 && b_scales.dtype() == a.dtype() &&
                         b_scales.IsContiguous(),
                     "`MarlinGemm` received invalid weight scales");
    if (b_bias) {
      INFINI_OPS_CHECK(b_bias->numel() == static_cast<Tensor::Size>(size_n_) && b_bias->dtype() == a.dtype() &&
                           b_bias->IsContiguous(),
                       "`MarlinGemm` received invalid bias");
    }
    if (b_zeros) {
      INFINI_OPS_CHECK(b_zeros->ndim() == 2 && b_zeros->size(0) == b_scales.size(0) &&
                           static_cast<int64_t>(b_zeros->size(1)) == size_n_ / pack &&
                           b_zeros->dtype() == DataType::kInt32 && b_zeros->IsContiguous(),
                       "`MarlinGemm` received invalid zero points");
    }
    INFINI_OPS_CHECK(!a_scales && !global_scale, "`MarlinGemm` does not take activation or global scales for 16-bit `a`");
    INFINI_OPS_CHECK(g_idx.has_value() == perm.has_value(), "`MarlinGemm` requires `g_idx` and `perm` together");
    if (g_idx && (g_idx->numel() != 0 || perm->numel() != 0)) {
      // activation order: one int32 entry per weight row
      for (const auto* t : {&*g_idx, &*perm}) {
        INFINI_OPS_CHECK(t->ndim() == 1 && static_cast<int64_t>(t->size(0)) == size_k_ && t->dtype() == DataType::kInt32 &&
                             t->IsContiguous() && SameDevice(*t, a),
                         "`MarlinGemm` requires contiguous int32 `g_idx` and `perm` of `size_k` entries");
      }
      INFINI_OPS_CHECK(b_scales.size(0) > 1, "`MarlinGemm` act-order needs grouped scales");
    }
    INFINI_OPS_CHECK(workspace.ndim() == 1 && workspace.dtype() == DataType::kInt32 && workspace.IsContiguous(),
                     "`MarlinGemm` requires an int32 workspace");
    INFINI_OPS_CHECK(out.shape() == Tensor::Shape({static_cast<Tensor::Size>(size_m_), static_cast<Tensor::Size>(size_n_)}) &&
                         out.dtype() == a.dtype() && out.IsContiguous(),
                     "`MarlinGemm` output metadata is invalid");
    for (const auto* t : {&b_q_weight, &b_scales, &workspace, static_cast<const Tensor*>(&out)}) {
      INFINI_OPS_CHECK(SameDevice(*t, a), "`MarlinGemm` requires all tensors on the input device");
    }
  }

  virtual void operator()(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias, const Tensor b_scales,
                          std::optional<Tensor> a_scales, std::optional<Tensor> global_scale,
                          std::optional<Tensor> b_zeros, std::optional<Tensor> g_idx, std::optional<Tensor> perm,
                          const Tensor workspace, const int64_t b_type_id, const int64_t size_m, const int64_t size_n,
                          const int64_t size_k, const bool is_k_full, const bool use_atomic_add,
                          const bool use_fp32_reduce, const bool is_zp_float, Tensor out) const = 0;

 protected:
  void ValidateCallMetadata(const Tensor (&tensors)[5], const std::optional<Tensor> (&optionals)[6],
                            const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                            const bool is_k_full, const bool use_atomic_add, const bool use_fp32_reduce,
                            const bool is_zp_float) const {
    INFINI_OPS_CHECK(b_type_id == b_type_id_ && size_m == size_m_ && size_n == size_n_ && size_k == size_k_ &&
                         is_k_full == is_k_full_ && use_atomic_add == use_atomic_add_ &&
                         use_fp32_reduce == use_fp32_reduce_ && is_zp_float == is_zp_float_,
                     "`MarlinGemm` attributes changed after descriptor creation");
    bool same = true;
    for (int i = 0; i < 5; ++i) same = same && SameMetadata(tensors_[i], tensors[i]);
    for (int i = 0; i < 6; ++i) same = same && SameMetadata(optionals_[i], optionals[i]);
    INFINI_OPS_CHECK(same, "`MarlinGemm` tensor metadata must match descriptor");
  }

  Tensor tensors_[5];  // a, b_q_weight, b_scales, workspace, out
  std::optional<Tensor> optionals_[6];
  int64_t b_type_id_, size_m_, size_n_, size_k_;
  bool is_k_full_, use_atomic_add_, use_fp32_reduce_, is_zp_float_;
  int device_index_;
};

}  // namespace infini::ops

#endif
