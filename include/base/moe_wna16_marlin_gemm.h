// Descriptor of `moe_wna16_marlin_gemm` (src/base/moe_wna16_marlin_gemm.h:16-358 of the reference).
#ifndef INFINI_OPS_BASE_MOE_WNA16_MARLIN_GEMM_H_
#define INFINI_OPS_BASE_MOE_WNA16_MARLIN_GEMM_H_

#include <cstdint>
#include <limits>
#include <optional>

#include "operator.h"

namespace infini::ops {

// vLLM scalar-type ids the reference accepts (src/base/moe_wna16_marlin_gemm.h:172-184).
namespace qtype {
constexpr int64_t kUint4B8 = 1125899907892224, kUint8B128 = 1125899923621888, kUint4 = 1125899906843648,
                  kUint8 = 1125899906844672, kInt4 = 1125899906908928, kInt8 = 1125899906909952,
                  kFloat8E4M3Fn = 2814749767172868, kFloat4E2M1F = 562949953487106;
}

class MoeWna16MarlinGemm : public Operator<MoeWna16MarlinGemm> {
 public:
  static constexpr const char* kName = "MoeWna16MarlinGemm";

  MoeWna16MarlinGemm(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias_or_none,
                     const Tensor b_scales, std::optional<Tensor> a_scales, std::optional<Tensor> global_scale,
                     std::optional<Tensor> b_zeros_or_none, std::optional<Tensor> g_idx_or_none,
                     std::optional<Tensor> perm_or_none, const Tensor workspace, const Tensor sorted_token_ids,
                     const Tensor expert_ids, const Tensor num_tokens_past_padded, const Tensor topk_weights,
                     const int64_t moe_block_size, const int64_t top_k, const bool mul_topk_weights,
                     const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                     const bool is_full_k, const bool use_atomic_add, const bool use_fp32_reduce,
                     const bool is_zp_float, const int64_t thread_k, const int64_t thread_n,
                     const int64_t blocks_per_sm, Tensor out)
      : tensors_{a, b_q_weight, b_scales, workspace, sorted_token_ids, expert_ids, num_tokens_past_padded,
                 topk_weights, out},
        optionals_{b_bias_or_none, a_scales, global_scale, b_zeros_or_none, g_idx_or_none, perm_or_none},
        moe_block_size_{moe_block_size}, top_k_{top_k}, mul_topk_weights_{mul_topk_weights}, b_type_id_{b_type_id},
        size_m_{size_m}, size_n_{size_n}, size_k_{size_k}, is_full_k_{is_full_k}, use_atomic_add_{use_atomic_add},
        use_fp32_reduce_{use_fp32_reduce}, is_zp_float_{is_zp_float}, thread_k_{thread_k}, thread_n_{thread_n},
        blocks_per_sm_{blocks_per_sm}, device_index_{a.device().index()} {
    INFINI_OPS_CHECK(a.ndim() == 2 && static_cast<int64_t>(a.size(0)) == size_m_ &&
                         static_cast<int64_t>(a.size(1)) == size_k_,
                     "`MoeWna16MarlinGemm` `a` shape must match `size_m` and `size_k`");
    const bool a_8bit = a.dtype() == DataType::kInt8;
    const DataType out_dtype = a_8bit ? b_scales.dtype() : a.dtype();
    INFINI_OPS_CHECK((a.dtype() == DataType::kFloat16 || a.dtype() == DataType::kBFloat16 || a_8bit) && a.IsContiguous(),
                     "`MoeWna16MarlinGemm` requires contiguous float16, bfloat16, or int8 `a`");
    INFINI_OPS_CHECK(size_m_ > 0 && size_n_ > 0 && size_k_ > 0 && top_k_ > 0 && size_k_ % 16 == 0 && size_n_ % 64 == 0,
                     "`MoeWna16MarlinGemm` received unsupported dimensions");
    INFINI_OPS_CHECK(moe_block_size_ == 8 || (moe_block_size_ >= 16 && moe_block_size_ <= 64 && moe_block_size_ % 16 == 0),
                     "`MoeWna16MarlinGemm` received an unsupported `moe_block_size`");
    using namespace qtype;
    const bool known = b_type_id_ == kUint4B8 || b_type_id_ == kUint8B128 || b_type_id_ == kUint4 || b_type_id_ == kUint8 ||
                       b_type_id_ == kInt4 || b_type_id_ == kInt8 || b_type_id_ == kFloat8E4M3Fn ||
                       b_type_id_ == kFloat4E2M1F;
    const bool has_zp = b_zeros_or_none.has_value();
    INFINI_OPS_CHECK(known && has_zp == (b_type_id_ == kUint4 || b_type_id_ == kUint8) &&
                         (!is_zp_float_ || (has_zp && a.dtype() == DataType::kFloat16)),
                     "`MoeWna16MarlinGemm` received an unsupported quantization configuration");
    const int64_t pack = (b_type_id_ == kUint8B128 || b_type_id_ == kUint8 || b_type_id_ == kInt8 ||
                          b_type_id_ == kFloat8E4M3Fn) ? 4 : 8;
    INFINI_OPS_CHECK(b_q_weight.ndim() == 3 && static_cast<int64_t>(b_q_weight.size(1)) == size_k_ / 16 &&
                         static_cast<int64_t>(b_q_weight.size(2)) == size_n_ * 16 / pack &&
                         b_q_weight.dtype() == DataType::kInt32 && b_q_weight.IsContiguous(),
                     "`MoeWna16MarlinGemm` received invalid packed weights");
    INFINI_OPS_CHECK(b_scales.ndim() == 3 && b_scales.size(0) == b_q_weight.size(0) && b_scales.size(1) > 0 &&
                         static_cast<int64_t>(b_scales.size(2)) == size_n_ &&
                         size_k_ % static_cast<int64_t>(b_scales.size(1)) == 0 &&
                         (out_dtype == DataType::kFloat16 || out_dtype == DataType::kBFloat16) &&
                         b_scales.dtype() == out_dtype && b_scales.IsContiguous(),
                     "`MoeWna16MarlinGemm` received invalid weight scales");
    INFINI_OPS_CHECK(a_scales.has_value() == a_8bit,
                     "`MoeWna16MarlinGemm` requires activation scales exactly for int8 `a`");
    if (b_bias_or_none) {
      INFINI_OPS_CHECK(b_bias_or_none->ndim() == 2 && b_bias_or_none->size(0) == b_q_weight.size(0) &&
                           static_cast<int64_t>(b_bias_or_none->size(1)) == size_n_ &&
                           b_bias_or_none->dtype() == out_dtype && b_bias_or_none->IsContiguous(),
                       "`MoeWna16MarlinGemm` received invalid bias");
    }
    if (b_zeros_or_none) {
      INFINI_OPS_CHECK(b_zeros_or_none->ndim() == 3 && b_zeros_or_none->size(0) == b_q_weight.size(0) &&
                           b_zeros_or_none->size(1) == b_scales.size(1) &&
                           static_cast<int64_t>(b_zeros_or_none->size(2)) == (is_zp_float_ ? size_n_ : size_n_ / pack) &&
                           (is_zp_float_ ? b_zeros_or_none->dtype() == out_dtype
                                         : b_zeros_or_none->dtype() == DataType::kInt32),
                       "`MoeWna16MarlinGemm` received invalid zero points");
    }
    for (const auto* t : {&b_q_weight, &b_scales, &workspace, &sorted_token_ids, &expert_ids, &num_tokens_past_padded,
                          &topk_weights, static_cast<const Tensor*>(&out)}) {
      INFINI_OPS_CHECK(SameDevice(*t, a), "`MoeWna16MarlinGemm` requires all tensors on the input device");
    }
    INFINI_OPS_CHECK(g_idx_or_none.has_value() == perm_or_none.has_value(),
                     "`MoeWna16MarlinGemm` requires `g_idx_or_none` and `perm_or_none` together");
    INFINI_OPS_CHECK(workspace.ndim() == 1 && workspace.numel() > 0 && workspace.dtype() == DataType::kInt32 &&
                         workspace.IsContiguous(),
                     "`MoeWna16MarlinGemm` requires a non-empty int32 workspace");
    INFINI_OPS_CHECK(sorted_token_ids.ndim() == 1 && sorted_token_ids.dtype() == DataType::kInt32 &&
                         sorted_token_ids.IsContiguous() && expert_ids.ndim() == 1 &&
                         expert_ids.dtype() == DataType::kInt32 && expert_ids.IsContiguous() &&
                         num_tokens_past_padded.numel() == 1 && num_tokens_past_padded.dtype() == DataType::kInt32,
                     "`MoeWna16MarlinGemm` received invalid routing metadata");
    INFINI_OPS_CHECK(static_cast<int64_t>(topk_weights.numel()) == size_m_ * top_k_ &&
                         ((!mul_topk_weights_ && (topk_weights.dtype() == DataType::kFloat16 ||
                                                  topk_weights.dtype() == DataType::kBFloat16)) ||
                          topk_weights.dtype() == DataType::kFloat32) &&
                         topk_weights.IsContiguous(),
                     "`MoeWna16MarlinGemm` received invalid top-k weights");
    INFINI_OPS_CHECK(out.shape() == Tensor::Shape({static_cast<Tensor::Size>(size_m_ * top_k_),
                                                   static_cast<Tensor::Size>(size_n_)}) &&
                         out.dtype() == out_dtype && out.IsContiguous(),
                     "`MoeWna16MarlinGemm` output metadata is invalid");
  }

  virtual void operator()(const Tensor a, const Tensor b_q_weight, std::optional<Tensor> b_bias_or_none,
                          const Tensor b_scales, std::optional<Tensor> a_scales, std::optional<Tensor> global_scale,
                          std::optional<Tensor> b_zeros_or_none, std::optional<Tensor> g_idx_or_none,
                          std::optional<Tensor> perm_or_none, const Tensor workspace, const Tensor sorted_token_ids,
                          const Tensor expert_ids, const Tensor num_tokens_past_padded, const Tensor topk_weights,
                          const int64_t moe_block_size, const int64_t top_k, const bool mul_topk_weights,
                          const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                          const bool is_full_k, const bool use_atomic_add, const bool use_fp32_reduce,
                          const bool is_zp_float, const int64_t thread_k, const int64_t thread_n,
                          const int64_t blocks_per_sm, Tensor out) const = 0;

 protected:
  // tensors in the order {a, b_q_weight, b_scales, workspace, sorted, expert_ids, npost, topk_weights, out};
  // optionals in the order {bias, a_scales, global_scale, zeros, g_idx, perm}
  void ValidateCallMetadata(const Tensor (&tensors)[9], const std::optional<Tensor> (&optionals)[6],
                            const int64_t moe_block_size, const int64_t top_k, const bool mul_topk_weights,
                            const int64_t b_type_id, const int64_t size_m, const int64_t size_n, const int64_t size_k,
                            const bool is_full_k, const bool use_atomic_add, const bool use_fp32_reduce,
                            const bool is_zp_float, const int64_t thread_k, const int64_t thread_n,
                            const int64_t blocks_per_sm) const {
    INFINI_OPS_CHECK(moe_block_size == moe_block_size_ && top_k == top_k_ && mul_topk_weights == mul_topk_weights_ &&
                         b_type_id == b_type_id_ && size_m == size_m_ && size_n == size_n_ && size_k == size_k_ &&
                         is_full_k == is_full_k_ && use_atomic_add == use_atomic_add_ &&
                         use_fp32_reduce == use_fp32_reduce_ && is_zp_float == is_zp_float_ &&
                         thread_k == thread_k_ && thread_n == thread_n_ && blocks_per_sm == blocks_per_sm_,
                     "`MoeWna16MarlinGemm` attributes changed after descriptor creation");
    bool same = true;
    for (int i = 0; i < 9; ++i) same = same && SameMetadata(tensors_[i], tensors[i]);
    for (int i = 0; i < 6; ++i) same = same && SameMetadata(optionals_[i], optionals[i]);
    INFINI_OPS_CHECK(same, "`MoeWna16MarlinGemm` tensor metadata must match descriptor");
  }

  Tensor tensors_[9];
  std::optional<Tensor> optionals_[6];
  int64_t moe_block_size_, top_k_;
  bool mul_topk_weights_;
  int64_t b_type_id_, size_m_, size_n_, size_k_;
  bool is_full_k_, use_atomic_add_, use_fp32_reduce_, is_zp_float_;
  int64_t thread_k_, thread_n_, blocks_per_sm_;
  int device_index_;
};

}  // namespace infini::ops

#endif
