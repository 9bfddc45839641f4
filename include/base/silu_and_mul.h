// Descriptor of `silu_and_mul` (src/base/silu_and_mul.h:9-72 of the reference).
#ifndef INFINI_OPS_BASE_SILU_AND_MUL_H_
#define INFINI_OPS_BASE_SILU_AND_MUL_H_

#include "operator.h"

namespace infini::ops {

class SiluAndMul : public Operator<SiluAndMul> {
 public:
  static constexpr const char* kName = "SiluAndMul";

  SiluAndMul(const Tensor input, Tensor out)
      : input_{input}, out_{out}, dtype_{input.dtype()}, device_index_{input.device().index()} {
    INFINI_OPS_CHECK(input.ndim() == out.ndim() && out.ndim() >= 1,
                     "`SiluAndMul` requires input and output ranks to match");
    INFINI_OPS_CHECK(input.dtype() == out.dtype(), "`SiluAndMul` requires input and output dtypes to match");
    INFINI_OPS_CHECK(input.size(-1) == 2 * out.size(-1),
                     "`SiluAndMul` requires input last dimension to be twice output last dimension");
    for (Tensor::Size i = 0; i + 1 < out.ndim(); ++i) {
      INFINI_OPS_CHECK(input.size(i) == out.size(i), "`SiluAndMul` requires matching leading dimensions");
    }
    INFINI_OPS_CHECK(dtype_ == DataType::kFloat32 || dtype_ == DataType::kFloat16 || dtype_ == DataType::kBFloat16,
                     "`SiluAndMul` supports float32, float16, and bfloat16");
    INFINI_OPS_CHECK(out.ndim() <= 8, "`SiluAndMul` supports at most 8 dimensions");
  }

  virtual void operator()(const Tensor input, Tensor out) const = 0;

  // An empty output for `input`, made by the caller's own tensor type: anything with `Shape`,
  // `shape()`, `dtype()`, `device()` and a static `Empty(shape, dtype, device)` (same contract as
  // src/base/silu_and_mul.h:38-46 of the reference; the view type `Tensor` itself owns no memory
  // and has no `Empty`).
  template <typename TensorLike>
  static auto MakeReturnValue(const TensorLike& input) {
    typename TensorLike::Shape out_shape{input.shape()};
    INFINI_OPS_CHECK(!out_shape.empty() && out_shape.back() % 2 == 0,
                     "`SiluAndMul` requires an even input last dimension");
    out_shape.back() /= 2;
    return TensorLike::Empty(out_shape, input.dtype(), input.device());
  }

  // Output geometry alone, for callers that hold plain views.
  static Tensor::Shape OutputShape(const Tensor& input) {
    Tensor::Shape shape{input.shape()};
    INFINI_OPS_CHECK(!shape.empty() && shape.back() % 2 == 0, "`SiluAndMul` requires an even input last dimension");
    shape.back() /= 2;
    return shape;
  }

 protected:
  Tensor input_, out_;
  DataType dtype_;
  int device_index_;
};

}  // namespace infini::ops

#endif
