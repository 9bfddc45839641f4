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

  // Output geometry for an input (the reference pairs this with an owning tensor type's `Empty`;
  // views do not allocate, so here it yields the shape only).
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
