// `infini::ops` names for the runtime types (src/tensor.h, src/device.h, src/data_type.h of the reference).
#ifndef INFINI_OPS_TENSOR_H_
#define INFINI_OPS_TENSOR_H_

#include <infini/rt.h>

namespace infini::ops {

using Tensor = infini::rt::TensorView;
using Device = infini::rt::Device;
using infini::rt::DataType;

}  // namespace infini::ops

#endif
