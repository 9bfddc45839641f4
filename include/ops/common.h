// Glue shared by the slot-0 NVIDIA implementations: device guard, type codes, status handling,
// scratch selection.  Everything below the operators goes through the C ABI of the CUDA library.
#ifndef INFINI_OPS_IMPL_COMMON_H_
#define INFINI_OPS_IMPL_COMMON_H_

#include <cstdio>
#include <cstdlib>

#include "infiniops_b200.h"
#include "operator.h"

namespace infini::ops::impl {

// Makes the tensors' device current for the launch and restores the caller's afterwards
// (the reference's launchers do the same, src/native/cuda/nvidia/ops/moe_sum/kernel.cu:14-41).
class DeviceGuard {
 public:
  explicit DeviceGuard(int device) {
    if (infiniops_b200_swap_device(device, &previous_) != IOB_OK) previous_ = -1;
    changed_ = previous_ >= 0 && previous_ != device;
  }
  ~DeviceGuard() {
    if (changed_) infiniops_b200_swap_device(previous_, nullptr);
  }
  DeviceGuard(const DeviceGuard&) = delete;
  DeviceGuard& operator=(const DeviceGuard&) = delete;

 private:
  int previous_{-1};
  bool changed_{false};
};

inline int TypeCode(DataType t) {
  switch (t) {
    case DataType::kFloat32: return IOB_F32;
    case DataType::kFloat16: return IOB_F16;
    case DataType::kBFloat16: return IOB_BF16;
    case DataType::kInt32: return IOB_I32;
    case DataType::kInt64: return IOB_I64;
    case DataType::kUInt32: return IOB_U32;
    default: return -1;
  }
}

// A launch that the library refuses is a programming error at this level: report and abort,
// as the reference does after a failed launch (`assert(cudaGetLastError() == cudaSuccess)`).
inline void Require(int status, const char* op) {
  if (status != IOB_OK) {
    std::fprintf(stderr, "`%s` failed (status %d): %s\n", op, status, infiniops_b200_last_error());
    std::fflush(stderr);
    std::abort();
  }
}

// Scratch for a call: the Handle's workspace when it is large enough, else the library's buffer
// for (thread, device, purpose, stream), which allocates on first use / growth.  A Handle
// workspace carries no promise about its content (other operators write it too), so for the GEMMs
// (purpose 0), whose kernels count split-K arrivals in it, the counter area is cleared on the
// stream first.
inline void* PickScratch(void* workspace, std::size_t workspace_bytes, std::size_t need, int purpose, void* stream,
                         std::size_t& bytes_out) {
  if (need == 0) {
    bytes_out = 0;
    return nullptr;
  }
  if (workspace != nullptr && workspace_bytes >= need) {
    bytes_out = workspace_bytes;
    if (purpose == 0) Require(infiniops_b200_gemm_scratch_prepare(workspace, workspace_bytes, stream), "scratch set-up");
    return workspace;
  }
  void* p = infiniops_b200_thread_scratch(purpose, need, stream);
  if (p == nullptr) Require(IOB_CUDA_ERROR, "scratch allocation");
  bytes_out = need;
  return p;
}

inline const void* DataOrNull(const std::optional<Tensor>& t) { return t ? t->data() : nullptr; }

}  // namespace infini::ops::impl

#endif
