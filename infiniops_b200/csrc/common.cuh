// Shared helpers for the C-ABI launchers: status reporting and small device utilities.
#ifndef INFINIOPS_B200_COMMON_CUH_
#define INFINIOPS_B200_COMMON_CUH_

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>

#include "infiniops_b200.h"

namespace iob {

// Records the message returned by infiniops_b200_last_error() and yields `code`.
int Fail(int code, const char* fmt, ...);

inline int CheckLaunch(const char* what) {
  const cudaError_t err = cudaGetLastError();
  if (err != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "%s: %s", what, cudaGetErrorString(err));
  }
  return IOB_OK;
}

#define IOB_REQUIRE(cond, ...)                                  \
  do {                                                          \
    if (!(cond)) return ::iob::Fail(IOB_INVALID_ARGUMENT, __VA_ARGS__); \
  } while (0)

inline int NumSms() {
  static thread_local int cached_device = -1;
  static thread_local int cached_sms = 0;
  int device = 0;
  cudaGetDevice(&device);
  if (device != cached_device) {
    cudaDeviceGetAttribute(&cached_sms, cudaDevAttrMultiProcessorCount, device);
    cached_device = device;
  }
  return cached_sms > 0 ? cached_sms : 148;
}

template <typename T>
__device__ __forceinline__ float ToFloat(T v);
template <>
__device__ __forceinline__ float ToFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ float ToFloat<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float ToFloat<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T FromFloat(float v);
template <>
__device__ __forceinline__ float FromFloat<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half FromFloat<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 FromFloat<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// silu(gate) * up from values already rounded to T, one rounding at the end: the arithmetic of
// `silu_and_mul`, shared with the GEMM epilogue that fuses it so that both give the same bits.
template <typename T>
__device__ __forceinline__ T SiluMulRounded(float g, float u) {
  const float sig = __frcp_rn(__fadd_rn(1.0f, __expf(-g)));
  return FromFloat<T>(__fmul_rn(__fmul_rn(g, sig), u));
}

}  // namespace iob

#endif  // INFINIOPS_B200_COMMON_CUH_
