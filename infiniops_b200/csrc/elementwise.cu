// silu_and_mul and moe_sum: pure HBM streams.
//
// Both move each byte once with 16-byte accesses when the innermost stride is 1 and the
// rows are 16-byte aligned, and fall back to element accesses for arbitrary strides.
#include "common.cuh"

namespace iob {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxDims = 8;

struct RowLayout {
  int ndim;  // number of leading (row) dimensions
  int64_t shape[kMaxDims];
  int64_t in_stride[kMaxDims];
  int64_t out_stride[kMaxDims];
};

__device__ __forceinline__ void RowOffsets(const RowLayout& l, int64_t row, int64_t& in_off, int64_t& out_off) {
  in_off = 0;
  out_off = 0;
  for (int d = l.ndim - 1; d >= 0; --d) {
    const int64_t i = row % l.shape[d];
    row /= l.shape[d];
    in_off += i * l.in_stride[d];
    out_off += i * l.out_stride[d];
  }
}

template <typename T>
__device__ __forceinline__ T SiluMul(T gate, T up) {
  return SiluMulRounded<T>(ToFloat<T>(gate), ToFloat<T>(up));
}

template <typename T, int kVec>
struct alignas(sizeof(T) * kVec) Pack {
  T v[kVec];
};

// Vector path: innermost stride 1 on both sides, H % kVec == 0, rows 16-byte aligned.  A thread
// handles two 16-byte pieces kThreads pieces apart (four loads in flight before the arithmetic), read
// and written with streaming accesses: every byte is touched once.
template <typename T, int kPieces>
__global__ void __launch_bounds__(kThreads)
SiluAndMulVecKernel(const T* __restrict__ in, T* __restrict__ out, RowLayout layout, int64_t hidden,
                    int blocks_per_row) {
  constexpr int kVec = 16 / sizeof(T);
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t col0 = (static_cast<int64_t>(blockIdx.x % blocks_per_row) * (kPieces * kThreads) + threadIdx.x) * kVec;
  const int64_t col1 = col0 + static_cast<int64_t>(kThreads) * kVec;
  if (col0 >= hidden) return;
  const bool second = kPieces == 2 && col1 < hidden;
  int64_t in_off, out_off;
  RowOffsets(layout, row, in_off, out_off);
  const uint4* src = reinterpret_cast<const uint4*>(in + in_off);
  const int64_t up_at = hidden / kVec;
  uint4 raw[4];
  raw[0] = __ldcs(src + col0 / kVec);
  raw[1] = __ldcs(src + up_at + col0 / kVec);
  if (second) {
    raw[2] = __ldcs(src + col1 / kVec);
    raw[3] = __ldcs(src + up_at + col1 / kVec);
  }
  using P = Pack<T, kVec>;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    if (half == 1 && !second) break;
    const P gate = *reinterpret_cast<const P*>(&raw[2 * half]);
    const P up = *reinterpret_cast<const P*>(&raw[2 * half + 1]);
    P result;
#pragma unroll
    for (int i = 0; i < kVec; ++i) result.v[i] = SiluMul<T>(gate.v[i], up.v[i]);
    __stcs(reinterpret_cast<uint4*>(out + out_off + (half ? col1 : col0)), *reinterpret_cast<const uint4*>(&result));
  }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
SiluAndMulScalarKernel(const T* __restrict__ in, T* __restrict__ out, RowLayout layout, int64_t hidden,
                       int64_t in_last_stride, int64_t out_last_stride, int blocks_per_row) {
  const int64_t row = blockIdx.x / blocks_per_row;
  const int64_t col = static_cast<int64_t>(blockIdx.x % blocks_per_row) * kThreads + threadIdx.x;
  if (col >= hidden) return;
  int64_t in_off, out_off;
  RowOffsets(layout, row, in_off, out_off);
  const T gate = in[in_off + col * in_last_stride];
  const T up = in[in_off + (hidden + col) * in_last_stride];
  out[out_off + col * out_last_stride] = SiluMul<T>(gate, up);
}

template <typename T>
int LaunchSilu(const void* input, void* out, int ndim, const int64_t* shape, const int64_t* in_strides,
               const int64_t* out_strides, cudaStream_t stream) {
  RowLayout layout{};
  layout.ndim = ndim - 1;
  int64_t rows = 1;
  for (int d = 0; d < ndim - 1; ++d) {
    layout.shape[d] = shape[d];
    layout.in_stride[d] = in_strides[d];
    layout.out_stride[d] = out_strides[d];
    rows *= shape[d];
  }
  const int64_t hidden = shape[ndim - 1];
  if (rows == 0 || hidden == 0) return IOB_OK;
  constexpr int kVec = 16 / sizeof(T);
  bool vec = in_strides[ndim - 1] == 1 && out_strides[ndim - 1] == 1 && hidden % kVec == 0 &&
             reinterpret_cast<uintptr_t>(input) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  for (int d = 0; d < ndim - 1 && vec; ++d) {
    vec = in_strides[d] % kVec == 0 && out_strides[d] % kVec == 0;
  }
  // (rows shorter than two pieces per thread keep one piece per thread, so that no half of a block idles)
  const int pieces = vec && hidden >= static_cast<int64_t>(2 * kThreads) * kVec ? 2 : 1;
  const int64_t per_block = vec ? static_cast<int64_t>(pieces * kThreads) * kVec : kThreads;
  const int64_t blocks_per_row = (hidden + per_block - 1) / per_block;
  IOB_REQUIRE(rows * blocks_per_row <= INT32_MAX, "silu_and_mul: tensor too large for one launch");
  const unsigned grid = static_cast<unsigned>(rows * blocks_per_row);
  if (vec) {
    auto kernel = pieces == 2 ? SiluAndMulVecKernel<T, 2> : SiluAndMulVecKernel<T, 1>;
    kernel<<<grid, kThreads, 0, stream>>>(static_cast<const T*>(input), static_cast<T*>(out), layout, hidden,
                                          static_cast<int>(blocks_per_row));
  } else {
    SiluAndMulScalarKernel<T><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(input), static_cast<T*>(out),
                                                           layout, hidden, in_strides[ndim - 1],
                                                           out_strides[ndim - 1], static_cast<int>(blocks_per_row));
  }
  return CheckLaunch("silu_and_mul launch");
}

// ------------------------------------------------------------------------------------------
struct SumArgs {
  int64_t topk, hidden;
  int64_t in_stride_t, in_stride_s, in_stride_h;
  const void* ids;
  int ids_are_i64;
  int64_t ids_stride_t, ids_stride_s;
  const int32_t* expert_map;
  int64_t expert_map_size, expert_map_stride;
};

__device__ __forceinline__ bool SlotActive(const SumArgs& a, int64_t token, int64_t slot) {
  if (a.ids == nullptr) return true;
  const int64_t at = token * a.ids_stride_t + slot * a.ids_stride_s;
  const int64_t id = a.ids_are_i64 ? static_cast<const int64_t*>(a.ids)[at]
                                   : static_cast<int64_t>(static_cast<const int32_t*>(a.ids)[at]);
  if (id < 0) return false;
  if (a.expert_map != nullptr && (id >= a.expert_map_size || a.expert_map[id * a.expert_map_stride] < 0)) {
    return false;
  }
  return true;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
MoeSumVecKernel(const T* __restrict__ in, T* __restrict__ out, SumArgs a, int blocks_per_row) {
  constexpr int kVec = 16 / sizeof(T);
  const int64_t token = blockIdx.x / blocks_per_row;
  const int64_t col = (static_cast<int64_t>(blockIdx.x % blocks_per_row) * kThreads + threadIdx.x) * kVec;
  if (col >= a.hidden) return;
  using P = Pack<T, kVec>;
  float acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = 0.0f;
  for (int64_t slot = 0; slot < a.topk; ++slot) {
    if (!SlotActive(a, token, slot)) continue;
    const P v = *reinterpret_cast<const P*>(in + token * a.in_stride_t + slot * a.in_stride_s + col);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] += ToFloat<T>(v.v[i]);
  }
  P result;
#pragma unroll
  for (int i = 0; i < kVec; ++i) result.v[i] = FromFloat<T>(acc[i]);
  *reinterpret_cast<P*>(out + token * a.hidden + col) = result;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
MoeSumScalarKernel(const T* __restrict__ in, T* __restrict__ out, SumArgs a, int blocks_per_row) {
  const int64_t token = blockIdx.x / blocks_per_row;
  const int64_t col = static_cast<int64_t>(blockIdx.x % blocks_per_row) * kThreads + threadIdx.x;
  if (col >= a.hidden) return;
  float acc = 0.0f;
  for (int64_t slot = 0; slot < a.topk; ++slot) {
    if (!SlotActive(a, token, slot)) continue;
    acc += ToFloat<T>(in[token * a.in_stride_t + slot * a.in_stride_s + col * a.in_stride_h]);
  }
  out[token * a.hidden + col] = FromFloat<T>(acc);
}

template <typename T>
int LaunchSum(const void* input, void* out, int64_t tokens, const SumArgs& a, cudaStream_t stream) {
  if (tokens == 0 || a.hidden == 0) return IOB_OK;
  constexpr int kVec = 16 / sizeof(T);
  const bool vec = a.in_stride_h == 1 && a.hidden % kVec == 0 && a.in_stride_t % kVec == 0 &&
                   a.in_stride_s % kVec == 0 && reinterpret_cast<uintptr_t>(input) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(out) % 16 == 0;
  const int64_t per_block = vec ? static_cast<int64_t>(kThreads) * kVec : kThreads;
  const int64_t blocks_per_row = (a.hidden + per_block - 1) / per_block;
  IOB_REQUIRE(tokens * blocks_per_row <= INT32_MAX, "moe_sum: tensor too large for one launch");
  const unsigned grid = static_cast<unsigned>(tokens * blocks_per_row);
  if (vec) {
    MoeSumVecKernel<T><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(input), static_cast<T*>(out), a,
                                                    static_cast<int>(blocks_per_row));
  } else {
    MoeSumScalarKernel<T><<<grid, kThreads, 0, stream>>>(static_cast<const T*>(input), static_cast<T*>(out), a,
                                                       static_cast<int>(blocks_per_row));
  }
  return CheckLaunch("moe_sum launch");
}

// moe_sum over rows that sit in sorted (expert) order: slot s of token t is row position[t * topk + s]
// of `in` [rows, hidden]; a negative position contributes nothing.  Same accumulation (fp32, slots in
// ascending order, one rounding) as moe_sum on the [T, topk, hidden] tensor those rows would form.
template <typename T>
__global__ void __launch_bounds__(kThreads)
MoeGatherSumKernel(const T* __restrict__ in, const int32_t* __restrict__ position, T* __restrict__ out, int topk,
                   int64_t hidden, int blocks_per_row) {
  constexpr int kVec = 16 / sizeof(T);
  const int64_t token = blockIdx.x / blocks_per_row;
  const int64_t col = (static_cast<int64_t>(blockIdx.x % blocks_per_row) * kThreads + threadIdx.x) * kVec;
  if (col >= hidden) return;
  using P = Pack<T, kVec>;
  float acc[kVec];
#pragma unroll
  for (int i = 0; i < kVec; ++i) acc[i] = 0.0f;
  for (int slot = 0; slot < topk; ++slot) {
    const int row = position[token * topk + slot];
    if (row < 0) continue;
    const P v = *reinterpret_cast<const P*>(in + static_cast<int64_t>(row) * hidden + col);
#pragma unroll
    for (int i = 0; i < kVec; ++i) acc[i] += ToFloat<T>(v.v[i]);
  }
  P result;
#pragma unroll
  for (int i = 0; i < kVec; ++i) result.v[i] = FromFloat<T>(acc[i]);
  *reinterpret_cast<P*>(out + token * hidden + col) = result;
}

template <typename T>
int LaunchGatherSum(const void* input, const int32_t* position, void* out, int64_t tokens, int64_t topk, int64_t hidden,
                    cudaStream_t stream) {
  constexpr int kVec = 16 / sizeof(T);
  IOB_REQUIRE(hidden % kVec == 0 && reinterpret_cast<uintptr_t>(input) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "moe_gather_sum: rows must be 16-byte aligned and `hidden` a multiple of %d", kVec);
  const int64_t per_block = static_cast<int64_t>(kThreads) * kVec;
  const int64_t blocks_per_row = (hidden + per_block - 1) / per_block;
  IOB_REQUIRE(tokens * blocks_per_row <= INT32_MAX, "moe_gather_sum: tensor too large for one launch");
  MoeGatherSumKernel<T><<<static_cast<unsigned>(tokens * blocks_per_row), kThreads, 0, stream>>>(
      static_cast<const T*>(input), position, static_cast<T*>(out), static_cast<int>(topk), hidden,
      static_cast<int>(blocks_per_row));
  return CheckLaunch("moe_gather_sum launch");
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_silu_and_mul(const void* input, void* out, int dtype, int ndim,
                                           const int64_t* out_shape, const int64_t* input_strides,
                                           const int64_t* out_strides, void* stream) {
  using namespace iob;
  IOB_REQUIRE(ndim >= 1 && ndim <= kMaxDims, "silu_and_mul: supports 1 to 8 dimensions");
  IOB_REQUIRE(out_shape && input_strides && out_strides, "silu_and_mul: null shape or stride array");
  for (int d = 0; d < ndim; ++d) {
    IOB_REQUIRE(out_shape[d] >= 0 && input_strides[d] >= 0 && out_strides[d] >= 0,
                "silu_and_mul: negative extent or stride");
  }
  auto s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case IOB_F32: return LaunchSilu<float>(input, out, ndim, out_shape, input_strides, out_strides, s);
    case IOB_F16: return LaunchSilu<__half>(input, out, ndim, out_shape, input_strides, out_strides, s);
    case IOB_BF16: return LaunchSilu<__nv_bfloat16>(input, out, ndim, out_shape, input_strides, out_strides, s);
    default: return Fail(IOB_INVALID_ARGUMENT, "silu_and_mul: supports float32, float16 and bfloat16");
  }
}

extern "C" int infiniops_b200_moe_sum(const void* input, int dtype, int64_t num_tokens, int64_t topk,
                                      int64_t hidden, int64_t in_stride_t, int64_t in_stride_s,
                                      int64_t in_stride_h, const void* topk_ids, int ids_dtype,
                                      int64_t ids_stride_t, int64_t ids_stride_s, const int32_t* expert_map,
                                      int64_t expert_map_size, int64_t expert_map_stride, void* out,
                                      void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_tokens >= 0 && topk >= 0 && hidden >= 0, "moe_sum: negative extent");
  IOB_REQUIRE(in_stride_t >= 0 && in_stride_s >= 0 && in_stride_h >= 0,
              "moe_sum: input requires non-negative strides");
  IOB_REQUIRE(expert_map == nullptr || topk_ids != nullptr, "moe_sum: expert_map requires topk_ids");
  IOB_REQUIRE(topk_ids == nullptr || ids_dtype == IOB_I32 || ids_dtype == IOB_I64,
              "moe_sum: topk_ids must have int32 or int64 dtype");
  SumArgs a{topk, hidden, in_stride_t, in_stride_s, in_stride_h, topk_ids, ids_dtype == IOB_I64 ? 1 : 0,
            ids_stride_t, ids_stride_s, expert_map, expert_map_size, expert_map_stride};
  auto s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case IOB_F32: return LaunchSum<float>(input, out, num_tokens, a, s);
    case IOB_F16: return LaunchSum<__half>(input, out, num_tokens, a, s);
    case IOB_BF16: return LaunchSum<__nv_bfloat16>(input, out, num_tokens, a, s);
    default: return Fail(IOB_INVALID_ARGUMENT, "moe_sum: supports float32, float16 and bfloat16");
  }
}

extern "C" int infiniops_b200_moe_gather_sum(const void* input, int dtype, const int32_t* position, int64_t num_tokens,
                                             int64_t topk, int64_t hidden, void* out, void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_tokens >= 0 && topk > 0 && topk <= INT32_MAX && hidden > 0, "moe_gather_sum: invalid extents");
  if (num_tokens == 0) return IOB_OK;
  IOB_REQUIRE(input && position && out, "moe_gather_sum: null tensor pointer");
  auto s = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case IOB_F32: return LaunchGatherSum<float>(input, position, out, num_tokens, topk, hidden, s);
    case IOB_F16: return LaunchGatherSum<__half>(input, position, out, num_tokens, topk, hidden, s);
    case IOB_BF16: return LaunchGatherSum<__nv_bfloat16>(input, position, out, num_tokens, topk, hidden, s);
    default: return Fail(IOB_INVALID_ARGUMENT, "moe_gather_sum: supports float32, float16 and bfloat16");
  }
}
