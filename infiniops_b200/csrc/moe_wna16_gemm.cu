// moe_wna16_gemm: routed weight-only GEMM on the plain (non-Marlin) layout.
//
//   b_qweight uint8 [E, N, K / (8 / bit)]   4-bit: low nibble = even k, high nibble = odd k
//   b_scales        [E, N, G]               G = K / group_size
//   b_qzeros  uint8 [E, N / (8 / bit), G]   4-bit: low nibble = even n; absent: zero point 2^(bit-1)
//   output          [M, top_k, N]           row r = flat routing id, zero where nothing was routed
//
// One thread block per (routing block, 128 output columns); a thread owns one column.  The block's
// activation rows are staged in shared memory 256 k at a time; every thread streams its own weight
// row (contiguous along k) one 32-bit word at a time, dequantises in fp32 -- (q - zero) * scale -- and
// accumulates in fp32, eight rows per pass.  Each output element is written exactly once, so the
// result does not depend on scheduling (the reference accumulates K-slices with atomics on a
// zeroed output; both start from a zero-filled output).
#include <algorithm>

#include "common.cuh"

namespace iob {
namespace {

constexpr int kCols = 128;   // output columns per block = threads
constexpr int kChunkK = 256; // k staged per step
constexpr int kRows = 8;     // rows accumulated per pass

template <typename T, int kBit>
__global__ void __launch_bounds__(kCols)
MoeWna16GemmKernel(const T* __restrict__ input, const uint8_t* __restrict__ qweight, const T* __restrict__ scales,
                   const uint8_t* __restrict__ qzeros, const float* __restrict__ topk_weights,
                   const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                   const int32_t* __restrict__ num_post_pad, long long sorted_size, int top_k, int block_m, int size_m,
                   int size_n, int size_k, int groups, T* __restrict__ output) {
  __shared__ float act[kRows][kChunkK];
  __shared__ int rows[64];
  __shared__ int n_valid;
  const long long first = static_cast<long long>(blockIdx.x) * block_m;
  if (first >= *num_post_pad) return;
  const int expert = expert_ids[blockIdx.x];
  if (expert < 0) return;
  if (threadIdx.x == 0) {
    int v = 0;
    for (; v < block_m; ++v) {
      if (first + v >= sorted_size) break;
      const int route = sorted_ids[first + v];
      if (route < 0 || route / top_k >= size_m) break;  // padding ends the block
      rows[v] = route;
    }
    n_valid = v;
  }
  __syncthreads();
  const int valid = n_valid;
  const int n = blockIdx.y * kCols + threadIdx.x;
  const bool n_ok = n < size_n;
  constexpr int kPerByte = 8 / kBit;
  const int group_size = size_k / groups;
  const uint8_t* wrow = qweight + (static_cast<size_t>(expert) * size_n + (n_ok ? n : 0)) * (size_k / kPerByte);
  const T* srow = scales + (static_cast<size_t>(expert) * size_n + (n_ok ? n : 0)) * groups;
  const uint8_t* zrow =
      qzeros == nullptr ? nullptr : qzeros + (static_cast<size_t>(expert) * (size_n / kPerByte) + (n_ok ? n : 0) / kPerByte) * groups;
  for (int r0 = 0; r0 < valid; r0 += kRows) {
    const int pass_rows = min(kRows, valid - r0);
    float acc[kRows];
#pragma unroll
    for (int r = 0; r < kRows; ++r) acc[r] = 0.0f;
    for (int k0 = 0; k0 < size_k; k0 += kChunkK) {
      const int chunk = min(kChunkK, size_k - k0);
      __syncthreads();
      for (int i = threadIdx.x; i < pass_rows * chunk; i += kCols) {
        const int r = i / chunk, kk = i - r * chunk;
        act[r][kk] = ToFloat<T>(input[static_cast<size_t>(rows[r0 + r] / top_k) * size_k + k0 + kk]);
      }
      __syncthreads();
      if (!n_ok) continue;
      // one 32-bit word of the weight row at a time (8 values of 4 bits, 4 of 8): K and the group
      // size are multiples of that, so a word never straddles a group
      constexpr int kPerWord = 32 / kBit;
      for (int kk = 0; kk < chunk; kk += kPerWord) {
        const int k = k0 + kk;
        const int g = k / group_size;
        const float scale = ToFloat<T>(srow[g]);
        float zero = static_cast<float>(1 << (kBit - 1));
        if (zrow != nullptr) {
          const uint8_t z = zrow[g];
          zero = static_cast<float>(kBit == 4 ? (z >> ((n & 1) * 4)) & 0xF : z);
        }
        const uint32_t word = *reinterpret_cast<const uint32_t*>(wrow + k / kPerByte);
        float w[kPerWord];
#pragma unroll
        for (int b = 0; b < kPerWord; ++b) {
          w[b] = (static_cast<float>((word >> (kBit * b)) & ((1u << kBit) - 1u)) - zero) * scale;
        }
#pragma unroll
        for (int r = 0; r < kRows; ++r) {
          if (r < pass_rows) {
            float sum = acc[r];
#pragma unroll
            for (int b = 0; b < kPerWord; ++b) sum = fmaf(w[b], act[r][kk + b], sum);
            acc[r] = sum;
          }
        }
      }
    }
    if (n_ok) {
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        if (r < pass_rows) {
          const int route = rows[r0 + r];
          float v = acc[r];
          if (topk_weights != nullptr) v *= topk_weights[route];
          output[static_cast<size_t>(route) * size_n + n] = FromFloat<T>(v);
        }
      }
    }
  }
}

template <typename T>
int Launch(int bit, dim3 grid, cudaStream_t s, const void* input, const uint8_t* qweight, const void* scales,
           const uint8_t* qzeros, const float* topk_weights, const int32_t* sorted_ids, const int32_t* expert_ids,
           const int32_t* npost, long long sorted_size, int top_k, int block_m, int m, int n, int k, int groups,
           void* output) {
  if (bit == 4) {
    MoeWna16GemmKernel<T, 4><<<grid, kCols, 0, s>>>(static_cast<const T*>(input), qweight, static_cast<const T*>(scales),
                                                    qzeros, topk_weights, sorted_ids, expert_ids, npost, sorted_size, top_k,
                                                    block_m, m, n, k, groups, static_cast<T*>(output));
  } else {
    MoeWna16GemmKernel<T, 8><<<grid, kCols, 0, s>>>(static_cast<const T*>(input), qweight, static_cast<const T*>(scales),
                                                    qzeros, topk_weights, sorted_ids, expert_ids, npost, sorted_size, top_k,
                                                    block_m, m, n, k, groups, static_cast<T*>(output));
  }
  return CheckLaunch("moe_wna16_gemm launch");
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_moe_wna16_gemm(const void* input, int dtype, const uint8_t* b_qweight, const void* b_scales,
                                             const uint8_t* b_qzeros, const float* topk_weights,
                                             const int32_t* sorted_token_ids, const int32_t* expert_ids,
                                             const int32_t* num_tokens_post_pad, int64_t sorted_size,
                                             int64_t expert_ids_size, int64_t top_k, int64_t block_size_m, int64_t bit,
                                             int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups,
                                             int64_t num_experts, void* output, void* stream) {
  using namespace iob;
  const char* op = "moe_wna16_gemm";
  IOB_REQUIRE(dtype == IOB_F16 || dtype == IOB_BF16, "%s: supports float16 and bfloat16 inputs", op);
  IOB_REQUIRE(bit == 4 || bit == 8, "%s: requires 4-bit or 8-bit weights", op);
  IOB_REQUIRE(size_m > 0 && size_n > 0 && size_k > 0 && num_experts > 0 && top_k > 0, "%s: requires positive dimensions", op);
  IOB_REQUIRE(num_groups > 0 && size_k % num_groups == 0, "%s: requires an integral quantization group size", op);
  const int64_t per_word = 32 / bit;
  IOB_REQUIRE(size_k % (8 / bit) == 0 && size_n % per_word == 0 && (size_k / num_groups) % per_word == 0,
              "%s: packed dimensions are incompatible with `bit`", op);
  IOB_REQUIRE(block_size_m > 0 && block_size_m <= 64, "%s: received unsupported block sizes", op);
  IOB_REQUIRE(size_m <= INT32_MAX / top_k && size_n <= INT32_MAX && size_k <= INT32_MAX, "%s: dimensions exceed int32", op);
  IOB_REQUIRE(input && b_qweight && b_scales && sorted_token_ids && expert_ids && num_tokens_post_pad && output,
              "%s: null tensor pointer", op);
  int64_t effective = sorted_size;
  if (size_m <= block_size_m) effective = std::min<int64_t>(effective, size_m * block_size_m * top_k);
  const int64_t blocks = (effective + block_size_m - 1) / block_size_m;
  IOB_REQUIRE(sorted_size > 0 && expert_ids_size >= blocks, "%s: routing metadata is too small", op);
  auto s = static_cast<cudaStream_t>(stream);
  // rows nothing is routed to read as zero, as in the reference (which also clears the output first)
  if (cudaMemsetAsync(output, 0, static_cast<size_t>(size_m) * top_k * size_n * 2, s) != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "%s: clearing the output failed", op);
  }
  const dim3 grid(static_cast<unsigned>(blocks), static_cast<unsigned>((size_n + kCols - 1) / kCols));
  if (dtype == IOB_BF16) {
    return Launch<__nv_bfloat16>(static_cast<int>(bit), grid, s, input, b_qweight, b_scales, b_qzeros, topk_weights,
                                 sorted_token_ids, expert_ids, num_tokens_post_pad, sorted_size, static_cast<int>(top_k),
                                 static_cast<int>(block_size_m), static_cast<int>(size_m), static_cast<int>(size_n),
                                 static_cast<int>(size_k), static_cast<int>(num_groups), output);
  }
  return Launch<__half>(static_cast<int>(bit), grid, s, input, b_qweight, b_scales, b_qzeros, topk_weights,
                        sorted_token_ids, expert_ids, num_tokens_post_pad, sorted_size, static_cast<int>(top_k),
                        static_cast<int>(block_size_m), static_cast<int>(size_m), static_cast<int>(size_n),
                        static_cast<int>(size_k), static_cast<int>(num_groups), output);
}
