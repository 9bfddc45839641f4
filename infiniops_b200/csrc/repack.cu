// GPTQ / AWQ -> Marlin tile layout repacking.
//
// One thread block owns a strip of TK quantised rows (16, or 32 for the 8-bit-activation
// layouts) by up to 256 columns.  It first expands that strip from the source packing into
// an unpacked byte tile in shared memory with coalesced word loads, then every thread
// assembles four consecutive output words from the tile and writes them with one 16-byte
// store.  The strip maps to one contiguous range of the output, so global traffic is one
// coalesced read and one coalesced write of the weights.
#include "common.cuh"

namespace iob {
namespace {

constexpr int kTileN = 256;
constexpr int kThreads = 256;

enum class Source { kGptq, kGptqPerm, kAwq };

// Which (k, n) of a 1024-element chunk sits in bit-field `field` of chunk word `inner`.
// 16-bit activations: chunk = 16 k x 64 n; 8-bit activations: chunk = 32 k x 32 n.
template <int kBits, bool kA8>
__device__ __forceinline__ void ChunkSource(int inner, int field, int& k, int& n) {
  if constexpr (!kA8 && kBits == 4) {
    const int lane = inner >> 2, sub = inner & 3;
    k = 2 * (lane & 3) + (field >> 2) + 8 * (field & 1);
    n = (lane >> 2) + 8 * ((field >> 1) & 1) + 16 * sub;
  } else if constexpr (!kA8 && kBits == 8) {
    const int lane = inner >> 3, sub = (inner >> 1) & 3, half = inner & 1;
    k = 2 * (lane & 3) + (field >> 1) + 8 * (field & 1);
    n = (lane >> 2) + 8 * half + 16 * sub;
  } else if constexpr (kA8 && kBits == 4) {
    const int lane = inner >> 2, sub = (inner >> 1) & 1, half = inner & 1;
    k = 4 * (lane & 3) + (field >> 1) + 16 * (field & 1);
    n = (lane >> 2) + 8 * half + 16 * sub;
  } else {
    const int lane = inner >> 3, sub = (inner >> 2) & 1, q = inner & 3;
    k = 4 * (lane & 3) + field + 16 * (q & 1);
    n = (lane >> 2) + 8 * (q >> 1) + 16 * sub;
  }
}

template <int kBits, bool kA8, Source kSource>
__global__ void __launch_bounds__(kThreads)
RepackKernel(const uint32_t* __restrict__ in, const int32_t* __restrict__ perm,
             uint32_t* __restrict__ out, int size_k, int size_n) {
  constexpr int kPf = 32 / kBits;
  constexpr int kTileK = kA8 ? 32 : 16;
  constexpr int kChunkN = kA8 ? 32 : 64;
  constexpr int kWordsPerChunk = 1024 / kPf;
  constexpr uint32_t kMask = (1u << kBits) - 1u;
  constexpr int kPitch = kTileN + 4;
  __shared__ __align__(16) uint8_t tile[kTileK][kPitch];

  const int n0 = blockIdx.x * kTileN;
  const int k0 = blockIdx.y * kTileK;
  const int tn = min(kTileN, size_n - n0);

  if constexpr (kSource == Source::kGptq) {
    constexpr int kRows = kTileK / kPf;
    for (int idx = threadIdx.x; idx < kRows * tn; idx += kThreads) {
      const int r = idx / tn, c = idx - r * tn;
      const uint32_t word = in[static_cast<int64_t>(k0 / kPf + r) * size_n + n0 + c];
#pragma unroll
      for (int i = 0; i < kPf; ++i) {
        tile[r * kPf + i][c] = static_cast<uint8_t>((word >> (kBits * i)) & kMask);
      }
    }
  } else if constexpr (kSource == Source::kGptqPerm) {
    for (int idx = threadIdx.x; idx < kTileK * tn; idx += kThreads) {
      const int k = idx / tn, c = idx - k * tn;
      const int src = perm[k0 + k];
      const uint32_t word = in[static_cast<int64_t>(src / kPf) * size_n + n0 + c];
      tile[k][c] = static_cast<uint8_t>((word >> (kBits * (src % kPf))) & kMask);
    }
  } else {
    // AWQ: logical column j of a word lives in field kOrder[j].
    constexpr int kOrder4[8] = {0, 4, 1, 5, 2, 6, 3, 7};
    constexpr int kOrder8[4] = {0, 2, 1, 3};
    const int words = tn / kPf;
    const int row_words = size_n / kPf;
    for (int idx = threadIdx.x; idx < kTileK * words; idx += kThreads) {
      const int k = idx / words, cw = idx - k * words;
      const uint32_t word = in[static_cast<int64_t>(k0 + k) * row_words + n0 / kPf + cw];
#pragma unroll
      for (int j = 0; j < kPf; ++j) {
        const int field = kBits == 4 ? kOrder4[j] : kOrder8[j & 3];
        tile[k][cw * kPf + j] = static_cast<uint8_t>((word >> (kBits * field)) & kMask);
      }
    }
  }
  __syncthreads();

  int64_t out_start;
  if constexpr (kA8) {
    out_start = (static_cast<int64_t>(k0 / 32) * (size_n / 32) + n0 / 32) * kWordsPerChunk;
  } else {
    out_start = static_cast<int64_t>(k0 / 16) * (static_cast<int64_t>(size_n) * 16 / kPf) +
                static_cast<int64_t>(n0) * 16 / kPf;
  }
  const int total_words = kTileK * tn / kPf;
  for (int w4 = threadIdx.x * 4; w4 < total_words; w4 += kThreads * 4) {
    uint32_t words[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int wi = w4 + u;
      const int chunk = wi / kWordsPerChunk;
      const int inner = wi - chunk * kWordsPerChunk;
      uint32_t word = 0;
#pragma unroll
      for (int field = 0; field < kPf; ++field) {
        int k, n;
        ChunkSource<kBits, kA8>(inner, field, k, n);
        word |= static_cast<uint32_t>(tile[k][chunk * kChunkN + n]) << (kBits * field);
      }
      words[u] = word;
    }
    *reinterpret_cast<uint4*>(out + out_start + w4) = make_uint4(words[0], words[1], words[2], words[3]);
  }
}

template <int kBits, bool kA8, Source kSource>
int Launch(const int32_t* in, const int32_t* perm, int32_t* out, int64_t size_k, int64_t size_n,
           cudaStream_t stream) {
  constexpr int kTileK = kA8 ? 32 : 16;
  const dim3 grid(static_cast<unsigned>((size_n + kTileN - 1) / kTileN),
                  static_cast<unsigned>(size_k / kTileK));
  RepackKernel<kBits, kA8, kSource><<<grid, kThreads, 0, stream>>>(
      reinterpret_cast<const uint32_t*>(in), perm, reinterpret_cast<uint32_t*>(out),
      static_cast<int>(size_k), static_cast<int>(size_n));
  return CheckLaunch("marlin repack launch");
}

int CheckCommon(const void* in, const void* out, int64_t size_k, int64_t size_n, int num_bits,
                int is_a_8bit) {
  IOB_REQUIRE(in != nullptr && out != nullptr, "marlin repack: null weight pointer");
  IOB_REQUIRE(num_bits == 4 || num_bits == 8, "marlin repack: `num_bits` must be 4 or 8");
  IOB_REQUIRE(size_k > 0 && size_n > 0 && size_k % 16 == 0 && size_n % 64 == 0,
              "marlin repack: needs positive `size_k` divisible by 16 and `size_n` divisible by 64");
  IOB_REQUIRE(!is_a_8bit || size_k % 32 == 0,
              "marlin repack: `size_k` must be divisible by 32 for 8-bit-activation layouts");
  IOB_REQUIRE(size_k <= INT32_MAX && size_n <= INT32_MAX && size_k / 16 <= 65535,
              "marlin repack: dimensions exceed kernel limits");
  IOB_REQUIRE(reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(in) % 4 == 0,
              "marlin repack: output must be 16-byte aligned");
  return IOB_OK;
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_gptq_marlin_repack(const int32_t* b_q_weight, const int32_t* perm,
                                                 int64_t size_k, int64_t size_n, int num_bits,
                                                 int is_a_8bit, int32_t* out, void* stream) {
  using namespace iob;
  if (const int rc = CheckCommon(b_q_weight, out, size_k, size_n, num_bits, is_a_8bit)) return rc;
  IOB_REQUIRE(!(is_a_8bit && perm != nullptr),
              "gptq_marlin_repack: `perm` is not supported for 8-bit-activation layouts");
  auto s = static_cast<cudaStream_t>(stream);
  if (perm != nullptr) {
    return num_bits == 4 ? Launch<4, false, Source::kGptqPerm>(b_q_weight, perm, out, size_k, size_n, s)
                         : Launch<8, false, Source::kGptqPerm>(b_q_weight, perm, out, size_k, size_n, s);
  }
  if (num_bits == 4) {
    return is_a_8bit ? Launch<4, true, Source::kGptq>(b_q_weight, nullptr, out, size_k, size_n, s)
                     : Launch<4, false, Source::kGptq>(b_q_weight, nullptr, out, size_k, size_n, s);
  }
  return is_a_8bit ? Launch<8, true, Source::kGptq>(b_q_weight, nullptr, out, size_k, size_n, s)
                   : Launch<8, false, Source::kGptq>(b_q_weight, nullptr, out, size_k, size_n, s);
}

extern "C" int infiniops_b200_awq_marlin_repack(const int32_t* b_q_weight, int64_t size_k,
                                                int64_t size_n, int num_bits, int is_a_8bit,
                                                int32_t* out, void* stream) {
  using namespace iob;
  if (const int rc = CheckCommon(b_q_weight, out, size_k, size_n, num_bits, is_a_8bit)) return rc;
  auto s = static_cast<cudaStream_t>(stream);
  if (num_bits == 4) {
    return is_a_8bit ? Launch<4, true, Source::kAwq>(b_q_weight, nullptr, out, size_k, size_n, s)
                     : Launch<4, false, Source::kAwq>(b_q_weight, nullptr, out, size_k, size_n, s);
  }
  return is_a_8bit ? Launch<8, true, Source::kAwq>(b_q_weight, nullptr, out, size_k, size_n, s)
                   : Launch<8, false, Source::kAwq>(b_q_weight, nullptr, out, size_k, size_n, s);
}
