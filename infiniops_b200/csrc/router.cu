// MoE routers: topk_softmax and grouped_topk.
//
// Both run one warp per token.  The warp keeps the token's per-expert scores in shared
// memory, so the logits are read from HBM exactly once, and performs every reduction
// (max, sum, arg-max rounds, top-2 per group) with register shuffles; there is no
// block-wide barrier and no serial single-thread scan over experts.
#include <cfloat>
#include <algorithm>
#include <cmath>

#include "align_block.cuh"
#include "common.cuh"

namespace iob {
namespace {

constexpr unsigned kFull = 0xffffffffu;
constexpr int kMaxGroups = 32;

// Candidate ordering shared by both routers: larger value wins, equal values go to the
// smaller index; an empty slot (index < 0) never wins and always loses.
__device__ __forceinline__ bool IsBetter(float value, int index, float best_value, int best_index) {
  if (index < 0) return false;
  if (best_index < 0) return true;
  return value > best_value || (value == best_value && index < best_index);
}

__device__ __forceinline__ void WarpArgBest(float& value, int& index) {
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) {
    const float other_value = __shfl_xor_sync(kFull, value, offset);
    const int other_index = __shfl_xor_sync(kFull, index, offset);
    if (IsBetter(other_value, other_index, value, index)) {
      value = other_value;
      index = other_index;
    }
  }
  // Every lane continues with lane 0's winner, so the warp never disagrees (NaN scores
  // make the pairwise comparison non-commutative).
  value = __shfl_sync(kFull, value, 0);
  index = __shfl_sync(kFull, index, 0);
}

template <typename Index>
__device__ __forceinline__ void StoreIndex(Index* p, int v) { *p = static_cast<Index>(v); }

// ------------------------------------------------------------------------------------------
// topk_softmax and topk_sigmoid
// ------------------------------------------------------------------------------------------
// kSigmoid: the per-expert score is sigmoid(x) = 1 / (1 + exp(-x)) instead of the softmax over the
// row, the selection adds the correction bias in the same way, and the selected weights are
// multiplied by `scaling` (after the optional renormalisation).
template <typename In, typename Index, bool kSigmoid = false>
__device__ __forceinline__ void RouteTokenSoftmax(unsigned char* smem_raw, int warp, int warps_per_block, int token,
                                                  const In* __restrict__ gating, const float* __restrict__ bias,
                                                  const uint8_t* __restrict__ is_padding, float* topk_weights,
                                                  Index* topk_indices, int32_t* token_expert_indices, int num_tokens,
                                                  int num_experts, int topk, bool renormalize, float scaling) {
  const int lane = threadIdx.x & 31;
  const int padded = (num_experts + 3) & ~3;
  float* score = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warp) * num_experts;
  uint8_t* taken = smem_raw + static_cast<size_t>(warps_per_block) * (num_experts + kMaxGroups) * sizeof(float) +
                   static_cast<size_t>(warp) * padded;

  const In* row = gating + static_cast<int64_t>(token) * num_experts;
  if constexpr (kSigmoid) {
    for (int e = lane; e < num_experts; e += 32) {
      float sc = 1.0f / (1.0f + expf(-ToFloat<In>(row[e])));
      if (!isfinite(sc)) sc = 0.0f;
      score[e] = sc;
      taken[e] = 0;
    }
  } else {
  float row_max = -FLT_MAX;
  for (int e = lane; e < num_experts; e += 32) {
    const float v = ToFloat<In>(row[e]);
    score[e] = v;
    taken[e] = 0;
    row_max = fmaxf(row_max, v);
  }
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(kFull, row_max, offset));
  float row_sum = 0.0f;
  for (int e = lane; e < num_experts; e += 32) row_sum += expf(score[e] - row_max);
#pragma unroll
  for (int offset = 16; offset > 0; offset >>= 1) row_sum += __shfl_xor_sync(kFull, row_sum, offset);
  for (int e = lane; e < num_experts; e += 32) {
    float s = expf(score[e] - row_max) / row_sum;
    if (!isfinite(s)) s = 0.0f;
    score[e] = s;
  }
  }
  __syncwarp();

  const int64_t out = static_cast<int64_t>(token) * topk;
  float selected_sum = 0.0f;
  for (int rank = 0; rank < topk; ++rank) {
    float best = -FLT_MAX;
    int best_index = -1;
    for (int e = lane; e < num_experts; e += 32) {
      if (taken[e]) continue;
      const float candidate = score[e] + (bias != nullptr ? bias[e] : 0.0f);
      if (IsBetter(candidate, e, best, best_index)) {
        best = candidate;
        best_index = e;
      }
    }
    WarpArgBest(best, best_index);
    if (lane == 0) {
      const float weight = score[best_index];
      taken[best_index] = 1;
      topk_weights[out + rank] = weight;
      StoreIndex(topk_indices + out + rank, best_index);
      token_expert_indices[out + rank] = rank * num_tokens + token;
      selected_sum += weight;
    }
    __syncwarp();
  }
  if (lane == 0) {
    float scale = renormalize && selected_sum > 0.0f ? 1.0f / selected_sum : 1.0f;
    if constexpr (kSigmoid) scale = renormalize ? scaling / (selected_sum > 0.0f ? selected_sum : 1.0f) : scaling;
    const bool padding = is_padding != nullptr && is_padding[token] != 0;
    for (int rank = 0; rank < topk; ++rank) {
      topk_weights[out + rank] *= scale;
      if (padding) StoreIndex(topk_indices + out + rank, -1);
    }
  }
}

template <typename In, typename Index, bool kSigmoid = false>
__global__ void TopkSoftmaxKernel(const In* __restrict__ gating, const float* __restrict__ bias,
                                  const uint8_t* __restrict__ is_padding,
                                  float* __restrict__ topk_weights, Index* __restrict__ topk_indices,
                                  int32_t* __restrict__ token_expert_indices, int num_tokens,
                                  int num_experts, int topk, bool renormalize, int warps_per_block,
                                  float scaling = 1.0f) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int token = blockIdx.x * warps_per_block + warp;
  if (token >= num_tokens) return;
  RouteTokenSoftmax<In, Index, kSigmoid>(smem_raw, warp, warps_per_block, token, gating, bias, is_padding, topk_weights,
                                         topk_indices, token_expert_indices, num_tokens, num_experts, topk, renormalize,
                                         scaling);
}

// Shared memory per warp: one float and one flag byte (padded to 4) per expert, plus one
// float per expert group.
inline size_t RouterSmemBytes(int warps, int64_t num_experts) {
  return static_cast<size_t>(warps) *
         ((num_experts + kMaxGroups) * sizeof(float) + ((num_experts + 3) & ~3));
}

template <typename Kernel>
int PickWarps(Kernel kernel, int64_t num_experts, int& warps, size_t& smem) {
  warps = 4;
  smem = RouterSmemBytes(warps, num_experts);
  if (smem > 48 * 1024) {
    warps = 1;
    smem = RouterSmemBytes(warps, num_experts);
  }
  if (smem > 200 * 1024) {
    return Fail(IOB_UNSUPPORTED, "router: %lld experts exceed the shared-memory budget",
                static_cast<long long>(num_experts));
  }
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 static_cast<int>(smem));
    if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "router: %s", cudaGetErrorString(err));
  }
  return IOB_OK;
}

template <typename In, typename Index, bool kSigmoid = false>
int LaunchTopkSoftmax(const void* gating, const float* bias, const uint8_t* is_padding, bool renormalize,
                      float* weights, void* indices, int32_t* tei, int64_t t, int64_t e, int64_t k,
                      cudaStream_t stream, float scaling = 1.0f) {
  auto kernel = TopkSoftmaxKernel<In, Index, kSigmoid>;
  int warps;
  size_t smem;
  if (const int rc = PickWarps(kernel, e, warps, smem)) return rc;
  const unsigned grid = static_cast<unsigned>((t + warps - 1) / warps);
  kernel<<<grid, warps * 32, smem, stream>>>(static_cast<const In*>(gating), bias, is_padding, weights,
                                             static_cast<Index*>(indices), tei, static_cast<int>(t),
                                             static_cast<int>(e), static_cast<int>(k), renormalize, warps, scaling);
  return CheckLaunch(kSigmoid ? "topk_sigmoid launch" : "topk_softmax launch");
}

template <typename In, bool kSigmoid = false>
int DispatchTopkIndex(int index_dtype, const void* gating, const float* bias, const uint8_t* is_padding,
                      bool renormalize, float* weights, void* indices, int32_t* tei, int64_t t, int64_t e,
                      int64_t k, cudaStream_t stream, float scaling = 1.0f) {
  switch (index_dtype) {
    case IOB_I32:
      return LaunchTopkSoftmax<In, int32_t, kSigmoid>(gating, bias, is_padding, renormalize, weights, indices, tei, t, e, k, stream, scaling);
    case IOB_U32:
      return LaunchTopkSoftmax<In, uint32_t, kSigmoid>(gating, bias, is_padding, renormalize, weights, indices, tei, t, e, k, stream, scaling);
    case IOB_I64:
      return LaunchTopkSoftmax<In, int64_t, kSigmoid>(gating, bias, is_padding, renormalize, weights, indices, tei, t, e, k, stream, scaling);
    default:
      return Fail(IOB_INVALID_ARGUMENT, "top-k router: `topk_indices` must be int32, uint32 or int64");
  }
}

// ------------------------------------------------------------------------------------------
// grouped_topk
// ------------------------------------------------------------------------------------------
template <typename Score, int kScoring>
__device__ __forceinline__ Score ApplyScoring(Score v) {
  if constexpr (kScoring == 0) {
    return v;
  } else {
    const float x = ToFloat<Score>(v);
    return FromFloat<Score>(0.5f * tanhf(0.5f * x) + 0.5f);
  }
}

// score (+ bias), every intermediate rounded to the score type before the fp32 comparison.
template <typename Score, typename Bias, int kScoring>
__device__ __forceinline__ float SelectionScore(Score s, Bias b) {
  const Score routed = ApplyScoring<Score, kScoring>(s);
  const Score routed_bias = FromFloat<Score>(ToFloat<Bias>(b));
  return ToFloat<Score>(FromFloat<Score>(ToFloat<Score>(routed) + ToFloat<Score>(routed_bias)));
}

__device__ __forceinline__ void InsertTopTwo(float v, float& first, float& second) {
  if (v > first) {
    second = first;
    first = v;
  } else if (v > second) {
    second = v;
  }
}

template <typename Score, typename Bias, int kScoring>
__device__ __forceinline__ void RouteTokenGrouped(unsigned char* smem_raw, int warp, int warps_per_block, int token,
                                                  const Score* __restrict__ scores, const Bias* __restrict__ bias,
                                                  float* topk_values, int32_t* topk_indices, int num_experts,
                                                  int num_groups, int topk_group, int topk, bool renormalize,
                                                  float routed_scaling_factor) {
  const int lane = threadIdx.x & 31;
  const int padded = (num_experts + 3) & ~3;
  float* sel = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warp) * num_experts;
  float* group_scores = reinterpret_cast<float*>(smem_raw) + static_cast<size_t>(warps_per_block) * num_experts +
                        warp * kMaxGroups;
  uint8_t* skip = smem_raw + static_cast<size_t>(warps_per_block) * (num_experts + kMaxGroups) * sizeof(float) +
                  static_cast<size_t>(warp) * padded;
  const Score* row = scores + static_cast<int64_t>(token) * num_experts;
  const int per_group = num_experts / num_groups;
  const int64_t out = static_cast<int64_t>(token) * topk;

  for (int e = lane; e < num_experts; e += 32) sel[e] = SelectionScore<Score, Bias, kScoring>(row[e], bias[e]);
  __syncwarp();

  // Group score = rounded sum of the group's two largest selection scores.
  for (int g = 0; g < num_groups; ++g) {
    float first = -INFINITY, second = -INFINITY;
    for (int i = lane; i < per_group; i += 32) InsertTopTwo(sel[g * per_group + i], first, second);
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other_first = __shfl_xor_sync(kFull, first, offset);
      const float other_second = __shfl_xor_sync(kFull, second, offset);
      InsertTopTwo(other_first, first, second);
      InsertTopTwo(other_second, first, second);
    }
    if (lane == 0) group_scores[g] = ToFloat<Score>(FromFloat<Score>(first + second));
  }
  __syncwarp();

  // Pick `topk_group` groups.  There are at most 32 groups, so every lane repeats the same
  // short serial scan (first unselected group opens the round, later ones must beat it).
  unsigned selected_groups = 0;
  bool proceed = true;
  for (int rank = 0; rank < topk_group; ++rank) {
    float best = -INFINITY;
    int best_group = -1;
    for (int g = 0; g < num_groups; ++g) {
      if (!((selected_groups >> g) & 1u) && IsBetter(group_scores[g], g, best, best_group)) {
        best = group_scores[g];
        best_group = g;
      }
    }
    if (best_group < 0 || best == -INFINITY) {
      proceed = false;
      break;
    }
    selected_groups |= 1u << best_group;
  }
  if (!proceed) {
    for (int r = lane; r < topk; r += 32) {
      topk_indices[out + r] = r;
      topk_values[out + r] = 1.0f / static_cast<float>(topk);
    }
    return;
  }

  for (int e = lane; e < num_experts; e += 32) {
    const bool in_group = (selected_groups >> (e / per_group)) & 1u;
    skip[e] = (!in_group || !isfinite(ToFloat<Score>(row[e]))) ? 1 : 0;
  }
  __syncwarp();

  for (int rank = 0; rank < topk; ++rank) {
    float best = -INFINITY;
    int best_expert = -1;
    for (int e = lane; e < num_experts; e += 32) {
      if (skip[e]) continue;
      if (IsBetter(sel[e], e, best, best_expert)) {
        best = sel[e];
        best_expert = e;
      }
    }
    WarpArgBest(best, best_expert);
    if (lane == 0) {
      if (best_expert < 0) {
        best_expert = 0;
      } else {
        skip[best_expert] = 1;
      }
      topk_indices[out + rank] = best_expert;
      topk_values[out + rank] = ToFloat<Score>(ApplyScoring<Score, kScoring>(row[best_expert]));
    }
    __syncwarp();
  }

  if (lane == 0) {
    float scale = routed_scaling_factor;
    if (renormalize) {
      float sum = 1e-20f;
      for (int rank = 0; rank < topk; ++rank) sum += topk_values[out + rank];
      scale /= sum;
    }
    for (int rank = 0; rank < topk; ++rank) topk_values[out + rank] *= scale;
  }
}

template <typename Score, typename Bias, int kScoring>
__global__ void GroupedTopkKernel(const Score* __restrict__ scores, const Bias* __restrict__ bias,
                                  float* __restrict__ topk_values, int32_t* __restrict__ topk_indices,
                                  int num_tokens, int num_experts, int num_groups, int topk_group, int topk,
                                  bool renormalize, float routed_scaling_factor, int warps_per_block) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  const int token = blockIdx.x * warps_per_block + warp;
  if (token >= num_tokens) return;
  RouteTokenGrouped<Score, Bias, kScoring>(smem_raw, warp, warps_per_block, token, scores, bias, topk_values,
                                           topk_indices, num_experts, num_groups, topk_group, topk, renormalize,
                                           routed_scaling_factor);
}

template <typename Score, typename Bias, int kScoring>
int LaunchGroupedTopk(const void* scores, const void* bias, int64_t t, int64_t e, int64_t groups,
                      int64_t topk_group, int64_t topk, bool renormalize, double scaling, float* values,
                      int32_t* indices, cudaStream_t stream) {
  auto kernel = GroupedTopkKernel<Score, Bias, kScoring>;
  int warps;
  size_t smem;
  if (const int rc = PickWarps(kernel, e, warps, smem)) return rc;
  const unsigned grid = static_cast<unsigned>((t + warps - 1) / warps);
  kernel<<<grid, warps * 32, smem, stream>>>(static_cast<const Score*>(scores), static_cast<const Bias*>(bias),
                                             values, indices, static_cast<int>(t), static_cast<int>(e),
                                             static_cast<int>(groups), static_cast<int>(topk_group),
                                             static_cast<int>(topk), renormalize, static_cast<float>(scaling),
                                             warps);
  return CheckLaunch("grouped_topk launch");
}

template <typename Score, typename Bias>
int DispatchScoring(int scoring, const void* scores, const void* bias, int64_t t, int64_t e, int64_t groups,
                    int64_t topk_group, int64_t topk, bool renormalize, double scaling, float* values,
                    int32_t* indices, cudaStream_t stream) {
  return scoring == 0 ? LaunchGroupedTopk<Score, Bias, 0>(scores, bias, t, e, groups, topk_group, topk,
                                                          renormalize, scaling, values, indices, stream)
                      : LaunchGroupedTopk<Score, Bias, 1>(scores, bias, t, e, groups, topk_group, topk,
                                                          renormalize, scaling, values, indices, stream);
}

template <typename Score>
int DispatchBias(int bias_dtype, int scoring, const void* scores, const void* bias, int64_t t, int64_t e,
                 int64_t groups, int64_t topk_group, int64_t topk, bool renormalize, double scaling,
                 float* values, int32_t* indices, cudaStream_t stream) {
  switch (bias_dtype) {
    case IOB_F32:
      return DispatchScoring<Score, float>(scoring, scores, bias, t, e, groups, topk_group, topk, renormalize, scaling, values, indices, stream);
    case IOB_F16:
      return DispatchScoring<Score, __half>(scoring, scores, bias, t, e, groups, topk_group, topk, renormalize, scaling, values, indices, stream);
    case IOB_BF16:
      return DispatchScoring<Score, __nv_bfloat16>(scoring, scores, bias, t, e, groups, topk_group, topk, renormalize, scaling, values, indices, stream);
    default:
      return Fail(IOB_INVALID_ARGUMENT, "grouped_topk: `bias` must be float32, float16 or bfloat16");
  }
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_topk_softmax(const void* gating_output, int gating_dtype, const float* bias,
                                           const uint8_t* is_padding, int renormalize, float* topk_weights,
                                           void* topk_indices, int index_dtype,
                                           int32_t* token_expert_indices, int64_t num_tokens,
                                           int64_t num_experts, int64_t topk, void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_tokens >= 0 && num_experts > 0 && topk > 0 && topk <= num_experts,
              "topk_softmax: requires `topk` in [1, num_experts]");
  IOB_REQUIRE(num_tokens <= INT32_MAX / topk && num_experts <= INT32_MAX,
              "topk_softmax: output indices must fit int32 indexing");
  if (num_tokens == 0) return IOB_OK;
  IOB_REQUIRE(gating_output && topk_weights && topk_indices && token_expert_indices,
              "topk_softmax: null tensor pointer");
  auto s = static_cast<cudaStream_t>(stream);
  const bool renorm = renormalize != 0;
  switch (gating_dtype) {
    case IOB_F32:
      return DispatchTopkIndex<float>(index_dtype, gating_output, bias, is_padding, renorm, topk_weights, topk_indices, token_expert_indices, num_tokens, num_experts, topk, s);
    case IOB_F16:
      return DispatchTopkIndex<__half>(index_dtype, gating_output, bias, is_padding, renorm, topk_weights, topk_indices, token_expert_indices, num_tokens, num_experts, topk, s);
    case IOB_BF16:
      return DispatchTopkIndex<__nv_bfloat16>(index_dtype, gating_output, bias, is_padding, renorm, topk_weights, topk_indices, token_expert_indices, num_tokens, num_experts, topk, s);
    default:
      return Fail(IOB_INVALID_ARGUMENT, "topk_softmax: supports float32, float16 and bfloat16 input");
  }
}

extern "C" int infiniops_b200_topk_sigmoid(const void* gating_output, int gating_dtype,
                                           const float* e_score_correction_bias, const uint8_t* is_padding,
                                           int renormalize, double routed_scaling_factor, float* topk_weights,
                                           void* topk_ids, int index_dtype, int32_t* token_expert_indices,
                                           int64_t num_tokens, int64_t num_experts, int64_t topk, void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_tokens >= 0 && num_experts > 0 && topk > 0 && topk <= num_experts,
              "topk_sigmoid: requires `topk` in [1, num_experts]");
  IOB_REQUIRE(num_tokens <= INT32_MAX / topk && num_experts <= INT32_MAX,
              "topk_sigmoid: output indices must fit int32 indexing");
  IOB_REQUIRE(std::isfinite(routed_scaling_factor), "topk_sigmoid: requires a finite `routed_scaling_factor`");
  if (num_tokens == 0) return IOB_OK;
  IOB_REQUIRE(gating_output && topk_weights && topk_ids && token_expert_indices, "topk_sigmoid: null tensor pointer");
  auto s = static_cast<cudaStream_t>(stream);
  const bool renorm = renormalize != 0;
  const float scaling = static_cast<float>(routed_scaling_factor);
  switch (gating_dtype) {
    case IOB_F32:
      return DispatchTopkIndex<float, true>(index_dtype, gating_output, e_score_correction_bias, is_padding, renorm, topk_weights, topk_ids, token_expert_indices, num_tokens, num_experts, topk, s, scaling);
    case IOB_F16:
      return DispatchTopkIndex<__half, true>(index_dtype, gating_output, e_score_correction_bias, is_padding, renorm, topk_weights, topk_ids, token_expert_indices, num_tokens, num_experts, topk, s, scaling);
    case IOB_BF16:
      return DispatchTopkIndex<__nv_bfloat16, true>(index_dtype, gating_output, e_score_correction_bias, is_padding, renorm, topk_weights, topk_ids, token_expert_indices, num_tokens, num_experts, topk, s, scaling);
    default:
      return Fail(IOB_INVALID_ARGUMENT, "topk_sigmoid: supports float32, float16 and bfloat16 input");
  }
}

extern "C" int infiniops_b200_grouped_topk(const void* scores, int scores_dtype, const void* bias,
                                           int bias_dtype, int64_t num_tokens, int64_t num_experts,
                                           int64_t num_expert_group, int64_t topk_group, int64_t topk,
                                           int renormalize, double routed_scaling_factor, int scoring_func,
                                           float* topk_values, int32_t* topk_indices, void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_tokens >= 0 && num_experts > 0 && num_expert_group > 0 &&
                  num_expert_group <= kMaxGroups && num_experts % num_expert_group == 0,
              "grouped_topk: `num_expert_group` must be in [1, 32] and divide `num_experts`");
  IOB_REQUIRE(num_experts / num_expert_group >= 2, "grouped_topk: requires at least two experts per group");
  IOB_REQUIRE(topk_group > 0 && topk_group <= num_expert_group, "grouped_topk: invalid `topk_group`");
  IOB_REQUIRE(topk > 0 && topk <= num_experts && num_tokens <= INT32_MAX / topk,
              "grouped_topk: invalid `topk`");
  IOB_REQUIRE(scoring_func == 0 || scoring_func == 1, "grouped_topk: `scoring_func` must be 0 or 1");
  if (num_tokens == 0) return IOB_OK;
  IOB_REQUIRE(scores && bias && topk_values && topk_indices, "grouped_topk: null tensor pointer");
  auto s = static_cast<cudaStream_t>(stream);
  const bool renorm = renormalize != 0;
  switch (scores_dtype) {
    case IOB_F32:
      return DispatchBias<float>(bias_dtype, scoring_func, scores, bias, num_tokens, num_experts, num_expert_group, topk_group, topk, renorm, routed_scaling_factor, topk_values, topk_indices, s);
    case IOB_F16:
      return DispatchBias<__half>(bias_dtype, scoring_func, scores, bias, num_tokens, num_experts, num_expert_group, topk_group, topk, renorm, routed_scaling_factor, topk_values, topk_indices, s);
    case IOB_BF16:
      return DispatchBias<__nv_bfloat16>(bias_dtype, scoring_func, scores, bias, num_tokens, num_experts, num_expert_group, topk_group, topk, renorm, routed_scaling_factor, topk_values, topk_indices, s);
    default:
      return Fail(IOB_INVALID_ARGUMENT, "grouped_topk: `scores` must be float32, float16 or bfloat16");
  }
}

// ------------------------------------------------------------------------------------------
// router + token sort in one launch
// ------------------------------------------------------------------------------------------
// At decode sizes (tokens x top_k <= 1024) the router and moe_align_block_size are each a few
// microseconds of work behind a launch; here one block of 1024 threads does both: its 32 warps
// route the tokens (one token per warp at a time, the same per-token code as the operators above),
// and after a block barrier the same threads sort the routing ids they have just written.
namespace iob {
namespace {

inline size_t FusedAlignBytes(int64_t num_experts) { return (align::SmemBytes(num_experts) + 15) & ~size_t{15}; }

template <typename In, bool kSigmoid>
__global__ void __launch_bounds__(align::kChunk)
SoftmaxAlignKernel(const In* __restrict__ gating, const float* __restrict__ bias, const uint8_t* __restrict__ is_padding,
                   float* topk_weights, int32_t* topk_ids, int32_t* token_expert_indices, int num_tokens, int num_experts,
                   int topk, bool renormalize, float scaling, const int32_t* __restrict__ expert_map, int block_size,
                   int32_t* sorted_token_ids, int64_t sorted_size, int32_t* experts_ids, int64_t experts_size,
                   int32_t* num_tokens_post_pad, unsigned align_bytes) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  for (int token = warp; token < num_tokens; token += align::kWarps) {
    RouteTokenSoftmax<In, int32_t, kSigmoid>(smem_raw + align_bytes, warp, align::kWarps, token, gating, bias, is_padding,
                                             topk_weights, topk_ids, token_expert_indices, num_tokens, num_experts, topk,
                                             renormalize, scaling);
    __syncwarp();
  }
  __syncthreads();  // the ids are in global memory and visible to the whole block
  align::AlignOneBlock(smem_raw, topk_ids, expert_map, num_tokens * topk, num_experts, block_size, sorted_token_ids,
                       sorted_size, experts_ids, experts_size, num_tokens_post_pad);
}

template <typename Score, int kScoring>
__global__ void __launch_bounds__(align::kChunk)
GroupedAlignKernel(const Score* __restrict__ scores, const float* __restrict__ bias, float* topk_values,
                   int32_t* topk_ids, int num_tokens, int num_experts, int num_groups, int topk_group, int topk,
                   bool renormalize, float scaling, const int32_t* __restrict__ expert_map, int block_size,
                   int32_t* sorted_token_ids, int64_t sorted_size, int32_t* experts_ids, int64_t experts_size,
                   int32_t* num_tokens_post_pad, unsigned align_bytes) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int warp = threadIdx.x >> 5;
  for (int token = warp; token < num_tokens; token += align::kWarps) {
    RouteTokenGrouped<Score, float, kScoring>(smem_raw + align_bytes, warp, align::kWarps, token, scores, bias, topk_values,
                                              topk_ids, num_experts, num_groups, topk_group, topk, renormalize, scaling);
    __syncwarp();
  }
  __syncthreads();
  align::AlignOneBlock(smem_raw, topk_ids, expert_map, num_tokens * topk, num_experts, block_size, sorted_token_ids,
                       sorted_size, experts_ids, experts_size, num_tokens_post_pad);
}

// Whether the fused launch applies, and its shared memory.
bool FusedFits(int64_t num_tokens, int64_t num_experts, int64_t topk, size_t& smem) {
  if (num_tokens <= 0 || topk <= 0 || num_tokens * topk > align::kChunk || num_experts <= 0 || num_experts >= 1024) {
    return false;
  }
  smem = FusedAlignBytes(num_experts) + RouterSmemBytes(align::kWarps, num_experts);
  return smem <= 200 * 1024;
}

template <typename Kernel>
int AllowFusedSmem(Kernel kernel, size_t smem) {
  if (smem > 48 * 1024) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "router + sort: %s", cudaGetErrorString(err));
  }
  return IOB_OK;
}

int CheckSortOutputs(const char* op, int64_t numel, int64_t num_experts, int64_t block_size, const int32_t* sorted,
                     int64_t sorted_size, const int32_t* experts_ids, int64_t experts_size, const int32_t* npost) {
  IOB_REQUIRE(block_size > 0 && block_size <= INT32_MAX, "%s: requires a positive `block_size`", op);
  int64_t need_sorted = numel + num_experts * (block_size - 1);
  if (numel < num_experts) need_sorted = std::min(need_sorted, numel * block_size);
  const int64_t need_blocks = (need_sorted + block_size - 1) / block_size;
  IOB_REQUIRE(sorted_size >= need_sorted && experts_size >= need_blocks, "%s: the sort's output tensors are too small", op);
  IOB_REQUIRE(npost != nullptr && sorted != nullptr && experts_ids != nullptr, "%s: null tensor pointer", op);
  return IOB_OK;
}

template <typename In>
int LaunchSoftmaxAlign(bool sigmoid, const void* gating, const float* bias, const uint8_t* is_padding, float* w,
                       int32_t* ids, int32_t* tei, int t, int e, int k, bool renorm, float scaling,
                       const int32_t* expert_map, int bs, int32_t* sorted, int64_t sorted_size, int32_t* experts_ids,
                       int64_t experts_size, int32_t* npost, size_t smem, cudaStream_t s) {
  const unsigned align_bytes = static_cast<unsigned>(FusedAlignBytes(e));
  auto launch = [&](auto kernel) {
    if (const int rc = AllowFusedSmem(kernel, smem)) return rc;
    kernel<<<1, align::kChunk, smem, s>>>(static_cast<const In*>(gating), bias, is_padding, w, ids, tei, t, e, k, renorm,
                                          scaling, expert_map, bs, sorted, sorted_size, experts_ids, experts_size, npost,
                                          align_bytes);
    return CheckLaunch("router + sort launch");
  };
  return sigmoid ? launch(SoftmaxAlignKernel<In, true>) : launch(SoftmaxAlignKernel<In, false>);
}

template <typename Score>
int LaunchGroupedAlign(int scoring, const void* scores, const float* bias, float* values, int32_t* ids, int t, int e,
                       int groups, int topk_group, int k, bool renorm, float scaling, const int32_t* expert_map, int bs,
                       int32_t* sorted, int64_t sorted_size, int32_t* experts_ids, int64_t experts_size, int32_t* npost,
                       size_t smem, cudaStream_t s) {
  const unsigned align_bytes = static_cast<unsigned>(FusedAlignBytes(e));
  auto launch = [&](auto kernel) {
    if (const int rc = AllowFusedSmem(kernel, smem)) return rc;
    kernel<<<1, align::kChunk, smem, s>>>(static_cast<const Score*>(scores), bias, values, ids, t, e, groups, topk_group, k,
                                          renorm, scaling, expert_map, bs, sorted, sorted_size, experts_ids, experts_size,
                                          npost, align_bytes);
    return CheckLaunch("grouped router + sort launch");
  };
  return scoring == 1 ? launch(GroupedAlignKernel<Score, 1>) : launch(GroupedAlignKernel<Score, 0>);
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_moe_align_block_size(const int32_t*, const int32_t*, int64_t, int64_t, int64_t, int32_t*,
                                                   int64_t, int32_t*, int64_t, int32_t*, void*, size_t, void*);

extern "C" int infiniops_b200_topk_softmax_align(const void* gating_output, int gating_dtype, const float* bias,
                                                 const uint8_t* is_padding, int renormalize, int sigmoid,
                                                 double routed_scaling_factor, float* topk_weights, int32_t* topk_ids,
                                                 int32_t* token_expert_indices, int64_t num_tokens, int64_t num_experts,
                                                 int64_t topk, const int32_t* expert_map, int64_t block_size,
                                                 int32_t* sorted_token_ids, int64_t sorted_size, int32_t* experts_ids,
                                                 int64_t experts_size, int32_t* num_tokens_post_pad, void* scratch,
                                                 size_t scratch_bytes, void* stream) {
  using namespace iob;
  size_t smem = 0;
  const bool known = gating_dtype == IOB_F32 || gating_dtype == IOB_F16 || gating_dtype == IOB_BF16;
  if (!known || !FusedFits(num_tokens, num_experts, topk, smem) || topk > num_experts) {
    // two launches (or three): the operators themselves, which also report what is wrong with the arguments
    const int rc = sigmoid ? infiniops_b200_topk_sigmoid(gating_output, gating_dtype, bias, is_padding, renormalize,
                                                         routed_scaling_factor, topk_weights, topk_ids, IOB_I32,
                                                         token_expert_indices, num_tokens, num_experts, topk, stream)
                           : infiniops_b200_topk_softmax(gating_output, gating_dtype, bias, is_padding, renormalize,
                                                         topk_weights, topk_ids, IOB_I32, token_expert_indices, num_tokens,
                                                         num_experts, topk, stream);
    if (rc != IOB_OK) return rc;
    return infiniops_b200_moe_align_block_size(topk_ids, expert_map, num_tokens * topk, num_experts, block_size,
                                               sorted_token_ids, sorted_size, experts_ids, experts_size,
                                               num_tokens_post_pad, scratch, scratch_bytes, stream);
  }
  IOB_REQUIRE(gating_output && topk_weights && topk_ids && token_expert_indices, "topk_softmax_align: null tensor pointer");
  IOB_REQUIRE(!sigmoid || std::isfinite(routed_scaling_factor), "topk_softmax_align: requires a finite scaling factor");
  if (const int rc = CheckSortOutputs("topk_softmax_align", num_tokens * topk, num_experts, block_size, sorted_token_ids,
                                      sorted_size, experts_ids, experts_size, num_tokens_post_pad)) {
    return rc;
  }
  auto s = static_cast<cudaStream_t>(stream);
  const int t = static_cast<int>(num_tokens), e = static_cast<int>(num_experts), k = static_cast<int>(topk);
  const float scaling = sigmoid ? static_cast<float>(routed_scaling_factor) : 1.0f;
  const bool renorm = renormalize != 0, sig = sigmoid != 0;
  const int bs = static_cast<int>(block_size);
  switch (gating_dtype) {
    case IOB_F32:
      return LaunchSoftmaxAlign<float>(sig, gating_output, bias, is_padding, topk_weights, topk_ids, token_expert_indices, t, e, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
    case IOB_F16:
      return LaunchSoftmaxAlign<__half>(sig, gating_output, bias, is_padding, topk_weights, topk_ids, token_expert_indices, t, e, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
    default:
      return LaunchSoftmaxAlign<__nv_bfloat16>(sig, gating_output, bias, is_padding, topk_weights, topk_ids, token_expert_indices, t, e, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
  }
}

extern "C" int infiniops_b200_grouped_topk_align(const void* scores, int scores_dtype, const void* bias, int bias_dtype,
                                                 int64_t num_tokens, int64_t num_experts, int64_t num_expert_group,
                                                 int64_t topk_group, int64_t topk, int renormalize,
                                                 double routed_scaling_factor, int scoring_func, float* topk_values,
                                                 int32_t* topk_ids, const int32_t* expert_map, int64_t block_size,
                                                 int32_t* sorted_token_ids, int64_t sorted_size, int32_t* experts_ids,
                                                 int64_t experts_size, int32_t* num_tokens_post_pad, void* scratch,
                                                 size_t scratch_bytes, void* stream) {
  using namespace iob;
  size_t smem = 0;
  const bool known = scores_dtype == IOB_F32 || scores_dtype == IOB_F16 || scores_dtype == IOB_BF16;
  const bool valid = num_expert_group > 0 && num_expert_group <= kMaxGroups && num_experts > 0 &&
                     num_experts % num_expert_group == 0 && num_experts / num_expert_group >= 2 && topk_group > 0 &&
                     topk_group <= num_expert_group && topk > 0 && topk <= num_experts &&
                     (scoring_func == 0 || scoring_func == 1) && scores && bias && topk_values && topk_ids;
  if (!known || !valid || bias_dtype != IOB_F32 || !FusedFits(num_tokens, num_experts, topk, smem)) {
    const int rc = infiniops_b200_grouped_topk(scores, scores_dtype, bias, bias_dtype, num_tokens, num_experts,
                                               num_expert_group, topk_group, topk, renormalize, routed_scaling_factor,
                                               scoring_func, topk_values, topk_ids, stream);
    if (rc != IOB_OK) return rc;
    return infiniops_b200_moe_align_block_size(topk_ids, expert_map, num_tokens * topk, num_experts, block_size,
                                               sorted_token_ids, sorted_size, experts_ids, experts_size,
                                               num_tokens_post_pad, scratch, scratch_bytes, stream);
  }
  if (const int rc = CheckSortOutputs("grouped_topk_align", num_tokens * topk, num_experts, block_size, sorted_token_ids,
                                      sorted_size, experts_ids, experts_size, num_tokens_post_pad)) {
    return rc;
  }
  auto s = static_cast<cudaStream_t>(stream);
  const int t = static_cast<int>(num_tokens), e = static_cast<int>(num_experts), k = static_cast<int>(topk);
  const int groups = static_cast<int>(num_expert_group), tg = static_cast<int>(topk_group);
  const float scaling = static_cast<float>(routed_scaling_factor);
  const bool renorm = renormalize != 0;
  const int bs = static_cast<int>(block_size);
  const float* fbias = static_cast<const float*>(bias);
  switch (scores_dtype) {
    case IOB_F32:
      return LaunchGroupedAlign<float>(scoring_func, scores, fbias, topk_values, topk_ids, t, e, groups, tg, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
    case IOB_F16:
      return LaunchGroupedAlign<__half>(scoring_func, scores, fbias, topk_values, topk_ids, t, e, groups, tg, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
    default:
      return LaunchGroupedAlign<__nv_bfloat16>(scoring_func, scores, fbias, topk_values, topk_ids, t, e, groups, tg, k, renorm, scaling, expert_map, bs, sorted_token_ids, sorted_size, experts_ids, experts_size, num_tokens_post_pad, smem, s);
  }
}
