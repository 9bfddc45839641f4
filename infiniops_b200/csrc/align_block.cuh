// Device pieces of moe_align_block_size shared by the stand-alone operator and by the fused
// router + sort launch: the stable per-expert ranking of up to 1024 routing ids by one thread block,
// the padded offsets, and the whole single-block sort.
#ifndef INFINIOPS_B200_ALIGN_BLOCK_CUH_
#define INFINIOPS_B200_ALIGN_BLOCK_CUH_

#include "common.cuh"

namespace iob {
namespace align {

constexpr int kChunk = 1024;
constexpr int kWarps = kChunk / 32;
constexpr unsigned kFull = 0xffffffffu;

__device__ __forceinline__ int MapExpert(int id, const int32_t* expert_map, int num_experts) {
  if (id < 0 || id >= num_experts) return -1;
  if (expert_map != nullptr) id = expert_map[id];
  return id >= 0 && id < num_experts ? id : -1;
}

struct Smem {
  uint16_t* warp_count;  // [kWarps][num_experts]: per-warp counts, then exclusive prefixes over warps
  int* expert_base;      // [num_experts]: first padded position of every expert
  int* expert_total;     // [num_experts]: ids routed to every expert
  int* warp_sums;        // [kWarps] scratch of the block scan
};

__device__ __forceinline__ Smem CarveSmem(unsigned char* raw, int num_experts) {
  Smem s;
  const int table = ((kWarps * num_experts + 1) & ~1);
  s.warp_count = reinterpret_cast<uint16_t*>(raw);
  s.expert_base = reinterpret_cast<int*>(raw + static_cast<size_t>(table) * sizeof(uint16_t));
  s.expert_total = s.expert_base + num_experts;
  s.warp_sums = s.expert_total + num_experts;
  return s;
}

inline size_t SmemBytes(int64_t num_experts) {
  const size_t table = ((kWarps * num_experts + 1) & ~1);
  return table * sizeof(uint16_t) + (2 * num_experts + kWarps) * sizeof(int);
}

// Stable rank of this thread's id among the chunk's ids with the same expert.  On return
// s.warp_count[w][e] holds the number of such ids in warps before w, and `chunk_total(e)`
// has been handed to `emit` for every expert.
template <typename Emit>
__device__ __forceinline__ int ChunkRank(const Smem& s, int expert, int num_experts, Emit emit) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < kWarps * num_experts; i += kChunk) s.warp_count[i] = 0;
  __syncthreads();
  const unsigned same = __match_any_sync(kFull, expert);
  const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
  if (expert >= 0 && rank_in_warp == 0) {
    s.warp_count[warp * num_experts + expert] = static_cast<uint16_t>(__popc(same));
  }
  __syncthreads();
  for (int e = tid; e < num_experts; e += kChunk) {
    int run = 0;
#pragma unroll 8
    for (int w = 0; w < kWarps; ++w) {
      const int c = s.warp_count[w * num_experts + e];
      s.warp_count[w * num_experts + e] = static_cast<uint16_t>(run);
      run += c;
    }
    emit(e, run);
  }
  __syncthreads();
  return expert >= 0 ? s.warp_count[warp * num_experts + expert] + rank_in_warp : 0;
}

// From s.expert_total: padded exclusive scan -> s.expert_base, block owners -> experts_ids,
// padded total -> num_tokens_post_pad.  Requires num_experts <= kChunk.
__device__ __forceinline__ void PadAndPublish(const Smem& s, int num_experts, int block_size,
                                              int32_t* experts_ids, int32_t* num_tokens_post_pad) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int count = tid < num_experts ? s.expert_total[tid] : 0;
  const int padded = (count + block_size - 1) / block_size * block_size;
  int incl = padded;
#pragma unroll
  for (int offset = 1; offset < 32; offset <<= 1) {
    const int up = __shfl_up_sync(kFull, incl, offset);
    if (lane >= offset) incl += up;
  }
  if (lane == 31) s.warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int v = s.warp_sums[lane];
#pragma unroll
    for (int offset = 1; offset < 32; offset <<= 1) {
      const int up = __shfl_up_sync(kFull, v, offset);
      if (lane >= offset) v += up;
    }
    s.warp_sums[lane] = v;  // inclusive over warps
  }
  __syncthreads();
  const int before = warp == 0 ? 0 : s.warp_sums[warp - 1];
  if (tid < num_experts) s.expert_base[tid] = before + incl - padded;
  const int total = s.warp_sums[kWarps - 1];
  __syncthreads();
  if (tid == 0) *num_tokens_post_pad = total;
  // Owner of block b = last expert whose base is <= b * block_size.
  for (int b = tid; b < total / block_size; b += kChunk) {
    const int pos = b * block_size;
    int lo = 0, hi = num_experts;  // first expert with base > pos
    while (lo < hi) {
      const int mid = (lo + hi) >> 1;
      if (s.expert_base[mid] <= pos) lo = mid + 1; else hi = mid;
    }
    experts_ids[b] = lo - 1;
  }
}

__device__ __forceinline__ void FillOutputs(int32_t* sorted_token_ids, int64_t sorted_size,
                                            int32_t* experts_ids, int64_t experts_size, int numel) {
  const int64_t stride = static_cast<int64_t>(gridDim.x) * kChunk;
  const int64_t start = static_cast<int64_t>(blockIdx.x) * kChunk + threadIdx.x;
  for (int64_t i = start; i < sorted_size; i += stride) sorted_token_ids[i] = numel;
  for (int64_t i = start; i < experts_size; i += stride) experts_ids[i] = -1;
}

// The whole operator for numel <= kChunk, run by one block of kChunk threads.  `topk_ids` may have
// been written earlier in this launch by this block (plain loads, after a block barrier).
__device__ __forceinline__ void AlignOneBlock(unsigned char* smem_raw, const int32_t* topk_ids, const int32_t* expert_map,
                                              int numel, int num_experts, int block_size, int32_t* sorted_token_ids,
                                              int64_t sorted_size, int32_t* experts_ids, int64_t experts_size,
                                              int32_t* num_tokens_post_pad) {
  const Smem s = CarveSmem(smem_raw, num_experts);
  FillOutputs(sorted_token_ids, sorted_size, experts_ids, experts_size, numel);
  const int tid = threadIdx.x;
  const int expert = tid < numel ? MapExpert(topk_ids[tid], expert_map, num_experts) : -1;
  const int rank = ChunkRank(s, expert, num_experts, [&](int e, int total) { s.expert_total[e] = total; });
  PadAndPublish(s, num_experts, block_size, experts_ids, num_tokens_post_pad);
  __syncthreads();
  if (expert >= 0) sorted_token_ids[s.expert_base[expert] + rank] = tid;
}

}  // namespace align
}  // namespace iob

#endif
