// moe_align_block_size: stable grouping of routing ids by expert, padded to blocks.
//
// The ids are cut into chunks of 1024 (one per thread block, one id per thread).  Inside a
// chunk a thread finds its stable rank among the ids of the same expert from a warp
// `match.any` ballot plus a per-warp / per-expert count table in shared memory -- no atomics
// on the ordering path, so the result is deterministic and equals the ascending-index order
// a serial scan would give.  Up to 1024 ids the whole operator is ONE launch of ONE block.
// Beyond that, a counting launch leaves per-chunk histograms in scratch, its last-arriving
// block (an atomic ticket, no spinning) turns them into offsets, and a second launch scatters.
#include "align_block.cuh"
#include "common.cuh"

namespace iob {
namespace {

using namespace align;

// Whole operator in one block (numel <= kChunk).
__global__ void __launch_bounds__(kChunk)
AlignSingleBlockKernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map,
                       int numel, int num_experts, int block_size, int32_t* __restrict__ sorted_token_ids,
                       int64_t sorted_size, int32_t* __restrict__ experts_ids, int64_t experts_size,
                       int32_t* __restrict__ num_tokens_post_pad) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  AlignOneBlock(smem_raw, topk_ids, expert_map, numel, num_experts, block_size, sorted_token_ids, sorted_size,
                experts_ids, experts_size, num_tokens_post_pad);
}

// Scratch layout (int32): [0] ticket, [1 .. E] expert_base, then [chunks][E] histograms.
__global__ void __launch_bounds__(kChunk)
AlignCountKernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map, int numel,
                 int num_experts, int block_size, int32_t* __restrict__ sorted_token_ids,
                 int64_t sorted_size, int32_t* __restrict__ experts_ids, int64_t experts_size,
                 int32_t* __restrict__ num_tokens_post_pad, int32_t* __restrict__ scratch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ int is_last;
  const Smem s = CarveSmem(smem_raw, num_experts);
  FillOutputs(sorted_token_ids, sorted_size, experts_ids, experts_size, numel);
  const int tid = threadIdx.x;
  const int idx = blockIdx.x * kChunk + tid;
  const int expert = idx < numel ? MapExpert(topk_ids[idx], expert_map, num_experts) : -1;
  int32_t* hist = scratch + 1 + num_experts;
  ChunkRank(s, expert, num_experts,
            [&](int e, int total) { hist[static_cast<int64_t>(blockIdx.x) * num_experts + e] = total; });
  __threadfence();
  __syncthreads();
  if (tid == 0) is_last = atomicAdd(scratch, 1) == static_cast<int>(gridDim.x) - 1;
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // Exclusive prefix over chunks, in place; totals to shared memory.
  for (int e = tid; e < num_experts; e += kChunk) {
    int run = 0;
    for (unsigned c = 0; c < gridDim.x; ++c) {
      const int64_t at = static_cast<int64_t>(c) * num_experts + e;
      const int v = hist[at];
      hist[at] = run;
      run += v;
    }
    s.expert_total[e] = run;
  }
  __syncthreads();
  PadAndPublish(s, num_experts, block_size, experts_ids, num_tokens_post_pad);
  __syncthreads();
  for (int e = tid; e < num_experts; e += kChunk) scratch[1 + e] = s.expert_base[e];
  if (tid == 0) scratch[0] = 0;
}

__global__ void __launch_bounds__(kChunk)
AlignScatterKernel(const int32_t* __restrict__ topk_ids, const int32_t* __restrict__ expert_map, int numel,
                   int num_experts, int32_t* __restrict__ sorted_token_ids,
                   const int32_t* __restrict__ scratch) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const Smem s = CarveSmem(smem_raw, num_experts);
  const int idx = blockIdx.x * kChunk + threadIdx.x;
  const int expert = idx < numel ? MapExpert(topk_ids[idx], expert_map, num_experts) : -1;
  const int rank = ChunkRank(s, expert, num_experts, [](int, int) {});
  if (expert >= 0) {
    const int32_t* hist = scratch + 1 + num_experts;
    const int at = scratch[1 + expert] + hist[static_cast<int64_t>(blockIdx.x) * num_experts + expert] + rank;
    sorted_token_ids[at] = idx;
  }
}

// get_cutlass_moe_mm_data: per-expert row counts and offsets, the two grouped-GEMM problem-size
// tables, and the permutation that groups the routes by expert.  One block; the routes are walked
// twice in chunks of 1024 (count, then place) with the same stable ranking as the sort above, so the
// placement inside an expert is by ascending route index and does not vary from run to run (the
// reference places with atomics, in any order).
__global__ void __launch_bounds__(kChunk)
MmDataKernel(const int32_t* __restrict__ topk_ids, int32_t* __restrict__ expert_offsets,
             int32_t* __restrict__ problem_sizes1, int32_t* __restrict__ problem_sizes2,
             int32_t* __restrict__ input_permutation, int32_t* __restrict__ output_permutation,
             int32_t* __restrict__ blockscale_offsets, int numel, int topk, int num_experts, int n, int k,
             bool is_gated) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const Smem s = CarveSmem(smem_raw, num_experts);
  const int tid = threadIdx.x;
  const bool swap_ab = blockscale_offsets == nullptr && numel <= 64;
  const int count_index = swap_ab ? 1 : 0;
  const int n1 = is_gated ? 2 * n : n;
  for (int e = tid; e < num_experts; e += kChunk) s.expert_total[e] = 0;
  for (int i = tid; i < numel; i += kChunk) input_permutation[i] = -1;
  __syncthreads();
  auto expert_of = [&](int i) {
    if (i >= numel) return -1;
    const int e = topk_ids[i];
    return e >= 0 && e < num_experts ? e : -1;
  };
  for (int start = 0; start < numel; start += kChunk) {
    ChunkRank(s, expert_of(start + tid), num_experts, [&](int e, int total) { s.expert_total[e] += total; });
  }
  __syncthreads();
  if (tid == 0) {
    int offset = 0, scale_offset = 0;
    expert_offsets[0] = 0;
    if (blockscale_offsets != nullptr) blockscale_offsets[0] = 0;
    for (int e = 0; e < num_experts; ++e) {
      const int count = s.expert_total[e];
      s.expert_base[e] = offset;
      offset += count;
      expert_offsets[e + 1] = offset;
      if (blockscale_offsets != nullptr) {
        scale_offset += (count + 127) / 128 * 128;
        blockscale_offsets[e + 1] = scale_offset;
      }
    }
    s.warp_sums[0] = offset;
  }
  __syncthreads();
  const int valid_total = s.warp_sums[0];
  for (int e = tid; e < num_experts; e += kChunk) {
    const int count = s.expert_total[e];
    int* p1 = problem_sizes1 + 3 * e;
    int* p2 = problem_sizes2 + 3 * e;
    p1[0] = swap_ab ? n1 : count;
    p1[1] = swap_ab ? count : n1;
    p1[2] = k;
    p2[0] = swap_ab ? k : count;
    p2[1] = swap_ab ? count : k;
    p2[2] = n;
    (void)count_index;
  }
  __syncthreads();
  for (int start = 0; start < numel; start += kChunk) {
    const int i = start + tid;
    const int expert = expert_of(i);
    const int rank = ChunkRank(s, expert, num_experts, [&](int e, int total) { s.expert_total[e] = total; });
    if (i < numel) {
      if (expert >= 0) {
        const int destination = s.expert_base[expert] + rank;
        input_permutation[destination] = i / topk;
        output_permutation[i] = destination;
      } else {
        output_permutation[i] = topk_ids[i] == -1 ? valid_total : -1;
      }
    }
    __syncthreads();
    for (int e = tid; e < num_experts; e += kChunk) s.expert_base[e] += s.expert_total[e];
  }
}

template <typename Kernel>
int AllowSmem(Kernel kernel, size_t bytes) {
  if (bytes > 48 * 1024) {
    const cudaError_t err =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(bytes));
    if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "moe_align_block_size: %s", cudaGetErrorString(err));
  }
  return IOB_OK;
}

}  // namespace
}  // namespace iob

extern "C" size_t infiniops_b200_moe_align_block_size_scratch_bytes(int64_t numel, int64_t num_experts) {
  if (numel <= iob::kChunk) return 0;
  const int64_t chunks = (numel + iob::kChunk - 1) / iob::kChunk;
  return static_cast<size_t>(1 + num_experts + chunks * num_experts) * sizeof(int32_t);
}

extern "C" int infiniops_b200_moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map,
                                                   int64_t numel, int64_t num_experts, int64_t block_size,
                                                   int32_t* sorted_token_ids, int64_t sorted_size,
                                                   int32_t* experts_ids, int64_t experts_size,
                                                   int32_t* num_tokens_post_pad, void* scratch,
                                                   size_t scratch_bytes, void* stream) {
  using namespace iob;
  IOB_REQUIRE(num_experts > 0 && num_experts < 1024, "moe_align_block_size: requires `num_experts` in [1, 1023]");
  IOB_REQUIRE(block_size > 0 && block_size <= INT32_MAX, "moe_align_block_size: requires a positive `block_size`");
  IOB_REQUIRE(numel >= 0 && numel <= INT32_MAX, "moe_align_block_size: requires int32-addressable token indices");
  int64_t need_sorted = numel + num_experts * (block_size - 1);
  if (numel < num_experts) need_sorted = numel * block_size < need_sorted ? numel * block_size : need_sorted;
  const int64_t need_blocks = (need_sorted + block_size - 1) / block_size;
  IOB_REQUIRE(need_sorted <= INT32_MAX, "moe_align_block_size: requires int32-addressable padded indices");
  IOB_REQUIRE(sorted_size >= need_sorted && experts_size >= need_blocks,
              "moe_align_block_size: output tensors are too small");
  IOB_REQUIRE(num_tokens_post_pad != nullptr && (sorted_size == 0 || sorted_token_ids != nullptr) &&
                  (experts_size == 0 || experts_ids != nullptr) && (numel == 0 || topk_ids != nullptr),
              "moe_align_block_size: null tensor pointer");
  auto s = static_cast<cudaStream_t>(stream);
  const size_t smem = SmemBytes(num_experts);
  const int n = static_cast<int>(numel), e = static_cast<int>(num_experts), bs = static_cast<int>(block_size);
  if (numel <= kChunk) {
    if (const int rc = AllowSmem(AlignSingleBlockKernel, smem)) return rc;
    AlignSingleBlockKernel<<<1, kChunk, smem, s>>>(topk_ids, expert_map, n, e, bs, sorted_token_ids, sorted_size,
                                                  experts_ids, experts_size, num_tokens_post_pad);
    return CheckLaunch("moe_align_block_size launch");
  }
  const size_t need = infiniops_b200_moe_align_block_size_scratch_bytes(numel, num_experts);
  if (scratch == nullptr || scratch_bytes < need) {
    return Fail(IOB_SCRATCH_TOO_SMALL, "moe_align_block_size: needs %zu bytes of scratch, got %zu", need,
                scratch_bytes);
  }
  auto* scratch_i32 = static_cast<int32_t*>(scratch);
  const unsigned chunks = static_cast<unsigned>((numel + kChunk - 1) / kChunk);
  if (cudaMemsetAsync(scratch_i32, 0, sizeof(int32_t), s) != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "moe_align_block_size: ticket reset failed");
  }
  if (const int rc = AllowSmem(AlignCountKernel, smem)) return rc;
  if (const int rc = AllowSmem(AlignScatterKernel, smem)) return rc;
  AlignCountKernel<<<chunks, kChunk, smem, s>>>(topk_ids, expert_map, n, e, bs, sorted_token_ids, sorted_size,
                                               experts_ids, experts_size, num_tokens_post_pad, scratch_i32);
  if (const int rc = CheckLaunch("moe_align_block_size count launch")) return rc;
  AlignScatterKernel<<<chunks, kChunk, smem, s>>>(topk_ids, expert_map, n, e, sorted_token_ids, scratch_i32);
  return CheckLaunch("moe_align_block_size scatter launch");
}

extern "C" int infiniops_b200_get_cutlass_moe_mm_data(const int32_t* topk_ids, int64_t numel, int64_t topk,
                                                      int64_t num_experts, int64_t n, int64_t k, int is_gated,
                                                      int32_t* expert_offsets, int32_t* problem_sizes1,
                                                      int32_t* problem_sizes2, int32_t* input_permutation,
                                                      int32_t* output_permutation, int32_t* blockscale_offsets,
                                                      void* stream) {
  using namespace iob;
  const char* op = "get_cutlass_moe_mm_data";
  IOB_REQUIRE(numel > 0 && topk > 0 && numel <= INT32_MAX, "%s: requires non-empty int32-addressable `topk_ids`", op);
  IOB_REQUIRE(num_experts > 0 && n > 0 && k > 0 && k <= INT32_MAX && n <= (is_gated ? INT32_MAX / 2 : INT32_MAX),
              "%s: requires positive int32 GEMM dimensions", op);
  if (num_experts >= 1024) return Fail(IOB_UNSUPPORTED, "%s: more than 1023 experts are not implemented", op);
  IOB_REQUIRE(topk_ids && expert_offsets && problem_sizes1 && problem_sizes2 && input_permutation && output_permutation,
              "%s: null tensor pointer", op);
  const size_t smem = SmemBytes(num_experts);
  if (const int rc = AllowSmem(MmDataKernel, smem)) return rc;
  MmDataKernel<<<1, kChunk, smem, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, expert_offsets, problem_sizes1, problem_sizes2, input_permutation, output_permutation,
      blockscale_offsets, static_cast<int>(numel), static_cast<int>(topk), static_cast<int>(num_experts),
      static_cast<int>(n), static_cast<int>(k), is_gated != 0);
  return CheckLaunch("get_cutlass_moe_mm_data launch");
}
