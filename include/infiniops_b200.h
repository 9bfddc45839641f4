/*
 * infiniops_b200.h -- C ABI of the B200 (sm_100a) int4 weight-only linear and
 * mixture-of-experts kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream
 * (`cudaStream_t` passed as `void*`, NULL = legacy default stream), launches
 * asynchronously on that stream on the CURRENT device, allocates nothing and
 * returns an `iob_status`.  The C++ `infini::ops` operators and the Python
 * module `infini.ops` shipped with this library are thin callers of these
 * functions.
 *
 * Each declaration names the reference interface it stands in for (paths are
 * relative to the InfiniOps source tree).
 */
#ifndef INFINIOPS_B200_H_
#define INFINIOPS_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  IOB_OK = 0,
  IOB_INVALID_ARGUMENT = 1, /* a shape / pointer / attribute the op cannot accept */
  IOB_UNSUPPORTED = 2,      /* valid for the reference, not implemented here */
  IOB_CUDA_ERROR = 3,       /* a CUDA runtime call or launch failed */
  IOB_SCRATCH_TOO_SMALL = 4 /* caller-provided scratch smaller than *_scratch_bytes() */
} iob_status;

/* Element types, for pointers whose type is chosen at run time. */
typedef enum {
  IOB_F32 = 0,
  IOB_F16 = 1,
  IOB_BF16 = 2,
  IOB_I32 = 3,
  IOB_I64 = 4,
  IOB_U32 = 5
} iob_dtype;

/* Quantised weight types (the two 4-bit types of
 * src/base/moe_wna16_marlin_gemm.h:172-184). */
#define IOB_QTYPE_UINT4B8 1125899907892224LL /* GPTQ symmetric: w = (q - 8) * s      */
#define IOB_QTYPE_UINT4 1125899906843648LL   /* AWQ: w = (q - z) * s, z in `b_zeros` */
#define IOB_QTYPE_UINT8B128 1125899923621888LL /* 8-bit symmetric: w = (q - 128) * s; b_q_weight [.., K/16, 4N] */
#define IOB_QTYPE_UINT8 1125899906844672LL     /* 8-bit with zero points: w = (q - z) * s; b_zeros [.., G, N/4], byte n % 4 of word n / 4 */
#define IOB_QTYPE_FLOAT8_E4M3FN 2814749767172868LL /* 8-bit float weights: w = float8_e4m3fn(byte) * s; layout as uint8b128, no zero points */

/* Text of the last non-OK status returned on the calling thread. */
const char* infiniops_b200_last_error(void);

/* Library version string. */
const char* infiniops_b200_version(void);

/* ---- runtime helpers (for hosts that do not link the CUDA runtime themselves) ------------------- */

/* Makes `device` the current CUDA device (no-op if negative or already current) and reports the
 * previous one, so that a caller can restore it afterwards.
 * Replaces: the DeviceGuard of the reference's launchers,
 * src/native/cuda/nvidia/ops/moe_sum/kernel.cu:14-41. */
int infiniops_b200_swap_device(int device, int* previous);

/* A zero-initialised scratch buffer of at least `bytes` on the current device, owned by the
 * library, one per (calling thread, device, purpose, stream); purpose 0 = GEMM, 1 = token sort.
 * Keyed by stream so that two operator calls that may overlap on the GPU never share split-K
 * counters.  It only grows; growing ALLOCATES (cudaMalloc + cudaMemset, frees the old buffer) and
 * therefore must not happen during stream capture, and a graph captured earlier that used the old
 * buffer must be captured again -- size it once up front.  Returns NULL on failure.  This is what
 * the C++ / Python operators fall back to when the Handle carries no workspace; the kernel entry
 * points themselves never allocate.  No counterpart in the reference (its operators that need
 * device scratch allocate it in their constructors, src/native/cuda/ops/silu_and_mul/kernel.h:19-46). */
void* infiniops_b200_thread_scratch(int purpose, size_t bytes, void* stream);

/* ---- weight repacking -------------------------------------------------------------------- */

/* GPTQ-packed int32 [K/pf, N] (pf = 32/num_bits; field i of a word = row pf*(k/pf)+i),
 * optional act-order row permutation `perm` (int32 [K], NULL = none), into the
 * Marlin tile layout int32 [K/16, N*16/pf].  num_bits 4 or 8; K % 16 == 0 (32 with
 * `is_a_8bit`), N % 64 == 0; `perm` is not accepted together with `is_a_8bit`.
 * Replaces: GptqMarlinRepack::operator(), src/base/gptq_marlin_repack.h:34-37
 * (implemented in the reference by vLLM `_C::gptq_marlin_repack`,
 * src/linked/torch/nvidia/ops/gptq_marlin_repack/vllm.cc:15-24). */
int infiniops_b200_gptq_marlin_repack(const int32_t* b_q_weight, const int32_t* perm,
                                      int64_t size_k, int64_t size_n, int num_bits,
                                      int is_a_8bit, int32_t* out, void* stream);

/* AWQ-packed int32 [K, N/pf] (logical column j of a word in field (0,4,1,5,2,6,3,7)[j]
 * for 4 bits, (0,2,1,3)[j] for 8) into the same Marlin tile layout.
 * Replaces: AwqMarlinRepack::operator(), src/base/awq_marlin_repack.h:32-34
 * (vLLM `_C::awq_marlin_repack`, src/linked/torch/nvidia/ops/awq_marlin_repack/vllm.cc:15-23). */
int infiniops_b200_awq_marlin_repack(const int32_t* b_q_weight, int64_t size_k, int64_t size_n,
                                     int num_bits, int is_a_8bit, int32_t* out, void* stream);

/* ---- routers ------------------------------------------------------------------------------- */

/* Softmax over experts, then top-k on softmax+bias; weights are the un-biased softmax
 * (optionally renormalised), ties go to the smaller expert index, rows flagged in
 * `is_padding` get index -1, token_expert_indices[t, r] = r * T + t.
 * gating [T, E] of `gating_dtype` (F32/F16/BF16); bias float [E] or NULL; is_padding
 * uint8 [T] or NULL; topk_weights float [T, k]; topk_indices [T, k] of `index_dtype`
 * (I32/U32/I64); token_expert_indices int32 [T, k].
 * Replaces: TopkSoftmax::operator(), src/base/topk_softmax.h:38-43 and the kernel
 * src/native/cuda/ops/topk_softmax/kernel.cuh:93-182. */
int infiniops_b200_topk_softmax(const void* gating_output, int gating_dtype, const float* bias,
                                const uint8_t* is_padding, int renormalize, float* topk_weights,
                                void* topk_indices, int index_dtype, int32_t* token_expert_indices,
                                int64_t num_tokens, int64_t num_experts, int64_t topk,
                                void* stream);

/* Sigmoid router: score = 1 / (1 + exp(-x)) (non-finite -> 0), top-k on score + correction bias,
 * ties to the smaller index; weights are the un-biased scores, optionally renormalised (divided by
 * their sum when it is positive), then multiplied by `routed_scaling_factor`; rows flagged in
 * `is_padding` get index -1; token_expert_indices[t, r] = r * T + t.  Types as for topk_softmax.
 * Replaces: TopkSigmoid::operator(), src/base/topk_sigmoid.h:41-47 and the kernel
 * src/native/cuda/nvidia/ops/topk_sigmoid/kernel.cuh:60-136. */
int infiniops_b200_topk_sigmoid(const void* gating_output, int gating_dtype,
                                const float* e_score_correction_bias, const uint8_t* is_padding,
                                int renormalize, double routed_scaling_factor, float* topk_weights,
                                void* topk_ids, int index_dtype, int32_t* token_expert_indices,
                                int64_t num_tokens, int64_t num_experts, int64_t topk, void* stream);

/* Group-limited top-k (DeepSeek style): score = x or sigmoid(x) rounded to the score type,
 * selection score = score + bias rounded to the score type, group score = sum of the two
 * largest selection scores of the group, `topk_group` best groups kept, `topk` best
 * finite experts inside them; values = un-biased score, optionally renormalised
 * (/(sum + 1e-20)) and scaled.  scores [T, E] of `scores_dtype`, bias [E] of `bias_dtype`
 * (both F32/F16/BF16); topk_values float [T, k]; topk_indices int32 [T, k].
 * scoring_func: 0 = none, 1 = sigmoid.
 * Replaces: GroupedTopk::operator(), src/base/grouped_topk.h:39-45 and the kernel
 * src/native/cuda/nvidia/ops/grouped_topk/kernel.cuh:143-261. */
int infiniops_b200_grouped_topk(const void* scores, int scores_dtype, const void* bias,
                                int bias_dtype, int64_t num_tokens, int64_t num_experts,
                                int64_t num_expert_group, int64_t topk_group, int64_t topk,
                                int renormalize, double routed_scaling_factor, int scoring_func,
                                float* topk_values, int32_t* topk_indices, void* stream);

/* ---- token sort / pad ---------------------------------------------------------------------- */

/* Bytes of scratch `infiniops_b200_moe_align_block_size` needs for `numel` routing ids
 * (0 for small inputs that one thread block handles). */
size_t infiniops_b200_moe_align_block_size_scratch_bytes(int64_t numel, int64_t num_experts);

/* Groups the flat routing ids 0..numel-1 by (mapped) expert, keeping ascending order inside
 * an expert, pads every expert's run to a multiple of `block_size` with the value `numel`,
 * writes the expert of every block (unused blocks -1) and the padded total.
 * topk_ids int32 [numel]; expert_map int32 [num_experts] or NULL; ids outside
 * [0, num_experts) or mapped outside it are dropped.  Every element of `sorted_token_ids`
 * [sorted_size] and `experts_ids` [experts_size] is written.
 * `scratch` may be NULL when *_scratch_bytes() is 0; its contents need no initialisation.
 * Replaces: MoeAlignBlockSize::operator(), src/base/moe_align_block_size.h:37-45 and the
 * kernel src/native/cuda/nvidia/ops/moe_align_block_size/kernel.cuh:23-78. */
int infiniops_b200_moe_align_block_size(const int32_t* topk_ids, const int32_t* expert_map,
                                        int64_t numel, int64_t num_experts, int64_t block_size,
                                        int32_t* sorted_token_ids, int64_t sorted_size,
                                        int32_t* experts_ids, int64_t experts_size,
                                        int32_t* num_tokens_post_pad, void* scratch,
                                        size_t scratch_bytes, void* stream);

/* Router and token sort as ONE launch: infiniops_b200_topk_softmax (or, with `sigmoid` != 0,
 * infiniops_b200_topk_sigmoid with `routed_scaling_factor`) followed by
 * infiniops_b200_moe_align_block_size on the [num_tokens, topk] int32 ids it has just produced.
 * Same outputs, bit for bit, as the two calls.  One thread block does both while
 * num_tokens * topk <= 1024 (the decode regime, where each operator is a few microseconds behind a
 * launch); beyond that the call issues the separate launches and needs the sort's scratch.
 * The reference has the two operators only (src/base/topk_softmax.h:89-153,
 * src/base/moe_align_block_size.h:37-45); the chain is the caller's. */
int infiniops_b200_topk_softmax_align(const void* gating_output, int gating_dtype, const float* bias,
                                      const uint8_t* is_padding, int renormalize, int sigmoid,
                                      double routed_scaling_factor, float* topk_weights,
                                      int32_t* topk_ids, int32_t* token_expert_indices,
                                      int64_t num_tokens, int64_t num_experts, int64_t topk,
                                      const int32_t* expert_map, int64_t block_size,
                                      int32_t* sorted_token_ids, int64_t sorted_size,
                                      int32_t* experts_ids, int64_t experts_size,
                                      int32_t* num_tokens_post_pad, void* scratch,
                                      size_t scratch_bytes, void* stream);

/* The same for infiniops_b200_grouped_topk (src/base/grouped_topk.h:92-150).  The single-block form
 * needs a float32 `bias`; other bias types take the separate launches. */
int infiniops_b200_grouped_topk_align(const void* scores, int scores_dtype, const void* bias,
                                      int bias_dtype, int64_t num_tokens, int64_t num_experts,
                                      int64_t num_expert_group, int64_t topk_group, int64_t topk,
                                      int renormalize, double routed_scaling_factor, int scoring_func,
                                      float* topk_values, int32_t* topk_ids, const int32_t* expert_map,
                                      int64_t block_size, int32_t* sorted_token_ids,
                                      int64_t sorted_size, int32_t* experts_ids, int64_t experts_size,
                                      int32_t* num_tokens_post_pad, void* scratch,
                                      size_t scratch_bytes, void* stream);

/* Bookkeeping for a grouped GEMM over routed tokens: expert_offsets [E + 1] (exclusive prefix of the
 * per-expert route counts), problem_sizes1 / problem_sizes2 [E, 3] ((count, 2n or n, k) and
 * (count, k, n); with at most 64 routes and no `blockscale_offsets` the first two entries are
 * swapped), input_permutation [numel] (source token of every grouped row, -1 beyond the routed
 * rows), output_permutation [numel] (grouped row of every route; the total for id -1, -1 for any
 * other id outside [0, E)), blockscale_offsets [E + 1] or NULL (prefix of the counts rounded up
 * to 128).  Routes of one expert are placed by ascending route index.  E < 1024.
 * Replaces: GetCutlassMoeMmData::operator(), src/base/get_cutlass_moe_mm_data.h:69-75 and the
 * kernel src/native/cuda/nvidia/ops/get_cutlass_moe_mm_data/kernel.cuh:15-100. */
int infiniops_b200_get_cutlass_moe_mm_data(const int32_t* topk_ids, int64_t numel, int64_t topk,
                                           int64_t num_experts, int64_t n, int64_t k, int is_gated,
                                           int32_t* expert_offsets, int32_t* problem_sizes1,
                                           int32_t* problem_sizes2, int32_t* input_permutation,
                                           int32_t* output_permutation, int32_t* blockscale_offsets,
                                           void* stream);

/* ---- activation and combine ------------------------------------------------------------------ */

/* out[..., j] = silu(in[..., j]) * in[..., H + j]; fp32 math, one rounding.
 * `ndim` <= 8; shape is the OUTPUT shape ([..., H]); strides in elements, any non-negative
 * values (16-byte vector accesses are used when the last stride is 1 and rows are aligned).
 * dtype F32/F16/BF16.
 * Replaces: SiluAndMul::operator(), src/base/silu_and_mul.h:36 and the kernel
 * src/native/cuda/ops/silu_and_mul/kernel.cuh:31-81. */
int infiniops_b200_silu_and_mul(const void* input, void* out, int dtype, int ndim,
                                const int64_t* out_shape, const int64_t* input_strides,
                                const int64_t* out_strides, void* stream);

/* out[t, h] = sum over slots s of in[t, s, h] (fp32 accumulation, slot order), skipping
 * slots whose id in `topk_ids` is negative, or -- with `expert_map` -- not below
 * `expert_map_size` or mapped to a negative value.  Input strides in elements, any
 * non-negative values; output contiguous [T, H].  topk_ids of `ids_dtype` (I32/I64) or NULL.
 * Replaces: MoeSum::operator() (both overloads), src/base/moe_sum.h:132-138 and the kernel
 * src/native/cuda/ops/moe_sum/kernel.cuh:10-48. */
int infiniops_b200_moe_sum(const void* input, int dtype, int64_t num_tokens, int64_t topk,
                           int64_t hidden, int64_t in_stride_t, int64_t in_stride_s,
                           int64_t in_stride_h, const void* topk_ids, int ids_dtype,
                           int64_t ids_stride_t, int64_t ids_stride_s, const int32_t* expert_map,
                           int64_t expert_map_size, int64_t expert_map_stride, void* out,
                           void* stream);

/* moe_sum over rows kept in sorted (expert) order: out[t] = sum over s < topk of
 * input[position[t * topk + s]] (rows of [rows, hidden]; a negative position contributes nothing),
 * accumulated in fp32 in slot order and rounded once -- the arithmetic of infiniops_b200_moe_sum on
 * the [num_tokens, topk, hidden] tensor those rows would form.  `position` as written by
 * iob_routed_options::route_position.  No counterpart in the reference (its layer scatters the
 * rows first and then calls moe_sum, src/base/moe_sum.h:14-208). */
int infiniops_b200_moe_gather_sum(const void* input, int dtype, const int32_t* position,
                                  int64_t num_tokens, int64_t topk, int64_t hidden, void* out,
                                  void* stream);

/* ---- W4A16 GEMM ------------------------------------------------------------------------------ */

/* The GEMM kernels bound every on-device wait.  If one expires (it never should) the kernel
 * records a non-zero code in the first int of its scratch buffer and returns early, leaving
 * the output incomplete.  This helper copies that int back on `stream`, synchronises the
 * stream and returns it (0 = no wait ever expired, -1 = the copy failed).
 * No counterpart in the reference. */
int infiniops_b200_scratch_status(const void* scratch, void* stream);

/* Self-test of the bounded device-side wait the GEMM kernels use: launches a one-block kernel in
 * which one thread waits, for a few thousand polls, on a barrier nobody arrives at (no copy and
 * no tensor-core work is involved).  The wait gives up, records code 7 with (block 0, thread 0,
 * detail 42) in the status header at the start of `scratch` (>= 256 bytes, zeroed) -- read it with
 * infiniops_b200_scratch_status -- and the kernel ends normally, writing result[0] = 0 (the wait
 * reported failure) and result[1] = 1 (the block's give-up flag) to the device ints at `result`.
 * No counterpart in the reference. */
int infiniops_b200_selftest_bounded_wait(void* scratch, size_t scratch_bytes, int* result, void* stream);

/* Clears (asynchronously, on `stream`) the part of a GEMM scratch buffer that the kernels expect
 * to find zero: the status header and the split-K arrival counters, 16 640 bytes from the start.
 * For scratch whose previous content is unknown -- e.g. a Handle workspace that other operators
 * also write (src/handle.h:10-41 gives no zeroing contract).  No counterpart in the reference. */
int infiniops_b200_gemm_scratch_prepare(void* scratch, size_t scratch_bytes, void* stream);

/* Bytes of scratch the dense GEMM needs for an [M, K] x [K, N] problem on the current
 * device (partial sums of K-split tiles and their arrival counters). */
size_t infiniops_b200_marlin_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k);
/* The same with room for the column-permuted copy of `a` that a problem with `g_idx` / `perm` makes. */
size_t infiniops_b200_marlin_gemm_act_order_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k);

/* C[M, N] = A[M, K] * dequant(W)[K, N] (+ bias[N]), fp32 accumulation, C in A's type.
 * a: [M, K] F16/BF16 row-major.  b_q_weight: Marlin layout int32 [K/16, 2N] as produced by
 * the repack functions above (4-bit).  b_scales: [G, N] in A's type, plain row-major,
 * G = K / group_size; this build needs K % 128 == 0 and a group size of 64 or a multiple of 128
 * (G = 1 for per-channel) and answers IOB_UNSUPPORTED otherwise (the reference contract allows any
 * K % 16 == 0).  b_zeros: int32 [G, N/8], field j of a word = column 8*(n/8)+j, required for
 * IOB_QTYPE_UINT4 and NULL for IOB_QTYPE_UINT4B8.  b_bias: [N] in A's type or NULL.  N % 64 == 0.
 * `scratch` must hold *_scratch_bytes(); its first use must find the header and counter area
 * zeroed (cudaMemset once after allocation, or infiniops_b200_gemm_scratch_prepare on memory of
 * unknown content); every completed call leaves it zeroed again.
 * The reference has no dense Marlin GEMM operator; this follows the argument set of its MoE
 * form (src/base/moe_wna16_marlin_gemm.h:18-34) without the routing arguments, and the value
 * semantics of tests/test_moe_wna16_gemm.py:397-404,437. */
int infiniops_b200_marlin_gemm(const void* a, int a_dtype, const int32_t* b_q_weight,
                               const void* b_bias, const void* b_scales, const int32_t* b_zeros,
                               int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k,
                               int64_t num_groups, void* out, void* scratch, size_t scratch_bytes,
                               void* stream);

/* One dense problem with its output placement, for infiniops_b200_marlin_gemm_placed and
 * infiniops_b200_marlin_gemm_batch.  Tensors as for infiniops_b200_marlin_gemm.  `out` is a matrix
 * of `out_ld` columns (0 = size_n) of which this problem writes columns [out_col0, out_col0 +
 * size_n): a column-parallel shard writes its slice of the full-width result directly.  The same
 * slice is also stored, with plain global stores from the GEMM's epilogue, into `n_peers` further
 * matrices of the same shape -- the result buffers of the other GPUs of a tensor-parallel group,
 * mapped into this process (infiniops_b200_peer_open) -- which replaces the all-gather that would
 * otherwise follow the GEMM.  Zero-initialise the struct; unused fields stay zero.
 * No counterpart in the reference (it has no communication layer). */
#define IOB_MAX_PEERS 7
typedef struct {
  const void* a;
  const int32_t* b_q_weight;
  const void* b_bias;
  const void* b_scales;
  const int32_t* b_zeros;
  void* out;
  int64_t size_m, size_n, size_k, num_groups;
  int64_t out_ld, out_col0;
  int n_peers;
  void* peer_out[IOB_MAX_PEERS];
  int scale_layout; /* 0 = plain scales / zero points, 1 = vLLM Marlin layouts (see iob_routed_options) */
  /* Activation order (both or neither; int32 [size_k]): `perm` is the row order the weights were
   * repacked with (gptq_marlin_repack's `perm`), the GEMM reads activation column perm[k] against
   * weight row k; `g_idx[k]` must be the group of row k in that order (k / group_size), any other
   * table is reported as code 9 in the scratch status header.  Needs
   * infiniops_b200_marlin_gemm_act_order_scratch_bytes of scratch (a permuted copy of `a`); not
   * accepted by the batch entry. */
  const int32_t* g_idx;
  const int32_t* perm;
} iob_gemm_problem;

/* Completion signal of a launch towards the other GPUs.  When the last thread block of the launch
 * has finished -- all stores into the peers' matrices issued and fenced -- it adds one to `*epoch`
 * (device int, owned by the caller, starts at 0) and stores the new value, with release semantics
 * at system scope, into word `flag_slot` of each `peer_flags[r]` (a device int array on GPU r,
 * mapped into this process).  `done_counter` is a zeroed device int the launch counts its blocks
 * in.  The receiving side waits with infiniops_b200_peer_wait.  No counterpart in the reference. */
typedef struct {
  int* done_counter;
  int* epoch;
  int n_peers;
  int* peer_flags[IOB_MAX_PEERS];
  int flag_slot;
} iob_peer_signal;

/* infiniops_b200_marlin_gemm for a problem given as a struct, with output placement, peer outputs
 * and an optional completion signal (NULL = none).  No counterpart in the reference. */
int infiniops_b200_marlin_gemm_placed(const iob_gemm_problem* problem, int a_dtype,
                                      int64_t b_type_id, const iob_peer_signal* signal,
                                      void* scratch, size_t scratch_bytes, void* stream);

/* Scratch bytes of infiniops_b200_marlin_gemm_batch on the current device (any problem list). */
size_t infiniops_b200_marlin_gemm_batch_scratch_bytes(void);

/* `count` independent dense problems of decode size (at most 64 rows each, group sizes that are
 * multiples of 128, one activation type and one weight type) in as few launches as possible: the
 * problems with up to 16 rows form one persistent launch, those with 17..64 rows another (16
 * problems per launch at most).  Inside a launch the (tile, k-stage) units of all problems form
 * one sequence cut into equal ranges, one per thread block, so pipelines never drain between
 * problems and launch, set-up and tail are paid once per launch instead of once per GEMM.
 * Results are identical to calling infiniops_b200_marlin_gemm per problem up to the order of the
 * fp32 split-K additions (deterministic for a given problem list).  `signal` (or NULL) rides on
 * the last launch.  Same scratch rules as infiniops_b200_marlin_gemm.
 * No counterpart in the reference. */
int infiniops_b200_marlin_gemm_batch(const iob_gemm_problem* problems, int count, int a_dtype,
                                     int64_t b_type_id, const iob_peer_signal* signal,
                                     void* scratch, size_t scratch_bytes, void* stream);

/* ---- peer memory (one process per GPU, NVLink) ------------------------------------------------- */

/* Device buffers that other processes on the same machine can map: allocate (zero-filled) / free
 * on the current device, export a 64-byte handle to send to the other processes by any host
 * channel, open a handle received from another process (enables peer access on first use) /
 * close the mapping.  Wrappers of cudaMalloc, cudaIpcGetMemHandle, cudaIpcOpenMemHandle and their
 * inverses, so that a host without the CUDA runtime headers can set up the peer outputs above.
 * No counterpart in the reference. */
int infiniops_b200_peer_alloc(size_t bytes, void** ptr);
int infiniops_b200_peer_free(void* ptr);
int infiniops_b200_peer_export(const void* ptr, unsigned char handle[64]);
int infiniops_b200_peer_open(const unsigned char handle[64], void** ptr);
int infiniops_b200_peer_close(void* ptr);

/* Receiving side of iob_peer_signal: a one-warp kernel on `stream` that adds one to `*wait_epoch`
 * (device int, starts at 0) and waits until words 0..n_slots-1 of `flags` (this GPU's flag array,
 * written by the peers), except `skip_slot`, have all reached that value.  The wait is bounded
 * (about a second): on expiry the kernel stores code 8 and the missing slot in `status[0..1]`
 * (a zeroed device int[2]) and returns, so the stream never hangs.  No counterpart in the reference. */
int infiniops_b200_peer_wait(const int* flags, int n_slots, int skip_slot, int* wait_epoch,
                             int* status, void* stream);

/* One rectangular slice to send to the other GPUs: `rows` rows of `row_bytes` bytes at a row pitch of
 * `pitch_bytes`, starting at `src` (local) and going to the same offsets from `dst[r]` (GPU r's
 * matrix as mapped into this process).  Sizes and addresses are multiples of 16 bytes. */
#define IOB_MAX_COPIES 16
typedef struct {
  const void* src;
  void* dst[IOB_MAX_PEERS];
  int64_t rows, row_bytes, pitch_bytes;
} iob_peer_copy;

/* Sends up to IOB_MAX_COPIES slices to `n_peers` GPUs each in one launch, with whole-warp 16-byte
 * stores (the coalesced alternative to iob_gemm_problem::peer_out, whose stores leave the GEMM
 * epilogue as 64-byte pieces; for decode-sized results the extra launch costs more than it saves --
 * it pays when the slices are large), then raises `signal` (or NULL) the way a GEMM launch does.  The column-parallel step is then: GEMMs with local placement only ->
 * infiniops_b200_peer_broadcast -> infiniops_b200_peer_wait.  No counterpart in the reference. */
int infiniops_b200_peer_broadcast(const iob_peer_copy* copies, int count, int n_peers,
                                  const iob_peer_signal* signal, void* stream);

/* The same dense GEMM for callers that have no device memory to lend and may not allocate any:
 * an engine whose arena already owns the whole GPU, or code that only runs while its host is
 * recording work and cudaMalloc is off limits.  The scratch is a 10 MiB array inside the library
 * image (every GPU that loads the library holds it until the process ends); this call allocates
 * nothing, on the device or through any library.  Limits: problems whose
 * infiniops_b200_marlin_gemm_scratch_bytes() exceeds 10 MiB -- more than 64 activation rows on a
 * 148-SM GPU -- are refused with IOB_SCRATCH_TOO_SMALL.  The first call on each device looks up
 * the array's device address (cudaGetSymbolAddress), so make that first call outside any stream
 * capture.  All calls share the one array: calls that can overlap on the GPU (different streams,
 * no dependency) race on it and must be serialised by the caller; the split-K counters are
 * cleared on `stream` at the start of every call.  Arguments as infiniops_b200_marlin_gemm.
 * This entry point has no counterpart in the reference. */
int infiniops_b200_marlin_gemm_static_scratch(const void* a, int a_dtype, const int32_t* b_q_weight,
                                              const void* b_bias, const void* b_scales,
                                              const int32_t* b_zeros, int64_t b_type_id,
                                              int64_t size_m, int64_t size_n, int64_t size_k,
                                              int64_t num_groups, void* out, void* stream);

/* Status word of the built-in array used by infiniops_b200_marlin_gemm_static_scratch on the
 * current device: copies it back on `stream`, clears the status header behind the copy,
 * synchronises the stream and returns the word (0 = no wait expired since the last query,
 * -1 = the query itself failed).  A non-zero answer means the output of some call since the last
 * query is incomplete.  This entry point has no counterpart in the reference. */
int infiniops_b200_static_scratch_status(void* stream);

/* Bytes of scratch the routed (MoE) GEMM needs. */
size_t infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(int64_t size_m, int64_t top_k,
                                                          int64_t size_n, int64_t size_k,
                                                          int64_t num_experts,
                                                          int64_t moe_block_size);

/* Routed GEMM: for every block b of `moe_block_size` entries of `sorted_token_ids` below
 * `num_tokens_past_padded[0]`, with e = expert_ids[b] >= 0, and every entry r < M*top_k of
 * the block: out[r, :] = A[r / top_k, :] * dequant(W[e]) (+ bias[e]) (* topk_weights[r] when
 * `mul_topk_weights`).  Rows of `out` that no entry names are left untouched.
 * a: [M, K]; b_q_weight: [E, K/16, 2N]; b_scales: [E, G, N]; b_zeros: [E, G, N/8] or NULL;
 * b_bias: [E, N] or NULL; topk_weights float [M*top_k]; out: [M*top_k, N].
 * Replaces: MoeWna16MarlinGemm::operator(), src/base/moe_wna16_marlin_gemm.h:71-85
 * (vLLM `_moe_C::moe_wna16_marlin_gemm`, src/linked/torch/nvidia/ops/moe_wna16_marlin_gemm/vllm.h:53-93). */
int infiniops_b200_moe_wna16_marlin_gemm(
    const void* a, int a_dtype, const int32_t* b_q_weight, const void* b_bias,
    const void* b_scales, const int32_t* b_zeros, const int32_t* sorted_token_ids,
    const int32_t* expert_ids, const int32_t* num_tokens_past_padded, const float* topk_weights,
    int64_t moe_block_size, int64_t top_k, int mul_topk_weights, int64_t b_type_id,
    int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups, int64_t num_experts,
    int64_t sorted_size, void* out, void* scratch, size_t scratch_bytes, void* stream);

/* Routed weight-only GEMM on the plain layout: b_qweight uint8 [E, N, K / (8 / bit)] (4-bit: low
 * nibble = even k), b_scales [E, N, G] in the input type, b_qzeros uint8 [E, N / (8 / bit), G]
 * (4-bit: low nibble = even n) or NULL (zero point 2^(bit-1)), topk_weights float [M * top_k] or NULL,
 * output [M * top_k, N]: cleared, then row r of every routing block below num_tokens_post_pad whose
 * expert is not -1 gets input[r / top_k] * dequant(W[expert])^T (x topk_weights[r]); a route id of
 * M * top_k or more ends its block.  bit 4 or 8, block_size_m <= 64, fp32 accumulation.
 * Replaces: MoeWna16Gemm::operator(), src/base/moe_wna16_gemm.h:47-54 and the kernel
 * src/native/cuda/nvidia/ops/moe_wna16_gemm/kernel.cuh:173-378. */
int infiniops_b200_moe_wna16_gemm(const void* input, int dtype, const uint8_t* b_qweight,
                                  const void* b_scales, const uint8_t* b_qzeros,
                                  const float* topk_weights, const int32_t* sorted_token_ids,
                                  const int32_t* expert_ids, const int32_t* num_tokens_post_pad,
                                  int64_t sorted_size, int64_t expert_ids_size, int64_t top_k,
                                  int64_t block_size_m, int64_t bit, int64_t size_m, int64_t size_n,
                                  int64_t size_k, int64_t num_groups, int64_t num_experts,
                                  void* output, void* stream);

/* Options of the routed GEMM beyond the reference's argument list.
 * `scale_layout`: 0 = `b_scales` [E, G, N] and `b_zeros` [E, G, N/8] in plain column order (field j
 * of a zero-point word = column 8 (n/8) + j); 1 = the layouts vLLM's Marlin kernels take, i.e. what
 * a checkpoint prepared for the reference's linked provider holds (scale columns permuted inside
 * blocks of 64 -- 32 with a single group --, zero points permuted alike and interleaved inside each
 * word; src/base/moe_wna16_marlin_gemm.h:204-210,231-240 fix only their shapes).
 * `row_dest` (or NULL): where the result rows go when they do not stay on this GPU -- the combine
 * step of expert parallelism fused into the epilogue.  Per output row (a flat routing id of this
 * call) two int32: the GPU the row belongs to and its row in that GPU's destination matrix
 * [rows, size_n]; `dest_base[g]` is that matrix of GPU g as mapped into this process (this GPU's
 * own included), `n_dest` their number (at most 8).  With a `row_dest`, `out` is only validated.
 * `signal` (or NULL) is raised when the launch has finished.
 * `a_sorted`: `a` is not [size_m, K] but already holds one row per position of `sorted_token_ids`
 * ([>= sorted_size rows, K]: row i belongs to entry i), so the GEMM reads it in place instead of
 * gathering.  `out_sorted`: the result is written as [sorted_size, N] in the same sorted order (row i
 * = entry i, padding entries included) with tile stores instead of one scattered row per entry; not
 * together with `mul_topk_weights` or `row_dest`.  Chaining w13 (out_sorted) -> silu_and_mul -> w2
 * (a_sorted) keeps the intermediate in expert order and scatters only once, at the end.
 * `fuse_silu` (with `out_sorted`, `size_n` a multiple of 128): the weight, scale and zero-point
 * columns of this call are the gate and up halves of a gated MLP interleaved in runs of 16 --
 * column 32 b + c holds gate feature 16 b + c for c < 16 and up feature 16 b + c - 16 for c >= 16 --
 * and the epilogue applies `silu_and_mul` itself: `out` is [sorted_size, size_n / 2], each value
 * silu(gate) * up computed from the two products rounded to the activation type, bit for bit what
 * infiniops_b200_silu_and_mul makes of the stored product.  The [rows, size_n] intermediate never
 * exists.
 * `g_idx`, `perm` (both or neither; int32 [num_experts, size_k]): activation order, the
 * `g_idx_or_none` / `perm_or_none` of src/base/moe_wna16_marlin_gemm.h:258-271.  `perm[e]` is the row
 * order expert e's weights were repacked with (gptq_marlin_repack's `perm`): the GEMM reads
 * activation column perm[e][k] against weight row k.  `g_idx[e][k]` must be the group of row k in
 * that order, i.e. k / group_size (what a provider passes with `is_k_full`); any other table is
 * reported as code 9 in the scratch status word (expert in word 1), not misread.
 * `out_sorted` together with `mul_topk_weights` (128- or 256-row routing blocks): the rows are
 * multiplied by their routing weight and still stored as tiles in sorted order; a padding row stores
 * zeros.  `route_position` (or NULL; int32 [size_m * top_k], a call that gathers, i.e. not `a_sorted`):
 * receives, for every route that occurs in `sorted_token_ids`, its position there, and -1 for
 * the others (the call clears the array first, on the stream).  w13 (`out_sorted`, `route_position`) -> silu_and_mul ->
 * w2 (`a_sorted`, `out_sorted`, weights) -> infiniops_b200_moe_gather_sum is the layer with every
 * GEMM store a tile store and the scatter folded into the final sum.
 * `block_rows` (or NULL; int32, one entry per routing block): the live rows of every block.  A call
 * that gathers (not `a_sorted`, no `perm`) writes it; any call given it restricts the MMAs and the
 * epilogue of a block to its live rows rounded up to 16, so a partly filled last block of an expert
 * costs tensor-core time for its rows, not for the padding (256-row blocks on paired thread blocks
 * keep the full extent).  Rows of a sorted output beyond that extent are then left unwritten.  Pass the table the w13 call wrote to the w2 call.
 * Zero-initialise the struct.  No counterpart in the reference beyond `g_idx` / `perm`. */
typedef struct {
  int scale_layout;
  int a_sorted, out_sorted, fuse_silu;
  const int32_t* g_idx;
  const int32_t* perm;
  int32_t* route_position;
  int32_t* block_rows;
  const int32_t* row_dest;
  void* dest_base[IOB_MAX_PEERS + 1];
  int n_dest;
  const iob_peer_signal* signal;
} iob_routed_options;

/* infiniops_b200_moe_wna16_marlin_gemm with options (NULL = none).  No counterpart in the reference. */
int infiniops_b200_moe_wna16_marlin_gemm_ex(
    const void* a, int a_dtype, const int32_t* b_q_weight, const void* b_bias,
    const void* b_scales, const int32_t* b_zeros, const int32_t* sorted_token_ids,
    const int32_t* expert_ids, const int32_t* num_tokens_past_padded, const float* topk_weights,
    int64_t moe_block_size, int64_t top_k, int mul_topk_weights, int64_t b_type_id,
    int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups, int64_t num_experts,
    int64_t sorted_size, void* out, const iob_routed_options* options, void* scratch,
    size_t scratch_bytes, void* stream);

/* ---- expert-parallel MoE layer (one process per GPU, NVLink) ------------------------------------ */

/* Geometry and peer mappings of an expert-parallel group.  Rank r owns experts
 * [r * experts_per_rank, (r + 1) * experts_per_rank).  Every rank owns an arena of
 * infiniops_b200_ep_arena_bytes() that all ranks map (`arena[g]` = rank g's arena as seen from this
 * process) and a flag array of `world` ints that all ranks map (`flags[g]`); `ctrl` is a zeroed
 * local int[8] (block counter, epoch, wait epoch, wait status[2]).  `capacity` is the largest number
 * of routes (tokens x top_k) any one rank dispatches per layer call. */
typedef struct {
  int world, rank;
  int64_t top_k, hidden, inter, experts_per_rank, capacity, moe_block_size;
  int a_dtype;
  int64_t b_type_id;
  void* arena[IOB_MAX_PEERS + 1];
  int* flags[IOB_MAX_PEERS + 1];
  int* ctrl;
} iob_ep_context;

/* This rank's experts, Marlin layout: w13 [E, H/16, 2*2I], w2 [E, I/16, 2H], scales [E, G, N],
 * zero points [E, G, N/8] or NULL.  `w13_interleaved` != 0: the columns of w13 / s13 / z13 are gate
 * and up interleaved in runs of 16 (iob_routed_options::fuse_silu) and the layer applies
 * silu_and_mul in the first GEMM's epilogue. */
typedef struct {
  const int32_t* w13;
  const void* s13;
  const int32_t* z13;
  int64_t groups13;
  const int32_t* w2;
  const void* s2;
  const int32_t* z2;
  int64_t groups2;
  int w13_interleaved;
} iob_expert_weights;

size_t infiniops_b200_ep_arena_bytes(int world, int64_t capacity, int64_t hidden);
size_t infiniops_b200_ep_workspace_bytes(const iob_ep_context* ctx);

/* One expert-parallel MoE layer, entirely on the device and on `stream` (no host read-back, no
 * collective library): the routes of this rank's `tokens` tokens are placed per owner of their
 * expert (stable order), the token rows are stored straight into the owners' arenas with each
 * route's expert, weight and origin, completion flags are exchanged and awaited (bounded wait), the
 * received rows run through moe_align_block_size, the w13 GEMM, silu_and_mul and the w2 GEMM
 * (x routing weight) whose epilogue stores every result row back into the arena of the rank the
 * token came from, flags again, and moe_sum adds each token's top_k rows into `out` [tokens, hidden].
 * x [tokens, hidden], topk_ids int32 [tokens, top_k] (global expert ids), topk_weights float
 * [tokens, top_k].  Every rank of the group must make the same sequence of calls.
 * Stands for the chain topk -> moe_align_block_size ->
 * moe_wna16_marlin_gemm -> silu_and_mul -> moe_wna16_marlin_gemm -> moe_sum for a sharded layer;
 * the reference has no communication layer of its own. */
int infiniops_b200_ep_moe_layer(const iob_ep_context* ctx, const iob_expert_weights* weights,
                                const void* x, const int32_t* topk_ids, const float* topk_weights,
                                int64_t tokens, void* out, void* workspace, size_t workspace_bytes,
                                void* stream);

#ifdef __cplusplus
}
#endif

#endif /* INFINIOPS_B200_H_ */
