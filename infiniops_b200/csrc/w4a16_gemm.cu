// W4A16 GEMM for sm_100a: dense (marlin_gemm) and routed (moe_wna16_marlin_gemm).
//
// Orientation.  The product is computed transposed, D[n, m] = sum_k W[k, n] * A[m, k], so the
// 128 weight columns of a tile are the M dimension of a tcgen05 MMA (one TMEM lane each) and
// the tokens are its N dimension (16..256).  The dequantised weights are the MMA's A operand
// and live in TENSOR MEMORY; the activations are the B operand in shared memory (K-major,
// 128-byte swizzle, written by TMA); the fp32 accumulator is in tensor memory too.
//
// Why tensor memory for the weights: the Marlin layout stores, per 32-bit word, exactly the
// fragment a thread of an m16n8k16 MMA would hold (two columns 8 apart, k pairs {2c,2c+1} and
// {2c+8,2c+9}).  `tcgen05.st.16x128b` has the same thread<->element map, so a word goes
// global -> shared (bulk copy, still packed) -> one 8-byte shared load -> lop3/sub/mul in
// registers -> tensor memory, without any shuffle and without ever writing 16-bit weights to
// shared memory (which would cost 4x the bytes of the int4 stream on the store and again on the
// MMA's operand fetch).
//
// Pipeline per thread block (one per SM, persistent):
//   warp 0      producer: per 128-k stage one TMA tensor copy of the packed weights, two of the
//               activation tile, bulk copies of scales / zero points; mbarrier completion;
//               several lanes issue for consecutive stages at once
//   warp 1      MMA issuer (one thread) + owner of the tensor-memory allocation
//   warps 2..   dequantisers (two or three sets of 4 warps; a warp owns a 32-lane quarter)
//   last 4      epilogue: accumulator -> registers -> bias / routing weight -> global
//
// Work split (stream-K): the tiles x k-stages grid is cut into equal contiguous ranges, one
// per thread block.  A tile whose k range is shared by several blocks is finished by the block
// that arrives last at the tile's counter (no waiting on other blocks): every sharer writes its
// fp32 partial to scratch, the last one adds them in a fixed order, so results do not depend
// on arrival order.
//
// Every wait on an mbarrier is bounded; on expiry the block raises a flag in scratch (see
// infiniops_b200_scratch_status), lets copies in flight land, frees tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"

namespace iob {
namespace {

constexpr int kTileN = 128;              // weight columns per tile (= UMMA M)
constexpr int kBlockK = 128;             // k per pipeline stage (two 64-k activation atoms)
constexpr int kAStageCols = kBlockK / 2; // 32-bit columns per stage (two 16-bit values each)
// Polls before a wait gives up.  A failed try_wait returns after a hardware time-out of a few
// microseconds, so this is a few hundred milliseconds -- far beyond any legitimate wait.
constexpr uint32_t kSpinLimit = 1u << 16;
constexpr int kHeaderBytes = 256;        // scratch: status word first, then arrival counters
constexpr int kMaxGrid = 1024;           // counters are laid out for at most this many thread blocks

constexpr int kMaxPeers = 7;             // other GPUs whose buffers a dense launch can also write
constexpr int kMaxBatch = 16;            // problems one batched launch can hold

constexpr int kErrFull = 1, kErrEmpty = 2, kErrAFull = 3, kErrAEmpty = 4, kErrDFull = 5, kErrDEmpty = 6;

// 8-bit weights: a stage of packed weights is 16 KB instead of 8 KB, so the rings are shorter (still
// multiples of the set and issuer counts of the tile class).
__host__ __device__ constexpr int StagesFor8(int tok) { return tok <= 32 ? 9 : tok <= 64 ? 6 : 4; }
__host__ __device__ constexpr int StagesFor(int tok) {
  // As many as fit in 227 KB (decode needs ~90 KB of weights in flight per SM to cover HBM
  // latency at full rate) -- and a multiple of SetsFor(tok), see there.
  return tok <= 32 ? 12 : tok <= 64 ? 8 : tok <= 128 ? 4 : 3;
}
// Sets of four dequantiser warps; a set takes every kSets-th stage.
//
// Both ring sizes (shared-memory stages, tensor-memory weight stages) are multiples of the number
// of sets, so that a given ring slot is always served by the same set.  mbarrier waits carry one
// parity bit, which is only sound while a waiter is never more than one phase ahead of the
// barrier; a set that has itself produced phase k of a slot cannot reach the wait for phase k+1
// early, but a set that meets the slot for the first time could -- and would read the stale
// parity as "done".
__host__ __device__ constexpr int SetsFor(int tok) { return tok <= 32 ? 3 : tok <= 128 ? 2 : 3; }
// Tensor-memory stages of dequantised weights (64 columns each).
__host__ __device__ constexpr int AStagesFor(int tok) { return tok <= 32 ? 6 : tok <= 128 ? 4 : 3; }
// accumulator stages (so the epilogue of one segment overlaps the next); limited by the 512 columns
__host__ __device__ constexpr int AccStagesFor(int tok) { return tok == 32 || tok > 128 ? 1 : 2; }
// activations (two swizzle atoms of tok x 128 B) | packed weights 8 KB | 2 scale rows | 2 zero rows
__host__ __device__ constexpr int StageBytes(int tok, int bits = 4) { return tok * 256 + (bits == 8 ? 16384 : 8192); }
// MMA-issuing threads.  One thread cannot keep the tensor pipe busy when a stage is only a few
// hundred cycles of MMA work (its barrier wait and commits are not overlapped), so small token
// tiles use two or three issuers on alternating stages, each with its own accumulator; the epilogue
// adds them in a fixed order.
__host__ __device__ constexpr int IssuersFor(int tok) { return tok <= 32 ? 3 : tok <= 64 ? 2 : tok <= 128 ? 1 : 2; }
// With a 256-token tile the two issuers do not alternate stages: both take every stage and each
// issues the MMAs of one half of the token columns (N = 128 each, same total pipe time), writing
// disjoint columns of one accumulator.  (For N <= 128 an MMA costs 64 cycles whatever N is, so
// halving N would only double the pipe time; there the issuers alternate instead.)
__host__ __device__ constexpr bool SplitTokens(int tok) { return tok > 128; }
// independent accumulators per accumulator stage
__host__ __device__ constexpr int AccSetsFor(int tok) { return SplitTokens(tok) ? 1 : IssuersFor(tok); }
__host__ __device__ constexpr int TmemNeedFor(int tok) {
  return AccStagesFor(tok) * AccSetsFor(tok) * tok + AStagesFor(tok) * kAStageCols;
}
__host__ __device__ constexpr int TmemColsFor(int tok) {
  const int need = TmemNeedFor(tok);
  return need <= 32 ? 32 : need <= 64 ? 64 : need <= 128 ? 128 : need <= 256 ? 256 : 512;
}
// The accumulators and the weight stages (kAStageCols = 64 columns each) share the 512 columns of
// tensor memory; a ring that does not fit would be addressed past the allocation.
static_assert(TmemNeedFor(16) <= 512 && TmemNeedFor(32) <= 512 && TmemNeedFor(64) <= 512 && TmemNeedFor(128) <= 512 &&
                  TmemNeedFor(256) <= 512,
              "tensor-memory budget");

struct GemmParams {
  const uint32_t* wq;      // [E][K/16][2N]
  const void* scales;      // [E][G][N]
  const uint32_t* zeros;   // [E][G][N/8] or null
  const void* bias;        // [E][N] or null
  void* out;               // [rows][N]
  float* partial;          // [2 * grid][tok][128]
  int* counters;           // [kMaxGrid][4]: one per (first block of a split tile, lane quarter)
  int* status;
  int m, n, k, groups, group_size;
  // 0: scales [G, N] and zero points [G, N/8] in plain column order.  1: the layouts vLLM's Marlin
  // kernels take -- scale columns permuted inside blocks of 64 (32 for one group), zero-point
  // nibbles permuted the same way and interleaved inside each word (see ScaleColumn / ZeroNibble).
  int layout;
  int pair;            // dense 256-token tiles: blocks work in pairs (the activation map's box is 128 rows then)
  int g_mul, g_shift;  // scale row of k-stage ks = (ks * g_mul) >> g_shift; g_shift < 0: divide instead
  // Where the result goes.  `out` is a matrix with `out_ld` columns; this problem's N columns start
  // at column `out_col0` of it (a column-parallel shard writes its slice of the full-width matrix).
  // The same slice is also stored into `n_peers` other buffers of the same shape -- the full-width
  // matrices of the other GPUs, mapped into this process -- with plain global stores.
  int out_ld, out_col0, n_peers;
  void* peer_out[kMaxPeers];
  // Completion signal of a launch (null: none).  The block that finishes last adds one to `*epoch`
  // and stores the new value to `peer_flags[r][flag_slot]` of every peer, after all blocks' stores
  // to the peers' buffers.
  int* done_counter;
  int* epoch;
  int* peer_flags[kMaxPeers];
  int flag_slot, n_flag_peers;
  // routed form only
  int out_sorted;                   // 1: result rows stay in sorted order (row = position in `sorted_ids`), stored as tiles
  // 1 (sorted output only; kernels built with kSilu): the weight columns come as gate/up interleaved
  // in runs of 16 (columns 32b..32b+15 = gate features 16b.., columns 32b+16..32b+31 = the matching up
  // features) and the epilogue stores silu(gate) * up, [rows][N/2], instead of the [rows][N] product.
  int fuse_silu;
  int bits;                         // 4 or 8: width of a packed weight
  int fp8;                          // 8-bit weights are float8_e4m3fn bytes (no zero point)
  // routed form, optional: live rows of every routing block (the rest of a block is padding).  The
  // MMAs of a block then cover only its live token columns, rounded up to 16, and so does the epilogue.
  const int* block_rows;
  const int2* row_dest;             // null, or per output row: (GPU, row there) the result row is stored to
  void* dest_base[kMaxPeers + 1];   // with `row_dest`: the destination matrix of every GPU (own included)
  const int32_t* sorted_ids;
  const int32_t* expert_ids;
  const int32_t* num_post_pad;
  const float* topk_weights;
  int top_k, block_size, mul_weights, out_rows;
};

// One GEMM as the kernel sees it: its three tensor maps, its parameters and, in a batched launch,
// its place in the launch's sequence of work units.
struct alignas(64) Problem {
  CUtensorMap a_map, w_map, c_map;
  GemmParams p;
  int n_tiles, m_tiles, k_stages;  // batched launches
  long long unit_end;              // batched launches: units of this and all earlier problems
};
// A batched launch: independent dense problems of one token-tile class, worked through as ONE
// stream of (tile, k-stage) units cut into equal ranges, so that the pipelines of a block never
// drain between problems and the launch, set-up and tail costs are paid once.
struct BatchTable {
  int count;
  Problem prob[kMaxBatch];
};

// Position of logical column n inside a row of scales.  Provider layout: a row is cut into blocks
// of 64 columns stored as [n % 8][n / 8] (so that the four columns c, c + 8, c + 16, c + 24 an MMA
// thread owns are adjacent); with a single group, blocks of 32 stored as [(n % 8) / 2][n / 8][n % 2].
__device__ __forceinline__ int ScaleColumn(const GemmParams& p, int n) {
  if (p.layout == 0) return n;
  if (p.groups > 1) return (n & ~63) + ((n & 7) << 3) + ((n & 63) >> 3);
  return (n & ~31) + (((n & 7) >> 1) << 3) + (((n & 31) >> 3) << 1) + (n & 1);
}
// Provider layout of the zero points: word (n / 64) * 8 + n % 8 of a row holds the eight columns
// n % 8 + 8 j of the block, column j in nibble j / 2 + 4 (j % 2).
__device__ __forceinline__ int ZeroNibble(int j) { return (j >> 1) + 4 * (j & 1); }

// Scale / zero-point row that the first k of stage `ks` falls in.
// The same with the problem's constants held in registers: in a batched launch the parameters of
// the problem at hand sit behind a pointer that moves, and reading them stage after stage costs a
// chain of dependent constant loads in the roles that pace the pipeline.
struct GroupMap {
  int mul, shift, size, n;
  __device__ __forceinline__ int Of(int ks) const { return shift >= 0 ? (ks * mul) >> shift : ks * kBlockK / size; }
};
__device__ __forceinline__ GroupMap MakeGroupMap(const GemmParams& p) { return GroupMap{p.g_mul, p.g_shift, p.group_size, p.n}; }
__device__ __forceinline__ int GroupOf(const GemmParams& p, int ks) {
  return p.g_shift >= 0 ? (ks * p.g_mul) >> p.g_shift : ks * kBlockK / p.group_size;
}

// ---- PTX wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t SmemAddr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void MbarInit(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void MbarArrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void MbarExpectTx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool MbarTryWait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// try_wait that also acquires what the other block of the cluster released with its arrival.
__device__ __forceinline__ bool MbarTryWaitCluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool MbarTestWaitCluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while when it fails).
__device__ __forceinline__ bool MbarTestWait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Two phase tests (by the lanes with `tester` set) issued ahead of the warp-wide wait for this
// thread's tensor-memory stores, so the round trips overlap.  Bit 0: first barrier's phase is
// complete, bit 1: second's.  Lanes that do not test get 0.
__device__ __forceinline__ uint32_t TestTwoAndWaitSt(bool tester, uint32_t bar0, uint32_t parity0, uint32_t bar1,
                                                     uint32_t parity1) {
  uint32_t bits;
  asm volatile(
      "{\n .reg .pred t, p, q;\n .reg .u32 hi;\n"
      " setp.ne.u32 t, %1, 0;\n setp.ne.u32 p, 0, 0;\n setp.ne.u32 q, 0, 0;\n"
      " @t mbarrier.test_wait.parity.shared::cta.b64 p, [%2], %3;\n"
      " @t mbarrier.test_wait.parity.shared::cta.b64 q, [%4], %5;\n"
      " tcgen05.wait::st.sync.aligned;\n"
      " selp.u32 %0, 1, 0, p;\n selp.u32 hi, 2, 0, q;\n or.b32 %0, %0, hi;\n}"
      : "=r"(bits)
      : "r"(static_cast<uint32_t>(tester)), "r"(bar0), "r"(parity0), "r"(bar1), "r"(parity1)
      : "memory");
  return bits;
}
// One phase test (by the lanes with `tester` set) issued ahead of the warp-wide wait for this
// thread's tensor-memory loads.  1: the phase is complete.  Lanes that do not test get 0.
__device__ __forceinline__ uint32_t TestAndWaitLd(bool tester, uint32_t bar, uint32_t parity) {
  uint32_t bit;
  asm volatile(
      "{\n .reg .pred t, p;\n"
      " setp.ne.u32 t, %1, 0;\n setp.ne.u32 p, 0, 0;\n"
      " @t mbarrier.test_wait.parity.shared::cta.b64 p, [%2], %3;\n"
      " tcgen05.wait::ld.sync.aligned;\n"
      " selp.u32 %0, 1, 0, p;\n}"
      : "=r"(bit)
      : "r"(static_cast<uint32_t>(tester)), "r"(bar), "r"(parity)
      : "memory");
  return bit;
}
// Post-mortem aid: when a block gives up, every warp of that block that was blocked in a wait
// leaves (wait code, detail) in the scratch header at ints [8 + 2 * warp, 9 + 2 * warp].
__device__ __forceinline__ void NoteBlockedWarp(int* status, int code, int detail) {
  if (reinterpret_cast<volatile int*>(status)[1] == static_cast<int>(blockIdx.x)) {
    status[8 + 2 * (threadIdx.x >> 5)] = code;
    status[9 + 2 * (threadIdx.x >> 5)] = detail;
  }
}
// Bounded wait.  Returns false when the block is giving up (this wait expired, or another did).
// kHot: poll with the non-suspending test instead of try_wait.  A thread suspended in try_wait is
// woken with some delay; on a chain of hand-overs that is on the critical path (paired blocks:
// commit -> activation producer -> copy -> relay -> issuer) those delays add up to more than the
// MMAs they gate.  Only single threads wait this way, so the polling costs next to nothing.
// kPolls: a poll limit other than the default (the self-test below uses a short one).
template <bool kClusterScope = false, bool kHot = false, uint32_t kPolls = 0>
__device__ __forceinline__ bool MbarWait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                         int code, int detail = 0) {
  constexpr uint32_t kLimit = kPolls != 0 ? kPolls : kHot ? (kSpinLimit << 6) : kSpinLimit;
  for (uint32_t spin = 0;; ++spin) {
    if (kHot ? (kClusterScope ? MbarTestWaitCluster(bar, parity) : MbarTestWait(bar, parity))
             : (kClusterScope ? MbarTryWaitCluster(bar, parity) : MbarTryWait(bar, parity))) {
      return true;
    }
    if ((spin & 0xff) == 0xff) {
      if (*abort_flag) {
        NoteBlockedWarp(status, code, detail);
        return false;
      }
      if (spin > kLimit) {
        // first expiry wins: code, then who and where (block, thread, caller's detail word)
        if (atomicCAS(status, 0, code) == 0) {
          status[1] = static_cast<int>(blockIdx.x);
          status[2] = static_cast<int>(threadIdx.x);
          status[3] = detail;
          __threadfence();
        }
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// Warp-collective form: one lane polls, the warp learns the outcome through the shuffle (which is
// also the warp barrier that orders the other lanes' reads after the wait).  Many threads polling
// the same mbarrier slow every other barrier operation of the block, including TMA completions.
// `relaxed` waits (not on the critical path) back off between polls.
__device__ __forceinline__ bool MbarWaitWarp(unsigned mask, int leader, uint32_t bar, uint32_t parity,
                                             volatile int* abort_flag, int* status, int code, bool relaxed = false,
                                             int detail = 0) {
  int ok = 1;
  if (static_cast<int>(threadIdx.x & 31) == leader) {
    if (relaxed) {
      for (int quick = 0; quick < 4 && !(ok = MbarTryWait(bar, parity)); ++quick) {
      }
      uint32_t spin = 0;
      while (!ok) {
        __nanosleep(64);
        ok = MbarTryWait(bar, parity);
        if (!ok && ((++spin & 0xff) == 0xff)) {
          if (*abort_flag) {
            NoteBlockedWarp(status, code, detail);
            break;
          }
          if (spin > kSpinLimit) {
            if (atomicCAS(status, 0, code) == 0) {
              status[1] = static_cast<int>(blockIdx.x);
              status[2] = static_cast<int>(threadIdx.x);
              status[3] = detail;
              __threadfence();
            }
            *abort_flag = 1;
            break;
          }
        }
      }
    } else {
      ok = MbarWait(bar, parity, abort_flag, status, code, detail);
    }
  }
  return __shfl_sync(mask, ok, leader) != 0;
}
__device__ __forceinline__ void BulkLoad(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void TmaLoad2D(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
          dst),
      "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void TmaLoad3D(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
// Loads that must be issued where they are written (a look-ahead fetch whose value is used a
// whole stage later): the compiler is free to sink an ordinary read-only load to its first use.
__device__ __forceinline__ uint32_t LdGlobalU16Here(const void* ptr) {
  uint32_t v;
  asm volatile("ld.global.nc.u16 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
__device__ __forceinline__ uint4 LdGlobalV4Here(const void* ptr) {
  uint4 v;
  asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(ptr));
  return v;
}
// Both blocks of a cluster meet (all threads), with release / acquire ordering across the cluster.
__device__ __forceinline__ void ClusterSync() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address, valid from any block of the cluster, of a shared-memory location of block `target`.
__device__ __forceinline__ uint32_t MapToBlock(uint32_t smem_addr, uint32_t target) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(target));
  return r;
}
// Arrival on a barrier that may live in the other block of the cluster.
__device__ __forceinline__ void MbarArriveCluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// `cta_group::2` forms: the MMA spans both blocks of the pair; the commit counts the MMAs of both
// and its barrier address may point into either block.
__device__ __forceinline__ void MmaTsPair(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::2.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(
          d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void TcCommitPair(uint32_t cluster_bar) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}
// Waits until the kernels this launch depends on have completed and their writes are visible
// (a no-op for a launch without a programmatic dependency).
__device__ __forceinline__ void GridDependencyWait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Tensor copy of a paired block: the data lands in this block's shared memory, the bytes are
// counted on a barrier that may belong to the other block of the pair (`bar` is a cluster address).
__device__ __forceinline__ void TmaLoad3DPair(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
          dst),
      "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void PrefetchL2(const void* ptr) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(ptr) : "memory");
}
// Tile store (shared memory -> global, clipped at the tensor's edges) as a bulk-async group.
__device__ __forceinline__ void TmaStore2D(const CUtensorMap* map, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(x), "r"(y),
               "r"(src)
               : "memory");
}
__device__ __forceinline__ void BulkCommitGroup() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Until at most one (resp. none) of this thread's store groups still has to read its source.
__device__ __forceinline__ void BulkWaitRead1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void BulkWaitAll() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void FenceProxyAsyncShared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void StShared16(uint32_t addr, unsigned short v) {
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(addr), "h"(v) : "memory");
}
__device__ __forceinline__ void TcFenceBefore() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcFenceAfter() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void TcCommit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]; A is 128 x 16 (16-bit, two per column), B is N x 16 K-major.
__device__ __forceinline__ void MmaTs(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                      uint32_t accumulate) {
  asm volatile(
      "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}" ::"r"(
          d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void TmemStore16(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void TmemLoad16(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void TmemWaitLd() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void TmemWaitSt() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void NamedBarrierUnused(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void LdShared128(uint32_t addr, uint32_t& a, uint32_t& b, uint32_t& c, uint32_t& d) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(a), "=r"(b), "=r"(c), "=r"(d) : "r"(addr));
}
__device__ __forceinline__ void LdShared64(uint32_t addr, uint32_t& a, uint32_t& b) {
  asm volatile("ld.shared.v2.b32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "r"(addr));
}
__device__ __forceinline__ uint32_t LdShared32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t LdSharedU16(uint32_t addr) {
  uint16_t v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint32_t Lop3AndOr(uint32_t a, uint32_t and_mask, uint32_t or_mask) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(and_mask), "r"(or_mask));
  return r;
}

// ---- 16-bit type traits ------------------------------------------------------------------------
template <typename T>
struct Half2Of;
template <>
struct Half2Of<__half> {
  using type = __half2;
  static constexpr uint32_t kMagic = 0x64006400u;  // 1024.0 in both halves
  static constexpr float kBase = 1024.0f;
  static constexpr uint32_t kFormat = 0;  // instruction-descriptor code of the operand type
};
template <>
struct Half2Of<__nv_bfloat16> {
  using type = __nv_bfloat162;
  static constexpr uint32_t kMagic = 0x43004300u;  // 128.0 in both halves
  static constexpr float kBase = 128.0f;
  static constexpr uint32_t kFormat = 1;
};
template <typename T>
__device__ __forceinline__ uint32_t Splat(float v) {
  using H2 = typename Half2Of<T>::type;
  const T h = FromFloat<T>(v);
  H2 p;
  p.x = h;
  p.y = h;
  return *reinterpret_cast<uint32_t*>(&p);
}
template <typename T>
__device__ __forceinline__ uint32_t SplatRaw(T h) {
  using H2 = typename Half2Of<T>::type;
  H2 p;
  p.x = h;
  p.y = h;
  return *reinterpret_cast<uint32_t*>(&p);
}
// ((magic | nibbles) - zero_magic) * scale, both halves; exact until the final multiply.
template <typename T>
__device__ __forceinline__ uint32_t Dequant2(uint32_t shifted_word, uint32_t zero_magic, uint32_t scale2) {
  using H2 = typename Half2Of<T>::type;
  const uint32_t biased = Lop3AndOr(shifted_word, 0x000F000Fu, Half2Of<T>::kMagic);
  const H2 centred = __hsub2(*reinterpret_cast<const H2*>(&biased), *reinterpret_cast<const H2*>(&zero_magic));
  const H2 scaled = __hmul2(centred, *reinterpret_cast<const H2*>(&scale2));
  return *reinterpret_cast<const uint32_t*>(&scaled);
}

// (magic | nibbles) - zero_magic: the exact integer q - zero in both halves.
template <typename T>
__device__ __forceinline__ uint32_t Centre2(uint32_t shifted_word, uint32_t zero_magic) {
  using H2 = typename Half2Of<T>::type;
  const uint32_t biased = Lop3AndOr(shifted_word, 0x000F000Fu, Half2Of<T>::kMagic);
  const H2 centred = __hsub2(*reinterpret_cast<const H2*>(&biased), *reinterpret_cast<const H2*>(&zero_magic));
  return *reinterpret_cast<const uint32_t*>(&centred);
}
// float16 only: the nibbles at bits 4..7 of each half read in place, 1024 + 16 q, and brought to
// q - zero with one exact fused multiply-add: (1024 + 16 q) / 16 - (64 + zero).  Saves the shift.
__device__ __forceinline__ uint32_t CentreHigh2(uint32_t word, uint32_t minus_64_zero) {
  const uint32_t biased = Lop3AndOr(word, 0x00F000F0u, 0x64006400u);
  const uint32_t sixteenth = 0x2C002C00u;
  const __half2 r = __hfma2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&sixteenth),
                            *reinterpret_cast<const __half2*>(&minus_64_zero));
  return *reinterpret_cast<const uint32_t*>(&r);
}

// 8-bit weights: bytes (2 odd, 2 odd + ...) of `word` -- `odd` = 0: bytes 0 and 2 (k = 2t, 2t + 1), `odd` = 1:
// bytes 1 and 3 (k = 2t + 8, 2t + 9) -- as (q - 128) * scale, both halves in T.  `scale16` is the raw
// 16-bit scale.
template <typename T>
__device__ __forceinline__ uint32_t Dequant8(uint32_t word, int odd, uint32_t scale16, uint32_t zero);
template <>
__device__ __forceinline__ uint32_t Dequant8<__half>(uint32_t word, int odd, uint32_t scale16, uint32_t zero) {
  // 0x6400 | q is the float16 1024 + q; minus (1024 + zero) = q - zero, exact
  const uint32_t biased = __byte_perm(word, 0x64646464u, odd ? 0x4341u : 0x4240u);
  const uint32_t centre = (0x6400u | zero) * 0x10001u, scale2 = scale16 * 0x10001u;
  const __half2 c = __hsub2(*reinterpret_cast<const __half2*>(&biased), *reinterpret_cast<const __half2*>(&centre));
  const __half2 r = __hmul2(c, *reinterpret_cast<const __half2*>(&scale2));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t Dequant8<__nv_bfloat16>(uint32_t word, int odd, uint32_t scale16, uint32_t zero) {
  // eight significant bits do not fit the bfloat16 mantissa trick: go through float32
  // (0x4B000000 | q = 8388608 + q), centre and scale there, round once to bfloat16
  const float centre = __uint_as_float(0x4B000000u | zero);
  const float lo = __uint_as_float(__byte_perm(word, 0x4B000000u, odd ? 0x7541u : 0x7540u)) - centre;
  const float hi = __uint_as_float(__byte_perm(word, 0x4B000000u, odd ? 0x7543u : 0x7542u)) - centre;
  const float s = __uint_as_float(scale16 << 16);
  const __nv_bfloat162 r = __floats2bfloat162_rn(lo * s, hi * s);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// 8-bit floating-point weights (float8_e4m3fn; same byte positions as Dequant8): value * scale in T.
// The byte's exponent and mantissa go where T keeps its own, which leaves the exponent bias of the narrow
// type (7) in place of T's: a power of two, multiplied back in exactly (subnormal bytes become
// subnormals of T and come out right the same way).  The type's two NaN bytes are not weights.
template <typename T>
__device__ __forceinline__ uint32_t DequantF8(uint32_t word, int odd, uint32_t scale16);
template <>
__device__ __forceinline__ uint32_t DequantF8<__half>(uint32_t word, int odd, uint32_t scale16) {
  const uint32_t v = __byte_perm(word, 0u, odd ? 0x3414u : 0x2404u);   // the two bytes as the high bytes of the halves
  const uint32_t h = (v & 0x80008000u) | ((v >> 1) & 0x3F803F80u);
  const uint32_t two8 = 0x5C005C00u, scale2 = scale16 * 0x10001u;       // 256 = 2^(15 - 7)
  const __half2 c = __hmul2(*reinterpret_cast<const __half2*>(&h), *reinterpret_cast<const __half2*>(&two8));
  const __half2 r = __hmul2(c, *reinterpret_cast<const __half2*>(&scale2));
  return *reinterpret_cast<const uint32_t*>(&r);
}
template <>
__device__ __forceinline__ uint32_t DequantF8<__nv_bfloat16>(uint32_t word, int odd, uint32_t scale16) {
  const uint32_t v = __byte_perm(word, 0u, odd ? 0x3414u : 0x2404u);
  const uint32_t h = (v & 0x80008000u) | ((v >> 4) & 0x07F007F0u);
  const float two120 = __uint_as_float(0x7B800000u);                    // 2^(127 - 7)
  const float s = __uint_as_float(scale16 << 16);
  const float lo = __uint_as_float(h << 16) * two120, hi = __uint_as_float(h & 0xFFFF0000u) * two120;
  const __nv_bfloat162 r = __floats2bfloat162_rn(lo * s, hi * s);
  return *reinterpret_cast<const uint32_t*>(&r);
}

// ---- work walker ------------------------------------------------------------------------------
struct Segment {
  int tile, n_tile, m_tile, k_begin, k_end;
  int prob, k_stages;    // problem of a batched launch (else 0) and its number of k-stages
  long long tile_u0;     // unit number of the tile's first k-stage
};
// Walks a block's range of units.  In a batched launch the units of the problems follow one
// another (`probs[i].unit_end`); a segment never crosses a tile, hence never a problem.
struct Walker {
  long long u, u_end;
  int k_stages, m_tiles;
  const Problem* probs = nullptr;  // batched launch: the table
  int prob = 0;
  long long base = 0;              // first unit of problem `prob`
  template <bool kBatch = false>
  __device__ __forceinline__ bool Next(Segment& s) {
    if (u >= u_end) return false;
    if constexpr (kBatch) {
      while (u >= probs[prob].unit_end) {
        base = probs[prob].unit_end;
        ++prob;
        k_stages = probs[prob].k_stages;
        m_tiles = probs[prob].m_tiles;
      }
    }
    const unsigned local = static_cast<unsigned>(u - base);
    s.tile = static_cast<int>(local / static_cast<unsigned>(k_stages));
    s.k_begin = static_cast<int>(local - static_cast<unsigned>(s.tile) * static_cast<unsigned>(k_stages));
    const long long left = u_end - u;
    s.k_end = left < k_stages - s.k_begin ? s.k_begin + static_cast<int>(left) : k_stages;
    s.n_tile = s.tile / m_tiles;
    s.m_tile = s.tile - s.n_tile * m_tiles;
    s.prob = prob;
    s.k_stages = k_stages;
    s.tile_u0 = base + static_cast<long long>(s.tile) * k_stages;
    u += s.k_end - s.k_begin;
    return true;
  }
};
// Position of one warp (or lane) in the block's sequence of k-stages.  `it` counts the stages the
// block really processes (segments of expert-less blocks are skipped and not counted); Locate moves
// the walker forward until its segment holds stage `it`.
struct Cursor {
  Walker walk;
  Segment seg;
  uint32_t it, seg_it;
  int seg_len, expert;
  __device__ __forceinline__ int Ks() const { return seg.k_begin + static_cast<int>(it - seg_it); }
};
template <bool kMoe, bool kBatch = false>
__device__ __forceinline__ bool Locate(Cursor& c, const int32_t* expert_ids) {
  while (c.it >= c.seg_it + c.seg_len) {
    c.seg_it += c.seg_len;
    c.seg_len = 0;
    if (!c.walk.template Next<kBatch>(c.seg)) return false;
    if constexpr (kMoe) {
      c.expert = expert_ids[c.seg.m_tile];
      if (c.expert < 0) continue;
    }
    c.seg_len = c.seg.k_end - c.seg.k_begin;
  }
  return true;
}
// First unit of a block's range: floor(block * total / grid).  Written with the quotient and
// remainder of total / grid so that no 64-bit division is needed (block, grid <= 1024).
__device__ __forceinline__ long long RangeStart(long long block, long long total, long long grid) {
  const unsigned t = static_cast<unsigned>(total), g = static_cast<unsigned>(grid), b = static_cast<unsigned>(block);
  const unsigned quot = t / g, rem = t - quot * g;
  return static_cast<long long>(b * quot + b * rem / g);
}
// Block whose range holds unit u (largest b with RangeStart(b) <= u): floor(((u + 1) * grid - 1) / total).
__device__ __forceinline__ int OwnerOf(long long u, long long total, long long grid) {
  const unsigned long long num = (static_cast<unsigned long long>(u) + 1) * static_cast<unsigned>(grid) - 1;
  if (num < (1ull << 32)) return static_cast<int>(static_cast<unsigned>(num) / static_cast<unsigned>(total));
  return static_cast<int>(num / static_cast<unsigned long long>(total));
}

// Paired blocks (40 KB stages) run two dequantiser sets over four shared-memory and four
// tensor-memory stages: the depth of the shared-memory ring is what bounds the prefill kernel.
// Their activations (32 KB a stage) travel in a ring of their own, freed by the MMAs alone, so a
// slot is not held while its weights are being converted; the 8 KB weight stages are freed by
// the dequantisers.
constexpr int kPairStages = 6, kPairAStages = 4, kPairSets = 2, kPairActStages = 5;
template <int kTok, int kSets, bool kPair = false, int kBits = 4>
struct Shared {
  static constexpr int kStages = kPair ? kPairStages : kBits == 8 ? StagesFor8(kTok) : StagesFor(kTok);
  static constexpr int kAcc = AccStagesFor(kTok);
  uint64_t full[kStages], empty[kStages];
  static constexpr int kAStages = kPair ? kPairAStages : AStagesFor(kTok);
  uint64_t a_full[kAStages], a_empty[kAStages];
  static constexpr int kDBars = kAcc * AccSetsFor(kTok);  // per-segment use needs kAcc of them, per-stage use all
  uint64_t d_full[kDBars], d_empty[kDBars];
  static constexpr int kActStages = kPair ? kPairActStages : 1;
  uint64_t act_full[kActStages], act_empty[kActStages];  // kPair: activation ring
  uint32_t tmem_base;
  int abort_flag;
};

// kLate (token tiles <= 32, groups of 128 k or more): the dequantisers write the exact integers
// (q - zero) and every k-stage gets an accumulator of its own; the epilogue warps, idle otherwise,
// read it out stage by stage and apply the group's scale in fp32.  That takes the multiply off the
// dequantisers, whose instruction issue is what bounds small-M problems.
//
// kPair (256-token tiles, N a multiple of 256; dense, or routed with routing blocks of 256 rows): two
// blocks of a cluster work as one.  Each
// dequantises its own 128 output columns into its own tensor memory and loads only half of the
// 256 activation rows; one thread of the even block issues `cta_group::2` MMAs (M = 256, N = 256)
// that run on both SMs and read the two activation halves from the two shared memories.  Per
// block and stage that is 40 KB of copies for the arithmetic that costs 72 KB alone -- the
// single-block prefill kernel is bound by how fast an SM can pull operands out of L2.
//
// kBatch: `probs` is a table of `count` dense problems that are worked through as one sequence of
// units (see BatchTable); otherwise it points to the launch's single problem.  `cur` is the problem
// the executing thread is currently working on -- every role moves it forward with its own walker.
template <typename T, int kTok, bool kZeros, bool kMoe, int kSets, bool kLate, bool kPair, bool kBatch, int kEpi = 0, int kBits = 4>
__device__ __forceinline__ void GemmBody(const Problem* probs, int count) {
  static_assert(!kBatch || (!kMoe && !kPair && kLate), "batched launches: dense late-scale tiles only");
  // kEpi, routed form with sorted output: 1 = silu_and_mul applied by the epilogue, 2 = rows multiplied
  // by their routing weight.  Variants of their own, so that the other kernels carry none of the code.
  static_assert(kEpi == 0 || kMoe, "epilogue variants: routed form only (sorted output)");
  constexpr bool kSilu = kEpi == 1;
  constexpr bool kWeighted = kEpi == 2;
  const Problem* cur = probs;
  int* const status_word = probs->p.status;  // one status header per launch
  using Sh = Shared<kTok, kSets, kPair, kBits>;
  static_assert(kBits == 4 || (kBits == 8 && !kPair && !kBatch && !kLate && kTok <= 128),
                "8-bit weights: unpaired tiles with scaled weights");
  constexpr int kWeightBytes = kBits == 8 ? 16384 : 8192;  // packed weights of a stage (128 columns x 128 k)
  constexpr int kStages = Sh::kStages;
  constexpr int kAcc = Sh::kAcc;
  constexpr int kAStages = Sh::kAStages;
  static_assert(kStages % kSets == 0 && kAStages % kSets == 0, "a ring slot must always meet the same dequantiser set");
  static_assert(kPair || SplitTokens(kTok) || (kStages % IssuersFor(kTok) == 0 && kAStages % IssuersFor(kTok) == 0),
                "a ring slot must always meet the same issuer");
  static_assert(!kPair || (kTok == 256 && !kLate), "paired blocks: 256-token tiles only");
  constexpr int kActRows = kPair ? kTok / 2 : kTok;  // activation rows this block loads per stage
  constexpr int kAtomBytes = kActRows * 128;          // one 64-k activation atom
  constexpr int kActBytes = 2 * kAtomBytes;
  constexpr int kStage = kPair ? 8192 : kActBytes + kWeightBytes;  // bytes of a ring slot (kPair: weights only)
  constexpr int kWeightsAt = kPair ? 0 : kActBytes;         // where the packed weights sit in a slot
  constexpr int kActStages = Sh::kActStages;
  static_assert(kStage <= StageBytes(kTok, kBits), "stage layout");
  // The lanes of a pass wait for each other, so a pass must stay well below the ring size or the
  // ring would drain between passes.
  constexpr int kProdLanes = kStages >= 8 ? 4 : kStages >= 4 ? 2 : 1;
  constexpr int kTmemCols = kPair ? 512 : TmemColsFor(kTok);
  constexpr int kDequantWarps = 4 * kSets;
  constexpr int kIssuerWarps = IssuersFor(kTok);        // warps reserved for issuing
  constexpr int kIssuers = kPair ? 1 : kIssuerWarps;    // threads that really issue MMAs
  constexpr bool kSplit = !kPair && SplitTokens(kTok);
  constexpr int kAccSets = kPair ? 1 : AccSetsFor(kTok);
  constexpr int kIssueStride = kSplit ? 1 : kIssuers;  // an issuer takes every kIssueStride-th stage
  constexpr int kMmaN = kSplit ? kTok / 2 : kTok;
  constexpr int kFirstDq = 1 + kIssuerWarps;  // warp 0 producer, then the issuers, dequantisers, epilogue
  constexpr int kSlots = kAcc * kAccSets;  // kLate: accumulators, one per stage in flight
  static_assert(!kLate || (!kSplit && kSlots % kIssuers == 0 && kTok <= 64), "per-stage accumulators: small tiles only");
  constexpr int kPeers = kPair ? 2 : 1;  // blocks whose warps arrive on the issuing block's barriers
  constexpr uint32_t kIdesc = (1u << 4) | (Half2Of<T>::kFormat << 7) | (Half2Of<T>::kFormat << 10) |
                              (static_cast<uint32_t>(kMmaN >> 3) << 17) |
                              (static_cast<uint32_t>((kPair ? 2 * kTileN : kTileN) >> 4) << 24);

  extern __shared__ unsigned char smem_dyn[];
  __shared__ Sh sh;
  unsigned char* stages =
      reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_dyn) + 1023) & ~uintptr_t(1023));
  const uint32_t stages_addr = SmemAddr(stages);
  [[maybe_unused]] const uint32_t acts_addr = stages_addr + Sh::kStages * 8192;  // kPair: activation ring behind the weight ring
  // behind the rings: two 16-row x 32-column output staging tiles per epilogue warp (8 KB in all)
  [[maybe_unused]] const uint32_t out_stage_addr =
      stages_addr + (kPair ? Sh::kStages * 8192 + Sh::kActStages * (kTok * 128) : Sh::kStages * StageBytes(kTok, kBits));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  volatile int* abort_flag = &sh.abort_flag;

  // Programmatic dependent launch: a following kernel launched with the matching attribute may
  // be scheduled once every block here has passed this point, so that its launch and set-up
  // overlap this kernel's tail.  Nothing of this kernel is published by it: the follower still
  // has to wait (GridDependencyWait) before it touches global memory.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      MbarInit(SmemAddr(&sh.full[i]), 1);
      MbarInit(SmemAddr(&sh.empty[i]), kPair ? 4 : kSplit ? kIssuers : 1);  // kPair: freed by the four dequantiser warps
    }
    for (int i = 0; i < kAStages; ++i) {
      MbarInit(SmemAddr(&sh.a_full[i]), 4 * kPeers);
      MbarInit(SmemAddr(&sh.a_empty[i]), kSplit ? kIssuers : 1);
    }
    for (int i = 0; i < (kLate ? kSlots : kAcc); ++i) {
      MbarInit(SmemAddr(&sh.d_full[i]), kLate ? 1 : kIssuers);
      MbarInit(SmemAddr(&sh.d_empty[i]), 4 * kPeers);
    }
    if constexpr (kPair) {
      for (int i = 0; i < kActStages; ++i) {
        MbarInit(SmemAddr(&sh.act_full[i]), 1);
        MbarInit(SmemAddr(&sh.act_empty[i]), 1);
      }
    }
    sh.abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (threadIdx.x == 32) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(&cur->a_map) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&cur->w_map) : "memory");
  }
  if (warp == 1) {
    // paired blocks allocate together: the same warp of each block, the same columns in both
    if constexpr (kPair) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&sh.tmem_base)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(SmemAddr(&sh.tmem_base)),
                   "r"(kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  // Set-up rendezvous.  The producer warp, which initialised the barriers, only announces that
  // (it needs no tensor memory) and goes straight to requesting copies; everyone else waits for
  // the barriers and the tensor-memory address.
  constexpr int kThreads = (5 + IssuersFor(kTok) + 4 * kSets) * 32;
  if (warp == 0) {
    __threadfence_block();
    asm volatile("bar.arrive 1, %0;" ::"n"(kThreads) : "memory");
  } else {
    TcFenceBefore();
    asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory");
    TcFenceAfter();
  }
  // Paired blocks signal each other's barriers: nobody may start before both have initialised theirs.
  if constexpr (kPair) ClusterSync();
  const int k_stages = kBatch ? cur->k_stages : cur->p.k / kBlockK;  // (batched: of the first problem)
  // kPair: the two blocks of a cluster walk the same sequence of (tile pair, k-stage) units; block
  // `rank` owns output tile 2 * pair + rank.  `my_block` / `grid` below count clusters then.
  uint32_t rank = 0;
  if constexpr (kPair) asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
  const int my_block = kPair ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int blocks_launched = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int n_tiles = kPair ? cur->p.n / (2 * kTileN) : (cur->p.n + kTileN - 1) / kTileN;
  int m_tiles;
  if constexpr (kMoe) {
    GridDependencyWait();  // the block count itself is a predecessor's output
    m_tiles = *cur->p.num_post_pad / cur->p.block_size;
  } else if constexpr (kBatch) {
    m_tiles = cur->m_tiles;
  } else {
    m_tiles = (cur->p.m + kTok - 1) / kTok;
  }
  const long long total_units =
      kBatch ? probs[count - 1].unit_end : static_cast<long long>(n_tiles) * m_tiles * k_stages;
  // Never more ranges than units: an empty range between two sharers of a tile would break the
  // arrival count of the tile.  Surplus blocks get nothing to do.
  long long grid = total_units < static_cast<long long>(blocks_launched) ? (total_units > 0 ? total_units : 1)
                                                                          : static_cast<long long>(blocks_launched);
  // Few tiles: use a multiple of the tile count.  Then every range lies inside one tile (plain
  // split-K), so a block has a single segment and a single hand-over instead of two ragged ones --
  // worth more than the last few SMs when the whole GEMM is only a handful of stages per block.
  if constexpr (!kBatch) {
    const long long tiles = static_cast<long long>(n_tiles) * m_tiles;
    if (tiles > 0 && tiles <= grid) {
      const long long splits = grid / tiles < k_stages ? grid / tiles : k_stages;
      if (tiles * splits * 5 >= grid * 4) grid = tiles * splits;
    }
  }
  const bool idle = static_cast<long long>(my_block) >= grid || total_units == 0;
  const long long u_begin = idle ? 0 : RangeStart(my_block, total_units, grid);
  const long long u_end = idle ? 0 : RangeStart(my_block + 1, total_units, grid);
  // output tile of a walker segment, and the block (as launched) behind a walker block number
  auto tile_of = [&](int seg_n_tile) { return kPair ? 2 * seg_n_tile + static_cast<int>(rank) : seg_n_tile; };
  auto launched_block = [&](int b) { return kPair ? 2 * b + static_cast<int>(rank) : b; };
  // a walker over this block's range (batched: starting in the first problem, it finds its own)
  auto make_walker = [&]() {
    Walker w{u_begin, u_end, k_stages, m_tiles};
    if constexpr (kBatch) w.probs = probs;
    return w;
  };

  // From here on global memory is read and written: everything before was on-chip set-up.
  // (The producer warp waits later: its first ring of weight copies does not depend on the predecessor.)
  if constexpr (!kMoe) {
    if (warp != 0) GridDependencyWait();
  }
  const uint32_t tmem_base = warp == 0 ? 0u : sh.tmem_base;
  const uint32_t tmem_d = tmem_base;  // accumulators: kAcc stages x kIssuers x kTok columns
  const uint32_t tmem_a = tmem_base + kAcc * kAccSets * kTok;  // weights: kAStages x 64 columns

  if (warp == 0) {
    // ================= producer =================
    // SIMT over stages: lane j requests the stages with it % kProdLanes == j (each mbarrier / TMA
    // instruction costs a shared-memory round trip, which one thread alone cannot hide).  A lane
    // never blocks: every pass each lane tests its own slot once and issues if the slot is free,
    // so one slow slot does not hold back the requests for the others.
    if (lane < kProdLanes) {
      constexpr unsigned kMask = (1u << kProdLanes) - 1u;
      Cursor c{make_walker(), Segment{}, static_cast<uint32_t>(lane), 0u, 0, 0};
      bool active = Locate<kMoe, kBatch>(c, cur->p.expert_ids);
      const int grp_rows = cur->p.group_size == 64 ? 2 : 1;
      // The copies of one stage.  Packed weights, scales and zero points are constants of the model;
      // only the activations can be the output of the kernel before this one.
      auto request_weights = [&](const Cursor& at) {
        [[maybe_unused]] const Problem* cur = kBatch ? probs + at.seg.prob : probs;
        const int s = at.it % kStages;
        const int ks = at.Ks();
        const uint32_t full = SmemAddr(&sh.full[s]);
        // both boxes are always counted in full (rows past M and columns past N arrive as zeros)
        MbarExpectTx(full, (kPair ? 0 : kActBytes) + kWeightBytes);
        if constexpr (kBits == 8) {
          // [K/16, 4N] words: the tile's 512 words per row as two boxes of 256 (one per 64 columns)
          const int x0 = 4 * tile_of(at.seg.n_tile) * kTileN, y0 = at.expert * (cur->p.k / 16) + ks * 8;
          TmaLoad2D(stages_addr + s * kStage + kWeightsAt, &cur->w_map, x0, y0, full);
          TmaLoad2D(stages_addr + s * kStage + kWeightsAt + 8192, &cur->w_map, x0 + 256, y0, full);
        } else {
          TmaLoad2D(stages_addr + s * kStage + kWeightsAt, &cur->w_map, 2 * tile_of(at.seg.n_tile) * kTileN,
                    at.expert * (cur->p.k / 16) + ks * 8, full);
        }
        // The dequantisers read this stage's scales and zero points with plain loads one stage
        // ahead; pull the lines into L2 now, a whole ring ahead.
        const int n0 = tile_of(at.seg.n_tile) * kTileN;
        const size_t grow = static_cast<size_t>(at.expert) * cur->p.groups + GroupOf(cur->p, ks);
        const char* sc = reinterpret_cast<const char*>(static_cast<const T*>(cur->p.scales) + grow * cur->p.n + n0);
        const bool wide = n0 + 64 < cur->p.n;  // second 128-byte line of the tile's 256 bytes of scales
        for (int r = 0; r < grp_rows; ++r) {
          PrefetchL2(sc + static_cast<size_t>(r) * cur->p.n * 2);
          if (wide) PrefetchL2(sc + static_cast<size_t>(r) * cur->p.n * 2 + 128);
          if constexpr (kZeros) PrefetchL2(cur->p.zeros + (grow + r) * (cur->p.n / 8) + n0 / 8);
        }
      };
      auto request_activations = [&](const Cursor& at) {
        [[maybe_unused]] const Problem* cur = kBatch ? probs + at.seg.prob : probs;
        if constexpr (!kPair) {
          const int s = at.it % kStages;
          // a paired block loads its own half of the tile's token rows
          const int row0 =
              (kMoe ? at.seg.m_tile * cur->p.block_size : at.seg.m_tile * kTok) + static_cast<int>(rank) * kActRows;
          // two 64-k atoms, one after the other
          TmaLoad3D(stages_addr + s * kStage, &cur->a_map, 0, row0, 2 * at.Ks(), SmemAddr(&sh.full[s]));
        }
      };
      if constexpr (!kMoe) {
        // First trip round the ring (every slot is free): the weight copies go out before this
        // kernel waits for its predecessor, so they overlap that kernel's tail; the activation
        // copies follow once the predecessor's output is visible.
        Cursor ahead = c;
        bool ahead_active = active;
        while (ahead_active && ahead.it < static_cast<uint32_t>(kStages)) {
          request_weights(ahead);
          ahead.it += kProdLanes;
          ahead_active = Locate<kMoe, kBatch>(ahead, cur->p.expert_ids);
        }
        GridDependencyWait();
        while (active && c.it < static_cast<uint32_t>(kStages)) {
          request_activations(c);
          c.it += kProdLanes;
          active = Locate<kMoe, kBatch>(c, cur->p.expert_ids);
        }
      }
      uint32_t idle = 0;
      while (__any_sync(kMask, active)) {
        bool progressed = false;
        if (active) {
          const int s = c.it % kStages;
          if (MbarTestWait(SmemAddr(&sh.empty[s]), ((c.it / kStages) & 1) ^ 1)) {
            request_weights(c);
            request_activations(c);
            c.it += kProdLanes;
            active = Locate<kMoe, kBatch>(c, cur->p.expert_ids);
            progressed = true;
            idle = 0;
          }
        }
        if (!__any_sync(kMask, progressed)) {
          // nothing was free: back off briefly; give up when the block does or after a bounded wait
          __nanosleep(32);
          if ((++idle & 0xff) == 0xff) {
            if (*abort_flag) {
              if (active) NoteBlockedWarp(status_word, kErrEmpty, static_cast<int>(c.it));
              break;
            }
            if (idle > kSpinLimit) {
              if (active && atomicCAS(status_word, 0, kErrEmpty) == 0) {
                status_word[1] = static_cast<int>(blockIdx.x);
                status_word[2] = static_cast<int>(threadIdx.x);
                status_word[3] = static_cast<int>(c.it);
                __threadfence();
              }
              *abort_flag = 1;
              break;
            }
          }
        }
      }
    }
  } else if (warp <= kIssuerWarps) {
    // ================= MMA issuers =================
    if (lane == 0 && warp - 1 < kIssuers) {
      const int me = warp - 1;  // takes the stages with it % kIssuers == me
      // Paired blocks: the even block issues for both.  The odd block's thread only follows the
      // sequence, to know which of its own barriers the last commits will still arrive on.
      const bool issuing = !kPair || rank == 0;
      // barrier of this block and the same barrier of the other block of the pair
      auto commit = [&](uint64_t* bar) {
        if constexpr (kPair) {
          TcCommitPair(SmemAddr(bar));
          TcCommitPair(MapToBlock(SmemAddr(bar), 1));
        } else {
          TcCommit(SmemAddr(bar));
        }
      };
      int first_it = -1, last_it = -1;
      Walker walk = make_walker();
      Segment seg;
      uint32_t it = 0, seg_idx = 0;
      bool alive = true;
      if constexpr (kLate && !kMoe) {
        // Late-scale dense tiles: nothing the issuer does depends on where a tile or a problem ends
        // -- every stage has its own accumulator, and ring slots follow from the stage number --
        // so this thread walks its own stages (me, me + kIssuers, ...) of the block's range directly,
        // with ring positions kept incrementally.  This thread's latency from "weights converted"
        // to "MMAs issued" paces the pipeline, so its instruction count matters.
        const uint32_t total = static_cast<uint32_t>(u_end - u_begin);
        int s = me % kStages, a = me % kAStages, slot = me % kSlots;
        uint32_t a_phase = 0, slot_phase = 0;
        for (it = me; it < total; it += kIssuers) {
          if (!MbarWait(SmemAddr(&sh.d_empty[slot]), slot_phase ^ 1, abort_flag, status_word, kErrDEmpty,
                        static_cast<int>(it)) ||
              !MbarWait(SmemAddr(&sh.a_full[a]), a_phase, abort_flag, status_word, kErrAFull, static_cast<int>(it))) {
            alive = false;
            break;
          }
          TcFenceAfter();
          const uint32_t act = stages_addr + s * kStage;
          const uint64_t desc0 = static_cast<uint64_t>((act >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) | (1ull << 46) |
                                 (2ull << 61);
          const uint32_t d_addr = tmem_d + slot * kTok;
#pragma unroll
          for (int j = 0; j < kBlockK / 16; ++j) {
            const uint64_t desc = desc0 + static_cast<uint64_t>((j >> 2) * (kAtomBytes >> 4) + 2 * (j & 3));
            MmaTs(d_addr, tmem_a + a * kAStageCols + 8 * j, desc, kIdesc, j > 0 ? 1u : 0u);
          }
          TcCommit(SmemAddr(&sh.empty[s]));
          TcCommit(SmemAddr(&sh.a_empty[a]));
          TcCommit(SmemAddr(&sh.d_full[slot]));
          last_it = static_cast<int>(it);
          s += kIssuers;
          if (s >= kStages) s -= kStages;
          a += kIssuers;
          if (a >= kAStages) {
            a -= kAStages;
            a_phase ^= 1;
          }
          slot += kIssuers;
          if (slot >= kSlots) {
            slot -= kSlots;
            slot_phase ^= 1;
          }
        }
        if (last_it >= 0) first_it = me;
      } else
      while (alive && walk.template Next<kBatch>(seg)) {
        if constexpr (kMoe) {
          if (cur->p.expert_ids[seg.m_tile] < 0) continue;
        }
        int acc = 0;
        uint32_t d_addr = tmem_d;
        if constexpr (!kLate) {
          acc = seg_idx % kAcc;
          if (issuing) {
            // (paired blocks: arrivals come from both blocks, hence the cluster-scope acquire)
            if (!MbarWait<kPair>(SmemAddr(&sh.d_empty[acc]), ((seg_idx / kAcc) & 1) ^ 1, abort_flag, status_word, kErrDEmpty,
                                 static_cast<int>(seg_idx))) {
              break;
            }
            TcFenceAfter();
          }
          d_addr = kSplit ? tmem_d + acc * kTok + me * kMmaN : tmem_d + (acc * kIssuers + me) * kTok;
        }
        bool issued = false;
        [[maybe_unused]] uint32_t idesc = kIdesc;
        if constexpr (kMoe && !kSplit && !kPair) {
          // (not for paired blocks: their token columns are split between the two blocks' activation
          // halves, so a shorter extent would not be a prefix of the rows)
          if (cur->p.block_rows != nullptr) {
            // token extent of this block's MMAs: its live rows, in steps of 16 (at least 16)
            const int live = cur->p.block_rows[seg.m_tile];
            const int n_eff = live >= kMmaN ? kMmaN : live <= 16 ? 16 : (live + 15) & ~15;
            idesc = (kIdesc & ~(0x3Fu << 17)) | (static_cast<uint32_t>(n_eff >> 3) << 17);
          }
        }
        for (int ks = seg.k_begin; ks < seg.k_end; ++ks, ++it) {
          if (!kSplit && static_cast<int>(it % kIssuers) != me) continue;
          last_it = static_cast<int>(it);
          if (first_it < 0) first_it = last_it;
          [[maybe_unused]] const int sa = it % kActStages;
          [[maybe_unused]] const uint32_t sa_phase = (it / kActStages) & 1;
          if (!issuing) continue;
          const int s = it % kStages, a = it % kAStages;
          if constexpr (kLate) {
            // this stage's own accumulator must have been read out by the epilogue
            acc = it % kSlots;
            if (!MbarWait(SmemAddr(&sh.d_empty[acc]), ((it / kSlots) & 1) ^ 1, abort_flag, status_word, kErrDEmpty,
                          static_cast<int>(it))) {
              alive = false;
              break;
            }
            d_addr = tmem_d + acc * kTok;
          }
          // `a_full` is raised by warps that waited for this stage's copies themselves, so it
          // also covers the activation tile (in both blocks of a pair).
          if (!MbarWait<kPair, kPair>(SmemAddr(&sh.a_full[a]), (it / kAStages) & 1, abort_flag, status_word, kErrAFull,
                                      static_cast<int>(it))) {
            alive = false;
            break;
          }
          if constexpr (kPair) {
            // both halves of the activation tile (the other block's copy counts on this barrier too)
            if (!MbarWait<true, true>(SmemAddr(&sh.act_full[sa]), sa_phase, abort_flag, status_word, kErrFull,
                                      static_cast<int>(it))) {
              alive = false;
              break;
            }
          }
          TcFenceAfter();
          const uint32_t act = kPair ? acts_addr + sa * kActBytes : stages_addr + s * kStage;
          // in split mode issuer `me` reads token rows [me * kMmaN, ...) of each activation atom
          const uint32_t rows_at = act + (kSplit ? me * kMmaN * 128 : 0);
          const uint64_t desc0 = static_cast<uint64_t>((rows_at >> 4) & 0x3FFF) | (1ull << 16) | (64ull << 32) |
                                 (1ull << 46) | (2ull << 61);
#pragma unroll
          for (int j = 0; j < kBlockK / 16; ++j) {
            // 16-k slab j: atom j / 4, 32 bytes per slab inside the 128-byte swizzled row
            const uint64_t desc = desc0 + static_cast<uint64_t>((j >> 2) * (kAtomBytes >> 4) + 2 * (j & 3));
            const uint32_t accumulate = ((issued && !kLate) || j > 0) ? 1u : 0u;
            if constexpr (kPair) {
              MmaTsPair(d_addr, tmem_a + a * kAStageCols + 8 * j, desc, idesc, accumulate);
            } else {
              MmaTs(d_addr, tmem_a + a * kAStageCols + 8 * j, desc, idesc, accumulate);
            }
          }
          issued = true;
          if constexpr (kPair) {
            commit(&sh.act_empty[sa]);
          } else {
            commit(&sh.empty[s]);
          }
          commit(&sh.a_empty[a]);
          if constexpr (kLate) commit(&sh.d_full[acc]);
        }
        if (!alive) break;
        if constexpr (!kLate) {
          if (issuing) {
            // an issuer without a stage in this segment still has to count as arrived
            if (issued) {
              commit(&sh.d_full[acc]);
            } else {
              MbarArrive(SmemAddr(&sh.d_full[acc]));
            }
          }
        }
        ++seg_idx;
      }
      // Drain: the commits of the last stages are arrivals nobody waits for any more.  They are
      // asynchronous; if the block exited with one still on its way, it could land in the
      // barriers of the next block that gets this shared memory.  So see them arrive first.
      if (alive && last_it >= 0) {
        constexpr int kDrain = kPair ? (kActStages > kAStages ? kActStages : kAStages) : kStages;
        for (int d = 0; d * kIssueStride < kDrain; ++d) {  // only stages not reused since
          const int step = last_it - d * kIssueStride;
          if (step < first_it) break;
          if constexpr (kPair) {
            if (d < kActStages && !MbarWait(SmemAddr(&sh.act_empty[step % kActStages]), (step / kActStages) & 1, abort_flag,
                                            status_word, kErrEmpty, step)) {
              break;
            }
          } else if (!MbarWait(SmemAddr(&sh.empty[step % kStages]), (step / kStages) & 1, abort_flag, status_word, kErrEmpty,
                               step)) {
            break;
          }
          if (d * kIssueStride < kAStages &&
              !MbarWait(SmemAddr(&sh.a_empty[step % kAStages]), (step / kAStages) & 1, abort_flag, status_word, kErrAEmpty,
                        step)) {
            break;
          }
        }
      }
    }
    if constexpr (kPair) {
      if (lane == 0 && warp == 2) {
        // ================= activation producer (paired blocks) =================
        // this block's 128 token rows of every stage, into the activation ring
        Cursor c{make_walker(), Segment{}, 0u, 0u, 0, 0};
        while (Locate<kMoe, kBatch>(c, cur->p.expert_ids)) {
          const int sa = c.it % kActStages;
          if (!MbarWait<false, true>(SmemAddr(&sh.act_empty[sa]), ((c.it / kActStages) & 1) ^ 1, abort_flag, status_word,
                                     kErrEmpty, static_cast<int>(c.it))) {
            break;
          }
          // Both halves of the tile are counted on the even block's barrier, which that block arms
          // for the two of them; the odd block's copy reports there directly.
          if (rank == 0) MbarExpectTx(SmemAddr(&sh.act_full[sa]), 2 * kActBytes);
          TmaLoad3DPair(acts_addr + sa * kActBytes, &cur->a_map, 0,
                        (kMoe ? c.seg.m_tile * cur->p.block_size : c.seg.m_tile * kTok) + static_cast<int>(rank) * kActRows,
                        2 * c.Ks(), MapToBlock(SmemAddr(&sh.act_full[sa]), 0));
          ++c.it;
        }
      }
    }
  } else if (warp < kFirstDq + kDequantWarps) {
    // ================= dequantisers =================
    const int set = (warp - kFirstDq) / 4;
    const int q = warp & 3;  // tensor-memory lane quarter this warp may touch
    // symmetric types: implicit zero point 8
    const uint32_t zero_sym = Half2Of<T>::kMagic | 0x00080008u;
    const int rows = cur->p.group_size == 64 ? 2 : 1;  // scale / zero rows a 128-k stage spans
    // Scales and zero points come straight from global memory (they are tiny and mostly L2 hits),
    // one stage ahead of their use, so the producer has only the two big copies to request.
    // This thread owns tile columns c0 = 16 (2q + h) + lane / 4 and c0 + 8 for h = 0, 1; `sc`
    // packs their two 16-bit scales per (row, h), `zp` holds the four zero-point words of the
    // warp's 32 columns per row.
    struct GroupRegs {
      uint32_t sc[2][2];
      uint4 zp[2];
    };
    // Per-segment bases (tile and expert are fixed inside a segment); columns past N (a 64-wide
    // last tile) are redirected to valid ones: their results are never written out.
    uint32_t based_on = 0xffffffffu;
    const unsigned short* sbase = nullptr;
    const uint4* zbase = nullptr;
    const uint32_t* zword = nullptr;  // provider layout: the one word that holds this thread's four zero points
    int col = 0, sstride = 8;
    GroupMap gmap{};  // of the segment's problem
    auto fetch_groups = [&](const Cursor& c) {
      [[maybe_unused]] const Problem* cur = kBatch ? probs + c.seg.prob : probs;
      if (c.seg_it != based_on) {
        based_on = c.seg_it;
        gmap = MakeGroupMap(cur->p);
        const int n0 = tile_of(c.seg.n_tile) * kTileN;
        const size_t g0 = static_cast<size_t>(c.expert) * cur->p.groups;
        const bool inside = n0 + 32 * q < cur->p.n;
        const int r = lane >> 2;
        // this thread's columns 32 q + r + {0, 8, 16, 24}: first one and the step between them in a scale row
        if (cur->p.layout == 0) {
          col = 32 * q + r;
          sstride = 8;
        } else if (cur->p.groups > 1) {
          col = 64 * (q >> 1) + 8 * r + 4 * (q & 1);
          sstride = 1;
        } else {
          col = 32 * q + 8 * (r >> 1) + (r & 1);
          sstride = 2;
        }
        col -= inside ? 0 : 64;
        sbase = reinterpret_cast<const unsigned short*>(cur->p.scales) + g0 * cur->p.n + n0;
        if constexpr (kZeros) {
          zbase = reinterpret_cast<const uint4*>(cur->p.zeros + g0 * (cur->p.n / 8) + n0 / 8) + (inside ? q : q - 2);
          zword = cur->p.layout == 0 ? nullptr
                                     : cur->p.zeros + g0 * (cur->p.n / 8) + n0 / 8 + 8 * ((q >> 1) - (inside ? 0 : 1)) + r;
        }
      }
      // Zero points of the provider layout, rearranged to where the plain layout has them (nibble
      // lane / 4 of words x, y, z, w = this thread's columns +0, +8, +16, +24), so that the
      // conversion code below is the same for both.
      auto load_zeros = [&](uint32_t row) -> uint4 {
        if constexpr (kBits == 8) {
          // 8-bit zero points: one byte per column ([G, N/4] words, byte n % 4 of word n / 4); the four
          // bytes of this thread's columns +0, +8, +16, +24 packed into x (plain layout only)
          const unsigned char* zrow = reinterpret_cast<const unsigned char*>(cur->p.zeros) +
                                      (static_cast<size_t>(c.expert) * cur->p.groups + row) * static_cast<uint32_t>(gmap.n) +
                                      tile_of(c.seg.n_tile) * kTileN + col;
          uint32_t packed = 0;
#pragma unroll
          for (int j = 0; j < 4; ++j) packed |= static_cast<uint32_t>(__ldg(zrow + 8 * j)) << (8 * j);
          return make_uint4(packed, 0, 0, 0);
        }
        if (zword == nullptr) return LdGlobalV4Here(zbase + static_cast<size_t>(row) * static_cast<uint32_t>(gmap.n / 32));
        uint32_t w;
        asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(w) : "l"(zword + static_cast<size_t>(row) * static_cast<uint32_t>(gmap.n / 8)));
        const int j0 = 4 * (q & 1), at = 4 * (lane >> 2);
        return make_uint4(((w >> (4 * ZeroNibble(j0))) & 0xFu) << at, ((w >> (4 * ZeroNibble(j0 + 1))) & 0xFu) << at,
                          ((w >> (4 * ZeroNibble(j0 + 2))) & 0xFu) << at, ((w >> (4 * ZeroNibble(j0 + 3))) & 0xFu) << at);
      };
      GroupRegs g;
      const uint32_t grp = static_cast<uint32_t>(gmap.Of(c.Ks()));
      const unsigned short* sp = sbase + static_cast<size_t>(grp) * static_cast<uint32_t>(gmap.n) + col;
      g.sc[0][0] = g.sc[0][1] = g.sc[1][0] = g.sc[1][1] = 0;
      if constexpr (!kLate) {
        g.sc[0][0] = LdGlobalU16Here(sp) | (LdGlobalU16Here(sp + sstride) << 16);
        g.sc[0][1] = LdGlobalU16Here(sp + 2 * sstride) | (LdGlobalU16Here(sp + 3 * sstride) << 16);
      }
      g.zp[0] = g.zp[1] = make_uint4(0, 0, 0, 0);
      if constexpr (kZeros) g.zp[0] = load_zeros(grp);
      if (!kLate && rows == 2) {
        sp += gmap.n;
        g.sc[1][0] = LdGlobalU16Here(sp) | (LdGlobalU16Here(sp + sstride) << 16);
        g.sc[1][1] = LdGlobalU16Here(sp + 2 * sstride) | (LdGlobalU16Here(sp + 3 * sstride) << 16);
        if constexpr (kZeros) g.zp[1] = load_zeros(grp + 1);
      }
      return g;
    };
    Cursor nx{make_walker(), Segment{}, static_cast<uint32_t>(set), 0u, 0, 0};
    bool more = Locate<kMoe, kBatch>(nx, cur->p.expert_ids);
    GroupRegs coming{};
    if (more) coming = fetch_groups(nx);
    uint32_t early = 0;  // lane 0: early barrier tests for the coming stage
    // ring positions of the stage in hand and their phase bits, advanced by kSets per stage
    // (both rings are multiples of kSets, so no division is needed)
    int s = set % kStages, a = set % kAStages;
    uint32_t s_phase = 0, a_phase = 0;
    while (more) {
      const uint32_t it = nx.it;
      const GroupRegs gr = coming;
      nx.it += kSets;
      more = Locate<kMoe, kBatch>(nx, cur->p.expert_ids);
      if (more) coming = fetch_groups(nx);
      // `early` holds lane 0's tests of this stage's two barriers, made while the previous stage
      // was still being converted (bit 0: copies landed, bit 1: tensor-memory stage free), so
      // that the round trip of a barrier test is off the critical path whenever the pipeline
      // runs ahead of this warp.  The shuffle hands the outcome to the warp and orders the other
      // lanes' reads behind lane 0's acquire.
      const uint32_t seen = __shfl_sync(0xffffffffu, early, 0);
      if (!(seen & 1u) && !MbarWaitWarp(0xffffffffu, 0, SmemAddr(&sh.full[s]), s_phase, abort_flag, status_word, kErrFull,
                                        false, static_cast<int>(it))) {
        break;
      }
      // Explicit shared-space loads (32-bit addresses) keep these off the generic-address path.
      const uint32_t wbase = stages_addr + s * kStage + kWeightsAt;
      // The thread's words for sub-blocks 2q and 2q + 1 of a 16-k slab are adjacent: one 8-byte load.
      const uint32_t waddr = wbase + ((q >> 1) * 128 + lane * 4 + 2 * (q & 1)) * 4;
      const int row_step = rows - 1;  // second 64 k use the next scale row
      bool alive = true;
      // first store of the stage: this tensor-memory stage must have been read out by the MMAs
      // that used it last
      auto before_first_store = [&]() {
        if (!(seen & 2u) && !MbarWaitWarp(0xffffffffu, 0, SmemAddr(&sh.a_empty[a]), a_phase ^ 1, abort_flag, status_word,
                                          kErrAEmpty, false, static_cast<int>(it))) {
          alive = false;
        }
        TcFenceAfter();
      };
      if constexpr (kBits == 8) {
        // 8-bit weights (uint8b128: w = (q - 128) * s; uint8: (q - z) * s; float8_e4m3fn: float8(q) * s).  Per 16-k slab and 64 columns the thread owns
        // four adjacent words: [columns c0 | c0 + 8] of its first 16-column block, then of its second;
        // a word's bytes are k = 2t, 2t + 8, 2t + 1, 2t + 9 (t = lane % 4).  The two 64-column halves
        // of the tile lie 8 KB apart (one copy each).
        const uint32_t waddr8 = wbase + (q >> 1) * 8192 + (lane * 8 + 4 * (q & 1)) * 4;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w8[4][4];
#pragma unroll
          for (int kt = 0; kt < 4; ++kt) {
            LdShared128(waddr8 + (half * 4 + kt) * 1024, w8[kt][0], w8[kt][1], w8[kt][2], w8[kt][3]);
          }
          const int row = half * row_step;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t pair = row ? gr.sc[1][h] : gr.sc[0][h];
            // zero points of columns c0 and c0 + 8 (128 for the symmetric type)
            uint32_t z0 = 128, z1 = 128;
            if constexpr (kZeros) {
              const uint32_t zp = row ? gr.zp[1].x : gr.zp[0].x;
              z0 = (zp >> (16 * h)) & 0xFFu;
              z1 = (zp >> (16 * h + 8)) & 0xFFu;
            }
            uint32_t regs[16];
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              const uint32_t w0 = w8[kt][2 * h], w1 = w8[kt][2 * h + 1];    // columns c0 and c0 + 8
              bool done = false;
              if constexpr (!kZeros) {
                if (cur->p.fp8) {
                  regs[4 * kt + 0] = DequantF8<T>(w0, 0, pair & 0xFFFFu);
                  regs[4 * kt + 1] = DequantF8<T>(w1, 0, pair >> 16);
                  regs[4 * kt + 2] = DequantF8<T>(w0, 1, pair & 0xFFFFu);
                  regs[4 * kt + 3] = DequantF8<T>(w1, 1, pair >> 16);
                  done = true;
                }
              }
              if (!done) {
                regs[4 * kt + 0] = Dequant8<T>(w0, 0, pair & 0xFFFFu, z0);    // k pair t
                regs[4 * kt + 1] = Dequant8<T>(w1, 0, pair >> 16, z1);
                regs[4 * kt + 2] = Dequant8<T>(w0, 1, pair & 0xFFFFu, z0);    // k pair t + 4
                regs[4 * kt + 3] = Dequant8<T>(w1, 1, pair >> 16, z1);
              }
            }
            if (half == 0 && h == 0) before_first_store();
            if (alive) {
              TmemStore16(tmem_a + (static_cast<uint32_t>(32 * q + 16 * h) << 16) + a * kAStageCols + half * 32, regs);
            }
          }
        }
      } else if constexpr (kLate) {
        // Integers only: (q - zero) for the thread's four columns; the scale is applied to the
        // stage's accumulator by the epilogue warps.
        constexpr bool kHalf = Half2Of<T>::kFormat == 0;
        uint32_t zm[2][2], zh[2][2];  // [h][column c0 / c0 + 8]: magic + zero, and -(64 + zero) for float16
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int c2 = 0; c2 < 2; ++c2) {
            uint32_t zz = 0x00080008u;
            if constexpr (kZeros) {
              const uint32_t zw = h ? (c2 ? gr.zp[0].w : gr.zp[0].z) : (c2 ? gr.zp[0].y : gr.zp[0].x);
              zz = ((zw >> (4 * (lane >> 2))) & 0xFu) * 0x10001u;
            }
            zm[h][c2] = Half2Of<T>::kMagic | zz;
            zh[h][c2] = 0xD400D400u | (zz << 4);
          }
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[4][2];
#pragma unroll
          for (int kt = 0; kt < 4; ++kt) LdShared64(waddr + (half * 4 + kt) * 1024, w[kt][0], w[kt][1]);
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t regs[16];
#pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              const uint32_t word = w[kt][h];
              const uint32_t word8 = word >> 8;
              regs[4 * kt + 0] = Centre2<T>(word, zm[h][0]);   // column c0,     k pair lane % 4
              regs[4 * kt + 1] = Centre2<T>(word8, zm[h][1]);  // column c0 + 8, k pair lane % 4
              if constexpr (kHalf) {
                regs[4 * kt + 2] = CentreHigh2(word, zh[h][0]);   // column c0,     k pair lane % 4 + 4
                regs[4 * kt + 3] = CentreHigh2(word8, zh[h][1]);  // column c0 + 8, k pair lane % 4 + 4
              } else {
                regs[4 * kt + 2] = Centre2<T>(word >> 4, zm[h][0]);
                regs[4 * kt + 3] = Centre2<T>(word >> 12, zm[h][1]);
              }
            }
            if (half == 0 && h == 0) before_first_store();
            if (alive) {
              TmemStore16(tmem_a + (static_cast<uint32_t>(32 * q + 16 * h) << 16) + a * kAStageCols + half * 32, regs);
            }
          }
        }
      } else {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t w[4][2];
  #pragma unroll
          for (int kt = 0; kt < 4; ++kt) LdShared64(waddr + (half * 4 + kt) * 1024, w[kt][0], w[kt][1]);
          const int row = half * row_step;
  #pragma unroll
          for (int h = 0; h < 2; ++h) {
            const uint32_t pair = row ? gr.sc[1][h] : gr.sc[0][h];
            const uint32_t s_lo = __byte_perm(pair, 0, 0x1010), s_hi = __byte_perm(pair, 0, 0x3232);
            // magic | z is the 16-bit float (base + z) for z < 16, the same trick as for the weights
            uint32_t z_lo = zero_sym, z_hi = zero_sym;
            if constexpr (kZeros) {
              const uint4 zw = row ? gr.zp[1] : gr.zp[0];
              const uint32_t shift = 4 * (lane >> 2);
              z_lo = Half2Of<T>::kMagic | ((((h ? zw.z : zw.x) >> shift) & 0xFu) * 0x10001u);
              z_hi = Half2Of<T>::kMagic | ((((h ? zw.w : zw.y) >> shift) & 0xFu) * 0x10001u);
            }
            uint32_t regs[16];
  #pragma unroll
            for (int kt = 0; kt < 4; ++kt) {
              const uint32_t word = w[kt][h];
              regs[4 * kt + 0] = Dequant2<T>(word, z_lo, s_lo);        // column c0,     k pair lane % 4
              regs[4 * kt + 1] = Dequant2<T>(word >> 8, z_hi, s_hi);   // column c0 + 8, k pair lane % 4
              regs[4 * kt + 2] = Dequant2<T>(word >> 4, z_lo, s_lo);   // column c0,     k pair lane % 4 + 4
              regs[4 * kt + 3] = Dequant2<T>(word >> 12, z_hi, s_hi);  // column c0 + 8, k pair lane % 4 + 4
            }
            if (half == 0 && h == 0) before_first_store();
            if (alive) {
              TmemStore16(tmem_a + (static_cast<uint32_t>(32 * q + 16 * h) << 16) + a * kAStageCols + half * 32, regs);
            }
          }
        }
      }
      if (!alive) break;
      if constexpr (kPair) {
        // every word of the stage is in registers: the weight slot can be refilled
        __syncwarp();
        if (lane == 0) MbarArrive(SmemAddr(&sh.empty[s]));
      }
      // Lane 0 tests the two barriers of this warp's next stage while the warp waits for its
      // tensor-memory stores, so the two latencies overlap; the answer is used on the next pass.
      const int a_done = a;
      s += kSets;
      if (s >= kStages) {
        s -= kStages;
        s_phase ^= 1;
      }
      a += kSets;
      if (a >= kAStages) {
        a -= kAStages;
        a_phase ^= 1;
      }
      early = TestTwoAndWaitSt(lane == 0, SmemAddr(&sh.full[s]), s_phase, SmemAddr(&sh.a_empty[a]), a_phase ^ 1);
      TcFenceBefore();
      __syncwarp();
      if (lane == 0) {
        if constexpr (kPair) {
          // the issuing thread lives in the even block and counts the warps of both
          MbarArriveCluster(MapToBlock(SmemAddr(&sh.a_full[a_done]), 0));
        } else {
          MbarArrive(SmemAddr(&sh.a_full[a_done]));
        }
      }
    }
  } else {
    // ================= epilogue =================
    const int q = warp & 3;
    Walker walk = make_walker();
    Segment seg;
    uint32_t seg_idx = 0, it = 0;
    uint32_t early = 0;  // kLate, lane 0: early test of the coming stage's accumulator barrier
    uint32_t staged = 0;  // output chunks this warp has sent through its staging buffers
    while (walk.template Next<kBatch>(seg)) {
      if constexpr (kBatch) cur = probs + seg.prob;
      T* out = static_cast<T*>(cur->p.out);
      int expert = 0;
      if constexpr (kMoe) {
        expert = cur->p.expert_ids[seg.m_tile];
        if (expert < 0) continue;
      }
      const int n_local = 32 * q + lane;
      const int n = tile_of(seg.n_tile) * kTileN + n_local;
      const bool n_ok = n < cur->p.n;
      const int row0 = kMoe ? seg.m_tile * cur->p.block_size : seg.m_tile * kTok;
      int m_valid = kMoe ? cur->p.block_size : min(kTok, cur->p.m - row0);
      if constexpr (kMoe && !kSplit && !kPair) {
        // (only the token columns the block's MMAs wrote: see the issuer)
        if (cur->p.block_rows != nullptr) m_valid = min(m_valid, max(16, (cur->p.block_rows[seg.m_tile] + 15) & ~15));
      }
      const bool whole = seg.k_begin == 0 && seg.k_end == seg.k_stages;
      const int n_steps = seg.k_end - seg.k_begin;
      float bias_v = 0.0f;
      if (cur->p.bias != nullptr && n_ok) bias_v = ToFloat<T>(static_cast<const T*>(cur->p.bias)[static_cast<size_t>(expert) * cur->p.n + n]);

      // Writes one finished value; `j` is the token column of the tile.
      auto emit = [&](int j, float v) {
        v += bias_v;
        if constexpr (kMoe) {
          if constexpr (kSilu) {
            // lanes 0..15 hold gate features, lanes 16..31 the matching up features (sorted output)
            const float mine = ToFloat<T>(FromFloat<T>(v));
            const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
            if (lane < 16) {
              out[static_cast<size_t>(row0 + j) * (cur->p.n >> 1) + ((n - lane) >> 1) + lane] = SiluMulRounded<T>(mine, other);
            }
            return;
          }
          if constexpr (kWeighted) {
            const int id = cur->p.sorted_ids[row0 + j];
            const float w = id < cur->p.out_rows ? cur->p.topk_weights[id] : 0.0f;
            out[static_cast<size_t>(row0 + j) * cur->p.n + n] = FromFloat<T>(v * w);
            return;
          }
          if (cur->p.out_sorted) {
            out[static_cast<size_t>(row0 + j) * cur->p.n + n] = FromFloat<T>(v);
            return;
          }
          const int id = cur->p.sorted_ids[row0 + j];
          if (id < cur->p.out_rows) {
            if (cur->p.mul_weights) v *= cur->p.topk_weights[id];
            if (cur->p.row_dest != nullptr) {
              // expert-parallel combine: the row goes back to the GPU the token came from, to the
              // row its route has there (a plain store into that GPU's mapped buffer)
              const int2 dest = cur->p.row_dest[id];
              static_cast<T*>(cur->p.dest_base[dest.x])[static_cast<size_t>(dest.y) * cur->p.n + n] = FromFloat<T>(v);
            } else {
              out[static_cast<size_t>(id) * cur->p.n + n] = FromFloat<T>(v);
            }
          }
        } else {
          const size_t at = static_cast<size_t>(row0 + j) * cur->p.out_ld + cur->p.out_col0 + n;
          const T value = FromFloat<T>(v);
          out[at] = value;
          for (int r = 0; r < cur->p.n_peers; ++r) static_cast<T*>(cur->p.peer_out[r])[at] = value;
        }
      };

      const bool first_of_block = walk.u - (seg.k_end - seg.k_begin) == u_begin;
      // partial slot layout: [kTok tokens][128 tile columns] -- a warp's 32 columns of one token are one
      // 128-byte line, for the stores here and for the loads of the block that sums the tile
      float* my_partial =
          cur->p.partial + static_cast<size_t>(2 * blockIdx.x + (first_of_block ? 0 : 1)) * kTileN * kTok + n_local;
      // 16 token columns of this thread's output row, summed over the segment: final values of a
      // whole tile, else this block's partial
      auto finish_chunk = [&](int c, const uint32_t (&r)[16]) {
        if (whole) {
          if (!kMoe || cur->p.out_sorted) {
            // Dense output: the warp's 16 rows x 32 columns are transposed through shared memory
            // and leave as one asynchronous tile store (clipped at M and N by the tensor map), so
            // the warp is not held up by 16 strided 64-byte store instructions per chunk and the
            // accumulator is handed back as soon as it has been read.
            if (n_ok) {
              const uint32_t buf = out_stage_addr + q * 2048 + (staged & 1) * 1024;
              if (lane == 0) BulkWaitRead1();  // the store that used this buffer two chunks ago has read it
              __syncwarp();
              if constexpr (kSilu) {
                // 16 rows x 16 features: gate (lanes 0..15) meets up (lanes 16..31) by shuffle, both
                // rounded to the storage type first, as a stored-then-reloaded product would be
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float mine = ToFloat<T>(FromFloat<T>(__uint_as_float(r[j]) + bias_v));
                  const float other = __shfl_xor_sync(0xffffffffu, mine, 16);
                  const T v = SiluMulRounded<T>(mine, other);
                  if (lane < 16) StShared16(buf + j * 32 + lane * 2, *reinterpret_cast<const unsigned short*>(&v));
                }
              } else if constexpr (kWeighted) {
                // lane j fetches the routing weight of row j of the chunk (0 for a padding row)
                float w_lane = 0.0f;
                if (lane < 16) {
                  const int id = cur->p.sorted_ids[row0 + c + lane];
                  if (id < cur->p.out_rows) w_lane = cur->p.topk_weights[id];
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const float wj = __shfl_sync(0xffffffffu, w_lane, j);
                  const T v = FromFloat<T>((__uint_as_float(r[j]) + bias_v) * wj);
                  StShared16(buf + j * 64 + lane * 2, *reinterpret_cast<const unsigned short*>(&v));
                }
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                  const T v = FromFloat<T>(__uint_as_float(r[j]) + bias_v);
                  StShared16(buf + j * 64 + lane * 2, *reinterpret_cast<const unsigned short*>(&v));
                }
              }
              FenceProxyAsyncShared();
              __syncwarp();
              if (lane == 0) {
                TmaStore2D(&cur->c_map, buf, kSilu ? (n - lane) >> 1 : cur->p.out_col0 + n - lane, row0 + c);
                BulkCommitGroup();
              }
              if (cur->p.n_peers > 0) {
                // The same 16 x 32 tile into the other GPUs' matrices: read back from the staging
                // buffer as 16-byte pieces (four per row) and stored with plain global stores.
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                  const int row = half * 8 + (lane >> 2), part = lane & 3;
                  if (row0 + c + row < cur->p.m) {
                    uint4 piece;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(piece.x), "=r"(piece.y), "=r"(piece.z), "=r"(piece.w)
                                 : "r"(buf + row * 64 + part * 16));
                    const size_t at = static_cast<size_t>(row0 + c + row) * cur->p.out_ld + cur->p.out_col0 + (n - lane) + part * 8;
                    for (int r = 0; r < cur->p.n_peers; ++r) {
                      *reinterpret_cast<uint4*>(static_cast<T*>(cur->p.peer_out[r]) + at) = piece;
                    }
                  }
                }
              }
              ++staged;
            }
          } else if (n_ok) {
            if constexpr (kMoe) {
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c + j < m_valid) emit(c + j, __uint_as_float(r[j]));
              }
            }
          }
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) my_partial[(c + j) * kTileN] = __uint_as_float(r[j]);
        }
      };

      if constexpr (kLate) {
        // Every stage has its own accumulator: read it, hand it back, add scale * value.  The
        // scale of the thread's row comes from global memory one stage ahead of its use.
        float sum[kTok];
#pragma unroll
        for (int j = 0; j < kTok; ++j) sum[j] = 0.0f;
        const T* srow = static_cast<const T*>(cur->p.scales) + static_cast<size_t>(expert) * cur->p.groups * cur->p.n +
                        ScaleColumn(cur->p, n_ok ? n : n - 64);  // a column past N borrows a valid one; it is never written
        const GroupMap gmap = MakeGroupMap(cur->p);
        uint32_t coming = LdGlobalU16Here(srow + static_cast<size_t>(gmap.Of(seg.k_begin)) * gmap.n);
        bool alive = true;
        for (int ks = seg.k_begin; ks < seg.k_end; ++ks, ++it) {
          const unsigned short raw = static_cast<unsigned short>(coming);
          const float scale = ToFloat<T>(*reinterpret_cast<const T*>(&raw));
          if (ks + 1 < seg.k_end) coming = LdGlobalU16Here(srow + static_cast<size_t>(gmap.Of(ks + 1)) * gmap.n);
          const int slot = it % kSlots;
          const uint32_t seen = __shfl_sync(0xffffffffu, early, 0);
          if (!(seen & 1u) && !MbarWaitWarp(0xffffffffu, 0, SmemAddr(&sh.d_full[slot]), (it / kSlots) & 1, abort_flag,
                                            status_word, kErrDFull, /*relaxed=*/false, static_cast<int>(it))) {
            alive = false;
            break;
          }
          TcFenceAfter();
          // at most 32 columns in registers at a time (64-token tiles take two rounds)
          constexpr int kRound = kTok < 32 ? kTok : 32;
#pragma unroll
          for (int c0 = 0; c0 < kTok; c0 += kRound) {
            uint32_t r[kRound];
#pragma unroll
            for (int c = 0; c < kRound; c += 16) {
              TmemLoad16(tmem_d + slot * kTok + (static_cast<uint32_t>(32 * q) << 16) + c0 + c, &r[c]);
            }
            if (c0 + kRound >= kTok) {
              // last round: the next stage's barrier is tested while the loads are in flight,
              // then the accumulator goes back to the issuers
              early = TestAndWaitLd(lane == 0, SmemAddr(&sh.d_full[(it + 1) % kSlots]), ((it + 1) / kSlots) & 1);
              TcFenceBefore();
              __syncwarp();
              if (lane == 0) MbarArrive(SmemAddr(&sh.d_empty[slot]));
            } else {
              TmemWaitLd();
            }
#pragma unroll
            for (int j = 0; j < kRound; ++j) sum[c0 + j] = fmaf(scale, __uint_as_float(r[j]), sum[c0 + j]);
          }
        }
        if (!alive) break;
#pragma unroll
        for (int c = 0; c < kTok; c += 16) {
          if (c < m_valid) {
            uint32_t r[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(sum[c + j]);
            finish_chunk(c, r);
          }
        }
        ++seg_idx;
      } else {
        const int acc = seg_idx % kAcc;
        if (!MbarWaitWarp(0xffffffffu, 0, SmemAddr(&sh.d_full[acc]), (seg_idx / kAcc) & 1, abort_flag, status_word,
                          kErrDFull, /*relaxed=*/true, static_cast<int>(seg_idx))) {
          break;
        }
        TcFenceAfter();
        const uint32_t d_addr = tmem_d + acc * kAccSets * kTok + (static_cast<uint32_t>(32 * q) << 16);
        // which issuers contributed to this segment (they alternate stages, counted by `it`)
        bool present[kAccSets];
#pragma unroll
        for (int j = 0; j < kAccSets; ++j) {
          present[j] = n_steps >= kAccSets || static_cast<int>((j + kAccSets - it % kAccSets) % kAccSets) < n_steps;
        }
        it += n_steps;
        if constexpr (kAccSets == 1 && kTok >= 64) {
          // One accumulator, many columns: the load of the next 16 columns is in flight while
          // the current 16 are converted and stored (the tile's MMAs cannot restart before the
          // accumulator is drained, so this latency is on the critical path of every tile).
          const int c_end = min(kTok, (m_valid + 15) & ~15);
          uint32_t b0[16], b1[16];
          TmemLoad16(d_addr, b0);
#pragma unroll 1
          for (int c = 0; c < c_end; c += 32) {
            TmemWaitLd();
            if (c + 16 < c_end) TmemLoad16(d_addr + c + 16, b1);
            finish_chunk(c, b0);
            if (c + 16 < c_end) {
              TmemWaitLd();
              if (c + 32 < c_end) TmemLoad16(d_addr + c + 32, b0);
              finish_chunk(c + 16, b1);
            }
          }
        } else
#pragma unroll 1
        for (int c = 0; c < kTok; c += 16) {
          if (c >= m_valid) break;
          uint32_t r[16];
          if (present[0]) {
            TmemLoad16(d_addr + c, r);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) r[j] = 0u;
          }
          TmemWaitLd();
#pragma unroll
          for (int other = 1; other < kAccSets; ++other) {
            if (present[other]) {
              uint32_t r1[16];
              TmemLoad16(d_addr + other * kTok + c, r1);
              TmemWaitLd();
#pragma unroll
              for (int j = 0; j < 16; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) + __uint_as_float(r1[j]));
            }
          }
          finish_chunk(c, r);
        }
        // The accumulator is in registers / memory now: hand it back to the MMA warp.
        TcFenceBefore();
        __syncwarp();
        if (lane == 0) {
          if constexpr (kPair) {
            MbarArriveCluster(MapToBlock(SmemAddr(&sh.d_empty[acc]), 0));
          } else {
            MbarArrive(SmemAddr(&sh.d_empty[acc]));
          }
        }
        ++seg_idx;
      }

      if (!whole) {
        // Each lane quarter of the tile has its own arrival counter, so the four epilogue
        // warps never have to meet at a barrier: the warp that arrives last for its quarter
        // (over all blocks sharing the tile) sums that quarter.
        const long long tile_u0 = seg.tile_u0;
        const int first_block = OwnerOf(tile_u0, total_units, grid);
        const int last_block = OwnerOf(tile_u0 + seg.k_stages - 1, total_units, grid);
        // A split tile is identified by the first block working on it: no two split tiles share one.
        int* counter = cur->p.counters + 4 * launched_block(first_block) + q;
        // Publish the partial and take a ticket in one acquire-release atomic: the warp barrier
        // orders every lane's stores before lane 0's release, and the shuffle orders the other lanes'
        // loads after its acquire.
        __syncwarp();
        int ticket = 0;
        if (lane == 0) {
          asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
        }
        ticket = __shfl_sync(0xffffffffu, ticket, 0);
        if (ticket == last_block - first_block) {
          if (n_ok) {
            // a block's first segment uses slot 2b, any later one slot 2b + 1
            auto slot_of = [&](int b) -> const float* {
              const bool is_first = RangeStart(b, total_units, grid) >= tile_u0;
              return cur->p.partial + static_cast<size_t>(2 * launched_block(b) + (is_first ? 0 : 1)) * kTileN * kTok + n_local;
            };
            for (int c = 0; c < m_valid; c += 16) {
              float sum[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) sum[j] = 0.0f;
              // two sharers per round: their 8 loads are all in flight together; the additions
              // stay in ascending block order, so the result does not depend on who arrived last
              for (int b = first_block; b <= last_block; b += 2) {
                float v[2][16];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                  const bool on = b + u <= last_block;
                  const float* src = slot_of(on ? b + u : b) + c * kTileN;
#pragma unroll
                  for (int j = 0; j < 16; ++j) v[u][j] = on ? __ldcg(src + j * kTileN) : 0.0f;
                }
#pragma unroll
                for (int u = 0; u < 2; ++u) {
#pragma unroll
                  for (int j = 0; j < 16; ++j) sum[j] += v[u][j];
                }
              }
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                if (c + j < m_valid) emit(c + j, sum[j]);
              }
            }
          }
          if (lane == 0) *counter = 0;
        }
      }
    }
    // the staged tile stores of this warp must have left shared memory (and landed) before the block ends
    if (lane == 0) BulkWaitAll();
  }

  // ---- teardown -----------------------------------------------------------------------------
  {
    // Completion signal to the other GPUs (launches that were given one).  Every block makes its
    // own stores visible system-wide and counts itself done; the block that comes last bumps the
    // epoch and publishes it in every peer's flag word.  Nobody waits here.
    if (probs[0].p.done_counter != nullptr) {
      __syncthreads();
      if (threadIdx.x == 0) {
        const GemmParams& sp = probs[0].p;
        __threadfence_system();
        int arrived;
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(sp.done_counter) : "memory");
        if (arrived == static_cast<int>(gridDim.x) - 1) {
          *sp.done_counter = 0;
          const int epoch = *sp.epoch + 1;
          *sp.epoch = epoch;
          __threadfence_system();
          for (int r = 0; r < sp.n_flag_peers; ++r) {
            asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(sp.peer_flags[r] + sp.flag_slot), "r"(epoch) : "memory");
          }
        }
      }
    }
  }
  if (*abort_flag) {
    // give copies in flight time to land before shared memory is released
    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
  }
  TcFenceBefore();
  __syncthreads();
  if constexpr (kPair) {
    // neither block may free tensor memory, or leave, while the other could still signal it
    ClusterSync();
    if (warp == 1) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
  } else if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

// One problem per launch.
template <typename T, int kTok, bool kZeros, bool kMoe, int kSets, bool kLate, bool kPair = false, int kEpi = 0, int kBits = 4>
__global__ void __launch_bounds__((5 + IssuersFor(kTok) + 4 * kSets) * 32, 1)
W4A16GemmKernel(const __grid_constant__ Problem problem) {
  GemmBody<T, kTok, kZeros, kMoe, kSets, kLate, kPair, false, kEpi, kBits>(&problem, 1);
}
// A table of dense problems per launch.
template <typename T, int kTok, bool kZeros, int kSets>
__global__ void __launch_bounds__((5 + IssuersFor(kTok) + 4 * kSets) * 32, 1)
W4A16GemmBatchKernel(const __grid_constant__ BatchTable table) {
  GemmBody<T, kTok, kZeros, false, kSets, true, false, true>(table.prob, table.count);
}

// Self-test of the bounded wait: one thread waits, with a limit of a few thousand polls, on a
// barrier that nobody ever arrives at.  The wait must give up, record (code, block, thread, detail)
// in the status header and return false; the kernel then ends normally.  No copy engine and no
// tensor memory is involved, so nothing is left in flight.
constexpr int kErrSelfTest = 7;
__global__ void BoundedWaitSelfTestKernel(int* status, int* result) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    MbarInit(SmemAddr(&bar), 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = MbarWait<false, true, 4096>(SmemAddr(&bar), 0, &abort_flag, status, kErrSelfTest, 42);
  __syncthreads();
  // the other threads see the block's abort flag, as the roles of the GEMM kernel do
  if (threadIdx.x == 0) {
    result[0] = ok ? 1 : 0;
    result[1] = abort_flag;
  }
}

// Copies the routed rows of `a` into scratch in sorted order so a TMA box of consecutive rows
// is one routing block.
template <typename T>
__global__ void GatherRowsKernel(const T* __restrict__ a, T* __restrict__ gathered,
                                 const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ num_post_pad,
                                 int k, int top_k, int out_rows, int32_t* __restrict__ position,
                                 int32_t* __restrict__ block_rows, int block_size) {
  const int rows = *num_post_pad;
  const int vec_per_row = k / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int id = sorted_ids[row];
    uint4* dst = reinterpret_cast<uint4*>(gathered + static_cast<size_t>(row) * k);
    // by-product: the live rows of every routing block (they are a prefix of the block: the last live
    // row is the one followed by padding or by the block's end)
    if (block_rows != nullptr && threadIdx.x == 0 && id < out_rows) {
      const int in_block = row % block_size;
      if (in_block == block_size - 1 || sorted_ids[row + 1] >= out_rows) block_rows[row / block_size] = in_block + 1;
    }
    // by-product for the caller's combine step: where each route sits in sorted order
    if (position != nullptr && threadIdx.x == 0 && id < out_rows) position[id] = row;
    if (id < out_rows) {
      const uint4* src = reinterpret_cast<const uint4*>(a + static_cast<size_t>(id / top_k) * k);
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
    } else {
      for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    }
  }
}

// Act-order form of the gather: row `row` of the sorted layout is the token's activations with the
// columns in the order of its expert's weight rows, gathered[row][k] = a[token][perm[expert][k]]
// (`perm` = the row order the weights were repacked with; vLLM's `permute_cols`, fused into the gather
// this GEMM does anyway).  `from_sorted`: `a` already has one row per sorted position.  The scales
// are read per contiguous group of k, which is what `g_idx` says once the rows are in that order
// (g_idx[expert][k] == k / group_size); the first row of every routing block checks its expert's
// `g_idx` and a table of any other form is reported in the status header (code kErrGIdx), not
// silently misread.
constexpr int kErrGIdx = 9;
template <typename T>
__global__ void GatherPermutedRowsKernel(const T* __restrict__ a, T* __restrict__ gathered,
                                         const int32_t* __restrict__ sorted_ids, const int32_t* __restrict__ expert_ids,
                                         const int32_t* __restrict__ num_post_pad, const int32_t* __restrict__ perm,
                                         const int32_t* __restrict__ g_idx, int k, int top_k, int out_rows, int block_size,
                                         int group_size, int from_sorted, int* status) {
  const int rows = *num_post_pad;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const int id = sorted_ids[row];
    const int expert = expert_ids[row / block_size];
    T* dst = gathered + static_cast<size_t>(row) * k;
    if (id < out_rows && expert >= 0) {
      const T* src = a + static_cast<size_t>(from_sorted ? row : id / top_k) * k;
      const int32_t* order = perm + static_cast<size_t>(expert) * k;
      for (int i = threadIdx.x; i < k; i += blockDim.x) {
        const int from = order[i];
        dst[i] = from >= 0 && from < k ? src[from] : FromFloat<T>(0.0f);
      }
    } else {
      for (int i = threadIdx.x; i < k; i += blockDim.x) dst[i] = FromFloat<T>(0.0f);
    }
    if (expert >= 0 && row % block_size == 0) {
      const int32_t* groups = g_idx + static_cast<size_t>(expert) * k;
      bool ok = true;
      for (int i = threadIdx.x; i < k; i += blockDim.x) ok = ok && groups[i] == i / group_size;
      if (!ok && atomicCAS(status, 0, kErrGIdx) == 0) {
        status[1] = expert;
        __threadfence();
      }
    }
  }
}

// Act-order for the dense GEMM: permuted[row][k] = a[row][perm[k]], one table for the whole matrix;
// block 0 checks `g_idx` as above (status header: code kErrGIdx, detail -1).
template <typename T>
__global__ void PermuteColumnsKernel(const T* __restrict__ a, T* __restrict__ permuted, const int32_t* __restrict__ perm,
                                     const int32_t* __restrict__ g_idx, int m, int k, int group_size, int* status) {
  for (int row = blockIdx.x; row < m; row += gridDim.x) {
    const T* src = a + static_cast<size_t>(row) * k;
    T* dst = permuted + static_cast<size_t>(row) * k;
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
      const int from = perm[i];
      dst[i] = from >= 0 && from < k ? src[from] : FromFloat<T>(0.0f);
    }
  }
  if (blockIdx.x == 0) {
    bool ok = true;
    for (int i = threadIdx.x; i < k; i += blockDim.x) ok = ok && g_idx[i] == i / group_size;
    if (!ok && atomicCAS(status, 0, kErrGIdx) == 0) {
      status[1] = -1;
      __threadfence();
    }
  }
}

// ---- host side ----------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn GetEncode() {
  static EncodeFn fn = [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult result;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &result) != cudaSuccess ||
        result != cudaDriverEntryPointSuccess) {
      return static_cast<EncodeFn>(nullptr);
    }
    return reinterpret_cast<EncodeFn>(ptr);
  }();
  return fn;
}

struct MapKey {
  const void* ptr;
  int64_t rows, cols;
  int box_rows, box_cols, kind;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols &&
           kind == o.kind;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h ^= static_cast<size_t>(k.rows) * 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>(k.cols) * 0xC2B2AE3D27D4EB4Full + (h << 6) + (h >> 2);
    h ^= static_cast<size_t>((k.box_rows * 1024 + k.box_cols) * 4 + k.kind) + (h << 6) + (h >> 2);
    return h;
  }
};

constexpr int kMapF16 = 0, kMapBf16 = 1, kMapWords = 2;

// Tensor map of a row-major [rows, cols] matrix with a [box_rows, box_cols] box.  16-bit kinds use
// the 128-byte swizzle (activation tiles, box_cols = 64); 32-bit words are copied unswizzled.
// Encoded maps are cached per thread: encoding costs microseconds of host time.
int TensorMap2D(const void* ptr, int64_t rows, int64_t cols, int box_rows, int box_cols, int kind,
                CUtensorMap* out) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, box_rows, box_cols, kind};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return IOB_OK;
  }
  EncodeFn encode = GetEncode();
  if (encode == nullptr) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: cuTensorMapEncodeTiled is not available");
  const int elem_bytes = kind == kMapWords ? 4 : 2;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * elem_bytes};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  const CUtensorMapDataType type = kind == kMapWords  ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                   : kind == kMapBf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                      : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  const CUresult rc = encode(out, type, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                             CU_TENSOR_MAP_INTERLEAVE_NONE,
                             kind == kMapWords ? CU_TENSOR_MAP_SWIZZLE_NONE : CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: tensor map encode failed (%d)", static_cast<int>(rc));
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return IOB_OK;
}

// Activations [rows, cols] of a 16-bit type seen as [cols / 64][rows][64]: one copy of a
// (2, box_rows, 64) box fetches the two 64-k atoms of a 128-k stage, each [box_rows][128 bytes]
// with the 128-byte swizzle, one after the other in shared memory.
int ActivationMap(const void* ptr, int64_t rows, int64_t cols, int box_rows, int dtype, CUtensorMap* out) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, box_rows, 64, dtype == IOB_BF16 ? kMapBf16 : kMapF16};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return IOB_OK;
  }
  EncodeFn encode = GetEncode();
  if (encode == nullptr) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(cols / 64)};
  const cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, 128};
  const cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 2};
  const cuuint32_t elem[3] = {1, 1, 1};
  const CUresult rc = encode(out, dtype == IOB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                             3, const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: tensor map encode failed (%d)", static_cast<int>(rc));
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return IOB_OK;
}

// Output [rows, cols] of a 16-bit type, box = 16 rows x 32 columns: the tile one epilogue warp
// stages and stores at a time.
int OutputMap(const void* ptr, int64_t rows, int64_t cols, int dtype, CUtensorMap* out, int box_cols = 32) {
  static thread_local std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  const MapKey key{ptr, rows, cols, 16, box_cols, dtype == IOB_BF16 ? kMapBf16 : kMapF16};
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return IOB_OK;
  }
  EncodeFn encode = GetEncode();
  if (encode == nullptr) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: cuTensorMapEncodeTiled is not available");
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(cols) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), 16};
  const cuuint32_t elem[2] = {1, 1};
  const CUresult rc = encode(out, dtype == IOB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                             2, const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (rc != CUDA_SUCCESS) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: tensor map encode failed (%d)", static_cast<int>(rc));
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, *out);
  return IOB_OK;
}

// Packed weights [E * K/16, 2N] words, box = 8 rows (128 k) x 256 words (128 columns).
int WeightMap(const void* ptr, int64_t experts, int64_t k, int64_t n, CUtensorMap* out, int bits = 4) {
  // (8-bit: [E * K/16, 4N] words; the same 8 x 256 box holds 64 columns, a tile takes two)
  return TensorMap2D(ptr, experts * (k / 16), (bits == 8 ? 4 : 2) * n, 8, 256, kMapWords, out);
}

// Shift/multiply form of `ks * 128 / group_size` for the usual group sizes.
void SetGroupMap(GemmParams& p) {
  p.g_mul = 1;
  p.g_shift = -1;
  if (p.groups == 1) {
    p.g_mul = 0;
    p.g_shift = 0;
  } else if (p.group_size == 64) {
    p.g_mul = 2;
    p.g_shift = 0;
  } else {
    const int per = p.group_size / kBlockK;  // stages per group
    if (per > 0 && (per & (per - 1)) == 0) {
      p.g_shift = 0;
      while ((1 << p.g_shift) < per) ++p.g_shift;
    }
  }
}

// Token tile of the dense GEMM.  33..64 rows run as two 32-row tiles when the group size allows the
// late-scale variant and both row tiles of every column tile find an SM of their own: converting the
// weights twice that way is then cheaper than once through the 64-row kernel, whose dequantisers
// also multiply by the scales (measured: 16 vs 20 us at 4096 x 4096, but 54 vs 46 us at 4096 x 28672).
int DenseTokenTile(int64_t m, int64_t n, int64_t group_size);
int TokenTile(int64_t m) { return m <= 16 ? 16 : m <= 32 ? 32 : m <= 64 ? 64 : m <= 128 ? 128 : 256; }

int DenseTokenTile(int64_t m, int64_t n, int64_t group_size) {
  if (m > 32 && m <= 64 && group_size >= kBlockK && 2 * ((n + kTileN - 1) / kTileN) <= NumSms()) return 32;
  return TokenTile(m);
}

size_t Align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct ScratchPlan {
  size_t counters_off, partial_off, gathered_off, total;
};
ScratchPlan PlanScratch(int64_t tiles, int tok, int64_t gathered_bytes) {
  ScratchPlan plan;
  plan.counters_off = kHeaderBytes;
  // Fixed positions whatever the problem: the counters must never overlap an area that some
  // other call fills with data, because every call relies on finding them zero.
  (void)tiles;
  plan.partial_off = Align256(plan.counters_off + static_cast<size_t>(4) * kMaxGrid * sizeof(int));
  plan.gathered_off = Align256(plan.partial_off + static_cast<size_t>(2) * NumSms() * tok * kTileN * sizeof(float));
  plan.total = Align256(plan.gathered_off + gathered_bytes);
  return plan;
}

template <typename T, int kTok, bool kZeros, bool kMoe, bool kLate, bool kPair = false, int kEpi = 0, int kBits = 4>
int LaunchVariant(const CUtensorMap& map, const CUtensorMap& w_map, const CUtensorMap& c_map, const GemmParams& p,
                  int grid, cudaStream_t stream) {
  constexpr int kSets = kPair ? kPairSets : SetsFor(kTok);
  auto kernel = W4A16GemmKernel<T, kTok, kZeros, kMoe, kSets, kLate, kPair, kEpi, kBits>;
  // rings + 8 KB of output staging + slack for the 1024-byte alignment
  constexpr int smem =
      (kPair ? kPairStages * 8192 + kPairActStages * kTok * 128
             : kBits == 8 ? StagesFor8(kTok) * StageBytes(kTok, 8) : StagesFor(kTok) * StageBytes(kTok)) + 8192 + 1024;
  static_assert(smem <= 232448, "shared memory budget");
  static thread_local bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM: %s", cudaGetErrorString(err));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  // Launched as a programmatic dependent of whatever precedes it in the stream: the kernel does
  // its on-chip set-up at once and waits for its predecessors before the first global access.
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3((5 + IssuersFor(kTok) + 4 * kSets) * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  if constexpr (kPair) {
    // clusters of two blocks; the grid is a whole number of them
    config.gridDim = dim3(grid & ~1);
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = 2;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    config.numAttrs = 2;
  }
  Problem problem{};
  problem.a_map = map;
  problem.w_map = w_map;
  problem.c_map = c_map;
  problem.p = p;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, problem);
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM launch: %s", cudaGetErrorString(err));
  return CheckLaunch("W4A16 GEMM launch");
}

// A table of dense problems (late-scale tiles of kTok tokens) as one launch.
template <typename T, int kTok, bool kZeros>
int LaunchBatchVariant(const BatchTable& table, int grid, cudaStream_t stream) {
  constexpr int kSets = SetsFor(kTok);
  auto kernel = W4A16GemmBatchKernel<T, kTok, kZeros, kSets>;
  constexpr int smem = StagesFor(kTok) * StageBytes(kTok) + 8192 + 1024;
  static thread_local bool configured[64] = {};
  int device = 0;
  cudaGetDevice(&device);
  if (device < 0 || device >= 64 || !configured[device]) {
    const cudaError_t err = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM batch: %s", cudaGetErrorString(err));
    if (device >= 0 && device < 64) configured[device] = true;
  }
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3((5 + IssuersFor(kTok) + 4 * kSets) * 32);
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attr;
  config.numAttrs = 1;
  const cudaError_t err = cudaLaunchKernelEx(&config, kernel, table);
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "W4A16 GEMM batch launch: %s", cudaGetErrorString(err));
  return CheckLaunch("W4A16 GEMM batch launch");
}

template <typename T>
int LaunchBatchTyped(bool zeros, int tok, const BatchTable& table, int grid, cudaStream_t stream) {
  switch (tok) {
    case 16:
      return zeros ? LaunchBatchVariant<T, 16, true>(table, grid, stream) : LaunchBatchVariant<T, 16, false>(table, grid, stream);
    case 32:
      return zeros ? LaunchBatchVariant<T, 32, true>(table, grid, stream) : LaunchBatchVariant<T, 32, false>(table, grid, stream);
    default:
      return zeros ? LaunchBatchVariant<T, 64, true>(table, grid, stream) : LaunchBatchVariant<T, 64, false>(table, grid, stream);
  }
}
int LaunchBatch(int a_dtype, bool zeros, int tok, const BatchTable& table, int grid, cudaStream_t stream) {
  return a_dtype == IOB_BF16 ? LaunchBatchTyped<__nv_bfloat16>(zeros, tok, table, grid, stream)
                             : LaunchBatchTyped<__half>(zeros, tok, table, grid, stream);
}

// Token tiles up to 32 with groups of at least one k-stage take the variant that scales the
// accumulators instead of the weights.
template <typename T, int kTok, bool kZeros, bool kMoe, int kEpi = 0>
int LaunchKernel(const CUtensorMap& map, const CUtensorMap& w_map, const CUtensorMap& c_map, const GemmParams& p, int grid,
                 cudaStream_t stream) {
  // silu_and_mul in the epilogue is a kernel variant of its own (routed form only), so that the
  // kernels without it carry none of its code
  if constexpr (kEpi == 0 && kTok <= 128) {
    if (p.bits == 8) return LaunchVariant<T, kTok, kZeros, kMoe, false, false, 0, 8>(map, w_map, c_map, p, grid, stream);
  }
  if constexpr (kMoe && kEpi == 0) {
    if (p.fuse_silu) return LaunchKernel<T, kTok, kZeros, kMoe, 1>(map, w_map, c_map, p, grid, stream);
    if constexpr (kTok >= 128) {
      if (p.out_sorted && p.mul_weights) return LaunchKernel<T, kTok, kZeros, kMoe, 2>(map, w_map, c_map, p, grid, stream);
    }
  }
  // (64-row tiles: dense only -- the routed form, with its many whole tiles per block and its
  // scattered tile-end stores, measured 40 % slower that way than with scaled weights)
  if constexpr (kTok <= 32 || (kTok == 64 && !kMoe)) {
    if (p.group_size >= kBlockK) {
      return LaunchVariant<T, kTok, kZeros, kMoe, true, false, kEpi>(map, w_map, c_map, p, grid, stream);
    }
  }
  if constexpr (kTok == 256) {
    if (p.pair) return LaunchVariant<T, kTok, kZeros, kMoe, false, true, kEpi>(map, w_map, c_map, p, grid, stream);
  }
  return LaunchVariant<T, kTok, kZeros, kMoe, false, false, kEpi>(map, w_map, c_map, p, grid, stream);
}

template <typename T, bool kZeros, bool kMoe>
int DispatchTok(int tok, const CUtensorMap& map, const CUtensorMap& w_map, const CUtensorMap& c_map, const GemmParams& p, int grid,
                cudaStream_t stream) {
  switch (tok) {
    case 16: return LaunchKernel<T, 16, kZeros, kMoe>(map, w_map, c_map, p, grid, stream);
    case 32: return LaunchKernel<T, 32, kZeros, kMoe>(map, w_map, c_map, p, grid, stream);
    case 64: return LaunchKernel<T, 64, kZeros, kMoe>(map, w_map, c_map, p, grid, stream);
    default: break;
  }
  if (tok == 128) return LaunchKernel<T, 128, kZeros, kMoe>(map, w_map, c_map, p, grid, stream);
  if (tok == 256) return LaunchKernel<T, 256, kZeros, kMoe>(map, w_map, c_map, p, grid, stream);
  return Fail(IOB_UNSUPPORTED, "W4A16 GEMM: no kernel for a token tile of %d", tok);
}

template <bool kMoe>
int Dispatch(int a_dtype, bool zeros, int tok, const CUtensorMap& map, const CUtensorMap& w_map,
             const CUtensorMap& c_map, const GemmParams& p, int grid, cudaStream_t stream) {
  if (a_dtype == IOB_BF16) {
    return zeros ? DispatchTok<__nv_bfloat16, true, kMoe>(tok, map, w_map, c_map, p, grid, stream)
                 : DispatchTok<__nv_bfloat16, false, kMoe>(tok, map, w_map, c_map, p, grid, stream);
  }
  return zeros ? DispatchTok<__half, true, kMoe>(tok, map, w_map, c_map, p, grid, stream)
               : DispatchTok<__half, false, kMoe>(tok, map, w_map, c_map, p, grid, stream);
}

int BitsOf(int64_t b_type_id) {
  return b_type_id == IOB_QTYPE_UINT8B128 || b_type_id == IOB_QTYPE_UINT8 || b_type_id == IOB_QTYPE_FLOAT8_E4M3FN ? 8 : 4;
}

int CheckProblem(const char* op, const void* a, int a_dtype, const void* wq, const void* scales, const void* zeros,
                 int64_t b_type_id, int64_t m, int64_t n, int64_t k, int64_t groups, const void* out) {
  IOB_REQUIRE(a && wq && scales && out, "%s: null tensor pointer", op);
  IOB_REQUIRE(a_dtype == IOB_F16 || a_dtype == IOB_BF16, "%s: requires float16 or bfloat16 `a`", op);
  IOB_REQUIRE(m > 0 && n > 0 && k > 0 && k % 16 == 0 && n % 64 == 0, "%s: received unsupported dimensions", op);
  IOB_REQUIRE(m <= INT32_MAX && n <= INT32_MAX && k <= INT32_MAX, "%s: dimensions exceed int32", op);
  if (b_type_id != IOB_QTYPE_UINT4B8 && b_type_id != IOB_QTYPE_UINT4 && b_type_id != IOB_QTYPE_UINT8B128 &&
      b_type_id != IOB_QTYPE_UINT8 && b_type_id != IOB_QTYPE_FLOAT8_E4M3FN) {
    return Fail(IOB_UNSUPPORTED,
                "%s: only the weight types uint4b8, uint4, uint8b128, uint8 and float8_e4m3fn are implemented", op);
  }
  IOB_REQUIRE((zeros != nullptr) == (b_type_id == IOB_QTYPE_UINT4 || b_type_id == IOB_QTYPE_UINT8),
              "%s: zero points are required for uint4 / uint8 and not accepted for uint4b8 / uint8b128 / float8_e4m3fn", op);
  IOB_REQUIRE(groups > 0 && k % groups == 0, "%s: `size_k` must be a multiple of the number of scale groups", op);
  if (k % kBlockK != 0 || ((k / groups) != 64 && (k / groups) % kBlockK != 0)) {
    return Fail(IOB_UNSUPPORTED, "%s: needs `size_k` to be a multiple of 128 and the group size 64 or a multiple of 128", op);
  }
  IOB_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(wq) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(scales) % 16 == 0 && reinterpret_cast<uintptr_t>(zeros) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "%s: tensors must be 16-byte aligned", op);
  return IOB_OK;
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_scratch_status(const void* scratch, void* stream) {
  int code = 0;
  auto s = static_cast<cudaStream_t>(stream);
  if (cudaMemcpyAsync(&code, scratch, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaStreamSynchronize(s) != cudaSuccess) {
    return -1;
  }
  return code;
}

extern "C" int infiniops_b200_selftest_bounded_wait(void* scratch, size_t scratch_bytes, int* result, void* stream) {
  using namespace iob;
  IOB_REQUIRE(scratch != nullptr && scratch_bytes >= static_cast<size_t>(kHeaderBytes) && result != nullptr,
              "selftest_bounded_wait: needs a scratch header of %d bytes and a result pointer", kHeaderBytes);
  BoundedWaitSelfTestKernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<int*>(scratch), result);
  return CheckLaunch("selftest_bounded_wait launch");
}

extern "C" int infiniops_b200_gemm_scratch_prepare(void* scratch, size_t scratch_bytes, void* stream) {
  using namespace iob;
  const size_t need = kHeaderBytes + static_cast<size_t>(4) * kMaxGrid * sizeof(int);
  IOB_REQUIRE(scratch != nullptr && scratch_bytes >= need, "gemm_scratch_prepare: the buffer is smaller than %zu bytes", need);
  if (cudaMemsetAsync(scratch, 0, need, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "gemm_scratch_prepare: clearing the header failed");
  }
  return IOB_OK;
}

extern "C" size_t infiniops_b200_marlin_gemm_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k) {
  using namespace iob;
  (void)size_k;
  const int tok = TokenTile(size_m);
  const int64_t tiles = ((size_n + kTileN - 1) / kTileN) * ((size_m + tok - 1) / tok);
  return PlanScratch(tiles, tok, 0).total;
}

extern "C" size_t infiniops_b200_marlin_gemm_act_order_scratch_bytes(int64_t size_m, int64_t size_n, int64_t size_k) {
  using namespace iob;
  const int tok = TokenTile(size_m);
  const int64_t tiles = ((size_n + kTileN - 1) / kTileN) * ((size_m + tok - 1) / tok);
  return PlanScratch(tiles, tok, size_m * size_k * 2).total;
}

namespace iob {
namespace {

// Validates the placement and peer fields of a problem and copies them into the kernel parameters.
int SetPlacement(const char* op, const iob_gemm_problem& g, GemmParams& p) {
  const int64_t ld = g.out_ld > 0 ? g.out_ld : g.size_n;
  IOB_REQUIRE(g.out_col0 >= 0 && g.out_col0 + g.size_n <= ld && ld % 8 == 0 && g.out_col0 % 8 == 0 && ld <= INT32_MAX,
              "%s: columns [out_col0, out_col0 + size_n) must lie inside a row of out_ld elements, both multiples of 8", op);
  IOB_REQUIRE(g.n_peers >= 0 && g.n_peers <= kMaxPeers, "%s: at most %d peer outputs", op, kMaxPeers);
  IOB_REQUIRE(g.scale_layout == 0 || g.scale_layout == 1, "%s: `scale_layout` must be 0 (plain) or 1 (provider)", op);
  p.layout = g.scale_layout;
  p.out_ld = static_cast<int>(ld);
  p.out_col0 = static_cast<int>(g.out_col0);
  p.n_peers = g.n_peers;
  for (int r = 0; r < g.n_peers; ++r) {
    IOB_REQUIRE(g.peer_out[r] != nullptr && reinterpret_cast<uintptr_t>(g.peer_out[r]) % 16 == 0,
                "%s: peer outputs must be non-null and 16-byte aligned", op);
    p.peer_out[r] = g.peer_out[r];
  }
  return IOB_OK;
}

int SetSignal(const char* op, const iob_peer_signal* signal, GemmParams& p) {
  if (signal == nullptr) return IOB_OK;
  IOB_REQUIRE(signal->done_counter != nullptr && signal->epoch != nullptr && signal->n_peers >= 0 &&
                  signal->n_peers <= kMaxPeers && signal->flag_slot >= 0,
              "%s: incomplete completion signal", op);
  p.done_counter = signal->done_counter;
  p.epoch = signal->epoch;
  p.flag_slot = signal->flag_slot;
  p.n_flag_peers = signal->n_peers;
  for (int r = 0; r < signal->n_peers; ++r) {
    IOB_REQUIRE(signal->peer_flags[r] != nullptr, "%s: null peer flag pointer", op);
    p.peer_flags[r] = signal->peer_flags[r];
  }
  return IOB_OK;
}

void FillDense(const iob_gemm_problem& g, unsigned char* scratch, const ScratchPlan& plan, GemmParams& p) {
  p.wq = reinterpret_cast<const uint32_t*>(g.b_q_weight);
  p.scales = g.b_scales;
  p.zeros = reinterpret_cast<const uint32_t*>(g.b_zeros);
  p.bias = g.b_bias;
  p.out = g.out;
  p.partial = reinterpret_cast<float*>(scratch + plan.partial_off);
  p.counters = reinterpret_cast<int*>(scratch + plan.counters_off);
  p.status = reinterpret_cast<int*>(scratch);
  p.m = static_cast<int>(g.size_m);
  p.n = static_cast<int>(g.size_n);
  p.k = static_cast<int>(g.size_k);
  p.groups = static_cast<int>(g.num_groups);
  p.group_size = static_cast<int>(g.size_k / g.num_groups);
  SetGroupMap(p);
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_marlin_gemm_placed(const iob_gemm_problem* problem, int a_dtype, int64_t b_type_id,
                                                 const iob_peer_signal* signal, void* scratch, size_t scratch_bytes,
                                                 void* stream) {
  using namespace iob;
  const char* op = "marlin_gemm";
  IOB_REQUIRE(problem != nullptr, "%s: null problem", op);
  const iob_gemm_problem& g = *problem;
  if (const int rc = CheckProblem(op, g.a, a_dtype, g.b_q_weight, g.b_scales, g.b_zeros, b_type_id, g.size_m, g.size_n,
                                  g.size_k, g.num_groups, g.out)) {
    return rc;
  }
  const int bits = BitsOf(b_type_id);
  IOB_REQUIRE(!(bits == 8 && g.b_zeros != nullptr && g.scale_layout != 0),
              "%s: 8-bit zero points are read in the plain layout only", op);
  IOB_REQUIRE(!(b_type_id == IOB_QTYPE_FLOAT8_E4M3FN && g.scale_layout != 0),
              "%s: float8_e4m3fn weights take their scales in the plain layout only", op);
  int tok = DenseTokenTile(g.size_m, g.size_n, g.size_k / (g.num_groups > 0 ? g.num_groups : 1));
  if (bits == 8 && tok > 128) tok = 128;  // 8-bit weights: no 256-row tiles (the stage ring would not fit)
  const int64_t n_tiles = (g.size_n + kTileN - 1) / kTileN, m_tiles = (g.size_m + tok - 1) / tok;
  // (the scratch query does not know the group size and answers for the larger plan)
  IOB_REQUIRE((g.perm == nullptr) == (g.g_idx == nullptr), "%s: requires `g_idx` and `perm` together", op);
  IOB_REQUIRE(g.perm == nullptr || g.num_groups > 1, "%s: activation order needs grouped scales", op);
  const ScratchPlan plan = PlanScratch(n_tiles * m_tiles, tok, g.perm != nullptr ? g.size_m * g.size_k * 2 : 0);
  if (scratch == nullptr || scratch_bytes < plan.total) {
    return Fail(IOB_SCRATCH_TOO_SMALL, "%s: needs %zu bytes of scratch, got %zu", op, plan.total, scratch_bytes);
  }
  GemmParams p{};
  if (const int rc = SetPlacement(op, g, p)) return rc;
  if (const int rc = SetSignal(op, signal, p)) return rc;
  const void* activations = g.a;
  if (g.perm != nullptr) {
    // Activation order: the weight rows are in `perm` order, so the GEMM runs on a copy of `a` with
    // its columns in that order (kept in the scratch buffer, behind the split-K partial sums).
    unsigned char* base = static_cast<unsigned char*>(scratch);
    const int rows_grid = static_cast<int>(std::min<int64_t>(g.size_m, 4 * NumSms()));
    auto launch = [&](auto* typed) {
      using T = std::remove_pointer_t<decltype(typed)>;
      PermuteColumnsKernel<T><<<rows_grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
          static_cast<const T*>(g.a), reinterpret_cast<T*>(base + plan.gathered_off), g.perm, g.g_idx,
          static_cast<int>(g.size_m), static_cast<int>(g.size_k), static_cast<int>(g.size_k / g.num_groups),
          reinterpret_cast<int*>(base));
    };
    if (a_dtype == IOB_BF16) {
      launch(static_cast<__nv_bfloat16*>(nullptr));
    } else {
      launch(static_cast<__half*>(nullptr));
    }
    if (const int rc = CheckLaunch("marlin_gemm column permutation launch")) return rc;
    activations = base + plan.gathered_off;
  }
  // Prefill-sized problems whose columns pair up run two blocks per 256 x 256 output tile.
  const bool pair = tok == 256 && g.size_n % (2 * kTileN) == 0 && NumSms() >= 2;
  CUtensorMap map;
  if (const int rc = ActivationMap(activations, g.size_m, g.size_k, pair ? tok / 2 : tok, a_dtype, &map)) return rc;
  CUtensorMap w_map;
  if (const int rc = WeightMap(g.b_q_weight, 1, g.size_k, g.size_n, &w_map, bits)) return rc;
  CUtensorMap c_map;
  if (const int rc = OutputMap(g.out, g.size_m, p.out_ld, a_dtype, &c_map)) return rc;
  p.pair = pair ? 1 : 0;
  p.bits = bits;
  p.fp8 = b_type_id == IOB_QTYPE_FLOAT8_E4M3FN ? 1 : 0;
  FillDense(g, static_cast<unsigned char*>(scratch), plan, p);
  const int64_t units = n_tiles * m_tiles * (g.size_k / kBlockK);
  const int grid = pair ? NumSms() : static_cast<int>(units < NumSms() ? units : NumSms());
  return Dispatch<false>(a_dtype, g.b_zeros != nullptr, tok, map, w_map, c_map, p, grid, static_cast<cudaStream_t>(stream));
}

extern "C" int infiniops_b200_marlin_gemm(const void* a, int a_dtype, const int32_t* b_q_weight, const void* b_bias,
                                          const void* b_scales, const int32_t* b_zeros, int64_t b_type_id,
                                          int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups,
                                          void* out, void* scratch, size_t scratch_bytes, void* stream) {
  iob_gemm_problem g{};
  g.a = a;
  g.b_q_weight = b_q_weight;
  g.b_bias = b_bias;
  g.b_scales = b_scales;
  g.b_zeros = b_zeros;
  g.out = out;
  g.size_m = size_m;
  g.size_n = size_n;
  g.size_k = size_k;
  g.num_groups = num_groups;
  return infiniops_b200_marlin_gemm_placed(&g, a_dtype, b_type_id, nullptr, scratch, scratch_bytes, stream);
}

extern "C" size_t infiniops_b200_marlin_gemm_batch_scratch_bytes(void) {
  using namespace iob;
  return PlanScratch(0, 64, 0).total;
}

extern "C" int infiniops_b200_marlin_gemm_batch(const iob_gemm_problem* problems, int count, int a_dtype,
                                                int64_t b_type_id, const iob_peer_signal* signal, void* scratch,
                                                size_t scratch_bytes, void* stream) {
  using namespace iob;
  const char* op = "marlin_gemm_batch";
  IOB_REQUIRE(BitsOf(b_type_id) == 4, "%s: 4-bit weights only; 8-bit problems go through marlin_gemm", op);
  IOB_REQUIRE(problems != nullptr && count > 0, "%s: no problems", op);
  const ScratchPlan plan = PlanScratch(0, 64, 0);
  if (scratch == nullptr || scratch_bytes < plan.total) {
    return Fail(IOB_SCRATCH_TOO_SMALL, "%s: needs %zu bytes of scratch, got %zu", op, plan.total, scratch_bytes);
  }
  // Three classes of token tile: up to 16 rows, 17..32 and 33..64 (inside one launch the whole grid
  // works on every tile in turn, so a 64-row tile -- each weight converted once -- beats two 32-row
  // ones).  Each class is one launch (or several, kMaxBatch problems at a time); the completion
  // signal rides on the last.
  constexpr int kClasses = 3;
  constexpr int kTokOf[kClasses] = {16, 32, 64};
  int order[kClasses][1024];
  int n_of[kClasses] = {0, 0, 0};
  IOB_REQUIRE(count <= 1024, "%s: at most 1024 problems per call", op);
  for (int i = 0; i < count; ++i) {
    const iob_gemm_problem& g = problems[i];
    if (const int rc = CheckProblem(op, g.a, a_dtype, g.b_q_weight, g.b_scales, g.b_zeros, b_type_id, g.size_m,
                                    g.size_n, g.size_k, g.num_groups, g.out)) {
      return rc;
    }
    if (g.size_m > 64 || (g.size_k / g.num_groups) % kBlockK != 0) {
      return Fail(IOB_UNSUPPORTED, "%s: problem %d: batched launches take at most 64 rows and group sizes that are "
                  "multiples of 128; use marlin_gemm", op, i);
    }
    IOB_REQUIRE(g.perm == nullptr && g.g_idx == nullptr, "%s: problem %d: activation order goes through marlin_gemm", op, i);
    const int cls = g.size_m <= 16 ? 0 : g.size_m <= 32 ? 1 : 2;
    order[cls][n_of[cls]++] = i;
  }
  int launches = 0;
  for (int cls = 0; cls < kClasses; ++cls) launches += (n_of[cls] + kMaxBatch - 1) / kMaxBatch;
  int launched = 0;
  for (int cls = 0; cls < kClasses; ++cls) {
    const int tok = kTokOf[cls];
    for (int first = 0; first < n_of[cls]; first += kMaxBatch) {
      BatchTable table{};
      table.count = std::min(kMaxBatch, n_of[cls] - first);
      long long units = 0;
      for (int j = 0; j < table.count; ++j) {
        const iob_gemm_problem& g = problems[order[cls][first + j]];
        Problem& pr = table.prob[j];
        if (const int rc = SetPlacement(op, g, pr.p)) return rc;
        if (const int rc = ActivationMap(g.a, g.size_m, g.size_k, tok, a_dtype, &pr.a_map)) return rc;
        if (const int rc = WeightMap(g.b_q_weight, 1, g.size_k, g.size_n, &pr.w_map)) return rc;
        if (const int rc = OutputMap(g.out, g.size_m, pr.p.out_ld, a_dtype, &pr.c_map)) return rc;
        FillDense(g, static_cast<unsigned char*>(scratch), plan, pr.p);
        pr.n_tiles = static_cast<int>((g.size_n + kTileN - 1) / kTileN);
        pr.m_tiles = static_cast<int>((g.size_m + tok - 1) / tok);
        pr.k_stages = static_cast<int>(g.size_k / kBlockK);
        units += static_cast<long long>(pr.n_tiles) * pr.m_tiles * pr.k_stages;
        IOB_REQUIRE(units < (1ll << 31), "%s: too many work units in one launch", op);
        pr.unit_end = units;
      }
      ++launched;
      if (launched == launches) {
        // the kernel reads the signal from the first problem of the table; its peers are those of the flags
        if (const int rc = SetSignal(op, signal, table.prob[0].p)) return rc;
      }
      const int grid = static_cast<int>(units < NumSms() ? units : NumSms());
      if (const int rc = LaunchBatch(a_dtype, problems[order[cls][first]].b_zeros != nullptr, tok, table, grid,
                                     static_cast<cudaStream_t>(stream))) {
        return rc;
      }
    }
  }
  return IOB_OK;
}

extern "C" size_t infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(int64_t size_m, int64_t top_k, int64_t size_n,
                                                                     int64_t size_k, int64_t num_experts,
                                                                     int64_t moe_block_size) {
  using namespace iob;
  int64_t sorted = size_m * top_k + num_experts * (moe_block_size - 1);
  if (size_m * top_k < num_experts) sorted = std::min(sorted, size_m * top_k * moe_block_size);
  const int tok = TokenTile(moe_block_size);
  const int64_t blocks = (sorted + moe_block_size - 1) / moe_block_size;
  const int64_t tiles = ((size_n + kTileN - 1) / kTileN) * blocks;
  // one extra box of rows so the last block's TMA box stays inside the buffer's tensor map
  return PlanScratch(tiles, tok, (sorted + tok) * size_k * 2).total;
}

extern "C" int infiniops_b200_moe_wna16_marlin_gemm(
    const void* a, int a_dtype, const int32_t* b_q_weight, const void* b_bias, const void* b_scales,
    const int32_t* b_zeros, const int32_t* sorted_token_ids, const int32_t* expert_ids,
    const int32_t* num_tokens_past_padded, const float* topk_weights, int64_t moe_block_size, int64_t top_k,
    int mul_topk_weights, int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups,
    int64_t num_experts, int64_t sorted_size, void* out, void* scratch, size_t scratch_bytes, void* stream) {
  return infiniops_b200_moe_wna16_marlin_gemm_ex(
      a, a_dtype, b_q_weight, b_bias, b_scales, b_zeros, sorted_token_ids, expert_ids, num_tokens_past_padded,
      topk_weights, moe_block_size, top_k, mul_topk_weights, b_type_id, size_m, size_n, size_k, num_groups, num_experts,
      sorted_size, out, nullptr, scratch, scratch_bytes, stream);
}

extern "C" int infiniops_b200_moe_wna16_marlin_gemm_ex(
    const void* a, int a_dtype, const int32_t* b_q_weight, const void* b_bias, const void* b_scales,
    const int32_t* b_zeros, const int32_t* sorted_token_ids, const int32_t* expert_ids,
    const int32_t* num_tokens_past_padded, const float* topk_weights, int64_t moe_block_size, int64_t top_k,
    int mul_topk_weights, int64_t b_type_id, int64_t size_m, int64_t size_n, int64_t size_k, int64_t num_groups,
    int64_t num_experts, int64_t sorted_size, void* out, const iob_routed_options* options, void* scratch,
    size_t scratch_bytes, void* stream) {
  using namespace iob;
  const char* op = "moe_wna16_marlin_gemm";
  if (const int rc = CheckProblem(op, a, a_dtype, b_q_weight, b_scales, b_zeros, b_type_id, size_m, size_n, size_k,
                                  num_groups, out)) {
    return rc;
  }
  IOB_REQUIRE(sorted_token_ids && expert_ids && num_tokens_past_padded, "%s: received invalid routing metadata", op);
  IOB_REQUIRE(top_k > 0 && num_experts > 0 && size_m <= INT32_MAX / top_k, "%s: output dimensions overflow", op);
  // (8..64: the sizes the reference accepts; 128 and 256: larger routing blocks for callers that sort
  // with them -- each weight is then converted once per 128 / 256 rows instead of once per 64)
  IOB_REQUIRE(moe_block_size == 8 || (moe_block_size >= 16 && moe_block_size <= 64 && moe_block_size % 16 == 0) ||
                  moe_block_size == 128 || moe_block_size == 256,
              "%s: received an unsupported `moe_block_size`", op);
  IOB_REQUIRE(!mul_topk_weights || topk_weights != nullptr, "%s: received invalid top-k weights", op);
  const int tok = TokenTile(moe_block_size);
  // rows the routing can occupy at most (the bound the sort operator guarantees)
  int64_t sorted_cap = size_m * top_k + num_experts * (moe_block_size - 1);
  if (size_m * top_k < num_experts) sorted_cap = std::min(sorted_cap, size_m * top_k * moe_block_size);
  IOB_REQUIRE(sorted_size >= sorted_cap, "%s: `sorted_token_ids` is smaller than the padded routing can be", op);
  const int64_t blocks = (sorted_cap + moe_block_size - 1) / moe_block_size;
  const int64_t n_tiles = (size_n + kTileN - 1) / kTileN;
  const ScratchPlan plan = PlanScratch(n_tiles * blocks, tok, (sorted_cap + tok) * size_k * 2);
  if (scratch == nullptr || scratch_bytes < plan.total) {
    return Fail(IOB_SCRATCH_TOO_SMALL, "%s: needs %zu bytes of scratch, got %zu", op, plan.total, scratch_bytes);
  }
  auto s = static_cast<cudaStream_t>(stream);
  auto* base = static_cast<unsigned char*>(scratch);
  const bool a_sorted = options != nullptr && options->a_sorted != 0;
  int32_t* position = options != nullptr ? options->route_position : nullptr;
  IOB_REQUIRE(position == nullptr || (!a_sorted && (options->perm == nullptr)),
              "%s: `route_position` is written by the plain row gather (not with `a_sorted` or `perm`)", op);
  // live rows per routing block: written by a call that gathers (plain gather), read by any call given it
  int32_t* block_rows = options != nullptr ? options->block_rows : nullptr;
  int32_t* block_rows_out = block_rows != nullptr && !a_sorted && (options->perm == nullptr) ? block_rows : nullptr;
  const int32_t* perm = options != nullptr ? options->perm : nullptr;
  const int32_t* g_idx = options != nullptr ? options->g_idx : nullptr;
  IOB_REQUIRE((perm == nullptr) == (g_idx == nullptr), "%s: requires `g_idx` and `perm` together", op);
  IOB_REQUIRE(perm == nullptr || num_groups > 1, "%s: activation order needs grouped scales", op);
  const void* gathered = a_sorted && perm == nullptr ? a : base + plan.gathered_off;
  const int out_rows = static_cast<int>(size_m * top_k);
  const int gather_grid = static_cast<int>(std::min<int64_t>(sorted_cap, 4 * NumSms()));
  if (position != nullptr &&
      cudaMemsetAsync(position, 0xFF, static_cast<size_t>(out_rows) * sizeof(int32_t), s) != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "%s: could not clear `route_position`", op);
  }
  if (perm != nullptr) {
    auto launch = [&](auto* typed) {
      using T = std::remove_pointer_t<decltype(typed)>;
      GatherPermutedRowsKernel<T><<<gather_grid, 256, 0, s>>>(
          static_cast<const T*>(a), reinterpret_cast<T*>(base + plan.gathered_off), sorted_token_ids, expert_ids,
          num_tokens_past_padded, perm, g_idx, static_cast<int>(size_k), static_cast<int>(top_k), out_rows,
          static_cast<int>(moe_block_size), static_cast<int>(size_k / num_groups), a_sorted ? 1 : 0,
          reinterpret_cast<int*>(base));
    };
    if (a_dtype == IOB_BF16) {
      launch(static_cast<__nv_bfloat16*>(nullptr));
    } else {
      launch(static_cast<__half*>(nullptr));
    }
  } else if (a_sorted) {
    // `a` already holds one row per sorted position: nothing to gather
  } else if (a_dtype == IOB_BF16) {
    GatherRowsKernel<__nv_bfloat16><<<gather_grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(a), reinterpret_cast<__nv_bfloat16*>(base + plan.gathered_off), sorted_token_ids,
        num_tokens_past_padded, static_cast<int>(size_k), static_cast<int>(top_k), out_rows, position, block_rows_out,
        static_cast<int>(moe_block_size));
  } else {
    GatherRowsKernel<__half><<<gather_grid, 256, 0, s>>>(static_cast<const __half*>(a), reinterpret_cast<__half*>(base + plan.gathered_off),
                                                        sorted_token_ids, num_tokens_past_padded,
                                                        static_cast<int>(size_k), static_cast<int>(top_k), out_rows, position,
                                                        block_rows_out, static_cast<int>(moe_block_size));
  }
  if (const int rc = CheckLaunch("moe_wna16_marlin_gemm gather launch")) return rc;
  // 256-row routing blocks whose columns pair up run two blocks of a cluster per 256 x 256 tile
  const bool pair = tok == 256 && size_n % (2 * kTileN) == 0 && NumSms() >= 2;
  CUtensorMap map;
  // (rows past the end of a caller's sorted buffer read as zeros; the scratch copy has a spare box of rows)
  if (const int rc = ActivationMap(gathered, a_sorted && perm == nullptr ? sorted_cap : sorted_cap + tok, size_k,
                                   pair ? tok / 2 : tok, a_dtype, &map)) {
    return rc;
  }
  CUtensorMap w_map;
  const int bits = BitsOf(b_type_id);
  IOB_REQUIRE(!(bits == 8 && b_zeros != nullptr && options != nullptr && options->scale_layout != 0),
              "%s: 8-bit zero points are read in the plain layout only", op);
  IOB_REQUIRE(!(b_type_id == IOB_QTYPE_FLOAT8_E4M3FN && options != nullptr && options->scale_layout != 0),
              "%s: float8_e4m3fn weights take their scales in the plain layout only", op);
  IOB_REQUIRE(bits == 4 || (moe_block_size <= 128 && (options == nullptr || !options->fuse_silu) &&
                            !(options != nullptr && options->out_sorted && mul_topk_weights)),
              "%s: 8-bit weights take routing blocks up to 128 rows and the plain epilogue", op);
  if (const int rc = WeightMap(b_q_weight, num_experts, size_k, size_n, &w_map, bits)) return rc;
  GemmParams p{};
  p.pair = pair ? 1 : 0;
  p.bits = bits;
  p.fp8 = b_type_id == IOB_QTYPE_FLOAT8_E4M3FN ? 1 : 0;
  p.block_rows = block_rows;
  p.wq = reinterpret_cast<const uint32_t*>(b_q_weight);
  p.scales = b_scales;
  p.zeros = reinterpret_cast<const uint32_t*>(b_zeros);
  p.bias = b_bias;
  p.out = out;
  p.partial = reinterpret_cast<float*>(base + plan.partial_off);
  p.counters = reinterpret_cast<int*>(base + plan.counters_off);
  p.status = reinterpret_cast<int*>(base);
  p.m = static_cast<int>(size_m);
  p.n = static_cast<int>(size_n);
  p.k = static_cast<int>(size_k);
  p.groups = static_cast<int>(num_groups);
  p.group_size = static_cast<int>(size_k / num_groups);
  SetGroupMap(p);
  p.sorted_ids = sorted_token_ids;
  p.expert_ids = expert_ids;
  p.num_post_pad = num_tokens_past_padded;
  p.topk_weights = topk_weights;
  p.top_k = static_cast<int>(top_k);
  p.block_size = static_cast<int>(moe_block_size);
  p.mul_weights = mul_topk_weights;
  p.out_rows = out_rows;
  if (options != nullptr) {
    IOB_REQUIRE(options->scale_layout == 0 || options->scale_layout == 1,
                "%s: `scale_layout` must be 0 (plain) or 1 (provider)", op);
    p.layout = options->scale_layout;
    p.out_sorted = options->out_sorted ? 1 : 0;
    IOB_REQUIRE(!p.out_sorted || options->row_dest == nullptr, "%s: sorted output takes no scatter", op);
    IOB_REQUIRE(!p.out_sorted || !mul_topk_weights || moe_block_size >= 128,
                "%s: sorted output with routing weights needs 128- or 256-row routing blocks", op);
    p.fuse_silu = options->fuse_silu ? 1 : 0;
    IOB_REQUIRE(!p.fuse_silu || (p.out_sorted && size_n % 128 == 0),
                "%s: the fused silu needs sorted output and `size_n` a multiple of 128", op);
    if (options->row_dest != nullptr) {
      IOB_REQUIRE(options->n_dest > 0 && options->n_dest <= kMaxPeers + 1, "%s: incomplete scatter description", op);
      p.row_dest = reinterpret_cast<const int2*>(options->row_dest);
      for (int r = 0; r < options->n_dest; ++r) {
        IOB_REQUIRE(options->dest_base[r] != nullptr, "%s: null scatter destination", op);
        p.dest_base[r] = options->dest_base[r];
      }
    }
    if (const int rc = SetSignal(op, options->signal, p)) return rc;
  }
  CUtensorMap c_map = w_map;  // unused while rows are scattered
  if (p.out_sorted) {
    if (const int rc = p.fuse_silu ? OutputMap(out, sorted_cap, size_n / 2, a_dtype, &c_map, 16)
                                   : OutputMap(out, sorted_cap, size_n, a_dtype, &c_map)) {
      return rc;
    }
  }
  return Dispatch<true>(a_dtype, b_zeros != nullptr, tok, map, w_map, c_map, p, NumSms(), s);
}

// ---- dense GEMM for callers that may not allocate device memory ---------------------------------
//
// Some hosts of this library cannot hand the GEMM a scratch buffer: an engine that gave all of
// the device's memory to its own arena at start-up and has no per-operator workspace to lend, or
// a plug-in that is only ever called from inside a region where cudaMalloc is not allowed (for
// example while the engine records its decode step).  For them the split-K scratch lives inside
// the library image itself, in the array below.  Every GPU that loads the library carries these
// 10 MiB until the process exits, which is why the size is kept to what decode-sized problems
// need: at most 64 rows of activations on a 148-SM part (the plan is 9.3 MiB there).
namespace iob {
namespace {

constexpr size_t kStaticScratchBytes = 10u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the symbol, not a device address, so the
// address each device gave the array is looked up once (with that device current) and kept.
int StaticScratchAddress(void** out) {
  static std::mutex mutex;
  static void* address[64] = {};
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    return Fail(IOB_CUDA_ERROR, "marlin_gemm_static_scratch: cannot identify the current device");
  }
  std::lock_guard<std::mutex> lock(mutex);
  if (address[device] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      return Fail(IOB_CUDA_ERROR, "marlin_gemm_static_scratch: cudaGetSymbolAddress failed: %s",
                  cudaGetErrorString(err));
    }
    address[device] = ptr;
  }
  *out = address[device];
  return IOB_OK;
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_marlin_gemm_static_scratch(const void* a, int a_dtype, const int32_t* b_q_weight,
                                                         const void* b_bias, const void* b_scales,
                                                         const int32_t* b_zeros, int64_t b_type_id, int64_t size_m,
                                                         int64_t size_n, int64_t size_k, int64_t num_groups,
                                                         void* out, void* stream) {
  using namespace iob;
  const size_t need = infiniops_b200_marlin_gemm_scratch_bytes(size_m, size_n, size_k);
  if (size_m <= 0 || need > kStaticScratchBytes) {
    return Fail(IOB_SCRATCH_TOO_SMALL,
                "marlin_gemm_static_scratch: a problem with %lld rows needs %zu bytes of scratch but the built-in "
                "buffer holds %zu (about 64 rows); call infiniops_b200_marlin_gemm with a buffer of your own",
                static_cast<long long>(size_m), need, kStaticScratchBytes);
  }
  void* scratch = nullptr;
  if (const int rc = StaticScratchAddress(&scratch)) return rc;
  // All calls share the buffer and find what the previous one left.  The arrival counters must
  // start at zero: a completed call leaves them so, but one that gave up on a wait may not, so
  // they are cleared on the stream first (a memset node, not an allocation).  The partial sums
  // are written before they are read and need no clearing.
  if (cudaMemsetAsync(static_cast<unsigned char*>(scratch) + kHeaderBytes, 0, 4 * kMaxGrid * sizeof(int),
                      static_cast<cudaStream_t>(stream)) != cudaSuccess) {
    return Fail(IOB_CUDA_ERROR, "marlin_gemm_static_scratch: clearing the counters failed");
  }
  return infiniops_b200_marlin_gemm(a, a_dtype, b_q_weight, b_bias, b_scales, b_zeros, b_type_id, size_m, size_n,
                                    size_k, num_groups, out, scratch, kStaticScratchBytes, stream);
}

extern "C" int infiniops_b200_static_scratch_status(void* stream) {
  using namespace iob;
  void* scratch = nullptr;
  if (StaticScratchAddress(&scratch) != IOB_OK) return -1;
  auto s = static_cast<cudaStream_t>(stream);
  int code = 0;
  // read the word, then clear the header (status and the blocked-warp notes) behind it on the same stream
  if (cudaMemcpyAsync(&code, scratch, sizeof(int), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
      cudaMemsetAsync(scratch, 0, kHeaderBytes, s) != cudaSuccess || cudaStreamSynchronize(s) != cudaSuccess) {
    return -1;
  }
  return code;
}
