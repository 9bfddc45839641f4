// Expert-parallel MoE layer over peer-mapped memory (one process per GPU, NVLink).
//
// Rank r owns experts [r * E_r, (r + 1) * E_r).  Tokens stay with the rank that holds them; each
// of their top_k routes travels to the owner of its expert and the result travels back:
//
//   plan      one block: stable position of every route among the routes to the same owner
//   dispatch  one block per route: the token row is stored into the owner's arena (region of the
//             sending rank), with the route's local expert, weight and origin; the last block to
//             finish publishes the sender's epoch in every rank's flag array
//   wait      bounded wait for every other rank's epoch
//   unpack    received (expert, weight, origin) -> the id / weight / destination arrays of the
//             routed GEMMs; slots beyond a sender's count become id -1
//   experts   moe_align_block_size -> w13 GEMM (result kept in sorted order, stored as tiles) ->
//             silu_and_mul -> w2 GEMM (reads the sorted rows in place) whose epilogue stores each
//             result row into the arena of the rank the token came from and raises the epoch again
//   wait, moe_sum
//
// Nothing is read back by the host and no collective library is involved, so the whole layer can
// be recorded once and replayed.  Arena layout (identical on every rank):
//   rows    [world][capacity][hidden]  16-bit   received token rows, one region per sender
//   meta    [world][capacity] int4              (local expert, weight bits, origin route, 0)
//   count   [world] int (padded to 256 bytes)   routes received from each sender
//   routed  [capacity][hidden]         16-bit   results coming back, row = origin route
#include <algorithm>

#include "common.cuh"

namespace iob {
namespace {

constexpr int kMaxWorld = IOB_MAX_PEERS + 1;
constexpr unsigned kFull = 0xffffffffu;

size_t Align256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }

struct ArenaLayout {
  size_t rows, meta, count, routed, total;
};
ArenaLayout PlanArena(int world, int64_t capacity, int64_t hidden) {
  ArenaLayout a;
  a.rows = 0;
  a.meta = Align256(a.rows + static_cast<size_t>(world) * capacity * hidden * 2);
  a.count = Align256(a.meta + static_cast<size_t>(world) * capacity * sizeof(int4));
  a.routed = Align256(a.count + 256);
  a.total = Align256(a.routed + static_cast<size_t>(capacity) * hidden * 2);
  return a;
}

struct PeerSet {
  unsigned char* arena[kMaxWorld];
  int* flags[kMaxWorld];
};

// Last-block-done completion signal (same protocol as the GEMM kernels): every block fences its
// stores system-wide and counts itself; the last one bumps the epoch and publishes it.
__device__ __forceinline__ void SignalWhenGridDone(int* ctrl, const PeerSet& peers, int world, int rank) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    int arrived;
    asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(ctrl) : "memory");
    if (arrived == static_cast<int>(gridDim.x) - 1) {
      ctrl[0] = 0;
      const int epoch = ctrl[1] + 1;
      ctrl[1] = epoch;
      __threadfence_system();
      for (int g = 0; g < world; ++g) {
        if (g != rank) asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(peers.flags[g] + rank), "r"(epoch) : "memory");
      }
    }
  }
}

// Position of every route among the routes of this rank that go to the same owner, in route
// order (stable: no atomics on the ordering path), and the number of routes per owner.
// One block of 1024 threads; routes with an expert id outside [0, world * experts_per_rank) get -1.
__global__ void __launch_bounds__(1024) EpPlanKernel(const int32_t* __restrict__ topk_ids, int routes,
                                                     int experts_per_rank, int world, int32_t* __restrict__ pos,
                                                     int32_t* __restrict__ send_count) {
  __shared__ int warp_count[32][kMaxWorld];
  __shared__ int base[kMaxWorld];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kMaxWorld) base[tid] = 0;
  for (int start = 0; start < routes; start += 1024) {
    if (tid < 32 * kMaxWorld) (&warp_count[0][0])[tid] = 0;
    __syncthreads();
    const int i = start + tid;
    int owner = -1;
    if (i < routes) {
      const int e = topk_ids[i];
      if (e >= 0 && e < world * experts_per_rank) owner = e / experts_per_rank;
    }
    const unsigned same = __match_any_sync(kFull, owner);
    const int rank_in_warp = __popc(same & ((1u << lane) - 1u));
    if (owner >= 0 && rank_in_warp == 0) warp_count[warp][owner] = __popc(same);
    __syncthreads();
    if (i < routes) {
      int before = 0;
      if (owner >= 0) {
        for (int w = 0; w < warp; ++w) before += warp_count[w][owner];
        before += base[owner] + rank_in_warp;
      }
      pos[i] = owner >= 0 ? before : -1;
    }
    __syncthreads();
    if (tid < world) {
      int total = 0;
      for (int w = 0; w < 32; ++w) total += warp_count[w][tid];
      base[tid] += total;
    }
    __syncthreads();
  }
  if (tid < world) send_count[tid] = base[tid];
}

// One block per route (grid-stride): copies the token row into the owner's arena and writes the
// route's metadata; block 0 also delivers this rank's counts.  Routes without an owner leave a
// zero row in this rank's own `routed` buffer so that the final sum sees nothing from them.
template <typename T>
__global__ void __launch_bounds__(256) EpDispatchKernel(const T* __restrict__ x, const int32_t* __restrict__ topk_ids,
                                                        const float* __restrict__ topk_weights,
                                                        const int32_t* __restrict__ pos,
                                                        const int32_t* __restrict__ send_count, int routes, int top_k,
                                                        int hidden, int experts_per_rank, int capacity, int world,
                                                        int rank, ArenaLayout lay, PeerSet peers, int* ctrl) {
  const int vec = hidden / 8;
  for (int i = blockIdx.x; i < routes; i += gridDim.x) {
    const int p = pos[i];
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(i / top_k) * hidden);
    if (p < 0) {
      uint4* dst = reinterpret_cast<uint4*>(peers.arena[rank] + lay.routed) + static_cast<size_t>(i) * vec;
      for (int v = threadIdx.x; v < vec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const int e = topk_ids[i];
    const int owner = e / experts_per_rank;
    const size_t slot = static_cast<size_t>(rank) * capacity + p;
    uint4* dst = reinterpret_cast<uint4*>(peers.arena[owner] + lay.rows) + slot * vec;
    for (int v = threadIdx.x; v < vec; v += blockDim.x) dst[v] = src[v];
    if (threadIdx.x == 0) {
      reinterpret_cast<int4*>(peers.arena[owner] + lay.meta)[slot] =
          make_int4(e - owner * experts_per_rank, __float_as_int(topk_weights[i]), i, 0);
    }
  }
  if (blockIdx.x == 0 && static_cast<int>(threadIdx.x) < world) {
    reinterpret_cast<int*>(peers.arena[threadIdx.x] + lay.count)[rank] = send_count[threadIdx.x];
  }
  SignalWhenGridDone(ctrl, peers, world, rank);
}

// Received metadata -> the arrays the routed GEMMs take: expert id per row (-1 for unused slots),
// routing weight per row, and (rank, row) the result row goes back to.
__global__ void EpUnpackKernel(const unsigned char* arena, ArenaLayout lay, int world, int capacity, int32_t* ids,
                               float* weights, int2* row_dest) {
  const int total = world * capacity;
  const int* count = reinterpret_cast<const int*>(arena + lay.count);
  const int4* meta = reinterpret_cast<const int4*>(arena + lay.meta);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
    const int sender = i / capacity, p = i - sender * capacity;
    if (p < count[sender]) {
      const int4 m = meta[i];
      ids[i] = m.x;
      weights[i] = __int_as_float(m.y);
      row_dest[i] = make_int2(sender, m.z);
    } else {
      ids[i] = -1;
      weights[i] = 0.0f;
      row_dest[i] = make_int2(0, 0);
    }
  }
}

// Combine step for layers whose second GEMM stores tiles in sorted order (128- / 256-row routing
// blocks): every result row goes from the local [sorted, hidden] buffer to the arena of the rank its
// token came from, to the row its route has there -- 16-byte plain stores into peer-mapped memory --
// and the last block raises the completion flags.  One block per row at a time.
__global__ void __launch_bounds__(256) EpCombineKernel(const uint4* __restrict__ rows, const int32_t* __restrict__ sorted_ids,
                                                       const int32_t* __restrict__ num_post_pad,
                                                       const int2* __restrict__ row_dest, int live_rows, int vec_per_row,
                                                       PeerSet peers, size_t routed_off, int world, int rank, int* ctrl) {
  const int total = *num_post_pad;
  for (int row = blockIdx.x; row < total; row += gridDim.x) {
    const int id = sorted_ids[row];
    if (id >= live_rows) continue;
    const int2 dest = row_dest[id];
    const uint4* src = rows + static_cast<size_t>(row) * vec_per_row;
    uint4* dst = reinterpret_cast<uint4*>(peers.arena[dest.x] + routed_off) + static_cast<size_t>(dest.y) * vec_per_row;
    for (int i = threadIdx.x; i < vec_per_row; i += blockDim.x) dst[i] = src[i];
  }
  if (world > 1) SignalWhenGridDone(ctrl, peers, world, rank);
}

struct Workspace {
  size_t pos, send_count, ids, weights, row_dest, sorted, experts, npost, live, g, h, gemm, align, total;
  size_t gemm_bytes, align_bytes;
  int64_t rows, sorted_size, blocks;
};
Workspace PlanWorkspace(const iob_ep_context& c) {
  Workspace w{};
  w.rows = static_cast<int64_t>(c.world) * c.capacity;
  w.sorted_size = w.rows + c.experts_per_rank * (c.moe_block_size - 1);
  if (w.rows < c.experts_per_rank) w.sorted_size = std::min(w.sorted_size, w.rows * c.moe_block_size);
  w.blocks = (w.sorted_size + c.moe_block_size - 1) / c.moe_block_size;
  size_t at = 0;
  auto take = [&](size_t bytes) {
    const size_t here = at;
    at = Align256(at + bytes);
    return here;
  };
  w.pos = take(static_cast<size_t>(c.capacity) * 4);
  w.send_count = take(kMaxWorld * 4);
  w.ids = take(static_cast<size_t>(w.rows) * 4);
  w.weights = take(static_cast<size_t>(w.rows) * 4);
  w.row_dest = take(static_cast<size_t>(w.rows) * 8);
  w.sorted = take(static_cast<size_t>(w.sorted_size) * 4);
  w.experts = take(static_cast<size_t>(w.blocks) * 4);
  w.npost = take(4);
  // the intermediates stay in sorted (expert) order: one row per position of the sorted id list
  w.live = take(static_cast<size_t>(w.blocks + 1) * sizeof(int32_t));
  // (also holds the second GEMM's [sorted, hidden] result when that is stored as tiles: see the combine step)
  w.g = take(static_cast<size_t>(w.sorted_size) * std::max<int64_t>(2 * c.inter, c.hidden) * 2);
  w.h = take(static_cast<size_t>(w.sorted_size) * c.inter * 2);
  w.gemm_bytes = std::max(
      infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(w.rows, 1, 2 * c.inter, c.hidden, c.experts_per_rank, c.moe_block_size),
      infiniops_b200_moe_wna16_marlin_gemm_scratch_bytes(w.rows, 1, c.hidden, c.inter, c.experts_per_rank, c.moe_block_size));
  w.gemm = take(w.gemm_bytes);
  w.align_bytes = infiniops_b200_moe_align_block_size_scratch_bytes(w.rows, c.experts_per_rank);
  w.align = take(w.align_bytes);
  w.total = at;
  return w;
}

int CheckContext(const iob_ep_context* c) {
  IOB_REQUIRE(c != nullptr, "ep: null context");
  IOB_REQUIRE(c->world >= 1 && c->world <= kMaxWorld && c->rank >= 0 && c->rank < c->world, "ep: bad world / rank");
  IOB_REQUIRE(c->top_k > 0 && c->hidden > 0 && c->hidden % 128 == 0 && c->inter > 0 && c->inter % 128 == 0 &&
                  c->experts_per_rank > 0 && c->capacity > 0,
              "ep: bad geometry (hidden and inter must be multiples of 128)");
  IOB_REQUIRE(c->a_dtype == IOB_F16 || c->a_dtype == IOB_BF16, "ep: float16 or bfloat16 activations");
  IOB_REQUIRE(c->ctrl != nullptr, "ep: null control block");
  for (int g = 0; g < c->world; ++g) {
    IOB_REQUIRE(c->arena[g] != nullptr && c->flags[g] != nullptr, "ep: rank %d's arena or flags are not mapped", g);
  }
  return IOB_OK;
}

}  // namespace
}  // namespace iob

extern "C" size_t infiniops_b200_ep_arena_bytes(int world, int64_t capacity, int64_t hidden) {
  return iob::PlanArena(world, capacity, hidden).total;
}

extern "C" size_t infiniops_b200_ep_workspace_bytes(const iob_ep_context* ctx) {
  if (iob::CheckContext(ctx) != IOB_OK) return 0;
  return iob::PlanWorkspace(*ctx).total;
}

extern "C" int infiniops_b200_ep_moe_layer(const iob_ep_context* ctx, const iob_expert_weights* weights, const void* x,
                                           const int32_t* topk_ids, const float* topk_weights, int64_t tokens,
                                           void* out, void* workspace, size_t workspace_bytes, void* stream) {
  using namespace iob;
  if (const int rc = CheckContext(ctx)) return rc;
  const iob_ep_context& c = *ctx;
  IOB_REQUIRE(weights != nullptr && x != nullptr && topk_ids != nullptr && topk_weights != nullptr && out != nullptr,
              "ep_moe_layer: null argument");
  const int64_t routes = tokens * c.top_k;
  IOB_REQUIRE(tokens > 0 && routes <= c.capacity, "ep_moe_layer: %lld routes exceed the context's capacity of %lld",
              static_cast<long long>(routes), static_cast<long long>(c.capacity));
  const Workspace w = PlanWorkspace(c);
  IOB_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, "ep_moe_layer: needs %zu bytes of workspace, got %zu",
              w.total, workspace_bytes);
  auto s = static_cast<cudaStream_t>(stream);
  auto* ws = static_cast<unsigned char*>(workspace);
  const ArenaLayout lay = PlanArena(c.world, c.capacity, c.hidden);
  PeerSet peers{};
  for (int g = 0; g < c.world; ++g) {
    peers.arena[g] = static_cast<unsigned char*>(c.arena[g]);
    peers.flags[g] = c.flags[g];
  }
  auto* pos = reinterpret_cast<int32_t*>(ws + w.pos);
  auto* send_count = reinterpret_cast<int32_t*>(ws + w.send_count);
  auto* ids = reinterpret_cast<int32_t*>(ws + w.ids);
  auto* row_weights = reinterpret_cast<float*>(ws + w.weights);
  auto* row_dest = reinterpret_cast<int2*>(ws + w.row_dest);
  auto* sorted = reinterpret_cast<int32_t*>(ws + w.sorted);
  auto* expert_ids = reinterpret_cast<int32_t*>(ws + w.experts);
  auto* npost = reinterpret_cast<int32_t*>(ws + w.npost);
  unsigned char* own = peers.arena[c.rank];

  // the GEMMs count split-K arrivals in their scratch: it must start zeroed whatever the workspace held
  if (const int rc = infiniops_b200_gemm_scratch_prepare(ws + w.gemm, w.gemm_bytes, stream)) return rc;
  // ---- dispatch ---------------------------------------------------------------------------------
  EpPlanKernel<<<1, 1024, 0, s>>>(topk_ids, static_cast<int>(routes), static_cast<int>(c.experts_per_rank), c.world, pos,
                                  send_count);
  if (const int rc = CheckLaunch("ep plan launch")) return rc;
  const int dispatch_grid = static_cast<int>(std::min<int64_t>(routes, 8 * NumSms()));
  if (c.a_dtype == IOB_BF16) {
    EpDispatchKernel<__nv_bfloat16><<<dispatch_grid, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), topk_ids, topk_weights, pos, send_count, static_cast<int>(routes),
        static_cast<int>(c.top_k), static_cast<int>(c.hidden), static_cast<int>(c.experts_per_rank),
        static_cast<int>(c.capacity), c.world, c.rank, lay, peers, c.ctrl);
  } else {
    EpDispatchKernel<__half><<<dispatch_grid, 256, 0, s>>>(
        static_cast<const __half*>(x), topk_ids, topk_weights, pos, send_count, static_cast<int>(routes),
        static_cast<int>(c.top_k), static_cast<int>(c.hidden), static_cast<int>(c.experts_per_rank),
        static_cast<int>(c.capacity), c.world, c.rank, lay, peers, c.ctrl);
  }
  if (const int rc = CheckLaunch("ep dispatch launch")) return rc;
  if (c.world > 1) {
    if (const int rc = infiniops_b200_peer_wait(c.flags[c.rank], c.world, c.rank, c.ctrl + 2, c.ctrl + 3, stream)) return rc;
  }

  // ---- this rank's experts on what it received -----------------------------------------------------
  EpUnpackKernel<<<static_cast<int>(std::min<int64_t>((w.rows + 255) / 256, 4 * NumSms())), 256, 0, s>>>(
      own, lay, c.world, static_cast<int>(c.capacity), ids, row_weights, row_dest);
  if (const int rc = CheckLaunch("ep unpack launch")) return rc;
  if (const int rc = infiniops_b200_moe_align_block_size(ids, nullptr, w.rows, c.experts_per_rank, c.moe_block_size, sorted,
                                                         w.sorted_size, expert_ids, w.blocks, npost,
                                                         w.align_bytes ? ws + w.align : nullptr, w.align_bytes, stream)) {
    return rc;
  }
  auto* live = reinterpret_cast<int32_t*>(ws + w.live);  // live rows per routing block, noted by the first GEMM's gather
  iob_routed_options first{};
  first.out_sorted = 1;
  first.block_rows = live;
  const bool fused = weights->w13_interleaved != 0 && (2 * c.inter) % 128 == 0;
  first.fuse_silu = fused ? 1 : 0;
  if (const int rc = infiniops_b200_moe_wna16_marlin_gemm_ex(
          own + lay.rows, c.a_dtype, weights->w13, nullptr, weights->s13, weights->z13, sorted, expert_ids, npost,
          row_weights, c.moe_block_size, 1, 0, c.b_type_id, w.rows, 2 * c.inter, c.hidden, weights->groups13,
          c.experts_per_rank, w.sorted_size, fused ? ws + w.h : ws + w.g, &first, ws + w.gemm, w.gemm_bytes, stream)) {
    return rc;
  }
  if (!fused) {
    const int64_t shape[2] = {w.sorted_size, c.inter};
    const int64_t in_strides[2] = {2 * c.inter, 1}, out_strides[2] = {c.inter, 1};
    if (const int rc = infiniops_b200_silu_and_mul(ws + w.g, ws + w.h, c.a_dtype, 2, shape, in_strides, out_strides, stream)) {
      return rc;
    }
  }
  iob_peer_signal signal{};
  signal.done_counter = c.ctrl;
  signal.epoch = c.ctrl + 1;
  signal.flag_slot = c.rank;
  for (int g = 0; g < c.world; ++g) {
    if (g != c.rank) signal.peer_flags[signal.n_peers++] = c.flags[g];
  }
  if (c.moe_block_size >= 128) {
    // tile stores out of the second GEMM too (rows x routing weight, sorted order), then the combine copy
    iob_routed_options tiles{};
    tiles.a_sorted = 1;
    tiles.out_sorted = 1;
    tiles.block_rows = live;
    if (const int rc = infiniops_b200_moe_wna16_marlin_gemm_ex(
            ws + w.h, c.a_dtype, weights->w2, nullptr, weights->s2, weights->z2, sorted, expert_ids, npost, row_weights,
            c.moe_block_size, 1, 1, c.b_type_id, w.rows, c.hidden, c.inter, weights->groups2, c.experts_per_rank,
            w.sorted_size, ws + w.g, &tiles, ws + w.gemm, w.gemm_bytes, stream)) {
      return rc;
    }
    const int vec_per_row = static_cast<int>(c.hidden * 2 / 16);
    EpCombineKernel<<<static_cast<int>(std::min<int64_t>(w.sorted_size, 8 * NumSms())), 256, 0, s>>>(
        reinterpret_cast<const uint4*>(ws + w.g), sorted, npost, row_dest, static_cast<int>(w.rows), vec_per_row, peers,
        lay.routed, c.world, c.rank, c.ctrl);
    if (const int rc = CheckLaunch("ep combine launch")) return rc;
    if (c.world > 1) {
      if (const int rc = infiniops_b200_peer_wait(c.flags[c.rank], c.world, c.rank, c.ctrl + 2, c.ctrl + 3, stream)) return rc;
    }
    return infiniops_b200_moe_sum(own + lay.routed, c.a_dtype, tokens, c.top_k, c.hidden, c.top_k * c.hidden, c.hidden, 1,
                                  nullptr, IOB_I32, 0, 0, nullptr, 0, 0, out, stream);
  }
  iob_routed_options scatter{};
  scatter.row_dest = reinterpret_cast<const int32_t*>(row_dest);
  scatter.n_dest = c.world;
  for (int g = 0; g < c.world; ++g) scatter.dest_base[g] = peers.arena[g] + lay.routed;
  scatter.signal = c.world > 1 ? &signal : nullptr;
  scatter.a_sorted = 1;
  scatter.block_rows = live;
  if (const int rc = infiniops_b200_moe_wna16_marlin_gemm_ex(
          ws + w.h, c.a_dtype, weights->w2, nullptr, weights->s2, weights->z2, sorted, expert_ids, npost, row_weights,
          c.moe_block_size, 1, 1, c.b_type_id, w.rows, c.hidden, c.inter, weights->groups2, c.experts_per_rank,
          w.sorted_size, ws + w.g /* validated only */, &scatter, ws + w.gemm, w.gemm_bytes, stream)) {
    return rc;
  }
  if (c.world > 1) {
    if (const int rc = infiniops_b200_peer_wait(c.flags[c.rank], c.world, c.rank, c.ctrl + 2, c.ctrl + 3, stream)) return rc;
  }
  // ---- sum each token's top_k rows ------------------------------------------------------------------
  return infiniops_b200_moe_sum(own + lay.routed, c.a_dtype, tokens, c.top_k, c.hidden, c.top_k * c.hidden, c.hidden, 1,
                                nullptr, IOB_I32, 0, 0, nullptr, 0, 0, out, stream);
}
