// Peer memory between the processes of one machine (one process per GPU): allocation, handle
// export / import, and the bounded wait for the completion flags that GEMM launches on other GPUs
// publish after storing their output slices into this GPU's buffers.
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace iob {
namespace {

constexpr int kErrPeerWait = 8;
// Polls before the wait gives up: with the pause between polls this is on the order of a second.
constexpr unsigned kPeerPolls = 1u << 22;

__global__ void PeerWaitKernel(const int* flags, int n_slots, int skip_slot, int* wait_epoch, int* status) {
  __shared__ int target;
  if (threadIdx.x == 0) {
    target = *wait_epoch + 1;
    *wait_epoch = target;
  }
  __syncthreads();
  const int slot = static_cast<int>(threadIdx.x);
  if (slot < n_slots && slot != skip_slot) {
    const int want = target;
    bool seen = false;
    for (unsigned poll = 0; poll < kPeerPolls; ++poll) {
      int v;
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flags + slot) : "memory");
      if (v >= want) {
        seen = true;
        break;
      }
      __nanosleep(200);
    }
    if (!seen && atomicCAS(status, 0, kErrPeerWait) == 0) status[1] = slot;
  }
}

// Slice broadcast: copies rectangular slices of local matrices ([rows, row_bytes] at a row pitch) to
// the same place in the other GPUs' matrices with whole-warp 16-byte stores -- 512 contiguous bytes
// per warp instruction, where a GEMM epilogue storing its own tiles to the peers sends 64-byte pieces
// -- and raises the completion flags when the last block is done.
struct BroadcastTable {
  int count, n_peers;
  long long first_unit[IOB_MAX_COPIES + 1];  // 16-byte units before each copy
  iob_peer_copy copy[IOB_MAX_COPIES];
  int* done_counter;
  int* epoch;
  int n_flag_peers;
  int* peer_flags[IOB_MAX_PEERS];
  int flag_slot;
};

__global__ void __launch_bounds__(256) PeerBroadcastKernel(const __grid_constant__ BroadcastTable t) {
  const long long total = t.first_unit[t.count];
  const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
  int c = 0;
  for (long long u = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; u < total; u += stride) {
    while (u >= t.first_unit[c + 1]) ++c;
    const iob_peer_copy& cp = t.copy[c];
    const long long local = u - t.first_unit[c];
    const long long per_row = cp.row_bytes / 16;
    const long long row = local / per_row, col = local - row * per_row;
    const size_t at = static_cast<size_t>(row) * cp.pitch_bytes + static_cast<size_t>(col) * 16;
    const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const unsigned char*>(cp.src) + at);
    for (int r = 0; r < t.n_peers; ++r) {
      *reinterpret_cast<uint4*>(static_cast<unsigned char*>(cp.dst[r]) + at) = v;
    }
  }
  if (t.done_counter != nullptr) {
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence_system();
      int arrived;
      asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(arrived) : "l"(t.done_counter) : "memory");
      if (arrived == static_cast<int>(gridDim.x) - 1) {
        *t.done_counter = 0;
        const int epoch = *t.epoch + 1;
        *t.epoch = epoch;
        __threadfence_system();
        for (int r = 0; r < t.n_flag_peers; ++r) {
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(t.peer_flags[r] + t.flag_slot), "r"(epoch) : "memory");
        }
      }
    }
  }
}

}  // namespace
}  // namespace iob

extern "C" int infiniops_b200_peer_broadcast(const iob_peer_copy* copies, int count, int n_peers,
                                             const iob_peer_signal* signal, void* stream) {
  using namespace iob;
  IOB_REQUIRE(copies != nullptr && count > 0 && count <= IOB_MAX_COPIES, "peer_broadcast: between 1 and %d copies per call",
              IOB_MAX_COPIES);
  IOB_REQUIRE(n_peers >= 0 && n_peers <= IOB_MAX_PEERS, "peer_broadcast: at most %d peers", IOB_MAX_PEERS);
  BroadcastTable t{};
  t.count = count;
  t.n_peers = n_peers;
  long long units = 0;
  for (int i = 0; i < count; ++i) {
    const iob_peer_copy& c = copies[i];
    IOB_REQUIRE(c.src != nullptr && c.rows >= 0 && c.row_bytes >= 0 && c.row_bytes % 16 == 0 && c.pitch_bytes % 16 == 0 &&
                    c.pitch_bytes >= c.row_bytes && reinterpret_cast<uintptr_t>(c.src) % 16 == 0,
                "peer_broadcast: copy %d: rows of 16-byte multiples at 16-byte aligned addresses", i);
    for (int r = 0; r < n_peers; ++r) {
      IOB_REQUIRE(c.dst[r] != nullptr && reinterpret_cast<uintptr_t>(c.dst[r]) % 16 == 0,
                  "peer_broadcast: copy %d: null or misaligned destination %d", i, r);
    }
    t.first_unit[i] = units;
    t.copy[i] = c;
    units += c.rows * (c.row_bytes / 16);
  }
  t.first_unit[count] = units;
  if (signal != nullptr) {
    IOB_REQUIRE(signal->done_counter != nullptr && signal->epoch != nullptr && signal->n_peers >= 0 &&
                    signal->n_peers <= IOB_MAX_PEERS,
                "peer_broadcast: incomplete signal");
    t.done_counter = signal->done_counter;
    t.epoch = signal->epoch;
    t.n_flag_peers = signal->n_peers;
    t.flag_slot = signal->flag_slot;
    for (int r = 0; r < signal->n_peers; ++r) t.peer_flags[r] = signal->peer_flags[r];
  }
  int device = 0, sms = 148;
  if (cudaGetDevice(&device) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
  const long long want = (units + 255) / 256;
  const int grid = static_cast<int>(std::max<long long>(1, std::min<long long>(want, 4LL * sms)));
  PeerBroadcastKernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(t);
  return CheckLaunch("peer_broadcast launch");
}

extern "C" int infiniops_b200_peer_alloc(size_t bytes, void** ptr) {
  using namespace iob;
  IOB_REQUIRE(ptr != nullptr && bytes > 0, "peer_alloc: bad arguments");
  void* p = nullptr;
  cudaError_t err = cudaMalloc(&p, bytes);
  if (err == cudaSuccess) err = cudaMemset(p, 0, bytes);
  if (err != cudaSuccess) {
    if (p != nullptr) cudaFree(p);
    return Fail(IOB_CUDA_ERROR, "peer_alloc(%zu): %s", bytes, cudaGetErrorString(err));
  }
  *ptr = p;
  return IOB_OK;
}

extern "C" int infiniops_b200_peer_free(void* ptr) {
  using namespace iob;
  const cudaError_t err = cudaFree(ptr);
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "peer_free: %s", cudaGetErrorString(err));
  return IOB_OK;
}

extern "C" int infiniops_b200_peer_export(const void* ptr, unsigned char handle[64]) {
  using namespace iob;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  IOB_REQUIRE(ptr != nullptr && handle != nullptr, "peer_export: bad arguments");
  cudaIpcMemHandle_t h;
  const cudaError_t err = cudaIpcGetMemHandle(&h, const_cast<void*>(ptr));
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "peer_export: %s", cudaGetErrorString(err));
  memcpy(handle, &h, sizeof(h));
  return IOB_OK;
}

extern "C" int infiniops_b200_peer_open(const unsigned char handle[64], void** ptr) {
  using namespace iob;
  IOB_REQUIRE(ptr != nullptr && handle != nullptr, "peer_open: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  const cudaError_t err = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "peer_open: %s", cudaGetErrorString(err));
  *ptr = p;
  return IOB_OK;
}

extern "C" int infiniops_b200_peer_close(void* ptr) {
  using namespace iob;
  const cudaError_t err = cudaIpcCloseMemHandle(ptr);
  if (err != cudaSuccess) return Fail(IOB_CUDA_ERROR, "peer_close: %s", cudaGetErrorString(err));
  return IOB_OK;
}

extern "C" int infiniops_b200_peer_wait(const int* flags, int n_slots, int skip_slot, int* wait_epoch, int* status,
                                        void* stream) {
  using namespace iob;
  IOB_REQUIRE(flags != nullptr && wait_epoch != nullptr && status != nullptr && n_slots > 0 && n_slots <= 32,
              "peer_wait: bad arguments (at most 32 flag slots)");
  PeerWaitKernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, n_slots, skip_slot, wait_epoch, status);
  return CheckLaunch("peer_wait launch");
}
