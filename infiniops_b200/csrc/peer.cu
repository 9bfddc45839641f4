// Peer memory between the processes of one machine (one process per GPU): allocation, handle
// export / import, and the bounded wait for the completion flags that GEMM launches on other GPUs
// publish after storing their output slices into this GPU's buffers.
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

}  // namespace
}  // namespace iob

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
