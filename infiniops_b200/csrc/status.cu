// Thread-local error text behind infiniops_b200_last_error().
#include <cstdarg>
#include <cstdio>
#include <unordered_map>

#include "common.cuh"

namespace iob {

static thread_local char g_last_error[512] = "";

int Fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_last_error, sizeof(g_last_error), fmt, args);
  va_end(args);
  return code;
}

}  // namespace iob

extern "C" const char* infiniops_b200_last_error(void) { return iob::g_last_error; }

extern "C" const char* infiniops_b200_version(void) { return "infiniops_b200 0.1 (sm_100a)"; }

// ---- small runtime helpers for hosts that do not link the CUDA runtime themselves ------------------

extern "C" int infiniops_b200_swap_device(int device, int* previous) {
  int current = 0;
  if (cudaGetDevice(&current) != cudaSuccess) return iob::Fail(IOB_CUDA_ERROR, "cudaGetDevice failed");
  if (previous != nullptr) *previous = current;
  if (device >= 0 && device != current && cudaSetDevice(device) != cudaSuccess) {
    return iob::Fail(IOB_CUDA_ERROR, "cudaSetDevice(%d) failed", device);
  }
  return IOB_OK;
}

extern "C" void* infiniops_b200_thread_scratch(int purpose, size_t bytes, void* stream) {
  struct Buffer {
    void* ptr = nullptr;
    size_t size = 0;
  };
  // One buffer per (calling thread, device, purpose, stream): two calls that can overlap on the GPU
  // (same thread, different streams) never share split-K counters or partial sums.
  static thread_local std::unordered_map<void*, Buffer> buffers[64][2];
  int device = 0;
  if (purpose < 0 || purpose > 1 || cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) {
    iob::Fail(IOB_INVALID_ARGUMENT, "thread_scratch: bad purpose or device");
    return nullptr;
  }
  Buffer& b = buffers[device][purpose][stream];
  if (b.size < bytes) {
    const size_t want = bytes < (size_t{1} << 20) ? (size_t{1} << 20) : bytes + bytes / 4;
    void* fresh = nullptr;
    if (cudaMalloc(&fresh, want) != cudaSuccess || cudaMemset(fresh, 0, want) != cudaSuccess) {
      iob::Fail(IOB_CUDA_ERROR, "thread_scratch: cannot allocate %zu bytes", want);
      return nullptr;
    }
    if (b.ptr != nullptr) cudaFree(b.ptr);  // synchronises the device: no kernel still uses the old buffer
    b.ptr = fresh;
    b.size = want;
  }
  return b.ptr;
}
