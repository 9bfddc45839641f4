// Thread-local error text behind infiniops_b200_last_error().
#include <cstdarg>
#include <cstdio>

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
