// Shared plumbing of the extern "C" entry points: thread-local error text and argument checks.
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include "../../../include/nvfp4_b200.h"

namespace nvfp4 {

char* last_error_buffer();  // thread-local, 512 bytes (defined in abi.cu)

inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

inline int launch_result(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
  return 0;
}

#define NVFP4_REQUIRE(cond, ...) \
  do {                           \
    if (!(cond)) return ::nvfp4::fail(-1, __VA_ARGS__); \
  } while (0)

}  // namespace nvfp4
