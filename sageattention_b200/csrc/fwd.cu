// Forward flash-attention kernel (placeholder while the kernel is being written).
#include "common/abi.cuh"
extern "C" size_t nvfp4_fwd_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int64_t, int) { return 0; }
extern "C" int nvfp4_fwd(const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*, const uint8_t*,
                         const uint8_t*, const float*, const int32_t*, const int32_t*, void*, int, int64_t,
                         int64_t, int64_t, float*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int,
                         float, int, void*, size_t, int*, nvfp4_stream_t) {
  return nvfp4::fail(-1, "nvfp4_fwd: kernel not built yet");
}
