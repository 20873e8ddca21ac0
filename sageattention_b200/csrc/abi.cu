// Library identification and the thread-local error text behind nvfp4_last_error().
#include "common/abi.cuh"

namespace nvfp4 {
char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}
}  // namespace nvfp4

extern "C" int nvfp4_abi_version(void) { return 1; }
extern "C" const char* nvfp4_last_error(void) { return nvfp4::last_error_buffer(); }
