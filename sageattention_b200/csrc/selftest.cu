// Self-test of the bounded-wait reporting path shared by every kernel of this library.
//
// The production kernels never spin forever: a wait on an mbarrier gives up after a probe budget,
// records KSTAT_WAIT_TIMEOUT | site in a CTA-shared word, every other role of the CTA then leaves
// its loops, and thread 0 publishes the word through the `status` pointer.  This file runs exactly
// that sequence on a barrier nobody ever completes -- no TMA copy, MMA or other asynchronous work
// is in flight, nothing traps, and the kernel returns by itself within microseconds -- so a host
// test can check that an expired wait really shows up in the status word and that the context stays
// usable afterwards.
#include "common/abi.cuh"
#include "common/sm100.cuh"

namespace nvfp4 {

__global__ void __launch_bounds__(128) selftest_wait_kernel(int site, uint32_t spins, int* status) {
  __shared__ uint64_t never;     // initialised for one arrival that no thread performs
  __shared__ int err;
  const int tid = threadIdx.x;
  if (tid == 0) {
    err = 0;
    mbar_init(&never, 1);
    mbar_fence_init();
  }
  __syncthreads();
  if (tid == 32) {
    // the role that times out
    mbar_wait_n(&never, 0, &err, site, spins);
  } else if (tid == 64) {
    // a second role waiting on the same barrier with a far larger budget: it must leave early
    // because the first one raised the CTA's error word
    mbar_wait_n(&never, 0, &err, site + 1, spins << 12);
  }
  __syncthreads();
  if (tid == 0 && err != 0 && status != nullptr) atomicExch(status, err);
}

}  // namespace nvfp4

extern "C" int nvfp4_selftest_wait_timeout(int site, unsigned spins, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(status != nullptr, "nvfp4_selftest_wait_timeout: status must not be NULL");
  NVFP4_REQUIRE(site >= 0 && site < 255, "nvfp4_selftest_wait_timeout: site must be in [0, 255)");
  NVFP4_REQUIRE(spins >= 1 && spins <= 4096, "nvfp4_selftest_wait_timeout: spins must be in [1, 4096]");
  selftest_wait_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(site, spins, status);
  return launch_result("nvfp4_selftest_wait_timeout");
}
