// Measured pipe rates of the device the library runs on: the denominators its kernels are judged
// against.  One entry point runs a resident-operand micro-kernel on every SM and the caller times
// it with CUDA events:
//   what = 0   tcgen05.mma kind::mxf4nvf4 (NVFP4 x NVFP4, e4m3 scale per 16), M128 N128 K64
//   what = 1   tcgen05.mma kind::f16 (bf16 x bf16), M128 N128 K16
//   what = 2   ex2.approx.ftz.f32            (the softmax exponentials)
//   what = 3   cvt.rn.satfinite.e2m1x2.f32   (the P / gradient packs)
//   what = 4   fma.rn.f32
//   what = 5   one ex2 plus one e2m1x2 convert per slot (pipe sharing: counts slots, i.e. pairs)
//   what = 6   cvt.rn.satfinite.e4m3x2.f32;  7  cvt.rn.f16x2.e4m3x2
// Operands stay in shared memory / registers, so nothing but the pipe under test is exercised.
#include "common/abi.cuh"
#include "common/sm100.cuh"

namespace nvfp4 {

constexpr int kPeakIlp = 8;

__device__ __forceinline__ void peak_umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// One CTA per SM; one thread issues `iters` MMAs back to back into three accumulators in turn.
template <bool kFp4>
__global__ void __launch_bounds__(128, 1) peak_mma_kernel(int iters, int* status) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_a = smem;            // 128 rows x 64 B (FP4: K = 128 nibbles) / 128 rows x 128 B (bf16: K = 64)
  uint8_t* s_b = smem + 16384;
  uint8_t* s_sf = smem + 32768;   // one 512-byte scale atom, every scale = 1.0 (0x38)
  __shared__ uint64_t done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  const int tid = threadIdx.x, warp = tid >> 5;
  // operands: every FP4 code = 1.0 (0x2 -> byte 0x22), every bf16 = 1.0 (0x3F80)
  for (int i = tid; i < 32768 / 4; i += blockDim.x)
    reinterpret_cast<uint32_t*>(smem)[i] = kFp4 ? 0x22222222u : 0x3F803F80u;
  for (int i = tid; i < 512 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(s_sf)[i] = 0x38383838u;
  if (tid == 0) {
    err = 0;
    mbar_init(&done, 1);
    mbar_fence_init();
  }
  if (warp == 0) tmem_alloc(&tmem_base_s, 512);
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  if (warp == 1) {
    if (elect_one()) {
      if constexpr (kFp4) {
        const uint32_t sfa = tmem + 384, sfb = tmem + 388;
        tmem_cp_32x128b_warpx4(sfa, smem_u32(s_sf));
        tmem_cp_32x128b_warpx4(sfb, smem_u32(s_sf));
        const uint32_t idesc = make_idesc_nvfp4(128, 128);
        const uint64_t ad0 = make_smem_desc(smem_u32(s_a), 16, 512, 4), bd0 = make_smem_desc(smem_u32(s_b), 16, 512, 4);
        for (int i = 0; i < iters; ++i) {
          const uint32_t acc = tmem + (uint32_t)(i % 3) * 128;
          const uint64_t off = (uint64_t)((i & 1) * 2);          // the two K = 64 halves of the 64-byte rows
          umma_nvfp4(acc, ad0 + off, bd0 + off, idesc, sfa, sfb, i >= 3 ? 1u : 0u);
        }
      } else {
        uint32_t idesc = 0;
        idesc |= 1u << 4;           // fp32 accumulate
        idesc |= 1u << 7;           // A bf16
        idesc |= 1u << 10;          // B bf16
        idesc |= (128u >> 3) << 17;
        idesc |= (128u >> 4) << 24;
        const uint64_t ad0 = make_smem_desc(smem_u32(s_a), 16, 1024, 2), bd0 = make_smem_desc(smem_u32(s_b), 16, 1024, 2);
        for (int i = 0; i < iters; ++i) {
          const uint32_t acc = tmem + (uint32_t)(i % 3) * 128;
          const uint64_t off = (uint64_t)((i & 3) * 2);          // the four K = 16 slices of the 128-byte rows
          peak_umma_bf16(acc, ad0 + off, bd0 + off, idesc, i >= 3 ? 1u : 0u);
        }
      }
      umma_commit(&done);
      mbar_wait(&done, 0, &err, 1);
    }
    __syncwarp();
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && status != nullptr) atomicExch(status, err);
  if (warp == 0) tmem_dealloc(tmem, 512);
}

template <int kWhat>
__global__ void __launch_bounds__(256) peak_alu_kernel(int iters, float seed, float* sink) {
  float x[kPeakIlp];
  uint32_t u[kPeakIlp];
#pragma unroll
  for (int i = 0; i < kPeakIlp; ++i) {
    x[i] = seed + threadIdx.x * 1e-3f + i;
    u[i] = 0u;
  }
  for (int it = 0; it < iters; ++it) {
#pragma unroll
    for (int i = 0; i < kPeakIlp; ++i) {
      if constexpr (kWhat == 2) {
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(x[i]));
      } else if constexpr (kWhat == 3) {
        uint16_t b;
        asm volatile("{.reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t;}"
                     : "=h"(b)
                     : "f"(x[i]), "f"(x[(i + 1) % kPeakIlp]));
        u[i] += b;
      } else if constexpr (kWhat == 5) {
        // one ex2 and one e2m1x2 convert per slot: do the two share a pipe?
        asm volatile("ex2.approx.ftz.f32 %0, %0;" : "+f"(x[i]));
        uint16_t b;
        asm volatile("{.reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u16.u8 %0, t;}"
                     : "=h"(b)
                     : "f"(x[(i + 3) % kPeakIlp]), "f"(x[(i + 1) % kPeakIlp]));
        u[i] += b;
      } else if constexpr (kWhat == 6) {
        uint16_t b;
        asm volatile("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(b) : "f"(x[i]), "f"(x[(i + 1) % kPeakIlp]));
        u[i] += b;
      } else if constexpr (kWhat == 7) {
        uint32_t h2;
        asm volatile("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)u[i]));
        u[i] = h2;
      } else {
        asm volatile("fma.rn.f32 %0, %0, %1, %2;" : "+f"(x[i]) : "f"(1.0001f), "f"(0.5f));
      }
    }
  }
  float s = 0.0f;
#pragma unroll
  for (int i = 0; i < kPeakIlp; ++i) s += x[i] + __uint_as_float(u[i]);
  if (s == 123.456f) sink[0] = s;   // keeps the loop alive
}

}  // namespace nvfp4

extern "C" int nvfp4_peak_probe(int what, int iters, double* work_per_launch, float* sink, int* status,
                                nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(what >= 0 && what <= 7, "nvfp4_peak_probe: what must be 0..7");
  NVFP4_REQUIRE(iters >= 1 && iters <= (1 << 16), "nvfp4_peak_probe: iters must be in [1, 65536]");
  NVFP4_REQUIRE(sink != nullptr, "nvfp4_peak_probe: sink must not be NULL");
  int dev = 0, sms = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (sms <= 0) return fail(-1, "nvfp4_peak_probe: no CUDA device");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (what <= 1) {
    const int smem = 32768 + 512 + 1024;
    if (what == 0) {
      peak_mma_kernel<true><<<sms, 128, smem, st>>>(iters, status);
      if (work_per_launch) *work_per_launch = (double)sms * iters * 2.0 * 128 * 128 * 64;   // FLOP
    } else {
      peak_mma_kernel<false><<<sms, 128, smem, st>>>(iters, status);
      if (work_per_launch) *work_per_launch = (double)sms * iters * 2.0 * 128 * 128 * 16;
    }
    return launch_result("nvfp4_peak_probe(mma)");
  }
  const int blocks = sms * 8;
  if (what == 2) peak_alu_kernel<2><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  else if (what == 3) peak_alu_kernel<3><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  else if (what == 5) peak_alu_kernel<5><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  else if (what == 6) peak_alu_kernel<6><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  else if (what == 7) peak_alu_kernel<7><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  else peak_alu_kernel<4><<<blocks, 256, 0, st>>>(iters, 1.0f, sink);
  if (work_per_launch) *work_per_launch = (double)blocks * 256 * iters * kPeakIlp;            // thread-instructions
  return launch_result("nvfp4_peak_probe(alu)");
}
