// Small device helpers shared by the backward kernels (high-precision and all-FP4 gradient GEMMs).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <cstring>
#include "fp4.cuh"
#include "sm100.cuh"

namespace nvfp4 {

__device__ __forceinline__ float ex2_bwd(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// K-major bf16 tile, rows of 128 bytes (64 elements), 128-byte swizzle: the MMA that consumes the
// 16 elements starting at element k16*16 of every row.
__device__ __forceinline__ uint64_t desc_sw128(const void* tile, int k16) {
  return make_smem_desc(smem_u32(tile) + (k16 & 3) * 32, 16, 1024, 2);
}
// The same kind of tile read as an MN-major operand: the contraction runs over the rows (16 rows
// = 2 KB per MMA), the 128 output columns are two 64-element sub-tiles `sub_bytes` apart.
__device__ __forceinline__ uint64_t desc_sw128_mn(const void* tile, int k16, uint32_t sub_bytes) {
  return make_smem_desc(smem_u32(tile) + k16 * 2048, sub_bytes, 1024, 2);
}
__device__ __forceinline__ uint64_t desc_sw64(const void* tile, int k64) {
  return make_smem_desc(smem_u32(tile) + (k64 & 1) * 32, 16, 512, 4);
}
// Instruction descriptor of kind::f16 (fp32 accumulate): 16-bit operands, bf16 unless `f16`.
__host__ __device__ inline uint32_t make_idesc_bf16(uint32_t m, uint32_t n, bool b_mn_major, bool f16 = false) {
  uint32_t d = 0;
  d |= 1u << 4;   // accumulator: fp32
  if (!f16) d |= (1u << 7) | (1u << 10);  // A and B: bf16 (0 = f16)
  if (b_mn_major) d |= 1u << 16;
  d |= (n >> 3) << 17;
  d |= (m >> 4) << 24;
  return d;
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// same, A operand read from TMEM (128 lanes x 8 columns of packed bf16 pairs per K = 16)
__device__ __forceinline__ void umma_bf16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc,
                                             uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ uint32_t pack_bf16x2(float a, float b) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// eight consecutive elements, one 16-byte load (two for fp32) when the address allows it
template <typename T>
__device__ __forceinline__ void load8(const T* src, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      const uint4 raw = *reinterpret_cast<const uint4*>(src);
      const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int e = 0; e < 8; ++e) v[e] = to_f32<T>(t[e]);
      return;
    }
  } else {
    if ((reinterpret_cast<uintptr_t>(src) & 15) == 0) {
      const float4 a = *reinterpret_cast<const float4*>(src), c = *reinterpret_cast<const float4*>(src + 4);
      v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = c.x; v[5] = c.y; v[6] = c.z; v[7] = c.w;
      return;
    }
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = to_f32<T>(src[e]);
}

// 32 fp32 accumulator columns -> 32 contiguous gradient elements
template <typename TG>
__device__ __forceinline__ void store_row32(TG* dst, const uint32_t (&r)[32], float mul) {
  if constexpr (sizeof(TG) == 2) {
    uint32_t w[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
      const TG a0 = from_f32<TG>(__uint_as_float(r[2 * e]) * mul);
      const TG a1 = from_f32<TG>(__uint_as_float(r[2 * e + 1]) * mul);
      w[e] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a0)) |
             ((uint32_t)(*reinterpret_cast<const uint16_t*>(&a1)) << 16);
    }
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int e = 0; e < 4; ++e) d4[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
  } else {
    float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int e = 0; e < 8; ++e)
      d4[e] = make_float4(__uint_as_float(r[4 * e]) * mul, __uint_as_float(r[4 * e + 1]) * mul,
                          __uint_as_float(r[4 * e + 2]) * mul, __uint_as_float(r[4 * e + 3]) * mul);
  }
}
template <typename TG>
__device__ __forceinline__ void zero_row(TG* dst, int n) {
  for (int e = 0; e < n; ++e) dst[e] = from_f32<TG>(0.0f);
}


// Smallest power of two >= a for a positive normal a; 1 for zero, denormals and non-finite input.
// Dividing a tensor by it is exact, which is what makes it usable as a global pre-scale of packs.
__host__ __device__ __forceinline__ float pow2_ceil(float a) {
#ifdef __CUDA_ARCH__
  uint32_t u = __float_as_uint(a) & 0x7FFFFFFFu;
#else
  uint32_t u;
  memcpy(&u, &a, 4);
  u &= 0x7FFFFFFFu;
#endif
  if (u < 0x00800000u || u >= 0x7F800000u) return 1.0f;
  uint32_t e = u >> 23;
  if (u & 0x7FFFFFu) ++e;
  if (e > 254u) e = 254u;
  const uint32_t r = e << 23;
#ifdef __CUDA_ARCH__
  return __uint_as_float(r);
#else
  float f;
  memcpy(&f, &r, 4);
  return f;
#endif
}

}  // namespace nvfp4
