// NVFP4 element arithmetic shared by every kernel that packs: IEEE fp32 scale computation, the
// e4m3 scale byte, the e2m1 convert.  Nothing here may be compiled with fast-math: packed bytes
// are compared bit for bit with an IEEE restatement (true divisions, round-to-nearest-even).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace nvfp4 {

constexpr float kScaleFloor = 0.001953125f;  // 2^-9, smallest positive e4m3 value
constexpr float kScaleMax = 448.0f;
constexpr float kF4Max = 6.0f;

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// e4m3 byte of clamp(amax / 6, 2^-9, 448), round-to-nearest-even.
__device__ __forceinline__ uint8_t scale_byte_from_amax(float amax) {
  float s = fminf(fmaxf(__fdiv_rn(amax, kF4Max), kScaleFloor), kScaleMax);
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(0.0f), "f"(s));
  return (uint8_t)(r & 0xFF);
}

// exact value of a (non-negative) e4m3 byte
__device__ __forceinline__ float e4m3_to_f32(uint8_t b) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"((uint16_t)b));
  return __half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF)));
}

// 8 fp32 -> 8 e2m1 codes in one 32-bit word, element 0 in the low nibble of byte 0.
__device__ __forceinline__ uint32_t e2m1x8(float x0, float x1, float x2, float x3, float x4,
                                           float x5, float x6, float x7) {
  uint32_t out;
  asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
      "mov.b32 %0, {b0, b1, b2, b3};\n\t}\n"
      : "=r"(out)
      : "f"(x0), "f"(x1), "f"(x2), "f"(x3), "f"(x4), "f"(x5), "f"(x6), "f"(x7));
  return out;
}

// ---- stochastic rounding (the fp4_legacy backward's gradient operands)
// 32 random bits for one quad of elements, a counter-based hash of (seed, a, b): the same
// (seed, position) always draws the same bits, different positions are decorrelated, and no state
// is kept anywhere.  Two multiply-xorshift rounds over both counters.
__device__ __forceinline__ uint32_t sr_bits(uint32_t seed, uint32_t a, uint32_t b) {
  uint32_t h = seed ^ (a * 0x9E3779B1u);
  h = (h ^ (h >> 15)) * 0x2C1B3C6Du;
  h += b * 0x85EBCA77u;
  h = (h ^ (h >> 12)) * 0x297A2D39u;
  h ^= h >> 15;
  h *= 0x9E3779B1u;
  h ^= h >> 16;
  return h;
}

// 4 fp32 -> 4 e2m1 codes, stochastically rounded by the hardware convert (each value goes to one
// of its two e2m1 neighbours with probability proportional to the distance to the other; exact
// values stay), element 0 in the low nibble.
__device__ __forceinline__ uint32_t e2m1x4_sr(float x0, float x1, float x2, float x3, uint32_t rbits) {
  uint16_t d;
  asm("cvt.rs.satfinite.e2m1x4.f32 %0, {%1, %2, %3, %4}, %5;"
      : "=h"(d)
      : "f"(x3), "f"(x2), "f"(x1), "f"(x0), "r"(rbits));
  return d;
}

// Correctly rounded x / sf from a correctly rounded reciprocal (one Markstein correction step):
// q = RN(x * inv), r = x - q * sf (exact in an FMA), result = RN(q + r * inv).  Three FMA-pipe
// instructions instead of the ~dozen of an IEEE divide.  |x| is clamped so the quotient cannot
// overflow (the clamp is far above 6 * sf, so the e2m1 code -- saturated -- is unchanged; it is
// only applied to groups whose amax could overflow), and the
// sign of x is restored so that -0.0 keeps its sign bit.
template <bool kClamp>
__device__ __forceinline__ float div_by_scale(float x, float sf, float inv) {
  const float xc = kClamp ? fminf(fmaxf(x, -1.0e30f), 1.0e30f) : x;
  const float q = xc * inv;
  const float r = fmaf(-q, sf, xc);
  return copysignf(fmaf(r, inv, q), x);
}

// Two quotients at once with packed fp32x2 instructions (each lane IEEE round-to-nearest, so the
// results are those of div_by_scale<false>): half the issue slots of the scalar form.
__device__ __forceinline__ float2 div2_by_scale(float2 x, float2 nsf, float2 inv) {
  const float2 q = __fmul2_rn(x, inv);
  const float2 r = __ffma2_rn(q, nsf, x);          // x - q * sf, exact
  const float2 y = __ffma2_rn(r, inv, q);
  return make_float2(copysignf(y.x, x.x), copysignf(y.y, x.y));
}

__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

// Pack one group of 16 fp32 values: returns the scale byte, writes 8 nibble bytes to lo/hi.
// Bit-exact with amax -> e4m3(clamp(amax / 6)) -> IEEE x / scale -> e2m1 RTNE.
__device__ __forceinline__ uint8_t pack_group16(const float (&x)[16], uint32_t& lo, uint32_t& hi) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; i += 2) amax = max3f(amax, fabsf(x[i]), fabsf(x[i + 1]));
  const uint8_t sb = scale_byte_from_amax(amax);
  const float sf = e4m3_to_f32(sb);
  const float inv = __frcp_rn(sf);
  float y[16];
  if (amax <= 1.0e30f) {   // the usual case: no quotient can overflow, skip the clamp
    const float2 nsf2 = make_float2(-sf, -sf), inv2 = make_float2(inv, inv);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
      const float2 q = div2_by_scale(make_float2(x[i], x[i + 1]), nsf2, inv2);
      y[i] = q.x;
      y[i + 1] = q.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) y[i] = div_by_scale<true>(x[i], sf, inv);
  }
  lo = e2m1x8(y[0], y[1], y[2], y[3], y[4], y[5], y[6], y[7]);
  hi = e2m1x8(y[8], y[9], y[10], y[11], y[12], y[13], y[14], y[15]);
  return sb;
}

// ---- MXFP8 (e4m3 values, one e8m0 power-of-two scale per 32): the gradient operands of the
// fp8_rownorm backward.  Scale exponent e = the smallest integer with amax / 2^e <= 448 (the exact
// form of ceil(log2(amax / 448)), flash.py:243-257), amax floored at 1e-30; stored as e + 127.
__device__ __forceinline__ uint8_t mx8_scale(float amax, float& inv) {
  const uint32_t b = __float_as_uint(fmaxf(amax, 1.0e-30f));
  const int k = (int)(b >> 23) - 127;                    // amax = m 2^k, 1 <= m < 2
  const int e = k - 8 + ((b & 0x7FFFFFu) > 0x600000u ? 1 : 0);   // 448 = 1.75 * 2^8
  inv = __uint_as_float((uint32_t)(127 - e) << 23);      // 2^-e, exact
  return (uint8_t)(e + 127);
}
// 4 fp32 -> 4 e4m3 bytes (RTNE, saturating), element 0 in the low byte
__device__ __forceinline__ uint32_t e4m3x4(float x0, float x1, float x2, float x3) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(x1), "f"(x0));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(x3), "f"(x2));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
// 32 values (two halves of 16) -> 8 words of e4m3 bytes; returns the e8m0 scale byte
__device__ __forceinline__ uint8_t pack_group32_mx8(const float* x0, const float* x1, uint32_t (&w)[8]) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fmaxf(fabsf(x0[i]), fabsf(x1[i])));
  float inv;
  const uint8_t sb = mx8_scale(amax, inv);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    w[i] = e4m3x4(x0[4 * i] * inv, x0[4 * i + 1] * inv, x0[4 * i + 2] * inv, x0[4 * i + 3] * inv);
    w[4 + i] = e4m3x4(x1[4 * i] * inv, x1[4 * i + 1] * inv, x1[4 * i + 2] * inv, x1[4 * i + 3] * inv);
  }
  return sb;
}

// pack_group16 with the e2m1 convert stochastically rounded (the scale byte is unchanged); the
// four quads of the group draw their bits from counters (ca, cb .. cb + 3).
__device__ __forceinline__ uint8_t pack_group16_sr(const float (&x)[16], uint32_t& lo, uint32_t& hi,
                                                   uint32_t seed, uint32_t ca, uint32_t cb) {
  float amax = 0.0f;
#pragma unroll
  for (int i = 0; i < 16; ++i) amax = fmaxf(amax, fabsf(x[i]));
  const uint8_t sb = scale_byte_from_amax(amax);
  const float sf = e4m3_to_f32(sb);
  const float inv = __frcp_rn(sf);
  uint32_t q[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    q[i] = e2m1x4_sr(div_by_scale<true>(x[4 * i], sf, inv), div_by_scale<true>(x[4 * i + 1], sf, inv),
                     div_by_scale<true>(x[4 * i + 2], sf, inv), div_by_scale<true>(x[4 * i + 3], sf, inv),
                     sr_bits(seed, ca, cb + i));
  lo = q[0] | (q[1] << 16);
  hi = q[2] | (q[3] << 16);
  return sb;
}

}  // namespace nvfp4
