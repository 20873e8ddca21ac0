// NVFP4 packer: strided [B, R, K] -> nibbles [B, R, Kp/2] + e4m3 scales [B, R, Kp/16].
//
// HBM-bound byte work (2 B read + 0.5625 B written per bf16 element).  Two kernels:
//   * pack_rows_kernel  -- contraction axis contiguous (Q, K along D): one thread per 16-group,
//     two 128-bit loads, one 64-bit nibble store;
//   * pack_cols_kernel  -- contraction axis strided, rows contiguous (V -> V^T along keys): a
//     128-key x 64-row tile is read with 128-bit loads along the contiguous axis, transposed
//     through shared memory, and written back as 64-byte row segments.
// A scalar kernel covers any other stride combination.
#include "common/abi.cuh"
#include "common/fp4.cuh"

namespace nvfp4 {

template <typename T> struct Vec8;  // 8 elements
template <> struct Vec8<__nv_bfloat16> { uint4 v; };
template <> struct Vec8<__half> { uint4 v; };
template <> struct Vec8<float> { uint4 v[2]; };

template <typename T>
__device__ __forceinline__ void load8(const T* p, bool vec_ok, int valid, float (&o)[8]) {
  if (vec_ok && valid >= 8) {
    Vec8<T> t = *reinterpret_cast<const Vec8<T>*>(p);
    const T* e = reinterpret_cast<const T*>(&t);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = to_f32<T>(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (i < valid) ? to_f32<T>(p[i]) : 0.0f;
  }
}

// ---------------------------------------------------------------- contraction contiguous
// grid = (blocks over the R * ngroups groups of one batch entry, B); ngroups_log2 >= 0 when the
// group count per row is a power of two (the usual D/16), which keeps 64-bit divisions out of
// a kernel that is otherwise a few dozen instructions per thread.
template <typename T>
__global__ void __launch_bounds__(256) pack_rows_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t ngroups, int ngroups_log2,
    int64_t per_batch, int64_t sxb, int64_t sxr, uint8_t* __restrict__ nib, int64_t snb,
    int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr, int vec_in) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= per_batch) return;
  const int64_t b = blockIdx.y;
  int64_t g, r;
  if (ngroups_log2 >= 0) {
    g = gid & (ngroups - 1);
    r = gid >> ngroups_log2;
  } else {
    g = gid % ngroups;
    r = gid / ngroups;
  }
  const T* p = x + b * sxb + r * sxr + g * 16;
  const int64_t left = k_read - g * 16;
  const int valid = left >= 16 ? 16 : (left > 0 ? (int)left : 0);
  float v[16];
  {
    float a[8], c[8];
    load8<T>(p, vec_in, valid, a);
    load8<T>(p + 8, vec_in, valid - 8, c);
#pragma unroll
    for (int i = 0; i < 8; ++i) { v[i] = a[i]; v[8 + i] = c[i]; }
  }
  uint32_t lo, hi;
  const uint8_t sb = pack_group16(v, lo, hi);
  uint8_t* pn = nib + b * snb + r * snr + g * 8;
  if ((reinterpret_cast<uintptr_t>(pn) & 7) == 0) {
    *reinterpret_cast<uint2*>(pn) = make_uint2(lo, hi);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) { pn[i] = (lo >> (8 * i)) & 0xFF; pn[4 + i] = (hi >> (8 * i)) & 0xFF; }
  }
  sc[b * ssb + r * ssr + g] = sb;
}

// ---------------------------------------------------------------- rows contiguous (V^T)
constexpr int kColsKeys = 128;  // contraction extent of a tile
constexpr int kColsRows = 64;   // row (head-dim) extent of a tile

template <typename T>
__global__ void __launch_bounds__(256) pack_cols_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t k_pad, int64_t sxb, int64_t sxk,
    uint8_t* __restrict__ nib, int64_t snb, int64_t snr, uint8_t* __restrict__ sc, int64_t ssb,
    int64_t ssr, int vec_in) {
  __shared__ float tile[kColsKeys][kColsRows + 1];
  __shared__ __align__(16) uint8_t onib[kColsRows][kColsKeys / 2];
  __shared__ __align__(8) uint8_t osc[kColsRows][kColsKeys / 16];
  const int tid = threadIdx.x;
  const int64_t k0 = (int64_t)blockIdx.x * kColsKeys;
  const int64_t r0 = (int64_t)blockIdx.y * kColsRows;
  const int64_t b = blockIdx.z;
  const T* xb = x + b * sxb;
  // load: 8 threads x 8 elements cover 64 rows of one key; 32 keys per pass
#pragma unroll
  for (int pass = 0; pass < kColsKeys / 32; ++pass) {
    const int key = pass * 32 + (tid >> 3);
    const int rc = (tid & 7) * 8;
    float v[8];
    const int64_t kk = k0 + key;
    int valid = 0;
    if (kk < k_read) {
      const int64_t left = R - (r0 + rc);
      valid = left >= 8 ? 8 : (left > 0 ? (int)left : 0);
    }
    if (valid > 0) {
      load8<T>(xb + kk * sxk + r0 + rc, vec_in, valid, v);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.0f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) tile[key][rc + i] = v[i];
  }
  __syncthreads();
  // quantise: thread -> (row = tid % 64, groups tid / 64 and tid / 64 + 4)
#pragma unroll
  for (int it = 0; it < 2; ++it) {
    const int row = tid & 63;
    const int g = (tid >> 6) + it * 4;
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = tile[g * 16 + j][row];
    uint32_t lo, hi;
    const uint8_t sb = pack_group16(v, lo, hi);
    *reinterpret_cast<uint2*>(&onib[row][g * 8]) = make_uint2(lo, hi);
    osc[row][g] = sb;
  }
  __syncthreads();
  // store: groups of this tile that exist in the output
  const int64_t gleft = (k_pad - k0) / 16;
  const int ng = gleft >= 8 ? 8 : (int)gleft;
  {
    const int row = tid >> 2, chunk = tid & 3;  // 16-byte chunk = 2 groups
    if (r0 + row < R) {
      uint8_t* pn = nib + b * snb + (r0 + row) * snr + k0 / 2 + chunk * 16;
      const int gv = ng - chunk * 2;  // groups valid in this chunk
      if (gv >= 2 && (reinterpret_cast<uintptr_t>(pn) & 15) == 0) {
        *reinterpret_cast<uint4*>(pn) = *reinterpret_cast<const uint4*>(&onib[row][chunk * 16]);
      } else if (gv > 0) {
        const int nb = (gv >= 2 ? 2 : gv) * 8;
        for (int i = 0; i < nb; ++i) pn[i] = onib[row][chunk * 16 + i];
      }
    }
  }
  if (tid < kColsRows && r0 + tid < R) {
    uint8_t* ps = sc + b * ssb + (r0 + tid) * ssr + k0 / 16;
    if (ng == 8 && (reinterpret_cast<uintptr_t>(ps) & 7) == 0) {
      *reinterpret_cast<uint2*>(ps) = *reinterpret_cast<const uint2*>(&osc[tid][0]);
    } else {
      for (int i = 0; i < ng; ++i) ps[i] = osc[tid][i];
    }
  }
}

// ---------------------------------------------------------------- any strides (scalar)
template <typename T>
__global__ void __launch_bounds__(256) pack_generic_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t ngroups, int64_t total, int64_t sxb,
    int64_t sxr, int64_t sxk, uint8_t* __restrict__ nib, int64_t snb, int64_t snr,
    uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= total) return;
  const int64_t g = gid % ngroups;
  const int64_t row = gid / ngroups;
  const int64_t r = row % R, b = row / R;
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const int64_t k = g * 16 + i;
    v[i] = k < k_read ? to_f32<T>(x[b * sxb + r * sxr + k * sxk]) : 0.0f;
  }
  uint32_t lo, hi;
  const uint8_t sb = pack_group16(v, lo, hi);
  uint8_t* pn = nib + b * snb + r * snr + g * 8;
#pragma unroll
  for (int i = 0; i < 4; ++i) { pn[i] = (lo >> (8 * i)) & 0xFF; pn[4 + i] = (hi >> (8 * i)) & 0xFF; }
  sc[b * ssb + r * ssr + g] = sb;
}

template <typename T>
int pack_dispatch(const T* x, int64_t B, int64_t R, int64_t k_read, int64_t k_pad, int64_t sxb,
                  int64_t sxr, int64_t sxk, uint8_t* nib, int64_t snb, int64_t snr, uint8_t* sc,
                  int64_t ssb, int64_t ssr, cudaStream_t st) {
  const int64_t ngroups = k_pad / 16;
  const int64_t total = B * R * ngroups;
  if (total == 0) return 0;
  constexpr int64_t kVecElems = 16 / sizeof(T);  // elements per 16 bytes
  const bool base_ok = (reinterpret_cast<uintptr_t>(x) & 15) == 0;
  if (sxk == 1 && B < 65536) {
    const int vec = base_ok && sxb % kVecElems == 0 && sxr % kVecElems == 0;
    const int64_t per_batch = R * ngroups;
    const int64_t blocks = (per_batch + 255) / 256;
    NVFP4_REQUIRE(blocks < (1LL << 31), "nvfp4_pack: tensor too large");
    int lg = -1;
    if ((ngroups & (ngroups - 1)) == 0) { lg = 0; while ((1LL << lg) < ngroups) ++lg; }
    dim3 grid((unsigned)blocks, (unsigned)B);
    pack_rows_kernel<T><<<grid, 256, 0, st>>>(x, R, k_read, ngroups, lg, per_batch, sxb, sxr, nib, snb,
                                              snr, sc, ssb, ssr, vec);
    return launch_result("nvfp4_pack(rows)");
  }
  if (sxr == 1 && B < 65536 && (R + kColsRows - 1) / kColsRows < 65536) {
    const int vec = base_ok && sxb % kVecElems == 0 && sxk % kVecElems == 0;
    dim3 grid((unsigned)((k_pad + kColsKeys - 1) / kColsKeys),
              (unsigned)((R + kColsRows - 1) / kColsRows), (unsigned)B);
    pack_cols_kernel<T><<<grid, 256, 0, st>>>(x, R, k_read, k_pad, sxb, sxk, nib, snb, snr, sc,
                                              ssb, ssr, vec);
    return launch_result("nvfp4_pack(cols)");
  }
  const int64_t blocks = (total + 255) / 256;
  NVFP4_REQUIRE(blocks < (1LL << 31), "nvfp4_pack: tensor too large");
  pack_generic_kernel<T><<<(unsigned)blocks, 256, 0, st>>>(x, R, k_read, ngroups, total, sxb, sxr,
                                                         sxk, nib, snb, snr, sc, ssb, ssr);
  return launch_result("nvfp4_pack(generic)");
}

}  // namespace nvfp4

extern "C" int nvfp4_pack(const void* x, int dtype, int64_t B, int64_t R, int64_t k_read,
                          int64_t k_pad, int64_t sxb, int64_t sxr, int64_t sxk, uint8_t* nib,
                          int64_t snb, int64_t snr, uint8_t* sc, int64_t ssb, int64_t ssr,
                          nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(B >= 0 && R >= 0 && k_read >= 0, "nvfp4_pack: negative extent");
  NVFP4_REQUIRE(k_pad % 16 == 0, "nvfp4_pack: padded contraction dim must be a multiple of 16");
  NVFP4_REQUIRE(k_pad >= k_read, "nvfp4_pack: k_pad < k_read");
  if (B * R * k_pad == 0) return 0;
  NVFP4_REQUIRE(x && nib && sc, "nvfp4_pack: null pointer");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NVFP4_DT_BF16:
      return pack_dispatch<__nv_bfloat16>(static_cast<const __nv_bfloat16*>(x), B, R, k_read, k_pad,
                                          sxb, sxr, sxk, nib, snb, snr, sc, ssb, ssr, st);
    case NVFP4_DT_FP16:
      return pack_dispatch<__half>(static_cast<const __half*>(x), B, R, k_read, k_pad, sxb, sxr,
                                   sxk, nib, snb, snr, sc, ssb, ssr, st);
    case NVFP4_DT_FP32:
      return pack_dispatch<float>(static_cast<const float*>(x), B, R, k_read, k_pad, sxb, sxr, sxk,
                                  nib, snb, snr, sc, ssb, ssr, st);
    default:
      return fail(-1, "nvfp4_pack: unknown dtype %d", dtype);
  }
}
