// NVFP4 packer: strided [B, R, K] -> nibbles [B, R, Kp/2] + e4m3 scales [B, R, Kp/16].
//
// HBM-bound byte work (2 B read + 0.5625 B written per bf16 element).  Kernels:
//   * pack_rows_quad_kernel -- contraction axis contiguous (Q, K along D), rows 32-byte aligned:
//     a thread packs four 16-groups that lie 32 groups apart, one 256-bit load per group, so the
//     lanes of a warp read consecutive sectors and write consecutive nibble words and scale bytes;
//   * pack_rows_kernel  -- the same axis for rows that are only 16-byte aligned, unaligned or have a
//     tail: one thread per 16-group;
//   * pack_cols_kernel  -- contraction axis strided, rows contiguous (V -> V^T along keys): runs of
//     128-key x 64-row tiles are read with 128-bit loads along the contiguous axis, transposed
//     through shared memory (16-bit inputs stay as loaded), and written back as 64-byte row
//     segments; the dual variant also emits the pack along the contiguous axis from the same read;
//   * pack_qkv_kernel   -- Q, K along D and V^T in one flat-grid launch (the forward's pre-pack);
//   * pack_mx8_cols_kernel -- MXFP8 (e4m3 + e8m0 per 32) along the strided axis.
// A scalar kernel covers any other stride combination.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/bwd_util.cuh"

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
struct RowsArgs {
  const void* x;
  int64_t R, k_read, ngroups, per_batch, sxb, sxr;
  int ngroups_log2, vec_in;
  uint8_t* nib;
  int64_t snb, snr;
  uint8_t* sc;
  int64_t ssb, ssr;
};

// group `gid` of batch entry `b`
template <typename T>
__device__ __forceinline__ void pack_rows_group(
    const T* __restrict__ x, int64_t k_read, int64_t ngroups, int ngroups_log2,
    int64_t sxb, int64_t sxr, uint8_t* __restrict__ nib, int64_t snb,
    int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr, int vec_in, int64_t gid, int64_t b) {
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

// 32 bytes with one 256-bit load (sm_100): a lane reads a whole 32-byte sector, so a warp whose
// lanes read consecutive sectors asks L1 for every sector once.
__device__ __forceinline__ void ldg256(const void* p, uint32_t (&r)[8]) {
  asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "l"(p));
}

// Four 16-groups per thread, 32 groups apart: in each of the four rounds the lanes of a warp take
// consecutive groups, so loads (one or two 256-bit loads per lane), nibble stores (8 bytes per lane)
// and scale stores (1 byte per lane) of a round cover consecutive memory, and the four rounds' loads
// are all issued before the first group is packed.  Needs whole groups (no tail), 32-byte aligned
// rows and a power-of-two group count per row.  `first` = first group of this thread's warp.
template <typename T>
__device__ __forceinline__ void pack_rows_quad(const T* __restrict__ x, int ng_log2, int64_t per_batch,
                                               int64_t sxb, int64_t sxr, uint8_t* __restrict__ nib, int64_t snb,
                                               int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr,
                                               int64_t first, int64_t b) {
  constexpr int kW = 16 * sizeof(T) / 4;          // 32-bit words per group
  const int lane = threadIdx.x & 31;
  uint32_t raw[4][kW];
  int64_t r[4];
  int g[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int64_t gid = first + i * 32 + lane;
    const int64_t gc = gid < per_batch ? gid : per_batch - 1;    // the tail re-reads the last group
    r[i] = gc >> ng_log2;
    g[i] = (int)(gc - (r[i] << ng_log2));
    const T* p = x + b * sxb + r[i] * sxr + g[i] * 16;
#pragma unroll
    for (int j = 0; j < kW / 8; ++j)
      ldg256(reinterpret_cast<const uint32_t*>(p) + 8 * j, *reinterpret_cast<uint32_t(*)[8]>(&raw[i][8 * j]));
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float v[16];
    const T* e = reinterpret_cast<const T*>(raw[i]);
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = to_f32<T>(e[j]);
    uint32_t lo, hi;
    const uint8_t sb = pack_group16(v, lo, hi);
    if (first + i * 32 + lane < per_batch) {
      *reinterpret_cast<uint2*>(nib + b * snb + r[i] * snr + g[i] * 8) = make_uint2(lo, hi);
      sc[b * ssb + r[i] * ssr + g[i]] = sb;
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256) pack_rows_quad_kernel(
    const T* __restrict__ x, int ng_log2, int64_t per_batch, int64_t sxb, int64_t sxr,
    uint8_t* __restrict__ nib, int64_t snb, int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr) {
  const int64_t first = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * 128;
  if (first >= per_batch) return;
  pack_rows_quad<T>(x, ng_log2, per_batch, sxb, sxr, nib, snb, snr, sc, ssb, ssr, first, blockIdx.y);
}

template <typename T>
__global__ void __launch_bounds__(256) pack_rows_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t ngroups, int ngroups_log2,
    int64_t per_batch, int64_t sxb, int64_t sxr, uint8_t* __restrict__ nib, int64_t snb,
    int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr, int vec_in) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= per_batch) return;
  pack_rows_group<T>(x, k_read, ngroups, ngroups_log2, sxb, sxr, nib, snb, snr, sc, ssb, ssr, vec_in, gid,
                     blockIdx.y);
}

// ---------------------------------------------------------------- rotary embedding + pack
// x [B, R, D] with the position of row r = pos0 + r (or positions[r]); cos / sin [P, D/2] fp32.
// Half-split convention ("rotate_half"): y[i] = x[i] cos[i] - x[i + D/2] sin[i] for i < D/2,
// y[i] = x[i] cos[i - D/2] + x[i - D/2] sin[i - D/2] otherwise; computed in fp32, rounded once to
// the input dtype (what an unfused rotary kernel would have stored), then packed like pack_rows.
template <typename T>
__global__ void __launch_bounds__(256) rope_pack_rows_kernel(
    const T* __restrict__ x, int64_t R, int d, int ngroups_log2, int64_t per_batch, int64_t sxb,
    int64_t sxr, const float* __restrict__ cs, const float* __restrict__ sn,
    const int32_t* __restrict__ positions, int64_t pos0, uint8_t* __restrict__ nib, int64_t snb,
    int64_t snr, uint8_t* __restrict__ sc, int64_t ssb, int64_t ssr, int vec_in) {
  const int64_t gid = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gid >= per_batch) return;
  const int64_t b = blockIdx.y;
  const int ngroups = d >> 4, half = d >> 1;
  const int g = (int)(gid & (ngroups - 1));
  const int64_t r = gid >> ngroups_log2;
  const bool upper = g * 16 >= half;
  const int gp = upper ? g - (ngroups >> 1) : g + (ngroups >> 1);      // partner group
  const T* row = x + b * sxb + r * sxr;
  const int64_t pos = positions ? (int64_t)positions[r] : pos0 + r;
  const float* c = cs + pos * half + (upper ? gp : g) * 16;
  const float* s_ = sn + pos * half + (upper ? gp : g) * 16;
  float a[16], pa[16];
  {
    float t0[8], t1[8];
    load8<T>(row + g * 16, vec_in, 16, t0);
    load8<T>(row + g * 16 + 8, vec_in, 8, t1);
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = t0[i]; a[8 + i] = t1[i]; }
    load8<T>(row + gp * 16, vec_in, 16, t0);
    load8<T>(row + gp * 16 + 8, vec_in, 8, t1);
#pragma unroll
    for (int i = 0; i < 8; ++i) { pa[i] = t0[i]; pa[8 + i] = t1[i]; }
  }
  float v[16];
#pragma unroll
  for (int i = 0; i < 16; i += 4) {
    const float4 c4 = *reinterpret_cast<const float4*>(c + i), s4 = *reinterpret_cast<const float4*>(s_ + i);
    const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float rot = upper ? pa[i + e] : -pa[i + e];
      v[i + e] = to_f32<T>(from_f32<T>(__fmaf_rn(rot, ss[e], a[i + e] * cc[e])));
    }
  }
  uint32_t lo, hi;
  const uint8_t sb = pack_group16(v, lo, hi);
  *reinterpret_cast<uint2*>(nib + b * snb + r * snr + g * 8) = make_uint2(lo, hi);
  sc[b * ssb + r * ssr + g] = sb;
}

// ---------------------------------------------------------------- rows contiguous (V^T)
constexpr int kColsKeys = 128;  // contraction extent of a tile
constexpr int kColsRows = 64;   // row (head-dim) extent of a tile
constexpr int kColsRun = 4;     // consecutive key tiles one block walks (the next tile's loads fly under the pack)

// The input tile: fp32 inputs as floats (one padding column); 16-bit inputs as loaded, two rows per
// 32-bit word, 144-byte key rows (16-byte aligned, and a quarter warp's 16-byte accesses to
// consecutive keys fall on different banks).
template <int kElemBytes> struct ColsTile { float tile[kColsKeys][kColsRows + 1]; };
template <> struct ColsTile<2> { __align__(16) uint32_t raw[kColsKeys][kColsRows / 2 + 4]; };

template <typename T>
struct ColsSmem : ColsTile<sizeof(T)> {
  __align__(16) uint8_t onib[kColsRows][kColsKeys / 2 + 16];
  __align__(8) uint8_t osc[kColsRows][kColsKeys / 16];
};

// two 16-bit elements of one word -> fp32 (element 0 in the low half)
template <typename T> __device__ __forceinline__ void unpack2(uint32_t w, float& a, float& b);
template <> __device__ __forceinline__ void unpack2<__nv_bfloat16>(uint32_t w, float& a, float& b) {
  a = __uint_as_float(w << 16);
  b = __uint_as_float(w & 0xFFFF0000u);
}
template <> __device__ __forceinline__ void unpack2<__half>(uint32_t w, float& a, float& b) {
  const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w));
  a = f.x;
  b = f.y;
}
template <> __device__ __forceinline__ void unpack2<float>(uint32_t, float&, float&) {}

// `nt` consecutive 128-key x 64-row tiles (tile coordinates bx .. bx + nt - 1, by of batch entry b);
// for 16-bit inputs the global loads of the next tile are issued before the current one is packed.
// With kDual every tile also yields the pack along the contiguous axis (rows of 16 consecutive
// elements of each key):
// dnib [B, keys, R/2], dsc [B, keys, R/16], from the one read of x.  sr_flags (kDual only): bit 0
// rounds the contiguous-axis pack stochastically, bit 1 the strided-axis pack; the random bits of
// an element depend only on (seed, which pack, its position in x).
template <typename T, bool kDual>
__device__ __forceinline__ void pack_cols_tile(
    ColsSmem<T>& sm, const T* __restrict__ x, int64_t R, int64_t k_read, int64_t k_pad, int64_t sxb, int64_t sxk,
    uint8_t* __restrict__ nib, int64_t snb, int64_t snr, uint8_t* __restrict__ sc, int64_t ssb,
    int64_t ssr, int vec_in, int64_t bx, int nt, int64_t by, int64_t b, uint8_t* __restrict__ dnib, int64_t dnb,
    int64_t dnr, uint8_t* __restrict__ dsc, int64_t dsb, int64_t dsr, const float* __restrict__ prescale_amax,
    int sr_flags = 0, uint32_t seed = 0) {
  // exact division by a power of two (1 when no pre-scale is asked for)
  const float pre = (kDual && prescale_amax != nullptr) ? __frcp_rn(pow2_ceil(*prescale_amax)) : 1.0f;
  auto& onib = sm.onib;
  auto& osc = sm.osc;
  const int tid = threadIdx.x;
  const int64_t r0 = by * kColsRows;
  const T* xb = x + b * sxb;
  // 16-bit inputs: 8 threads x 8 elements cover 64 rows of one key, 32 keys per pass, kept in
  // registers as loaded until the shared tile is free
  uint4 wreg[kColsKeys / 32];
  auto load16 = [&](int64_t k0) {
    if (vec_in && k0 + kColsKeys <= k_read && r0 + kColsRows <= R) {
      // interior tile: four unconditional 16-byte loads, all in flight together
      const T* src = xb + (k0 + (tid >> 3)) * sxk + r0 + (tid & 7) * 8;
#pragma unroll
      for (int pass = 0; pass < kColsKeys / 32; ++pass)
        wreg[pass] = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)pass * 32 * sxk));
      return;
    }
#pragma unroll
    for (int pass = 0; pass < kColsKeys / 32; ++pass) {
      const int key = pass * 32 + (tid >> 3);
      const int rc = (tid & 7) * 8;
      const int64_t kk = k0 + key;
      int valid = 0;
      if (kk < k_read) {
        const int64_t left = R - (r0 + rc);
        valid = left >= 8 ? 8 : (left > 0 ? (int)left : 0);
      }
      uint4 w = make_uint4(0u, 0u, 0u, 0u);
      const T* src = xb + kk * sxk + r0 + rc;
      if (valid >= 8 && vec_in) {
        w = __ldg(reinterpret_cast<const uint4*>(src));
      } else if (valid > 0) {
        uint16_t e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) e[i] = i < valid ? *reinterpret_cast<const uint16_t*>(src + i) : (uint16_t)0;
        w = make_uint4(e[0] | ((uint32_t)e[1] << 16), e[2] | ((uint32_t)e[3] << 16), e[4] | ((uint32_t)e[5] << 16),
                       e[6] | ((uint32_t)e[7] << 16));
      }
      wreg[pass] = w;
    }
  };
  if constexpr (sizeof(T) == 2) load16(bx * kColsKeys);
  // Shared-memory reuse across the tiles of a run needs no extra barrier: the input tile is rewritten
  // after the second barrier of the tile before (all its readers are past it), the output staging is
  // rewritten after the first barrier of this tile (its readers, the store phase, are before it).
  for (int ti = 0; ti < nt; ++ti) {
    const int64_t k0 = (bx + ti) * kColsKeys;
    if constexpr (sizeof(T) == 2) {
      auto& raw = sm.raw;
      // one 16-byte shared store per 16-byte load; then the next tile's loads are issued
#pragma unroll
      for (int pass = 0; pass < kColsKeys / 32; ++pass)
        *reinterpret_cast<uint4*>(&raw[pass * 32 + (tid >> 3)][(tid & 7) * 4]) = wreg[pass];
      if (ti + 1 < nt) load16(k0 + kColsKeys);
      __syncthreads();
      if constexpr (kDual) {
        // along the contiguous axis: thread -> (key = tid % 128, groups tid / 128 and tid / 128 + 2);
        // the 16 elements of a group are two 16-byte shared loads
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int key = tid & 127;
          const int g = (tid >> 7) + it * 2;
          if (k0 + key < k_read && r0 + g * 16 < R) {
            const uint4 w0 = *reinterpret_cast<const uint4*>(&raw[key][g * 8]);
            const uint4 w1 = *reinterpret_cast<const uint4*>(&raw[key][g * 8 + 4]);
            const uint32_t ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
            float v[16];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              unpack2<T>(ww[j], v[2 * j], v[2 * j + 1]);
              v[2 * j] *= pre;
              v[2 * j + 1] *= pre;
            }
            uint32_t lo, hi;
            const uint8_t sb = (sr_flags & 1)
                                   ? pack_group16_sr(v, lo, hi, seed, (uint32_t)(b * k_read + k0 + key) * 2u,
                                                     (uint32_t)(r0 / 4 + g * 4))
                                   : pack_group16(v, lo, hi);
            *reinterpret_cast<uint2*>(dnib + b * dnb + (k0 + key) * dnr + (r0 + g * 16) / 2) = make_uint2(lo, hi);
            dsc[b * dsb + (k0 + key) * dsr + (r0 + g * 16) / 16] = sb;
          }
        }
      }
      // quantise along the keys: thread -> (rows 2 (tid % 32) and the next, 16-key group tid / 32); one
      // 32-bit shared load brings a key's elements of both rows
      {
        const int rp = tid & 31, g = tid >> 5;
        float v0[16], v1[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          unpack2<T>(raw[g * 16 + j][rp], v0[j], v1[j]);
          if (kDual) {
            v0[j] *= pre;
            v1[j] *= pre;
          }
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int row = 2 * rp + h;
          uint32_t lo, hi;
          const uint8_t sb = (kDual && (sr_flags & 2))
                                 ? pack_group16_sr(h ? v1 : v0, lo, hi, seed, (uint32_t)(b * R + r0 + row) * 2u + 1u,
                                                   (uint32_t)(k0 / 4 + g * 4))
                                 : pack_group16(h ? v1 : v0, lo, hi);
          *reinterpret_cast<uint2*>(&onib[row][g * 8]) = make_uint2(lo, hi);
          osc[row][g] = sb;
        }
      }
    } else {
    auto& tile = sm.tile;
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
      for (int i = 0; i < 8; ++i) tile[key][rc + i] = kDual ? v[i] * pre : v[i];
    }
    __syncthreads();
    if constexpr (kDual) {
      // along the contiguous axis: thread -> (key = tid % 128, groups tid / 128 and tid / 128 + 2)
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int key = tid & 127;
        const int g = (tid >> 7) + it * 2;
        if (k0 + key < k_read && r0 + g * 16 < R) {
          float v[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = tile[key][g * 16 + j];
          uint32_t lo, hi;
          const uint8_t sb = (sr_flags & 1)
                                 ? pack_group16_sr(v, lo, hi, seed, (uint32_t)(b * k_read + k0 + key) * 2u,
                                                   (uint32_t)(r0 / 4 + g * 4))
                                 : pack_group16(v, lo, hi);
          *reinterpret_cast<uint2*>(dnib + b * dnb + (k0 + key) * dnr + (r0 + g * 16) / 2) = make_uint2(lo, hi);
          dsc[b * dsb + (k0 + key) * dsr + (r0 + g * 16) / 16] = sb;
        }
      }
    }
    // quantise: thread -> (row = tid % 64, groups tid / 64 and tid / 64 + 4)
#pragma unroll
    for (int it = 0; it < 2; ++it) {
      const int row = tid & 63;
      const int g = (tid >> 6) + it * 4;
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) v[j] = tile[g * 16 + j][row];
      uint32_t lo, hi;
      const uint8_t sb = (kDual && (sr_flags & 2))
                             ? pack_group16_sr(v, lo, hi, seed, (uint32_t)(b * R + r0 + row) * 2u + 1u,
                                               (uint32_t)(k0 / 4 + g * 4))
                             : pack_group16(v, lo, hi);
      *reinterpret_cast<uint2*>(&onib[row][g * 8]) = make_uint2(lo, hi);
      osc[row][g] = sb;
    }
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
  }  // tiles of the run
}

template <typename T, bool kDual>
__global__ void __launch_bounds__(256, 3) pack_cols_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t k_pad, int64_t sxb, int64_t sxk,
    uint8_t* __restrict__ nib, int64_t snb, int64_t snr, uint8_t* __restrict__ sc, int64_t ssb,
    int64_t ssr, int vec_in, uint8_t* __restrict__ dnib, int64_t dnb, int64_t dnr,
    uint8_t* __restrict__ dsc, int64_t dsb, int64_t dsr, const float* __restrict__ prescale_amax,
    int sr_flags, uint32_t seed) {
  __shared__ ColsSmem<T> sm;
  const int64_t tx = (k_pad + kColsKeys - 1) / kColsKeys, bx = (int64_t)blockIdx.x * kColsRun;
  pack_cols_tile<T, kDual>(sm, x, R, k_read, k_pad, sxb, sxk, nib, snb, snr, sc, ssb, ssr, vec_in, bx,
                           (int)(tx - bx < kColsRun ? tx - bx : kColsRun), blockIdx.y, blockIdx.z, dnib, dnb, dnr,
                           dsc, dsb, dsr, prescale_amax, sr_flags, seed);
}

// ---------------------------------------------------------------- MXFP8 along the strided axis
// x [B, S, R] (rows contiguous) -> e4m3 bytes [B, R, s_pad] + e8m0 scales [B, R, s_pad/32]: the
// transposed gradient operands (dO^T, Q^T, K^T) of the fp8_rownorm backward.  A 128-token x 64-row
// tile goes through shared memory; a thread packs one 32-token group of one row.  Tokens >= S read
// as +0.0; with prescale_amax every element is first divided by the power of two >= that value.
template <typename T>
__global__ void __launch_bounds__(256) pack_mx8_cols_kernel(
    const T* __restrict__ x, int64_t R, int64_t k_read, int64_t k_pad, int64_t sxb, int64_t sxk,
    uint8_t* __restrict__ out, uint8_t* __restrict__ sc, int vec_in, const float* __restrict__ prescale_amax) {
  __shared__ float tile[kColsKeys][kColsRows + 1];
  const float pre = prescale_amax != nullptr ? __frcp_rn(pow2_ceil(*prescale_amax)) : 1.0f;
  const int tid = threadIdx.x;
  const int64_t k0 = (int64_t)blockIdx.x * kColsKeys, r0 = (int64_t)blockIdx.y * kColsRows, b = blockIdx.z;
  const T* xb = x + b * sxb;
  bool loaded = false;
  if constexpr (sizeof(T) == 2) {
    if (vec_in && k0 + kColsKeys <= k_read && r0 + kColsRows <= R) {
      // interior tile: four unconditional 16-byte loads, all in flight together
      const T* src = xb + (k0 + (tid >> 3)) * sxk + r0 + (tid & 7) * 8;
      uint4 w[kColsKeys / 32];
#pragma unroll
      for (int pass = 0; pass < kColsKeys / 32; ++pass)
        w[pass] = __ldg(reinterpret_cast<const uint4*>(src + (int64_t)pass * 32 * sxk));
#pragma unroll
      for (int pass = 0; pass < kColsKeys / 32; ++pass) {
        const uint32_t ww[4] = {w[pass].x, w[pass].y, w[pass].z, w[pass].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float a, c;
          unpack2<T>(ww[i], a, c);
          tile[pass * 32 + (tid >> 3)][(tid & 7) * 8 + 2 * i] = a * pre;
          tile[pass * 32 + (tid >> 3)][(tid & 7) * 8 + 2 * i + 1] = c * pre;
        }
      }
      loaded = true;
    }
  }
  if (!loaded) {
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
      for (int i = 0; i < 8; ++i) tile[key][rc + i] = v[i] * pre;
    }
  }
  __syncthreads();
  const int row = tid & 63, g = tid >> 6;          // 32-token group g of row `row`
  if (r0 + row >= R || k0 + g * 32 >= k_pad) return;
  float v0[16], v1[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    v0[j] = tile[g * 32 + j][row];
    v1[j] = tile[g * 32 + 16 + j][row];
  }
  uint32_t w[8];
  const uint8_t sb = pack_group32_mx8(v0, v1, w);
  uint8_t* po = out + (b * R + r0 + row) * k_pad + k0 + g * 32;
  *reinterpret_cast<uint4*>(po) = make_uint4(w[0], w[1], w[2], w[3]);
  *reinterpret_cast<uint4*>(po + 16) = make_uint4(w[4], w[5], w[6], w[7]);
  sc[(b * R + r0 + row) * (k_pad / 32) + (k0 + g * 32) / 32] = sb;
}

// ---------------------------------------------------------------- Q, K along D and V^T in one launch
// A flat grid: the first nbq blocks pack Q's 16-groups, the next nbk blocks K's, the rest are the
// 128-key x 64-row tiles of V -> V^T.  Below a few thousand tokens three launches cost more than
// the packing itself; this is one.
struct QkvArgs {
  const void *q, *k, *v;
  int64_t rq, rk;            // rows of Q / K per batch entry
  int64_t bq, bk;            // batch entries of Q / K (= V)
  int d, ngroups_log2, vec_q, vec_k, vec_v;
  int quad_q, quad_k;        // Q / K packed four groups per thread (32-byte aligned rows)
  int64_t sqb, sqr, skb, skr, svb, svk;   // element strides
  int64_t bpq, bpk;          // 256-thread blocks per batch entry
  int64_t nbq, nbk;          // blocks of the Q and K parts
  int64_t s_kv, s_pad, tx, ty;            // V: keys, padded keys, tiles along keys / along D
  uint8_t *qnv, *qsc, *knv, *ksc, *vnv, *vsc;
};

template <typename T>
__global__ void __launch_bounds__(256, 3) pack_qkv_kernel(const QkvArgs a) {
  __shared__ ColsSmem<T> sm;
  const int64_t v = blockIdx.x;
  const int ngroups = a.d >> 4;
  if (v < a.nbq + a.nbk) {
    const bool is_q = v < a.nbq;
    const int64_t w = is_q ? v : v - a.nbq;
    const int64_t bp = is_q ? a.bpq : a.bpk;
    const int64_t b = w / bp;
    const int64_t gid = (w - b * bp) * 256 + threadIdx.x;
    const int64_t rows = is_q ? a.rq : a.rk;
    if (is_q ? a.quad_q : a.quad_k) {
      const int64_t first = ((w - b * bp) * 8 + (threadIdx.x >> 5)) * 128;    // first group of this warp
      if (first >= rows * ngroups) return;
      if (is_q)
        pack_rows_quad<T>(static_cast<const T*>(a.q), a.ngroups_log2, rows * ngroups, a.sqb, a.sqr, a.qnv,
                          rows * (a.d / 2), a.d / 2, a.qsc, rows * ngroups, ngroups, first, b);
      else
        pack_rows_quad<T>(static_cast<const T*>(a.k), a.ngroups_log2, rows * ngroups, a.skb, a.skr, a.knv,
                          rows * (a.d / 2), a.d / 2, a.ksc, rows * ngroups, ngroups, first, b);
      return;
    }
    if (gid >= rows * ngroups) return;
    if (is_q)
      pack_rows_group<T>(static_cast<const T*>(a.q), a.d, ngroups, a.ngroups_log2, a.sqb, a.sqr, a.qnv,
                         rows * (a.d / 2), a.d / 2, a.qsc, rows * ngroups, ngroups, a.vec_q, gid, b);
    else
      pack_rows_group<T>(static_cast<const T*>(a.k), a.d, ngroups, a.ngroups_log2, a.skb, a.skr, a.knv,
                         rows * (a.d / 2), a.d / 2, a.ksc, rows * ngroups, ngroups, a.vec_k, gid, b);
    return;
  }
  const int64_t w = v - a.nbq - a.nbk;
  const int64_t runs = (a.tx + kColsRun - 1) / kColsRun;      // runs of key tiles per row of tiles
  const int64_t per = runs * a.ty;
  const int64_t b = w / per;
  const int64_t rem = w - b * per;
  const int64_t by = rem / runs, bx = (rem - by * runs) * kColsRun;
  pack_cols_tile<T, false>(sm, static_cast<const T*>(a.v), a.d, a.s_kv, a.s_pad, a.svb, a.svk, a.vnv,
                           (int64_t)a.d * (a.s_pad / 2), a.s_pad / 2, a.vsc, (int64_t)a.d * (a.s_pad / 16),
                           a.s_pad / 16, a.vec_v, bx, (int)(a.tx - bx < kColsRun ? a.tx - bx : kColsRun), by, b,
                           nullptr, 0, 0, nullptr, 0, 0, nullptr);
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
    // whole groups, 32-byte aligned rows, a power-of-two group count: four groups per thread
    constexpr int64_t kVec32 = 32 / sizeof(T);
    if (lg >= 0 && k_read >= k_pad && (reinterpret_cast<uintptr_t>(x) & 31) == 0 && sxb % kVec32 == 0 &&
        sxr % kVec32 == 0 && (reinterpret_cast<uintptr_t>(nib) & 7) == 0 && snb % 8 == 0 && snr % 8 == 0) {
      dim3 qgrid((unsigned)((per_batch + 1023) / 1024), (unsigned)B);
      pack_rows_quad_kernel<T><<<qgrid, 256, 0, st>>>(x, lg, per_batch, sxb, sxr, nib, snb, snr, sc, ssb, ssr);
      return launch_result("nvfp4_pack(rows)");
    }
    dim3 grid((unsigned)blocks, (unsigned)B);
    pack_rows_kernel<T><<<grid, 256, 0, st>>>(x, R, k_read, ngroups, lg, per_batch, sxb, sxr, nib, snb,
                                              snr, sc, ssb, ssr, vec);
    return launch_result("nvfp4_pack(rows)");
  }
  if (sxr == 1 && B < 65536 && (R + kColsRows - 1) / kColsRows < 65536) {
    const int vec = base_ok && sxb % kVecElems == 0 && sxk % kVecElems == 0;
    dim3 grid((unsigned)((k_pad + kColsKeys * kColsRun - 1) / (kColsKeys * kColsRun)),
              (unsigned)((R + kColsRows - 1) / kColsRows), (unsigned)B);
    pack_cols_kernel<T, false><<<grid, 256, 0, st>>>(x, R, k_read, k_pad, sxb, sxk, nib, snb, snr, sc,
                                                     ssb, ssr, vec, nullptr, 0, 0, nullptr, 0, 0, nullptr, 0, 0u);
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

namespace nvfp4 {

template <typename T>
int pack_dual_launch(const void* x, int64_t B, int64_t S, int d, int64_t s_pad, int64_t sxb, int64_t sxs,
                     const float* prescale_amax, int sr_flags, uint32_t seed, uint8_t* dnib, uint8_t* dsc,
                     uint8_t* tnib, uint8_t* tsc, cudaStream_t st) {
  constexpr int64_t kVecElems = 16 / sizeof(T);
  const int vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && sxb % kVecElems == 0 && sxs % kVecElems == 0;
  dim3 grid((unsigned)((s_pad + kColsKeys * kColsRun - 1) / (kColsKeys * kColsRun)),
            (unsigned)((d + kColsRows - 1) / kColsRows), (unsigned)B);
  pack_cols_kernel<T, true><<<grid, 256, 0, st>>>(
      static_cast<const T*>(x), d, S, s_pad, sxb, sxs, tnib, (int64_t)d * (s_pad / 2), s_pad / 2, tsc,
      (int64_t)d * (s_pad / 16), s_pad / 16, vec, dnib, S * (int64_t)(d / 2), d / 2, dsc, S * (int64_t)(d / 16),
      d / 16, prescale_amax, sr_flags, seed);
  return launch_result("nvfp4_pack_dual");
}

template <typename T>
int pack_qkv_launch(QkvArgs a, cudaStream_t st) {
  constexpr int64_t kVecElems = 16 / sizeof(T);
  auto vec_ok = [&](const void* p, int64_t s0, int64_t s1) {
    return (int)((reinterpret_cast<uintptr_t>(p) & 15) == 0 && s0 % kVecElems == 0 && s1 % kVecElems == 0);
  };
  a.vec_q = vec_ok(a.q, a.sqb, a.sqr);
  a.vec_k = vec_ok(a.k, a.skb, a.skr);
  a.vec_v = vec_ok(a.v, a.svb, a.svk);
  // four groups per thread (a block covers 1024 groups) where the rows are 32-byte aligned
  constexpr int64_t kVec32 = 32 / sizeof(T);
  auto quad_ok = [&](const void* p, int64_t s0, int64_t s1) {
    return (int)((reinterpret_cast<uintptr_t>(p) & 31) == 0 && s0 % kVec32 == 0 && s1 % kVec32 == 0);
  };
  a.quad_q = quad_ok(a.q, a.sqb, a.sqr);
  a.quad_k = quad_ok(a.k, a.skb, a.skr);
  const int64_t ng = a.d / 16;
  a.bpq = (a.rq * ng + (a.quad_q ? 1023 : 255)) / (a.quad_q ? 1024 : 256);
  a.bpk = (a.rk * ng + (a.quad_k ? 1023 : 255)) / (a.quad_k ? 1024 : 256);
  a.nbq = a.bpq * a.bq;
  a.nbk = a.bpk * a.bk;
  const int64_t total = a.nbq + a.nbk + a.bk * ((a.tx + kColsRun - 1) / kColsRun) * a.ty;
  NVFP4_REQUIRE(total < (1LL << 31), "nvfp4_pack_qkv: tensors too large");
  pack_qkv_kernel<T><<<(unsigned)total, 256, 0, st>>>(a);
  return launch_result("nvfp4_pack_qkv");
}

}  // namespace nvfp4

extern "C" int nvfp4_pack_dual(const void* x, int dtype, int64_t B, int64_t S, int d, int64_t s_pad,
                               int64_t sxb, int64_t sxs, const float* prescale_amax, int sr_flags,
                               uint32_t seed, uint8_t* dnib, uint8_t* dsc, uint8_t* tnib, uint8_t* tsc,
                               nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(B >= 0 && S >= 0 && d >= 16 && d % 16 == 0, "nvfp4_pack_dual: head dim must be a positive multiple of 16");
  NVFP4_REQUIRE(s_pad % 16 == 0 && s_pad >= S, "nvfp4_pack_dual: s_pad must be a multiple of 16 >= S");
  if (B == 0 || s_pad == 0) return 0;
  NVFP4_REQUIRE(x && dnib && dsc && tnib && tsc, "nvfp4_pack_dual: null pointer");
  NVFP4_REQUIRE(B < 65536, "nvfp4_pack_dual: too many batch entries");
  NVFP4_REQUIRE(((uintptr_t)dnib & 7) == 0, "nvfp4_pack_dual: nibble buffers must be 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NVFP4_DT_BF16: return pack_dual_launch<__nv_bfloat16>(x, B, S, d, s_pad, sxb, sxs, prescale_amax, sr_flags, seed, dnib, dsc, tnib, tsc, st);
    case NVFP4_DT_FP16: return pack_dual_launch<__half>(x, B, S, d, s_pad, sxb, sxs, prescale_amax, sr_flags, seed, dnib, dsc, tnib, tsc, st);
    case NVFP4_DT_FP32: return pack_dual_launch<float>(x, B, S, d, s_pad, sxb, sxs, prescale_amax, sr_flags, seed, dnib, dsc, tnib, tsc, st);
    default: return fail(-1, "nvfp4_pack_dual: unknown dtype %d", dtype);
  }
}

extern "C" int nvfp4_pack_mx8_t(const void* x, int dtype, int64_t B, int64_t S, int d, int64_t s_pad,
                                int64_t sxb, int64_t sxs, const float* prescale_amax, uint8_t* out,
                                uint8_t* sc, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(B >= 0 && S >= 0 && d >= 1, "nvfp4_pack_mx8_t: bad extents");
  NVFP4_REQUIRE(s_pad % 32 == 0 && s_pad >= S, "nvfp4_pack_mx8_t: s_pad must be a multiple of 32 >= S");
  if (B == 0 || s_pad == 0) return 0;
  NVFP4_REQUIRE(x && out && sc, "nvfp4_pack_mx8_t: null pointer");
  NVFP4_REQUIRE(B < 65536 && ((uintptr_t)out & 15) == 0, "nvfp4_pack_mx8_t: too many batch entries or unaligned output");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((s_pad + kColsKeys - 1) / kColsKeys), (unsigned)((d + kColsRows - 1) / kColsRows), (unsigned)B);
#define NVFP4_MX8(T)                                                                                    \
  {                                                                                                     \
    constexpr int64_t kVecElems = 16 / sizeof(T);                                                       \
    const int vec = (reinterpret_cast<uintptr_t>(x) & 15) == 0 && sxb % kVecElems == 0 && sxs % kVecElems == 0; \
    pack_mx8_cols_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(x), d, S, s_pad, sxb, sxs, out, sc, vec, \
                                                  prescale_amax);                                       \
    return launch_result("nvfp4_pack_mx8_t");                                                           \
  }
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_MX8(__nv_bfloat16)
    case NVFP4_DT_FP16: NVFP4_MX8(__half)
    case NVFP4_DT_FP32: NVFP4_MX8(float)
    default: return fail(-1, "nvfp4_pack_mx8_t: unknown dtype %d", dtype);
  }
#undef NVFP4_MX8
}

extern "C" int nvfp4_pack_qkv(const void* q, const void* k, const void* v, int dtype, int64_t bq,
                              int64_t bk, int64_t s_q, int64_t s_kv, int64_t s_pad, int d,
                              int64_t sqb, int64_t sqr, int64_t skb, int64_t skr, int64_t svb,
                              int64_t svk, uint8_t* qnv, uint8_t* qsc, uint8_t* knv, uint8_t* ksc,
                              uint8_t* vnv, uint8_t* vsc, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d >= 16 && (d & (d - 1)) == 0, "nvfp4_pack_qkv: head dim must be a power of two >= 16");
  NVFP4_REQUIRE(bq >= 1 && bk >= 1 && s_q >= 1 && s_kv >= 1, "nvfp4_pack_qkv: empty problem");
  NVFP4_REQUIRE(s_pad % 16 == 0 && s_pad >= s_kv, "nvfp4_pack_qkv: s_pad must be a multiple of 16 >= s_kv");
  NVFP4_REQUIRE(q && k && v && qnv && qsc && knv && ksc && vnv && vsc, "nvfp4_pack_qkv: null pointer");
  NVFP4_REQUIRE((((uintptr_t)qnv | (uintptr_t)knv | (uintptr_t)vnv) & 15) == 0 && (((uintptr_t)vsc) & 7) == 0,
                "nvfp4_pack_qkv: outputs must be 16-byte aligned");
  QkvArgs a;
  a.q = q; a.k = k; a.v = v; a.rq = s_q; a.rk = s_kv; a.bq = bq; a.bk = bk; a.d = d;
  int lg = 0;
  while ((1 << lg) < d / 16) ++lg;
  a.ngroups_log2 = lg;
  a.sqb = sqb; a.sqr = sqr; a.skb = skb; a.skr = skr; a.svb = svb; a.svk = svk;
  a.bpq = a.bpk = a.nbq = a.nbk = 0;   // set by the launch, which knows the per-dtype alignment
  a.s_kv = s_kv; a.s_pad = s_pad;
  a.tx = (s_pad + kColsKeys - 1) / kColsKeys; a.ty = (d + kColsRows - 1) / kColsRows;
  a.qnv = qnv; a.qsc = qsc; a.knv = knv; a.ksc = ksc; a.vnv = vnv; a.vsc = vsc;
  a.vec_q = a.vec_k = a.vec_v = a.quad_q = a.quad_k = 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case NVFP4_DT_BF16: return pack_qkv_launch<__nv_bfloat16>(a, st);
    case NVFP4_DT_FP16: return pack_qkv_launch<__half>(a, st);
    case NVFP4_DT_FP32: return pack_qkv_launch<float>(a, st);
    default: return fail(-1, "nvfp4_pack_qkv: unknown dtype %d", dtype);
  }
}

extern "C" int nvfp4_rope_pack(const void* x, int dtype, int64_t B, int64_t R, int d, int64_t sxb,
                               int64_t sxr, const float* cos_tab, const float* sin_tab,
                               const int32_t* positions, int64_t pos0, uint8_t* nib, int64_t snb,
                               int64_t snr, uint8_t* sc, int64_t ssb, int64_t ssr,
                               nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(x && cos_tab && sin_tab && nib && sc, "nvfp4_rope_pack: null pointer");
  NVFP4_REQUIRE(d >= 32 && (d & (d - 1)) == 0, "nvfp4_rope_pack: head dim must be a power of two >= 32");
  NVFP4_REQUIRE(B >= 0 && R >= 0 && B < 65536, "nvfp4_rope_pack: bad extents");
  NVFP4_REQUIRE(((uintptr_t)nib & 7) == 0 && snb % 8 == 0 && snr % 8 == 0,
                "nvfp4_rope_pack: nibble rows must be 8-byte aligned");
  NVFP4_REQUIRE(((uintptr_t)cos_tab & 15) == 0 && ((uintptr_t)sin_tab & 15) == 0,
                "nvfp4_rope_pack: cos / sin tables must be 16-byte aligned");
  if (B == 0 || R == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int ngroups = d / 16;
  int lg = 0;
  while ((1 << lg) < ngroups) ++lg;
  const int64_t per_batch = R * ngroups;
  const int64_t blocks = (per_batch + 255) / 256;
  NVFP4_REQUIRE(blocks < (1LL << 31), "nvfp4_rope_pack: tensor too large");
  dim3 grid((unsigned)blocks, (unsigned)B);
  const int es = dtype == NVFP4_DT_FP32 ? 4 : 2;
  const int vec = ((uintptr_t)x % 16 == 0) && (sxb * es) % 16 == 0 && (sxr * es) % 16 == 0;
#define NVFP4_ROPE(T)                                                                              \
  rope_pack_rows_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(x), R, d, lg, per_batch, sxb, \
                                                 sxr, cos_tab, sin_tab, positions, pos0, nib, snb,  \
                                                 snr, sc, ssb, ssr, vec);                           \
  return launch_result("nvfp4_rope_pack")
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_ROPE(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_ROPE(__half);
    case NVFP4_DT_FP32: NVFP4_ROPE(float);
    default: return fail(-1, "nvfp4_rope_pack: unknown dtype %d", dtype);
  }
#undef NVFP4_ROPE
}
