// KV-cache kernels: the fused one-token append, the exact recent-window attention used by hybrid
// decode, and the log-sum-exp merge of two attention regions.
#include "common/abi.cuh"
#include "common/fp4.cuh"

namespace nvfp4 {

// One block per (z, kv-head) unit, one thread per head-dim element.
//  * threads [0, D/16) pack the new K row (one 16-group each);
//  * every thread stores its element of the new V token into the partial-group buffer and
//    re-packs "its" V^T row of the current 16-key group (8 bytes + 1 scale);
//  * ring slots are written when the rings exist.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new,
                                 int64_t s_new, int d, int64_t pos, uint8_t* __restrict__ knv,
                                 int64_t knv_unit, uint8_t* __restrict__ ksc, int64_t ksc_unit,
                                 uint8_t* __restrict__ vnv, int64_t vnv_unit, int64_t vnv_row,
                                 uint8_t* __restrict__ vsc, int64_t vsc_unit, int64_t vsc_row,
                                 T* __restrict__ partial, T* __restrict__ ring_k,
                                 T* __restrict__ ring_v, int64_t ring_cap) {
  const int64_t u = blockIdx.x;
  const int t = threadIdx.x;
  const T* kr = k_new + u * s_new;
  const T* vr = v_new + u * s_new;
  if (t < d / 16) {
    float v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = to_f32<T>(kr[t * 16 + i]);
    uint32_t lo, hi;
    const uint8_t sb = pack_group16(v, lo, hi);
    uint8_t* pn = knv + u * knv_unit + pos * (d / 2) + t * 8;
    *reinterpret_cast<uint2*>(pn) = make_uint2(lo, hi);
    ksc[u * ksc_unit + pos * (d / 16) + t] = sb;
  }
  const int slot = (int)(pos % 16);
  const int64_t gidx = pos / 16;
  T* pu = partial + u * 16 * d;
  const T vt = vr[t];
  float v[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    if (j < slot) {
      v[j] = to_f32<T>(pu[j * d + t]);
    } else if (j == slot) {
      v[j] = to_f32<T>(vt);
      pu[j * d + t] = vt;
    } else {
      v[j] = 0.0f;
      if (slot == 0) pu[j * d + t] = from_f32<T>(0.0f);
    }
  }
  uint32_t lo, hi;
  const uint8_t sb = pack_group16(v, lo, hi);
  uint8_t* pv = vnv + u * vnv_unit + (int64_t)t * vnv_row + gidx * 8;
  *reinterpret_cast<uint2*>(pv) = make_uint2(lo, hi);
  vsc[u * vsc_unit + (int64_t)t * vsc_row + gidx] = sb;
  if (ring_k != nullptr) {
    const int64_t rs = pos % ring_cap;
    ring_k[(u * ring_cap + rs) * d + t] = kr[t];
    ring_v[(u * ring_cap + rs) * d + t] = vt;
  }
}

// Exact attention of the G query rows of one kv head over `count` ring-resident keys.
// One block (512 threads) per (z, kv head): every K and V row of the window is read once and
// serves all G heads; scores live in shared memory ([G][count] floats).
// With `ws_acc` (partial mode) the window is cut into gridDim.y pieces of `chunk` keys and block
// (unit, j) writes the UN-normalised result of its piece -- sum exp(s - m) v, m, sum exp(s - m) -- as
// one more split-K partial of the unit (slot extra_base + unit * gridDim.y + j, the layout of the
// FP4 decode's partials), so the decode's combine merges prefix and window in one pass.
// This scalar kernel serves any dtype, head dim and GQA group <= 16; 16-bit caches with D = 128 / 256
// take window_mma_kernel below in partial mode.
template <typename T>
__global__ void __launch_bounds__(512) window_attention_kernel(
    const T* __restrict__ q, int64_t s_qz, int64_t s_qh, const T* __restrict__ rk,
    const T* __restrict__ rv, int hk, int g, int d, int64_t ring_cap, int64_t first_pos_all,
    int count_all, int chunk, float scaling, float* __restrict__ out, float* __restrict__ lse,
    float* __restrict__ ws_acc, float* __restrict__ ws_m, float* __restrict__ ws_l, int64_t extra_base) {
  extern __shared__ __align__(16) float sm[];
  const bool partial = ws_acc != nullptr;
  const int k0 = partial ? (int)blockIdx.y * chunk : 0;
  const int count = partial ? min(chunk, count_all - k0) : count_all;
  const int64_t first_pos = first_pos_all + k0;
  if (partial && count <= 0) {          // an empty piece: a partial that the combine ignores
    const int64_t slot = extra_base + (int64_t)blockIdx.x * gridDim.y + blockIdx.y;
    for (int i = threadIdx.x; i < g * d; i += 512) ws_acc[slot * 16 * d + i] = 0.0f;
    if (threadIdx.x < g) {
      ws_m[slot * 16 + threadIdx.x] = -INFINITY;
      ws_l[slot * 16 + threadIdx.x] = 0.0f;
    }
    return;
  }
  float* qs = sm;                 // [g][d]
  float* sc = sm + g * d;         // [g][count]
  float* part = sc + ((g * (partial ? chunk : count) + 3) & ~3);   // [4][g][d] partial outputs (four slots shared by the sixteen warps), 16-byte aligned
  __shared__ float row_m[16], row_l[16];
  const int zi = blockIdx.x / hk, kh = blockIdx.x % hk;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  for (int i = tid; i < g * d; i += 512) {
    const int gq = i / d, e = i - gq * d;
    qs[i] = to_f32<T>(q[zi * s_qz + (int64_t)(kh * g + gq) * s_qh + e]);
  }
  __syncthreads();
  const T* kb = rk + ((int64_t)(zi * hk + kh) * ring_cap) * d;
  const T* vb = rv + ((int64_t)(zi * hk + kh) * ring_cap) * d;
  const int cap = (int)ring_cap, first = (int)(first_pos % ring_cap);   // slot of key j: first + j, wrapped once
  auto slot = [&](int j) { const int sl = first + j; return sl >= cap ? sl - cap : sl; };
  // scores: a warp takes four keys at a time (four independent row loads in flight), a lane owns
  // four consecutive elements of every 128-element piece of the row; all heads per key
  for (int j0 = warp * 4; j0 < count; j0 += 64) {
    float acc[4][16];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int gq = 0; gq < 16; ++gq) acc[u][gq] = 0.0f;
    for (int c = 0; c < d; c += 128) {
      float kv[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + u, count - 1);
        const T* kr = kb + (int64_t)slot(j) * d + c + lane * 4;
        if constexpr (sizeof(T) == 2) {
          const uint2 raw = *reinterpret_cast<const uint2*>(kr);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int x = 0; x < 4; ++x) kv[u][x] = to_f32<T>(e[x]);
        } else {
#pragma unroll
          for (int x = 0; x < 4; ++x) kv[u][x] = to_f32<T>(kr[x]);
        }
      }
#pragma unroll
      for (int gq = 0; gq < 16; ++gq)
        if (gq < g) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + gq * d + c + lane * 4);
#pragma unroll
          for (int u = 0; u < 4; ++u)
            acc[u][gq] += q4.x * kv[u][0] + q4.y * kv[u][1] + q4.z * kv[u][2] + q4.w * kv[u][3];
        }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int gq = 0; gq < 16; ++gq)
        if (gq < g) {
          float v = acc[u][gq];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0 && j0 + u < count) sc[gq * count + j0 + u] = v * scaling;
        }
  }
  __syncthreads();
  // softmax statistics: one warp per head
  for (int gq = warp; gq < g; gq += 16) {
    float m = -INFINITY;
    for (int j = lane; j < count; j += 32) m = fmaxf(m, sc[gq * count + j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.0f;
    for (int j = lane; j < count; j += 32) {
      const float e = expf(sc[gq * count + j] - m);
      sc[gq * count + j] = e;
      l += e;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) { row_m[gq] = m; row_l[gq] = l; }
  }
  __syncthreads();
  // P.V: warp w takes keys w, w + 16, ... (four row loads in flight), a lane owns four consecutive
  // columns of each 128-column piece; the sixteen warps' partial sums meet in four shared slots
  // (warps w, w + 4, w + 8, w + 12 add into slot w & 3 in turn)
  for (int c = 0; c < d; c += 128) {
    float acc[16][4];
#pragma unroll
    for (int gq = 0; gq < 16; ++gq)
#pragma unroll
      for (int x = 0; x < 4; ++x) acc[gq][x] = 0.0f;
    for (int j0 = warp; j0 < count; j0 += 64) {
      float vv[4][4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = min(j0 + 16 * u, count - 1);
        const T* vr = vb + (int64_t)slot(j) * d + c + lane * 4;
        if constexpr (sizeof(T) == 2) {
          const uint2 raw = *reinterpret_cast<const uint2*>(vr);
          const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
          for (int x = 0; x < 4; ++x) vv[u][x] = to_f32<T>(e[x]);
        } else {
#pragma unroll
          for (int x = 0; x < 4; ++x) vv[u][x] = to_f32<T>(vr[x]);
        }
      }
#pragma unroll
      for (int gq = 0; gq < 16; ++gq)
        if (gq < g) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float pr = (j0 + 16 * u < count) ? sc[gq * count + j0 + 16 * u] : 0.0f;
#pragma unroll
            for (int x = 0; x < 4; ++x) acc[gq][x] = fmaf(pr, vv[u][x], acc[gq][x]);
          }
        }
    }
    for (int r = 0; r < 4; ++r) {
      if ((warp >> 2) == r) {
#pragma unroll
        for (int gq = 0; gq < 16; ++gq)
          if (gq < g) {
            float4* dst = reinterpret_cast<float4*>(part + ((warp & 3) * g + gq) * d + c + lane * 4);
            float4 v = make_float4(acc[gq][0], acc[gq][1], acc[gq][2], acc[gq][3]);
            if (r > 0) {
              const float4 o = *dst;
              v = make_float4(v.x + o.x, v.y + o.y, v.z + o.z, v.w + o.w);
            }
            *dst = v;
          }
      }
      __syncthreads();
    }
  }
  if (partial) {
    const int64_t slot = extra_base + (int64_t)blockIdx.x * gridDim.y + blockIdx.y;
    for (int i = tid; i < g * d; i += 512)
      ws_acc[slot * 16 * d + i] = part[i] + part[g * d + i] + part[2 * g * d + i] + part[3 * g * d + i];
    if (tid < g) {
      ws_m[slot * 16 + tid] = row_m[tid];
      ws_l[slot * 16 + tid] = row_l[tid];
    }
    return;
  }
  for (int i = tid; i < g * d; i += 512) {
    const int gq = i / d;
    out[((int64_t)(zi * hk + kh) * g) * d + i] =
        (part[i] + part[g * d + i] + part[2 * g * d + i] + part[3 * g * d + i]) / row_l[gq];
  }
  if (tid < g) lse[(int64_t)(zi * hk + kh) * g + tid] = row_m[tid] + logf(row_l[tid]);
}

// ---------------------------------------------------------------------------------------------
// Window partials on the (legacy) warp-level tensor path, for 16-bit caches with D = 128 or 256.
// The window is 34 MB at the decode benchmark's size -- HBM-bound byte work -- and the scalar kernel
// above spends ~250 issue slots per key on lane reductions.  Here a block (256 threads) owns one
// piece (<= kWinMaxKeys keys) of one (batch, kv head) unit:
//   1. all K and V rows of the piece go to shared memory in ONE burst of 16-byte cp.async (every
//      byte in flight at once; 16-byte chunks XOR-swizzled by the row so ldmatrix is conflict-free);
//   2. scores = Q[16 x D] K^T with mma.sync m16n8k16 (the <= 16 heads of the group are the M rows),
//      warps split the 8-key groups;
//   3. one warp per head: maximum, exponentials, sum; P is kept as a high + low pair of 16-bit
//      values so the product with V carries ~16 mantissa bits;
//   4. O = P V with V fragments from ldmatrix.trans, every warp owning D/8 output columns over all
//      keys, so no cross-warp reduction is needed.
// The block writes (sum exp(s - m) v, m, sum exp(s - m)) as one split-K partial of the unit.
template <typename T> struct WinMma;
template <> struct WinMma<__nv_bfloat16> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
template <> struct WinMma<__half> {
  static __device__ __forceinline__ void mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
};
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t saddr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(saddr));
}

constexpr int kWinThreads = 256;
// bytes of dynamic shared memory for a piece of `keys` (multiple of 16) keys
__host__ __device__ constexpr size_t win_mma_smem(int d, int keys) {
  return (size_t)16 * d * 2            // Q rows (16-bit), swizzled
         + 2 * (size_t)keys * d * 2    // K and V rows, swizzled
         + (size_t)16 * (keys + 4) * 4       // scores (fp32); P high / low reuse the K rows
         + 128;
}

template <typename T, int D>
__global__ void __launch_bounds__(kWinThreads, D == 128 ? 2 : 1) window_mma_kernel(
    const T* __restrict__ q, int64_t s_qz, int64_t s_qh, const T* __restrict__ rk,
    const T* __restrict__ rv, int hk, int g, int64_t ring_cap, int64_t first_pos_all, int count_all,
    int chunk, float scaling, float* __restrict__ ws_acc, float* __restrict__ ws_m,
    float* __restrict__ ws_l, int64_t extra_base) {
  constexpr int kRowB = D * 2;            // bytes of a row
  constexpr int kChunks = D / 8;          // 16-byte chunks of a row
  extern __shared__ __align__(128) uint8_t wsm[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int k0 = (int)blockIdx.y * chunk;
  const int count = min(chunk, count_all - k0);
  const int64_t slot = extra_base + (int64_t)blockIdx.x * gridDim.y + blockIdx.y;
  if (count <= 0) {                       // an empty piece: a partial that the combine ignores
    for (int i = tid; i < g * D; i += kWinThreads) ws_acc[slot * 16 * D + i] = 0.0f;
    if (tid < g) {
      ws_m[slot * 16 + tid] = -INFINITY;
      ws_l[slot * 16 + tid] = 0.0f;
    }
    return;
  }
  const int keys = (count + 15) & ~15;    // rows of the staged tiles that the MMAs touch
  uint8_t* qs = wsm;
  uint8_t* ks = qs + 16 * kRowB;
  uint8_t* vs = ks + (size_t)keys * kRowB;
  float* sc = reinterpret_cast<float*>(vs + (size_t)keys * kRowB);     // [16][keys + 4]
  const int scs = keys + 4;
  T* ph = reinterpret_cast<T*>(ks);            // [16][keys + 8], over the K rows once the scores exist
  const int ps = keys + 8;
  T* pl = ph + 16 * ps;
  __shared__ float row_m[16], row_l[16];
  const int zi = blockIdx.x / hk, kh = blockIdx.x % hk;
  const uint32_t qs_a = (uint32_t)__cvta_generic_to_shared(qs), ks_a = (uint32_t)__cvta_generic_to_shared(ks);
  const uint32_t vs_a = (uint32_t)__cvta_generic_to_shared(vs);
  const T* kb = rk + ((int64_t)(zi * hk + kh) * ring_cap) * D;
  const T* vb = rv + ((int64_t)(zi * hk + kh) * ring_cap) * D;
  const int cap = (int)ring_cap, first = (int)((first_pos_all + k0) % ring_cap);
  // ---- 1. stage: K first (its own group, so the scores can start while V is still landing)
  auto stage = [&](const T* base, uint32_t dst) {
    for (int idx = tid; idx < count * kChunks; idx += kWinThreads) {
      const int j = idx / kChunks, c = idx - j * kChunks;
      int sl = first + j;
      sl = sl >= cap ? sl - cap : sl;
      const char* src = reinterpret_cast<const char*>(base + (int64_t)sl * D) + c * 16;
      const uint32_t d_ = dst + j * kRowB + ((c ^ (j & 7)) << 4);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d_), "l"(src) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(kb, ks_a);
  stage(vb, vs_a);
  // Q rows (zero rows above the group) and zero V rows behind the last key: 0 * garbage must stay 0
  for (int idx = tid; idx < 16 * kChunks; idx += kWinThreads) {
    const int r = idx / kChunks, c = idx - r * kChunks;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < g) v = *reinterpret_cast<const uint4*>(q + zi * s_qz + (int64_t)(kh * g + r) * s_qh + c * 8);
    *reinterpret_cast<uint4*>(qs + r * kRowB + ((c ^ (r & 7)) << 4)) = v;
  }
  for (int idx = tid; idx < (keys - count) * kChunks; idx += kWinThreads) {
    const int r = count + idx / kChunks, c = idx % kChunks;
    *reinterpret_cast<uint4*>(vs + (size_t)r * kRowB + ((c ^ (r & 7)) << 4)) = make_uint4(0u, 0u, 0u, 0u);
  }
  asm volatile("cp.async.wait_group 1;" ::: "memory");
  __syncthreads();
  // ---- 2. scores, in base-2 units: warp w takes the 8-key groups w, w + 8, ...
  {
    uint32_t aq[D / 16][4];
#pragma unroll
    for (int s_ = 0; s_ < D / 16; ++s_) {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8, c = 2 * s_ + (lane >> 4);
      ldsm_x4(aq[s_], qs_a + r * kRowB + ((c ^ (r & 7)) << 4));
    }
    const float c2 = scaling * 1.4426950408889634f;
    for (int grp = warp; grp * 8 < count; grp += kWinThreads / 32) {
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      const int r = grp * 8 + (lane & 7);
#pragma unroll
      for (int jj = 0; jj < D / 32; ++jj) {
        uint32_t b[4];
        const int c = 4 * jj + (lane >> 3);
        ldsm_x4(b, ks_a + r * kRowB + ((c ^ (r & 7)) << 4));
        WinMma<T>::mma(acc, aq[2 * jj], b[0], b[1]);
        WinMma<T>::mma(acc, aq[2 * jj + 1], b[2], b[3]);
      }
      const int key = grp * 8 + 2 * (lane & 3), row = lane >> 2;
      const float s0 = key < count ? acc[0] * c2 : -INFINITY, s1 = key + 1 < count ? acc[1] * c2 : -INFINITY;
      const float s2 = key < count ? acc[2] * c2 : -INFINITY, s3 = key + 1 < count ? acc[3] * c2 : -INFINITY;
      *reinterpret_cast<float2*>(sc + row * scs + key) = make_float2(s0, s1);
      *reinterpret_cast<float2*>(sc + (row + 8) * scs + key) = make_float2(s2, s3);
    }
  }
  __syncthreads();
  // ---- 3. one warp per head (two when the group has more than 8): m, p = 2^(s - m) as high + low
  for (int r = warp; r < 16; r += kWinThreads / 32) {
    if (r < g) {
      float m = -INFINITY;
      for (int j = lane; j < count; j += 32) m = fmaxf(m, sc[r * scs + j]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      float l = 0.0f;
      for (int j = lane; j < keys; j += 32) {
        const float e = j < count ? exp2f(sc[r * scs + j] - m) : 0.0f;
        const T hi = from_f32<T>(e);
        ph[r * ps + j] = hi;
        pl[r * ps + j] = from_f32<T>(e - to_f32<T>(hi));
        l += e;
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
      if (lane == 0) { row_m[r] = m * 0.6931471805599453f; row_l[r] = l; }
    } else {
      for (int j = lane; j < keys; j += 32) {      // rows without a head: finite, never written out
        ph[r * ps + j] = from_f32<T>(0.0f);
        pl[r * ps + j] = from_f32<T>(0.0f);
      }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  // ---- 4. O = P V: warp w owns output columns [w D/8, (w + 1) D/8) over all keys
  constexpr int kTiles = D / 128;        // pairs of 8-column tiles per warp (one ldmatrix.x4.trans each)
  float o[2 * kTiles][4];
#pragma unroll
  for (int i = 0; i < 2 * kTiles; ++i)
#pragma unroll
    for (int x = 0; x < 4; ++x) o[i][x] = 0.0f;
  const uint32_t ph_a = (uint32_t)__cvta_generic_to_shared(ph), pl_a = (uint32_t)__cvta_generic_to_shared(pl);
  for (int kb16 = 0; kb16 < keys; kb16 += 16) {
    uint32_t ah[4], al[4];
    {
      const int r = (lane & 7) + ((lane >> 3) & 1) * 8, col = kb16 + (lane >> 4) * 8;
      ldsm_x4(ah, ph_a + (r * ps + col) * 2);
      ldsm_x4(al, pl_a + (r * ps + col) * 2);
    }
#pragma unroll
    for (int t = 0; t < kTiles; ++t) {
      uint32_t b[4];
      const int r = kb16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = warp * (kChunks / 8) + 2 * t + (lane >> 4);
      ldsm_x4_trans(b, vs_a + r * kRowB + ((c ^ (r & 7)) << 4));
      WinMma<T>::mma(o[2 * t], ah, b[0], b[1]);
      WinMma<T>::mma(o[2 * t], al, b[0], b[1]);
      WinMma<T>::mma(o[2 * t + 1], ah, b[2], b[3]);
      WinMma<T>::mma(o[2 * t + 1], al, b[2], b[3]);
    }
  }
  {
    const int row = lane >> 2;
#pragma unroll
    for (int i = 0; i < 2 * kTiles; ++i) {
      const int col = warp * (D / 8) + i * 8 + 2 * (lane & 3);
      if (row < g) *reinterpret_cast<float2*>(ws_acc + slot * 16 * D + row * D + col) = make_float2(o[i][0], o[i][1]);
      if (row + 8 < g)
        *reinterpret_cast<float2*>(ws_acc + slot * 16 * D + (row + 8) * D + col) = make_float2(o[i][2], o[i][3]);
    }
  }
  if (tid < g) {
    ws_m[slot * 16 + tid] = row_m[tid];
    ws_l[slot * 16 + tid] = row_l[tid];
  }
}

template <typename T>
__global__ void lse_merge_kernel(const T* __restrict__ o1, const float* __restrict__ l1,
                                 const T* __restrict__ o2, const float* __restrict__ l2,
                                 T* __restrict__ out, float* __restrict__ lse_out, int64_t rows, int d) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const int64_t r = i / d;
  const float a1 = l1[r], a2 = l2[r];
  const float m = fmaxf(a1, a2);
  if (m == -INFINITY) {   // a row neither side touched
    out[i] = from_f32<T>(0.0f);
    if (lse_out != nullptr && i == r * d) lse_out[r] = -INFINITY;
    return;
  }
  const float w1 = expf(a1 - m), w2 = expf(a2 - m);
  // a side with weight 0 may hold anything (an untouched row of an empty buffer)
  const float v1 = w1 > 0.0f ? w1 * to_f32<T>(o1[i]) : 0.0f;
  const float v2 = w2 > 0.0f ? w2 * to_f32<T>(o2[i]) : 0.0f;
  out[i] = from_f32<T>((v1 + v2) / (w1 + w2));
  if (lse_out != nullptr && i == r * d) lse_out[r] = m + logf(w1 + w2);
}

template <typename T>
int append_launch(const void* k_new, const void* v_new, int64_t s_new, int64_t zhk, int d,
                  int64_t pos, uint8_t* knv, int64_t knv_unit, uint8_t* ksc, int64_t ksc_unit,
                  uint8_t* vnv, int64_t vnv_unit, int64_t vnv_row, uint8_t* vsc, int64_t vsc_unit,
                  int64_t vsc_row, void* partial, void* ring_k, void* ring_v, int64_t ring_cap,
                  cudaStream_t st) {
  kv_append_kernel<T><<<(unsigned)zhk, d, 0, st>>>(
      static_cast<const T*>(k_new), static_cast<const T*>(v_new), s_new, d, pos, knv, knv_unit, ksc,
      ksc_unit, vnv, vnv_unit, vnv_row, vsc, vsc_unit, vsc_row, static_cast<T*>(partial),
      static_cast<T*>(ring_k), static_cast<T*>(ring_v), ring_cap);
  return launch_result("nvfp4_kv_append");
}

}  // namespace nvfp4

extern "C" int nvfp4_kv_append(const void* k_new, const void* v_new, int dtype, int64_t s_new,
                               int64_t zhk, int d, int64_t pos, uint8_t* knv, int64_t knv_unit,
                               uint8_t* ksc, int64_t ksc_unit, uint8_t* vnv, int64_t vnv_unit,
                               int64_t vnv_row, uint8_t* vsc, int64_t vsc_unit, int64_t vsc_row,
                               void* partial, void* ring_k, void* ring_v, int64_t ring_cap,
                               nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_kv_append: D must be 128 or 256");
  NVFP4_REQUIRE(zhk > 0 && zhk < (1LL << 31) && pos >= 0, "nvfp4_kv_append: bad extent");
  NVFP4_REQUIRE(k_new && v_new && knv && ksc && vnv && vsc && partial,
                "nvfp4_kv_append: null pointer");
  NVFP4_REQUIRE((ring_k == nullptr) == (ring_v == nullptr) && (ring_k == nullptr || ring_cap > 0),
                "nvfp4_kv_append: ring_k/ring_v/ring_cap inconsistent");
  NVFP4_REQUIRE(((uintptr_t)knv % 8) == 0 && knv_unit % 8 == 0 && ((uintptr_t)vnv % 8) == 0 &&
                    vnv_unit % 8 == 0 && vnv_row % 8 == 0,
                "nvfp4_kv_append: nibble buffers must be 8-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define NVFP4_APPEND(T)                                                                         \
  return append_launch<T>(k_new, v_new, s_new, zhk, d, pos, knv, knv_unit, ksc, ksc_unit, vnv,  \
                          vnv_unit, vnv_row, vsc, vsc_unit, vsc_row, partial, ring_k, ring_v,   \
                          ring_cap, st)
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_APPEND(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_APPEND(__half);
    case NVFP4_DT_FP32: NVFP4_APPEND(float);
    default: return fail(-1, "nvfp4_kv_append: unknown dtype %d", dtype);
  }
#undef NVFP4_APPEND
}

extern "C" int nvfp4_window_attention(const void* q, int dtype, int64_t s_qz, int64_t s_qh,
                                      const void* rk, const void* rv, int64_t z, int64_t hk, int g,
                                      int d, int64_t ring_cap, int64_t first_pos, int64_t count,
                                      float scaling, float* out, float* lse,
                                      nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(q && rk && rv && out && lse, "nvfp4_window_attention: null pointer");
  NVFP4_REQUIRE(count > 0 && count <= ring_cap, "nvfp4_window_attention: count must be in (0, ring_cap]");
  NVFP4_REQUIRE(z * hk * g < (1LL << 31), "nvfp4_window_attention: too many heads");
  const size_t smem = (size_t)(5 * g * d + g * count + 4) * sizeof(float);
  NVFP4_REQUIRE(g >= 1 && g <= 16, "nvfp4_window_attention: GQA group %d must be <= 16", g);
  NVFP4_REQUIRE(smem <= 200 * 1024, "nvfp4_window_attention: window too long (%lld keys)", (long long)count);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(z * hk);
#define NVFP4_WIN(T)                                                                              \
  if (smem > 48 * 1024) {                                                                         \
    cudaError_t e = cudaFuncSetAttribute(window_attention_kernel<T>,                              \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return fail((int)e, "nvfp4_window_attention: smem attribute: %s", cudaGetErrorString(e)); \
  }                                                                                               \
  window_attention_kernel<T><<<grid, 512, smem, st>>>(static_cast<const T*>(q), s_qz, s_qh,       \
                                                      static_cast<const T*>(rk),                  \
                                                      static_cast<const T*>(rv), (int)hk, g, d,   \
                                                      ring_cap, first_pos, (int)count, (int)count, \
                                                      scaling, out, lse, nullptr, nullptr,        \
                                                      nullptr, 0);                                \
  return launch_result("nvfp4_window_attention")
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_WIN(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_WIN(__half);
    case NVFP4_DT_FP32: NVFP4_WIN(float);
    default: return fail(-1, "nvfp4_window_attention: unknown dtype %d", dtype);
  }
#undef NVFP4_WIN
}

extern "C" int nvfp4_window_partials(const void* q, int dtype, int64_t s_qz, int64_t s_qh, const void* rk,
                                     const void* rv, int64_t z, int64_t hk, int g, int d,
                                     int64_t ring_cap, int64_t first_pos, int64_t count, float scaling,
                                     int pieces, void* workspace, int64_t total_slots,
                                     int64_t extra_base, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(q && rk && rv && workspace, "nvfp4_window_partials: null pointer");
  NVFP4_REQUIRE(count > 0 && count <= ring_cap, "nvfp4_window_partials: count must be in (0, ring_cap]");
  NVFP4_REQUIRE(g >= 1 && g <= 16, "nvfp4_window_partials: GQA group %d must be <= 16", g);
  NVFP4_REQUIRE(pieces >= 1 && pieces <= 64, "nvfp4_window_partials: pieces must be in [1, 64]");
  NVFP4_REQUIRE(z * hk < (1LL << 31) && extra_base >= 0 && extra_base + z * hk * pieces <= total_slots,
                "nvfp4_window_partials: partial slots out of range");
  float* ws = static_cast<float*>(workspace);
  float* ws_acc = ws;
  float* ws_m = ws + total_slots * 16 * d;
  float* ws_l = ws_m + total_slots * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)(z * hk), (unsigned)pieces);
  // 16-bit caches with D = 128 / 256: the staged tensor-path kernel, when a piece fits its tiles
  {
    const int chunk16 = (int)(((count + pieces - 1) / pieces + 15) / 16 * 16);
    const size_t smem16 = win_mma_smem(d, chunk16);
    const bool aligned = ((uintptr_t)q % 16) == 0 && ((uintptr_t)rk % 16) == 0 && ((uintptr_t)rv % 16) == 0 &&
                         s_qz % 8 == 0 && s_qh % 8 == 0;
    if ((dtype == NVFP4_DT_BF16 || dtype == NVFP4_DT_FP16) && (d == 128 || d == 256) && aligned &&
        smem16 <= 200 * 1024) {
#define NVFP4_WINM(T, DD)                                                                             \
  {                                                                                                   \
    cudaError_t e = cudaFuncSetAttribute(window_mma_kernel<T, DD>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         (int)smem16);                                                \
    if (e != cudaSuccess) return fail((int)e, "nvfp4_window_partials: smem attribute: %s", cudaGetErrorString(e)); \
    window_mma_kernel<T, DD><<<grid, kWinThreads, smem16, st>>>(                                      \
        static_cast<const T*>(q), s_qz, s_qh, static_cast<const T*>(rk), static_cast<const T*>(rv), (int)hk, g, \
        ring_cap, first_pos, (int)count, chunk16, scaling, ws_acc, ws_m, ws_l, extra_base);           \
    return launch_result("nvfp4_window_partials");                                                    \
  }
      if (dtype == NVFP4_DT_BF16) {
        if (d == 128) NVFP4_WINM(__nv_bfloat16, 128) else NVFP4_WINM(__nv_bfloat16, 256)
      } else {
        if (d == 128) NVFP4_WINM(__half, 128) else NVFP4_WINM(__half, 256)
      }
#undef NVFP4_WINM
    }
  }
  const int chunk = (int)(((count + pieces - 1) / pieces + 3) / 4 * 4);
  const size_t smem = (size_t)(5 * g * d + g * chunk + 4) * sizeof(float);
  NVFP4_REQUIRE(smem <= 200 * 1024, "nvfp4_window_partials: window piece too long (%d keys)", chunk);
#define NVFP4_WINP(T)                                                                               \
  {                                                                                                 \
    if (smem > 48 * 1024) {                                                                         \
      cudaError_t e = cudaFuncSetAttribute(window_attention_kernel<T>,                              \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) return fail((int)e, "nvfp4_window_partials: smem attribute: %s", cudaGetErrorString(e)); \
    }                                                                                               \
    window_attention_kernel<T><<<grid, 512, smem, st>>>(                                            \
        static_cast<const T*>(q), s_qz, s_qh, static_cast<const T*>(rk), static_cast<const T*>(rv), (int)hk, g, d, \
        ring_cap, first_pos, (int)count, chunk, scaling, nullptr, nullptr, ws_acc, ws_m, ws_l, extra_base); \
    return launch_result("nvfp4_window_partials");                                                  \
  }
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_WINP(__nv_bfloat16)
    case NVFP4_DT_FP16: NVFP4_WINP(__half)
    case NVFP4_DT_FP32: NVFP4_WINP(float)
    default: return fail(-1, "nvfp4_window_partials: unknown dtype %d", dtype);
  }
#undef NVFP4_WINP
}

extern "C" int nvfp4_lse_merge(const void* o1, const float* lse1, const void* o2, const float* lse2,
                               void* out, float* lse_out, int dtype, int64_t rows, int d,
                               nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(o1 && o2 && lse1 && lse2 && out, "nvfp4_lse_merge: null pointer");
  if (rows * d == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows * d + 255) / 256);
#define NVFP4_MERGE(T)                                                                           \
  lse_merge_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(o1), lse1,                     \
                                            static_cast<const T*>(o2), lse2, static_cast<T*>(out), \
                                            lse_out, rows, d);                                   \
  return launch_result("nvfp4_lse_merge")
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_MERGE(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_MERGE(__half);
    case NVFP4_DT_FP32: NVFP4_MERGE(float);
    default: return fail(-1, "nvfp4_lse_merge: unknown dtype %d", dtype);
  }
#undef NVFP4_MERGE
}
