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
// kStaged (partial mode only): the K and V rows of the piece are first copied to shared memory with
// one burst of 16-byte cp.async (every byte of the piece in flight at once), because walking them
// straight from global memory is a chain of dependent DRAM round trips -- 0.7 TB/s on a window that
// should stream at HBM rate.
template <typename T, bool kStaged>
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
  T* stage_k = reinterpret_cast<T*>(part + 4 * g * d);             // kStaged: [chunk][d], then V [chunk][d]
  T* stage_v = stage_k + (size_t)chunk * d;
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
  auto gslot = [&](int j) { const int sl = first + j; return sl >= cap ? sl - cap : sl; };
  if constexpr (kStaged) {
    const int per_row = d * (int)sizeof(T) / 16;         // 16-byte pieces of a row
    for (int idx = tid; idx < count * per_row; idx += 512) {
      const int j = idx / per_row, o = idx - j * per_row;
      const char* gk = reinterpret_cast<const char*>(kb + (int64_t)gslot(j) * d) + o * 16;
      const char* gv = reinterpret_cast<const char*>(vb + (int64_t)gslot(j) * d) + o * 16;
      const uint32_t sk = (uint32_t)__cvta_generic_to_shared(reinterpret_cast<char*>(stage_k) + (size_t)idx * 16);
      const uint32_t sv = (uint32_t)__cvta_generic_to_shared(reinterpret_cast<char*>(stage_v) + (size_t)idx * 16);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sk), "l"(gk) : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sv), "l"(gv) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    kb = stage_k;
    vb = stage_v;
  }
  auto slot = [&](int j) { return kStaged ? j : gslot(j); };
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
    cudaError_t e = cudaFuncSetAttribute(window_attention_kernel<T, false>,                       \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    if (e != cudaSuccess) return fail((int)e, "nvfp4_window_attention: smem attribute: %s", cudaGetErrorString(e)); \
  }                                                                                               \
  window_attention_kernel<T, false><<<grid, 512, smem, st>>>(static_cast<const T*>(q), s_qz, s_qh, \
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
  const int chunk = (int)(((count + pieces - 1) / pieces + 3) / 4 * 4);
  const size_t esz = dtype == NVFP4_DT_FP32 ? 4 : 2;
  const size_t smem_plain = (size_t)(5 * g * d + g * chunk + 4) * sizeof(float);
  const size_t smem_staged = smem_plain + 2 * (size_t)chunk * d * esz;
  const bool staged = smem_staged <= 200 * 1024 && (d * esz) % 16 == 0 && ((uintptr_t)rk % 16) == 0 &&
                      ((uintptr_t)rv % 16) == 0;
  const size_t smem = staged ? smem_staged : smem_plain;
  NVFP4_REQUIRE(smem <= 200 * 1024, "nvfp4_window_partials: window piece too long (%d keys)", chunk);
  float* ws = static_cast<float*>(workspace);
  float* ws_acc = ws;
  float* ws_m = ws + total_slots * 16 * d;
  float* ws_l = ws_m + total_slots * 16;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((unsigned)(z * hk), (unsigned)pieces);
  auto launch = [&](auto kern) -> int {
    if (smem > 48 * 1024) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return fail((int)e, "nvfp4_window_partials: smem attribute: %s", cudaGetErrorString(e));
    }
    return 0;
  };
#define NVFP4_WINP(T)                                                                               \
  {                                                                                                 \
    int rc = staged ? launch(window_attention_kernel<T, true>) : launch(window_attention_kernel<T, false>); \
    if (rc) return rc;                                                                              \
    if (staged)                                                                                     \
      window_attention_kernel<T, true><<<grid, 512, smem, st>>>(                                    \
          static_cast<const T*>(q), s_qz, s_qh, static_cast<const T*>(rk), static_cast<const T*>(rv), (int)hk, g, d, \
          ring_cap, first_pos, (int)count, chunk, scaling, nullptr, nullptr, ws_acc, ws_m, ws_l, extra_base); \
    else                                                                                            \
      window_attention_kernel<T, false><<<grid, 512, smem, st>>>(                                   \
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
