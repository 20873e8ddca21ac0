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

// Exact attention of one query row per head over `count` ring-resident keys.
// One block (128 threads) per (z, h); scores live in shared memory.
template <typename T>
__global__ void __launch_bounds__(128) window_attention_kernel(
    const T* __restrict__ q, int64_t s_qz, int64_t s_qh, const T* __restrict__ rk,
    const T* __restrict__ rv, int hk, int g, int d, int64_t ring_cap, int64_t first_pos,
    int count, float scaling, float* __restrict__ out, float* __restrict__ lse) {
  extern __shared__ float sm[];
  float* qs = sm;           // d
  float* sc = sm + d;       // count
  __shared__ float red[4];
  const int h_all = hk * g;
  const int zi = blockIdx.x / h_all, hi = blockIdx.x % h_all;
  const int kh = hi / g;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const T* qp = q + zi * s_qz + hi * s_qh;
  for (int i = tid; i < d; i += 128) qs[i] = to_f32<T>(qp[i]);
  __syncthreads();
  const T* kb = rk + ((int64_t)(zi * hk + kh) * ring_cap) * d;
  const T* vb = rv + ((int64_t)(zi * hk + kh) * ring_cap) * d;
  float mloc = -INFINITY;
  for (int j = warp; j < count; j += 4) {
    const T* kr = kb + ((first_pos + j) % ring_cap) * d;
    float s = 0.0f;
    for (int i = lane; i < d; i += 32) s += qs[i] * to_f32<T>(kr[i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    s *= scaling;
    if (lane == 0) sc[j] = s;
    mloc = fmaxf(mloc, s);
  }
  if (lane == 0) red[warp] = mloc;
  __syncthreads();
  const float m = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
  __syncthreads();
  float lsum = 0.0f;
  for (int j = tid; j < count; j += 128) {
    const float e = expf(sc[j] - m);
    sc[j] = e;
    lsum += e;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
  if (lane == 0) red[warp] = lsum;
  __syncthreads();
  const float l = red[0] + red[1] + red[2] + red[3];
  for (int i = tid; i < d; i += 128) {
    float acc = 0.0f;
    for (int j = 0; j < count; ++j) acc += sc[j] * to_f32<T>(vb[((first_pos + j) % ring_cap) * d + i]);
    out[(int64_t)blockIdx.x * d + i] = acc / l;
  }
  if (tid == 0) lse[blockIdx.x] = m + logf(l);
}

template <typename T>
__global__ void lse_merge_kernel(const T* __restrict__ o1, const float* __restrict__ l1,
                                 const T* __restrict__ o2, const float* __restrict__ l2,
                                 T* __restrict__ out, int64_t rows, int d) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= rows * d) return;
  const int64_t r = i / d;
  const float a1 = l1[r], a2 = l2[r];
  const float m = fmaxf(a1, a2);
  const float w1 = expf(a1 - m), w2 = expf(a2 - m);
  out[i] = from_f32<T>((w1 * to_f32<T>(o1[i]) + w2 * to_f32<T>(o2[i])) / (w1 + w2));
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
  const size_t smem = (size_t)(d + count) * sizeof(float);
  NVFP4_REQUIRE(smem <= 48 * 1024, "nvfp4_window_attention: window too long (%lld keys)", (long long)count);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)(z * hk * g);
#define NVFP4_WIN(T)                                                                              \
  window_attention_kernel<T><<<grid, 128, smem, st>>>(static_cast<const T*>(q), s_qz, s_qh,       \
                                                      static_cast<const T*>(rk),                  \
                                                      static_cast<const T*>(rv), (int)hk, g, d,   \
                                                      ring_cap, first_pos, (int)count, scaling,   \
                                                      out, lse);                                  \
  return launch_result("nvfp4_window_attention")
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_WIN(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_WIN(__half);
    case NVFP4_DT_FP32: NVFP4_WIN(float);
    default: return fail(-1, "nvfp4_window_attention: unknown dtype %d", dtype);
  }
#undef NVFP4_WIN
}

extern "C" int nvfp4_lse_merge(const void* o1, const float* lse1, const void* o2, const float* lse2,
                               void* out, int dtype, int64_t rows, int d, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(o1 && o2 && lse1 && lse2 && out, "nvfp4_lse_merge: null pointer");
  if (rows * d == 0) return 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)((rows * d + 255) / 256);
#define NVFP4_MERGE(T)                                                                           \
  lse_merge_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(o1), lse1,                     \
                                            static_cast<const T*>(o2), lse2, static_cast<T*>(out), \
                                            rows, d);                                            \
  return launch_result("nvfp4_lse_merge")
  switch (dtype) {
    case NVFP4_DT_BF16: NVFP4_MERGE(__nv_bfloat16);
    case NVFP4_DT_FP16: NVFP4_MERGE(__half);
    case NVFP4_DT_FP32: NVFP4_MERGE(float);
    default: return fail(-1, "nvfp4_lse_merge: unknown dtype %d", dtype);
  }
#undef NVFP4_MERGE
}
