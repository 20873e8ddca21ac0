// V projection with the NVFP4 pack as its epilogue: V = X W^T (+ bias) is computed on the tensor
// cores and leaves the kernel as the V^T pack along the keys that the attention kernels read (and,
// optionally, as the 16-bit V itself), so the projected tensor is never re-read for quantisation.
// This is the "v_proj epilogue" producer the reference's notes ask callers to fuse.
//
// The product is formed TRANSPOSED, V^T[feature, token] = W[feature, :] . X[token, :], so that the
// accumulator puts one output feature (one row of the V^T pack) on one TMEM lane and 128 consecutive
// tokens on its columns: the 16-token groups of the pack are thread-local in the epilogue and a
// thread writes 64 contiguous nibble bytes + 8 scale bytes of its row.
//
// One CTA = 128 features x 128 tokens of one batch entry; K loop over the hidden dim in 64-element
// stages (TMA, 128-byte swizzle, 4-stage ring), tcgen05.mma kind::f16 M128 N128 K16, accumulator in
// 128 TMEM columns.  Warps: 0 TMA producer, 1 MMA issuer, 2-5 epilogue.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"
#include "common/bwd_util.cuh"

namespace nvfp4 {

constexpr int kVpThreads = 192;
constexpr int kVpStages = 4;
constexpr int kVpTile = 128 * 64 * 2;      // bytes of one operand tile of a stage

struct VprojParams {
  const void* bias;      // [features] in the operand dtype, or null
  uint8_t* vnv;          // [Z*Hk, D, s_pad/2]
  uint8_t* vsc;          // [Z*Hk, D, s_pad/16]
  void* v_out;           // [Z, S, features] (element strides svb, svs; unit feature stride) or null
  int64_t svb, svs;
  int features, d, hk, s, s_pad, hidden;
  int f16;
  int* status;
};

template <typename T>
__global__ void __launch_bounds__(kVpThreads, 1)
vproj_pack_kernel(const __grid_constant__ CUtensorMap tm_w, const __grid_constant__ CUtensorMap tm_x,
                  const VprojParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  __shared__ uint64_t full[kVpStages], empty[kVpStages], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int f0 = blockIdx.x * 128, t0 = blockIdx.y * 128, zi = blockIdx.z;
  const int nstage = (p.hidden + 63) / 64;
  if (tid == 0) {
    err = 0;
    for (int i = 0; i < kVpStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 128);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  if (warp == 0) {
    if (elect_one()) {
      for (int st = 0; st < nstage; ++st) {
        const int s = st % kVpStages;
        if (st >= kVpStages) mbar_wait(&empty[s], ((st / kVpStages) & 1) ^ 1, &err, 1);
        uint8_t* sb = smem + s * 2 * kVpTile;
        mbar_expect_tx(&full[s], 2 * kVpTile);
        tma_load_3d(sb, &tm_w, &full[s], st * 64, f0, 0);
        tma_load_3d(sb + kVpTile, &tm_x, &full[s], st * 64, t0, zi);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(128, 128, false, p.f16 != 0);
      for (int st = 0; st < nstage; ++st) {
        const int s = st % kVpStages;
        mbar_wait(&full[s], (st / kVpStages) & 1, &err, 2);
        tc_fence_after();
        const uint8_t* sb = smem + s * 2 * kVpTile;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem, desc_sw128(sb, k), desc_sw128(sb + kVpTile, k), idesc, (st > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      umma_commit(&acc_done);
    }
    __syncwarp();
  } else {
    // epilogue: thread = feature row f0 + 32 (warp % 4) + lane, columns = 128 tokens
    const int wq = warp & 3;
    const int f = f0 + wq * 32 + lane;
    const bool f_ok = f < p.features;
    const float b = (f_ok && p.bias != nullptr) ? to_f32<T>(static_cast<const T*>(p.bias)[f]) : 0.0f;
    mbar_wait(&acc_done, 0, &err, 3);
    tc_fence_after();
    const int64_t unit = (int64_t)zi * p.hk + (f_ok ? f / p.d : 0);
    const int dr = f_ok ? f % p.d : 0;
    uint8_t* nrow = p.vnv + (unit * p.d + dr) * (int64_t)(p.s_pad / 2) + t0 / 2;
    uint8_t* srow = p.vsc + (unit * p.d + dr) * (int64_t)(p.s_pad / 16) + t0 / 16;
    T* vo = p.v_out ? static_cast<T*>(p.v_out) + (int64_t)zi * p.svb + f : nullptr;
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      uint32_t r[32];
      tmem_ld32(tmem + ((uint32_t)(wq * 32) << 16) + c * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        const int tok = t0 + c * 32 + gi * 16;
        if (tok >= p.s_pad) continue;       // groups behind the padded extent do not exist
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          // what an unfused projection would have stored: rounded once to the operand dtype;
          // tokens behind S are +0.0
          const T hv = from_f32<T>(__uint_as_float(r[gi * 16 + e]) + b);
          v[e] = (tok + e < p.s) ? to_f32<T>(hv) : 0.0f;
          if (vo != nullptr && f_ok && tok + e < p.s) vo[(int64_t)(tok + e) * p.svs] = hv;
        }
        uint32_t lo, hi;
        const uint8_t sb = pack_group16(v, lo, hi);
        if (f_ok) {
          *reinterpret_cast<uint2*>(nrow + (c * 32 + gi * 16) / 2) = make_uint2(lo, hi);
          srow[(c * 32 + gi * 16) / 16] = sb;
        }
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 128);
}

}  // namespace nvfp4

extern "C" int nvfp4_vproj_pack(const void* x, const void* w, const void* bias, int dtype, int64_t z,
                                int64_t s, int64_t hidden, int64_t hk, int d, int64_t sxb, int64_t sxs,
                                int64_t s_pad, uint8_t* vnv, uint8_t* vsc, void* v_out, int64_t svb,
                                int64_t svs, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(dtype == NVFP4_DT_BF16 || dtype == NVFP4_DT_FP16, "nvfp4_vproj_pack: operands must be bf16 or fp16");
  NVFP4_REQUIRE(x && w && vnv && vsc, "nvfp4_vproj_pack: null pointer");
  NVFP4_REQUIRE(z >= 1 && s >= 1 && hk >= 1 && d >= 16 && d % 16 == 0, "nvfp4_vproj_pack: bad extents");
  NVFP4_REQUIRE(hidden >= 8 && hidden % 8 == 0, "nvfp4_vproj_pack: hidden size must be a multiple of 8");
  NVFP4_REQUIRE(s_pad % 16 == 0 && s_pad >= s, "nvfp4_vproj_pack: s_pad must be a multiple of 16 >= s");
  NVFP4_REQUIRE(sxb % 8 == 0 && sxs % 8 == 0, "nvfp4_vproj_pack: activation strides must be multiples of 8 elements");
  NVFP4_REQUIRE(((uintptr_t)vnv & 7) == 0 && (s_pad / 2) % 8 == 0, "nvfp4_vproj_pack: nibble rows must be 8-byte aligned");
  const int64_t features = hk * d;
  NVFP4_REQUIRE(features < (1LL << 30) && s_pad < (1LL << 30) && z < 65536 && (s_pad + 127) / 128 < 65536,
                "nvfp4_vproj_pack: problem too large");
  CUtensorMap t_w, t_x;
  int rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_w, w, (uint64_t)hidden, (uint64_t)features, 1, (uint64_t)hidden * 2,
                                    (uint64_t)features * hidden * 2, 128, "nvfp4_vproj_pack(W)")))
    return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_x, x, (uint64_t)hidden, (uint64_t)s, (uint64_t)z, (uint64_t)sxs * 2,
                                    (uint64_t)(z > 1 ? sxb : s * sxs) * 2, 128, "nvfp4_vproj_pack(X)")))
    return rc;
  VprojParams p;
  p.bias = bias; p.vnv = vnv; p.vsc = vsc; p.v_out = v_out; p.svb = svb; p.svs = svs;
  p.features = (int)features; p.d = d; p.hk = (int)hk; p.s = (int)s; p.s_pad = (int)s_pad; p.hidden = (int)hidden;
  p.f16 = dtype == NVFP4_DT_FP16 ? 1 : 0; p.status = status;
  const int smem = kVpStages * 2 * kVpTile + 1024;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)((features + 127) / 128), (unsigned)((s_pad + 127) / 128), (unsigned)z);
#define NVFP4_VP(T)                                                                                       \
  {                                                                                                       \
    cudaError_t e = cudaFuncSetAttribute(vproj_pack_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
    if (e != cudaSuccess) return fail((int)e, "nvfp4_vproj_pack: smem attribute: %s", cudaGetErrorString(e)); \
    vproj_pack_kernel<T><<<grid, kVpThreads, smem, st>>>(t_w, t_x, p);                                    \
    return launch_result("nvfp4_vproj_pack");                                                             \
  }
  if (dtype == NVFP4_DT_BF16) NVFP4_VP(__nv_bfloat16)
  NVFP4_VP(__half)
#undef NVFP4_VP
}
