// Backward of the NVFP4 flash attention with ALL GEMMs in NVFP4 (tcgen05.mma kind::mxf4nvf4,
// e4m3 scale per 16), sm_100a.  The "fp4_rownorm" mode of the training entry.
//
//   S  = Q K^T                     from the forward's packs of Q and K (along D)
//   P  = exp2(S * scaling * log2e - lse * log2e)
//   dP = dO' V^T                   dO' = dO / 2^e packed along D, V packed along D
//   dS = P o (dP - delta') * scaling
//   dV = P^T dO',  dK = dS^T Q,  dQ = dS K     A operand packed IN THE KERNEL along the contraction
//                                              axis, B operand = the transposed pack (dO'^T, Q^T, K^T)
//
// One kernel template serves both passes.  A CTA owns 128 "rows" and streams "columns" in stages
// of 128 (two 64-column steps per stage):
//   dK/dV pass  rows = keys of a (batch, kv-head) unit, columns = queries of every head of the GQA
//               group in turn (dK / dV are reduced over the group in TMEM and written once);
//   dQ pass     rows = queries of a head, columns = keys.
// Per step the issuer thread queues S (or S^T) and dP as two N=64 block-scaled MMAs each; a
// softmax thread owns one row and 16-column chunks of the step's 64 columns, so the per-16 packs of
// P and dS along the columns are thread-local: nibbles and scale bytes go to shared memory in the
// operand layout and feed one M128 N128 K64 MMA per gradient.  Six FP4 MMAs per step replace the
// twenty bf16 MMAs of the high-precision kernels.  Two teams of softmax warps alternate steps, so
// the TMEM loads and barrier waits of one step hide behind the arithmetic of the other; at D = 128
// two threads share a row (sixteen softmax warps, four per SM sub-partition: the per-element exp +
// pack work is bound by how many warps a sub-partition has to interleave), at D = 256 one.
//
// Keeping the packed operands inside the e4m3 scale range (2^-9 .. 448) -- the job of the
// reference's per-row rms normalisation, flash.py:184-228 -- is done with factors that never change
// while a CTA accumulates, so the sums stay in TMEM:
//   * dO is divided once by 2^e, the smallest power of two >= max|dO| (exact; found by the pre-pass);
//   * P is packed as P * 2^11 and dS as dS * 2^9: with per-16 scales reaching down to 2^-9 this keeps
//     full precision for P >= 6e-6 (uniform attention over 170 k keys) and flushes only below 2e-7;
//   * the constant factors are undone on the accumulators in the epilogue.
// Causal masking is bottom-right aligned; packed varlen is block-diagonal; an additive key bias
// enters the recompute of P.  Head dim 128, or 256 as two 128-wide output halves per tile (both
// halves recompute S and dP).  No atomics: results are run-to-run identical.  Every barrier wait
// is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"
#include "common/bwd_util.cuh"

namespace nvfp4 {

constexpr float kB4Log2e = 1.4426950408889634f;
constexpr float kB4PShift = 11.0f;   // P is packed as P * 2^11
constexpr int kB4Prefetch = 2;       // stages prefetched into L2 ahead of the ring


// kFp8: the gradient GEMMs' operands (P^T, dS^T, dS packed in the kernel; dO'^T, Q^T, K^T from the
// pre-pass) are MXFP8 -- e4m3 bytes, e8m0 scale per 32 -- instead of NVFP4: tiles of 128-byte rows.
template <int D, bool kFp8 = false>
struct B4Cfg {
  static constexpr int KSUB = D / 128;      // 64-byte-wide sub-tiles of a pack row
  static constexpr int KB = D / 64;         // K = 64 MMAs per product over D
  static constexpr int X = KSUB * 8192;     // one pack tile: 128 rows x D/2 bytes
  static constexpr int AT = kFp8 ? 16384 : 8192;   // an in-kernel operand tile / a transposed-pack tile
  // resident part
  static constexpr int O_X1 = 0, O_X2 = X, O_A1 = 2 * X, O_A2 = 2 * X + AT;
  static constexpr int O_XSF = 2 * X + 2 * AT;            // X1 atoms [KB], X2 atoms [KB]
  static constexpr int O_ASF = O_XSF + 2 * KB * 512;      // A1 atoms [2 parities], A2 atoms [2]
  static constexpr int RES = ((O_ASF + 2048 + 1023) / 1024) * 1024;
  // one stage = 128 columns
  static constexpr int S_Y1 = 0, S_Y2 = X, S_T1 = 2 * X, S_T2 = 2 * X + AT;
  static constexpr int S_YSF = 2 * X + 2 * AT;            // Y1 atoms [2 steps][KB], then Y2 atoms [2][KB]
  static constexpr int S_TSF = S_YSF + 4 * KB * 512;      // T1 atoms [2 parities], T2 atoms [2] (MXFP8: one each)
  static constexpr int S_AUX = S_TSF + 2048;              // two float[128]
  static constexpr int STAGE = ((S_AUX + 1024 + 1023) / 1024) * 1024;
  static constexpr int NSTAGE = D == 128 ? 3 : 2;
  // softmax threads per row: at D = 128 two (each owns 32 of a step's 64 columns; sixteen softmax
  // warps, four on every SM sub-partition), at D = 256 one (eight warps: there the MMAs of a step
  // take long enough to cover one warp per sub-partition and team)
  static constexpr int NP = D == 128 ? 2 : 1;
  static constexpr int THREADS = 128 + 256 * NP;
  static constexpr int TOTAL = RES + NSTAGE * STAGE + 1024;
  // TMEM columns
  static constexpr uint32_t T_ACC1 = 0, T_ACC2 = 128, T_S = 256, T_G = 384;
  static constexpr uint32_t T_SFX1 = 448, T_SFX2 = T_SFX1 + KB * 4, T_SFY = T_SFX2 + KB * 4;
  static constexpr uint32_t T_SFA1 = T_SFY + KB * 4, T_SFT1 = T_SFA1 + 4, T_SFA2 = T_SFT1 + 4, T_SFT2 = T_SFA2 + 4;
  static_assert(T_SFT2 + 4 <= 512, "TMEM budget");
  static_assert(TOTAL <= 227 * 1024, "shared memory budget");
};

// kind::mxf8f6f4, e4m3 x e4m3, ue8m0 scale per 32, fp32 accumulate, both operands K-major; a_sf / b_sf
// pick the byte of the scale word in tensor memory that holds this K = 32 block's scale.
__host__ __device__ __forceinline__ uint32_t make_idesc_mx8(uint32_t m, uint32_t n, uint32_t a_sf, uint32_t b_sf) {
  uint32_t d = 0;
  d |= (b_sf & 3u) << 4;
  d |= (n >> 3) << 17;
  d |= 1u << 23;         // scale format: ue8m0
  d |= (m >> 4) << 24;
  d |= (a_sf & 3u) << 29;
  return d;              // A and B format 0 = e4m3
}
__device__ __forceinline__ void umma_mx8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t sfa_tmem, uint32_t sfb_tmem, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale.block32 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

struct B4Params {
  const uint8_t* x1sc;   // row side, along D: [RB, R, D/16]   (dK/dV: K scales; dQ: Q scales)
  const uint8_t* x2sc;   //                                    (dK/dV: V scales; dQ: dO' scales)
  const uint8_t* y1sc;   // column side, along D: [CB, C, D/16] (dK/dV: Q; dQ: K)
  const uint8_t* y2sc;   //                                    (dK/dV: dO'; dQ: V)
  const uint8_t* t1sc;   // transposed packs: [CB, D, c_pad/16] (dK/dV: dO'^T; dQ: unused)
  const uint8_t* t2sc;   //                                    (dK/dV: Q^T; dQ: K^T)
  const float* lse;      // [ZH, Sq] natural log
  const float* delta;    // [ZH, Sq] rowsum(dO o O), in units of dO
  const float* amax;     // device float: max|dO| (the pre-scale of the dO packs is 2^-ceil(log2 amax))
  const float* bias;     // [Z, Skv] additive key bias or null
  const int32_t* seq_start;  // [S] or null (packed varlen)
  const int32_t* seq_end;
  void* out1;            // dK/dV: dV [ZHk, Skv, D]
  void* out2;            // dK/dV: dK [ZHk, Skv, D]; dQ: dQ [ZH, Sq, D]
  int h, hk, g;
  int s_q, s_kv, c_pad;  // c_pad: padded column extent of the transposed packs
  float scaling;
  int causal;
  int sr_p, sr_ds;       // stochastic rounding of the in-kernel P / dS packs (fp4_legacy mode)
  uint32_t seed;
  int* status;
};

__device__ __forceinline__ float b4_max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float b4_absmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(fabsf(b)), "f"(fabsf(c)));
  return d;
}

// 16 values -> 8 nibble bytes (two words) and the e4m3 scale byte, with the packer's scale rule; the
// divisions are reciprocal multiplies here (these operands exist only inside the kernel).
// With sr the e2m1 convert rounds stochastically from the bits of (seed, ca, cb .. cb + 3).
template <bool kSigned>
__device__ __forceinline__ uint32_t b4_pack16(const float* x, uint32_t& lo, uint32_t& hi, bool sr = false,
                                              uint32_t seed = 0, uint32_t ca = 0, uint32_t cb = 0) {
  float m;
  if constexpr (kSigned) {
    m = fabsf(x[0]);
#pragma unroll
    for (int e = 1; e < 15; e += 2) m = b4_absmax3(m, x[e], x[e + 1]);
    m = fmaxf(m, fabsf(x[15]));
  } else {
    m = x[0];
#pragma unroll
    for (int e = 1; e < 15; e += 2) m = b4_max3(m, x[e], x[e + 1]);
    m = fmaxf(m, x[15]);
  }
  uint32_t sb;
  float inv;
  {
    const float s32 = fminf(fmaxf(m * 0.16666667f, kScaleFloor), kScaleMax);
    uint16_t sb16;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sb16) : "f"(0.0f), "f"(s32));
    uint32_t h2;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(sb16));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(__half2float(__ushort_as_half((unsigned short)(h2 & 0xFFFF)))));
    sb = sb16 & 0xFFu;
  }
  const float2 i2 = make_float2(inv, inv);
  float2 y[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) y[e] = __fmul2_rn(make_float2(x[2 * e], x[2 * e + 1]), i2);
  if (sr) {
    uint32_t q[4];
#pragma unroll
    for (int e = 0; e < 4; ++e)
      q[e] = e2m1x4_sr(y[2 * e].x, y[2 * e].y, y[2 * e + 1].x, y[2 * e + 1].y, sr_bits(seed, ca, cb + e));
    lo = q[0] | (q[1] << 16);
    hi = q[2] | (q[3] << 16);
    return sb;
  }
  lo = e2m1x8(y[0].x, y[0].y, y[1].x, y[1].y, y[2].x, y[2].y, y[3].x, y[3].y);
  hi = e2m1x8(y[4].x, y[4].y, y[5].x, y[5].y, y[6].x, y[6].y, y[7].x, y[7].y);
  return sb;
}

__device__ __forceinline__ void sts_v4(uint32_t saddr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(saddr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void sts_b8(uint32_t saddr, uint32_t a) {
  asm volatile("st.shared.b8 [%0], %1;" ::"r"(saddr), "h"((uint16_t)a) : "memory");
}
__device__ __forceinline__ void sts_b16(uint32_t saddr, uint32_t a) {
  asm volatile("st.shared.b16 [%0], %1;" ::"r"(saddr), "h"((uint16_t)a) : "memory");
}

// kDkdv = true: the dK/dV pass (rows = keys), false: the dQ pass (rows = queries).
// kMode: 0 = NVFP4 gradient operands rounded to nearest, 1 = NVFP4 with the stochastic-rounding
// flags honoured (a kernel of its own, so the common case carries none of it), 2 = MXFP8.
template <int D, bool kDkdv, typename TG, int kMode>
__global__ void __launch_bounds__((B4Cfg<D, kMode == 2>::THREADS), 1)
bwd4_kernel(const __grid_constant__ CUtensorMap tm_x1, const __grid_constant__ CUtensorMap tm_x2,
            const __grid_constant__ CUtensorMap tm_y1, const __grid_constant__ CUtensorMap tm_y2,
            const __grid_constant__ CUtensorMap tm_t1, const __grid_constant__ CUtensorMap tm_t2,
            const B4Params p) {
  constexpr bool kFp8 = kMode == 2, kSr = kMode == 1;
  using C = B4Cfg<D, kFp8>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_res = smem;
  uint8_t* s_stage = smem + C::RES;

  __shared__ uint64_t full_tma[C::NSTAGE], full_aux[C::NSTAGE], empty[C::NSTAGE];
  __shared__ uint64_t x_full, xsf_full, s_full[2], s_free[2], g_full, g_free, a_full[2], a_free[2], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  __shared__ float gs_s;      // the power-of-two pre-scale of dO

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int half = blockIdx.z;     // 128-wide slice of the head dim owned by this CTA (D = 256)
  const int shift = p.s_kv - p.s_q;
  const bool varlen = p.seq_start != nullptr;

  // ---- rows of this CTA, and the range of 128-column stages it has to visit
  int rb, row0, zi, kh = 0, cb0;     // row batch entry, first row, batch index, kv head, first column batch entry
  int R, Ccols;                      // row / column extents
  int c_lo = 0, c_hi = 0;
  if constexpr (kDkdv) {
    rb = blockIdx.x;                 // z * hk + kh
    row0 = blockIdx.y * 128;
    zi = rb / p.hk; kh = rb % p.hk;
    cb0 = zi * p.h + kh * p.g;
    R = p.s_kv; Ccols = p.s_q;
    c_lo = p.causal ? max(0, row0 - shift) : 0;
    c_hi = p.s_q;
    if (varlen) {
      c_lo = max(c_lo, (int)p.seq_start[min(row0, p.s_kv - 1)]);
      c_hi = min(c_hi, (int)p.seq_end[min(row0 + 127, p.s_kv - 1)]);
    }
  } else {
    rb = blockIdx.x;                 // z * h + hi
    row0 = (gridDim.y - 1 - blockIdx.y) * 128;   // late query tiles see the most keys: first
    zi = rb / p.h;
    cb0 = zi * p.hk + (rb % p.h) / p.g;
    R = p.s_q; Ccols = p.s_kv;
    c_hi = p.causal ? max(0, min(p.s_kv, row0 + 128 + shift)) : p.s_kv;
    if (varlen) {
      c_lo = p.seq_start[min(row0, p.s_q - 1)];
      c_hi = min(c_hi, (int)p.seq_end[min(row0 + 127, p.s_q - 1)]);
    }
  }
  const int i_lo = c_lo / 128;
  const int n_i = max((c_hi + 127) / 128 - i_lo, 0);
  const int nstage = (kDkdv ? p.g : 1) * n_i;
  const int nstep = 2 * nstage;

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(&full_tma[i], 1);
      mbar_init(&full_aux[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&x_full, 1);
    mbar_init(&xsf_full, 1);
    mbar_init(&g_full, 1);
    mbar_init(&g_free, 4 * C::NP);
    mbar_init(&acc_done, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_free[b], 4 * C::NP);
      mbar_init(&a_full[b], 4 * C::NP);
      mbar_init(&a_free[b], 1);
    }
    mbar_fence_init();
    gs_s = pow2_ceil(p.amax != nullptr ? *p.amax : 1.0f);
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const float gs = gs_s;

  // stage index -> (column batch entry, first column)
  auto stage_cols = [&](int sg, int& cb, int& col0) {
    if constexpr (kDkdv) {
      cb = cb0 + sg / n_i;
      col0 = (i_lo + sg % n_i) * 128;
    } else {
      cb = cb0;
      col0 = (i_lo + sg) * 128;
    }
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && nstep > 0) {
      mbar_expect_tx(&x_full, 2 * C::X);
#pragma unroll
      for (int c = 0; c < C::KSUB; ++c) {
        tma_load_3d(s_res + C::O_X1 + c * 8192, &tm_x1, &x_full, c * 64, row0, rb);
        tma_load_3d(s_res + C::O_X2 + c * 8192, &tm_x2, &x_full, c * 64, row0, rb);
      }
      auto prefetch = [&](int sg) {
        int cb, col0;
        stage_cols(sg, cb, col0);
#pragma unroll
        for (int c = 0; c < C::KSUB; ++c) {
          tma_prefetch_3d(&tm_y1, c * 64, col0, cb);
          tma_prefetch_3d(&tm_y2, c * 64, col0, cb);
        }
        if constexpr (kDkdv) tma_prefetch_3d(&tm_t1, kFp8 ? col0 : col0 / 2, half * 128, cb);
        tma_prefetch_3d(&tm_t2, kFp8 ? col0 : col0 / 2, half * 128, cb);
      };
      for (int sg = C::NSTAGE; sg < min(nstage, C::NSTAGE + kB4Prefetch); ++sg) prefetch(sg);
      for (int sg = 0; sg < nstage; ++sg) {
        const int s = sg % C::NSTAGE;
        int cb, col0;
        stage_cols(sg, cb, col0);
        if (sg + C::NSTAGE + kB4Prefetch < nstage) prefetch(sg + C::NSTAGE + kB4Prefetch);
        if (sg >= C::NSTAGE) mbar_wait(&empty[s], ((sg / C::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* sb = s_stage + s * C::STAGE;
        mbar_expect_tx(&full_tma[s], 2 * C::X + (kDkdv ? 2 : 1) * C::AT);
#pragma unroll
        for (int c = 0; c < C::KSUB; ++c) {
          tma_load_3d(sb + C::S_Y1 + c * 8192, &tm_y1, &full_tma[s], c * 64, col0, cb);
          tma_load_3d(sb + C::S_Y2 + c * 8192, &tm_y2, &full_tma[s], c * 64, col0, cb);
        }
        if constexpr (kDkdv) tma_load_3d(sb + C::S_T1, &tm_t1, &full_tma[s], kFp8 ? col0 : col0 / 2, half * 128, cb);
        tma_load_3d(sb + C::S_T2, &tm_t2, &full_tma[s], kFp8 ? col0 : col0 / 2, half * 128, cb);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale atoms, per-column statistics
    if (nstep > 0) {
      const uint32_t xsf = smem_u32(s_res + C::O_XSF);
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = lane + 32 * r4;
        const bool ok = row0 + r < R;
        const int64_t gi = ((int64_t)rb * R + (ok ? row0 + r : 0)) * (D / 16);
#pragma unroll
        for (int c = 0; c < C::KB; ++c) {
          cp_async_4(xsf + c * 512 + sf_atom_offset(r, 0), p.x1sc + gi + 4 * c, ok ? 4u : 0u);
          cp_async_4(xsf + (C::KB + c) * 512 + sf_atom_offset(r, 0), p.x2sc + gi + 4 * c, ok ? 4u : 0u);
        }
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&xsf_full);
      const float inv_gs = 1.0f / gs;
      const int csc = p.c_pad / (kFp8 ? 32 : 16);      // scale bytes per row of a transposed pack
      for (int sg = 0; sg < nstage; ++sg) {
        const int s = sg % C::NSTAGE;
        int cb, col0;
        stage_cols(sg, cb, col0);
        if (sg >= C::NSTAGE) mbar_wait(&empty[s], ((sg / C::NSTAGE) & 1) ^ 1, &err, 2);
        uint8_t* sb = s_stage + s * C::STAGE;
        const uint32_t ysf = smem_u32(sb + C::S_YSF), tsf = smem_u32(sb + C::S_TSF);
        float* aux = reinterpret_cast<float*>(sb + C::S_AUX);
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int r = lane + 32 * r4;            // column within the stage / row of a transposed tile
          const int col = col0 + r;
          const bool ok = col < Ccols;
          const int pp = r >> 6, rr = r & 63;
          const int64_t gi = ((int64_t)cb * Ccols + (ok ? col : 0)) * (D / 16);
#pragma unroll
          for (int c = 0; c < C::KB; ++c) {
            cp_async_4(ysf + (pp * C::KB + c) * 512 + sf_atom_offset(rr, 0), p.y1sc + gi + 4 * c, ok ? 4u : 0u);
            cp_async_4(ysf + ((2 + pp) * C::KB + c) * 512 + sf_atom_offset(rr, 0), p.y2sc + gi + 4 * c, ok ? 4u : 0u);
          }
          // transposed packs: row = feature (this CTA's 128-wide half), 8 scale bytes = this stage's columns
          if constexpr (kFp8) {     // one word = the four 32-column blocks of the stage
            const int64_t ti = ((int64_t)cb * D + half * 128 + r) * csc + col0 / 32;
            if constexpr (kDkdv) cp_async_4(tsf + sf_atom_offset(r, 0), p.t1sc + ti, 4u);
            cp_async_4(tsf + 2 * 512 + sf_atom_offset(r, 0), p.t2sc + ti, 4u);
          } else {
            const int64_t ti = ((int64_t)cb * D + half * 128 + r) * csc + col0 / 16;
#pragma unroll
            for (int pq = 0; pq < 2; ++pq) {
              if constexpr (kDkdv) cp_async_4(tsf + pq * 512 + sf_atom_offset(r, 0), p.t1sc + ti + 4 * pq, 4u);
              cp_async_4(tsf + (2 + pq) * 512 + sf_atom_offset(r, 0), p.t2sc + ti + 4 * pq, 4u);
            }
          }
          if constexpr (kDkdv) {
            // per query: -lse * log2e + 11 (exponent offset of P * 2^11) and -delta' * scaling / 4
            const int64_t qi = (int64_t)cb * p.s_q + (ok ? col : 0);
            aux[r] = ok ? fmaf(-p.lse[qi], kB4Log2e, kB4PShift) : 0.0f;
            aux[128 + r] = ok ? -p.delta[qi] * inv_gs * (p.scaling * 0.25f) : 0.0f;
          } else {
            // per key: the additive bias in base-2 units
            aux[r] = (p.bias != nullptr && ok) ? p.bias[(int64_t)zi * p.s_kv + col] * kB4Log2e : 0.0f;
          }
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_aux[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && nstep > 0) {
      const uint32_t id_n64 = make_idesc_nvfp4(128, 64);
      const uint32_t id_n128 = make_idesc_nvfp4(128, 128);
      mbar_wait(&x_full, 0, &err, 3);
      mbar_wait(&xsf_full, 0, &err, 4);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < C::KB; ++c) {
        tmem_cp_32x128b_warpx4(tmem + C::T_SFX1 + 4 * c, smem_u32(s_res + C::O_XSF + c * 512));
        tmem_cp_32x128b_warpx4(tmem + C::T_SFX2 + 4 * c, smem_u32(s_res + C::O_XSF + (C::KB + c) * 512));
      }
      const uint64_t d_x1 = desc_sw64(s_res + C::O_X1, 0), d_x2 = desc_sw64(s_res + C::O_X2, 0);
      const uint64_t d_a1 = kFp8 ? desc_sw128(s_res + C::O_A1, 0) : desc_sw64(s_res + C::O_A1, 0);
      const uint64_t d_a2 = kFp8 ? desc_sw128(s_res + C::O_A2, 0) : desc_sw64(s_res + C::O_A2, 0);
      const uint64_t d_y1 = desc_sw64(s_stage + C::S_Y1, 0), d_y2 = desc_sw64(s_stage + C::S_Y2, 0);
      const uint64_t d_t1 = kFp8 ? desc_sw128(s_stage + C::S_T1, 0) : desc_sw64(s_stage + C::S_T1, 0);
      const uint64_t d_t2 = kFp8 ? desc_sw128(s_stage + C::S_T2, 0) : desc_sw64(s_stage + C::S_T2, 0);
      // acc1 += A1 T1^T, acc2 += A2 T2^T for step t (columns [64 pp, 64 pp + 64) of its stage)
      auto grad_gemms = [&](int t) {
        const int pp = t & 1, s = (t >> 1) % C::NSTAGE;
        uint8_t* sb = s_stage + s * C::STAGE;
        mbar_wait(&a_full[pp], (t >> 1) & 1, &err, 8);
        tc_fence_after();
        const uint32_t acc = t > 0 ? 1u : 0u;
        if constexpr (kFp8) {
          // a step is two K = 32 blocks (32 bytes each) of the 128-byte operand rows; block j of step pp
          // reads byte j of the A atom (one atom per step parity) and byte 2 pp + j of the T atom
          const uint64_t sg = (uint64_t)(s * (C::STAGE >> 4));
          if constexpr (kDkdv) {
            tmem_cp_32x128b_warpx4(tmem + C::T_SFA1, smem_u32(s_res + C::O_ASF + pp * 512));
            tmem_cp_32x128b_warpx4(tmem + C::T_SFT1, smem_u32(sb + C::S_TSF));
          }
          tmem_cp_32x128b_warpx4(tmem + C::T_SFA2, smem_u32(s_res + C::O_ASF + (2 + pp) * 512));
          tmem_cp_32x128b_warpx4(tmem + C::T_SFT2, smem_u32(sb + C::S_TSF + 2 * 512));
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            const uint32_t kk = (uint32_t)(pp * 2 + j);
            const uint32_t id = make_idesc_mx8(128, 128, (uint32_t)j, kk);
            if constexpr (kDkdv)
              umma_mx8(tmem + C::T_ACC1, d_a1 + kk * 2, d_t1 + sg + kk * 2, id, tmem + C::T_SFA1, tmem + C::T_SFT1,
                       j > 0 ? 1u : acc);
            umma_mx8(tmem + C::T_ACC2, d_a2 + kk * 2, d_t2 + sg + kk * 2, id, tmem + C::T_SFA2, tmem + C::T_SFT2,
                     j > 0 ? 1u : acc);
          }
          umma_commit(&a_free[pp]);
          if (pp == 1) umma_commit(&empty[s]);
          return;
        }
        const uint64_t so = (uint64_t)(s * (C::STAGE >> 4)) + (uint64_t)(pp * 2);   // stage, then the 32-byte half of a row
        if constexpr (kDkdv) {
          tmem_cp_32x128b_warpx4(tmem + C::T_SFA1, smem_u32(s_res + C::O_ASF + pp * 512));
          tmem_cp_32x128b_warpx4(tmem + C::T_SFT1, smem_u32(sb + C::S_TSF + pp * 512));
          umma_nvfp4(tmem + C::T_ACC1, d_a1 + pp * 2, d_t1 + so, id_n128, tmem + C::T_SFA1, tmem + C::T_SFT1, acc);
        }
        tmem_cp_32x128b_warpx4(tmem + C::T_SFA2, smem_u32(s_res + C::O_ASF + (2 + pp) * 512));
        tmem_cp_32x128b_warpx4(tmem + C::T_SFT2, smem_u32(sb + C::S_TSF + (2 + pp) * 512));
        umma_nvfp4(tmem + C::T_ACC2, d_a2 + pp * 2, d_t2 + so, id_n128, tmem + C::T_SFA2, tmem + C::T_SFT2, acc);
        umma_commit(&a_free[pp]);
        if (pp == 1) umma_commit(&empty[s]);
      };
      for (int st = 0; st < nstep; ++st) {
        const int pp = st & 1, sg = st >> 1, s = sg % C::NSTAGE;
        uint8_t* sb = s_stage + s * C::STAGE;
        if (pp == 0) {
          const uint32_t ph = (sg / C::NSTAGE) & 1;
          mbar_wait(&full_tma[s], ph, &err, 5);
          mbar_wait(&full_aux[s], ph, &err, 6);
        }
        if (st >= 2) mbar_wait(&s_free[pp], ((st >> 1) - 1) & 1, &err, 7);
        tc_fence_after();
        const uint64_t so = (uint64_t)(s * (C::STAGE >> 4)) + (uint64_t)(pp * 256);   // 64 rows x 64 bytes further
        // S (or S^T): rows x this step's 64 columns
#pragma unroll
        for (int c = 0; c < C::KB; ++c)
          tmem_cp_32x128b_warpx4(tmem + C::T_SFY + 4 * c, smem_u32(sb + C::S_YSF + (pp * C::KB + c) * 512));
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          umma_nvfp4(tmem + C::T_S + pp * 64, d_x1 + (k >> 1) * 512 + (k & 1) * 2, d_y1 + so + (k >> 1) * 512 + (k & 1) * 2,
                     id_n64, tmem + C::T_SFX1 + k * 4, tmem + C::T_SFY + k * 4, k > 0);
        umma_commit(&s_full[pp]);
        if (st > 0) {
          mbar_wait(&g_free, (st - 1) & 1, &err, 9);
          tc_fence_after();
        }
        // dP (or dP^T)
#pragma unroll
        for (int c = 0; c < C::KB; ++c)
          tmem_cp_32x128b_warpx4(tmem + C::T_SFY + 4 * c, smem_u32(sb + C::S_YSF + ((2 + pp) * C::KB + c) * 512));
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          umma_nvfp4(tmem + C::T_G, d_x2 + (k >> 1) * 512 + (k & 1) * 2, d_y2 + so + (k >> 1) * 512 + (k & 1) * 2,
                     id_n64, tmem + C::T_SFX2 + k * 4, tmem + C::T_SFY + k * 4, k > 0);
        umma_commit(&g_full);
        // The gradient GEMMs trail by two steps: S and dP of step st are queued while the team that
        // will consume them is still finishing step st - 2, so it finds them ready when it is done;
        // waiting here for step st - 1 instead would put the whole MMA round trip between two steps
        // of a team.
        if (st > 1) grad_gemms(st - 2);
      }
      grad_gemms(nstep - 2);
      grad_gemms(nstep - 1);
      umma_commit(&acc_done);
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax teams, epilogue
    // Two teams alternate steps (team t owns the steps of parity t, hence S slot t and half t of the
    // operand tiles' rows), so one team's TMEM loads and barrier waits overlap the other team's
    // arithmetic.  NP threads share a row: thread h of a row owns 64 / NP of the step's 64 columns,
    // as 16-column chunks whose packs are thread-local.
    constexpr int NP = C::NP, NCH = 4 / NP;               // chunks per thread and step
    const int team = (warp - 4) / (4 * NP);
    const int h = ((warp - 4) >> 2) % NP;
    const int part = team * NP + h;       // epilogue: which 64 / NP accumulator columns this thread stores
    const int wq = warp & 3;
    const int row_in = wq * 32 + lane;
    const int row = row0 + row_in;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c2 = p.scaling * kB4Log2e;
    const float cds = p.scaling * 0.25f;           // dS * 2^9 = (P * 2^11) * (dP - delta') * scaling / 4
    const bool row_ok = row < R;
    const bool has_bias = p.bias != nullptr;
    // visible columns of this row: [lo, hi); per-row terms of the exponent and of dS
    int lo = 0, hi = 0;
    float row_e = 0.0f, row_nd = 0.0f;
    if constexpr (kDkdv) {
      if (row_ok) {
        lo = p.causal ? max(row - shift, 0) : 0;
        hi = p.s_q;
        if (varlen) {
          lo = max(lo, (int)p.seq_start[row]);
          hi = min(hi, (int)p.seq_end[row]);
        }
        hi = max(hi, lo);
        if (has_bias) row_e = p.bias[(int64_t)zi * p.s_kv + row] * kB4Log2e;
      }
    } else {
      if (row_ok) {
        hi = p.causal ? min(p.s_kv, row + shift + 1) : p.s_kv;
        if (varlen) {
          lo = p.seq_start[row];
          hi = min(hi, (int)p.seq_end[row]);
        }
        hi = max(hi, lo);
        row_e = fmaf(-p.lse[(int64_t)rb * p.s_q + row], kB4Log2e, kB4PShift);
        row_nd = -p.delta[(int64_t)rb * p.s_q + row] * (1.0f / gs) * cds;
      }
    }
    const uint32_t a1_s = smem_u32(s_res + C::O_A1), a2_s = smem_u32(s_res + C::O_A2);
    const uint32_t asf_s = smem_u32(s_res + C::O_ASF);
    const float2 c22 = make_float2(c2, c2), cds2 = make_float2(cds, cds);
    // dQ pass: the per-row exponent offset and -delta' term; dK/dV pass: these come per column from aux
    const float2 re2 = kDkdv ? make_float2(0.0f, 0.0f) : make_float2(row_e, row_e);
    const float2 rnd2 = make_float2(row_nd, row_nd);
    for (int st = team; st < nstep; st += 2) {
      const int pp = team, sg = st >> 1, s = sg % C::NSTAGE;
      int cb, col0;
      stage_cols(sg, cb, col0);
      const float* aux0 = reinterpret_cast<const float*>(s_stage + s * C::STAGE + C::S_AUX) + 64 * pp;
      const int cs0 = col0 + 64 * pp;                // first column of the step
      const bool masked = !__all_sync(0xffffffffu, cs0 >= lo && cs0 + 64 <= hi);
      mbar_wait(&full_aux[s], (sg / C::NSTAGE) & 1, &err, 10);
      mbar_wait(&s_full[pp], (st >> 1) & 1, &err, 11);
      mbar_wait(&g_full, st & 1, &err, 12);
      tc_fence_after();
      uint32_t wp[4], wd[4], scp = 0u, scd = 0u;
      float pkeep[kFp8 ? 16 : 1], dkeep[kFp8 ? 16 : 1];     // MXFP8: the even chunk of a 32-column group
      // one 16-column chunk: S and dP (or dP^T) values -> P, dS -> packs -> operand tiles
      auto chunk = [&](int ch, const uint32_t (&cur)[16], const uint32_t* gsrc) {
        const float* aux = aux0 + 16 * ch;
        float pf[16], ds[16];
#pragma unroll
        for (int e = 0; e < 16; e += 4) {
          float2 eo01 = re2, eo23 = re2, nd01 = rnd2, nd23 = rnd2;
          if constexpr (kDkdv) {
            const float4 a4 = *reinterpret_cast<const float4*>(aux + e);
            const float4 n4 = *reinterpret_cast<const float4*>(aux + 128 + e);
            eo01 = make_float2(a4.x, a4.y); eo23 = make_float2(a4.z, a4.w);
            nd01 = make_float2(n4.x, n4.y); nd23 = make_float2(n4.z, n4.w);
          }
          const float2 t01 = __ffma2_rn(make_float2(__uint_as_float(cur[e]), __uint_as_float(cur[e + 1])), c22, eo01);
          const float2 t23 = __ffma2_rn(make_float2(__uint_as_float(cur[e + 2]), __uint_as_float(cur[e + 3])), c22, eo23);
          const float2 a01 = __ffma2_rn(make_float2(__uint_as_float(gsrc[e]), __uint_as_float(gsrc[e + 1])), cds2, nd01);
          const float2 a23 = __ffma2_rn(make_float2(__uint_as_float(gsrc[e + 2]), __uint_as_float(gsrc[e + 3])), cds2, nd23);
          pf[e] = t01.x; pf[e + 1] = t01.y; pf[e + 2] = t23.x; pf[e + 3] = t23.y;
          ds[e] = a01.x; ds[e + 1] = a01.y; ds[e + 2] = a23.x; ds[e + 3] = a23.y;
        }
        if (has_bias) {           // row bias (dK/dV pass) or column bias (dQ pass), base-2 units
#pragma unroll
          for (int e = 0; e < 16; ++e) pf[e] += kDkdv ? row_e : aux[e];
        }
#pragma unroll
        for (int e = 0; e < 16; ++e) pf[e] = ex2_bwd(pf[e]);
        if (masked) {
#pragma unroll
          for (int e = 0; e < 16; ++e) pf[e] = (cs0 + 16 * ch + e >= lo && cs0 + 16 * ch + e < hi) ? pf[e] : 0.0f;
        }
#pragma unroll
        for (int e = 0; e < 16; e += 2) {
          const float2 d2 = __fmul2_rn(make_float2(pf[e], pf[e + 1]), make_float2(ds[e], ds[e + 1]));
          ds[e] = d2.x; ds[e + 1] = d2.y;
        }
        if constexpr (kFp8) {
          if (!(ch & 1)) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              if constexpr (kDkdv) pkeep[e] = pf[e];
              dkeep[e] = ds[e];
            }
          } else {
            if (ch == NCH * h + 1 && st >= 2) mbar_wait(&a_free[pp], ((st >> 1) - 1) & 1, &err, 13);
            const int gi = ch >> 1;                       // which 32 columns of the step
            const uint32_t byte0 = (uint32_t)(pp * 64 + gi * 32);
            uint32_t w[8];
            if constexpr (kDkdv) {
              const uint32_t sb8 = pack_group32_mx8(pkeep, pf, w);
              sts_v4(a1_s + sw128_offset(row_in, byte0), w[0], w[1], w[2], w[3]);
              sts_v4(a1_s + sw128_offset(row_in, byte0 + 16), w[4], w[5], w[6], w[7]);
              sts_b8(asf_s + pp * 512 + sf_atom_offset(row_in, gi), sb8);
            }
            const uint32_t sd8 = pack_group32_mx8(dkeep, ds, w);
            sts_v4(a2_s + sw128_offset(row_in, byte0), w[0], w[1], w[2], w[3]);
            sts_v4(a2_s + sw128_offset(row_in, byte0 + 16), w[4], w[5], w[6], w[7]);
            sts_b8(asf_s + (2 + pp) * 512 + sf_atom_offset(row_in, gi), sd8);
          }
        } else {
        // random-bit counters: (tensor, row of the CTA's unit) and the quad's column within the unit
        if constexpr (kSr) {
          const uint32_t sr_row = (uint32_t)((int64_t)rb * R + row) * 4u + (kDkdv ? 0u : 2u);
          const uint32_t sr_col = (uint32_t)(st * 16 + ch * 4);
          if constexpr (kDkdv)
            scp |= b4_pack16<false>(pf, wp[2 * (ch & 1)], wp[2 * (ch & 1) + 1], p.sr_p != 0, p.seed, sr_row + 1u, sr_col)
                   << (8 * (ch & 1));
          scd |= b4_pack16<true>(ds, wd[2 * (ch & 1)], wd[2 * (ch & 1) + 1], p.sr_ds != 0, p.seed, sr_row, sr_col)
                 << (8 * (ch & 1));
        } else {
          if constexpr (kDkdv) scp |= b4_pack16<false>(pf, wp[2 * (ch & 1)], wp[2 * (ch & 1) + 1]) << (8 * (ch & 1));
          scd |= b4_pack16<true>(ds, wd[2 * (ch & 1)], wd[2 * (ch & 1) + 1]) << (8 * (ch & 1));
        }
        if (ch & 1) {
          // the operand tiles of step st - 2 (same half of the rows' bytes) must have been consumed
          if (ch == NCH * h + 1 && st >= 2) mbar_wait(&a_free[pp], ((st >> 1) - 1) & 1, &err, 13);
          const int c2i = ch >> 1;      // which 32 columns of the step
          if constexpr (kDkdv) {
            sts_v4(a1_s + sw64_offset(row_in, pp * 32 + c2i * 16), wp[0], wp[1], wp[2], wp[3]);
            sts_b16(asf_s + pp * 512 + sf_atom_offset(row_in, c2i * 2), scp);
            scp = 0u;
          }
          sts_v4(a2_s + sw64_offset(row_in, pp * 32 + c2i * 16), wd[0], wd[1], wd[2], wd[3]);
          sts_b16(asf_s + (2 + pp) * 512 + sf_atom_offset(row_in, c2i * 2), scd);
          scd = 0u;
        }
        }
      };
      if constexpr (NP == 1) {
        // dP (or dP^T): all 64 columns at once, so the single slot goes back to the issuer right away;
        // S in 16-column chunks, the next one in flight while the current one is worked on
        uint32_t g0[32], g1[32], sa[16], sb[16];
        tmem_ld32(tmem + lane_addr + C::T_G, g0);
        tmem_ld32(tmem + lane_addr + C::T_G + 32, g1);
        tmem_ld16(tmem + lane_addr + C::T_S + pp * 64, sa);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&g_free);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          if (ch < 3) {
            if (ch & 1) tmem_ld16(tmem + lane_addr + C::T_S + pp * 64 + 16 * (ch + 1), sa);
            else tmem_ld16(tmem + lane_addr + C::T_S + pp * 64 + 16 * (ch + 1), sb);
          }
          chunk(ch, (ch & 1) ? sb : sa, ch < 2 ? g0 + 16 * ch : g1 + 16 * (ch - 2));
          if (ch < 3) {
            tmem_ld_wait();
            if (ch == 2) {          // the last chunk of S is in registers: the slot goes back
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&s_free[pp]);
            }
          }
        }
      } else {
        // this thread's 32 columns of dP (or dP^T) arrive with the first S chunk, so the single dP slot
        // goes back to the issuer after one round trip; the S slot follows with the second chunk
        uint32_t gq[32];
        tmem_ld32(tmem + lane_addr + C::T_G + 32 * h, gq);
#pragma unroll
        for (int cc = 0; cc < NCH; ++cc) {
          const int ch = NCH * h + cc;
          uint32_t cur[16];
          tmem_ld16(tmem + lane_addr + C::T_S + pp * 64 + 16 * ch, cur);
          tmem_ld_wait();
          if (cc == 0 || cc == NCH - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (cc == 0) mbar_arrive(&g_free);
              if (cc == NCH - 1) mbar_arrive(&s_free[pp]);
            }
          }
          chunk(ch, cur, gq + 16 * cc);
        }
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&a_full[pp]);
    }
    // ---- epilogue: thread `part` of a row writes gradient columns [EC part, EC part + EC), EC = 64 / NP,
    // of this CTA's 128-wide half
    const float m1 = gs * 4.8828125e-4f;       // 2^-11
    const float m2 = gs * 1.953125e-3f;        // 2^-9
    TG* o1 = nullptr;
    constexpr int EC = 64 / NP;
    TG* o2 = static_cast<TG*>(p.out2) + ((int64_t)rb * R + row) * D + half * 128 + part * EC;
    if constexpr (kDkdv) o1 = static_cast<TG*>(p.out1) + ((int64_t)rb * R + row) * D + half * 128 + part * EC;
    if (nstep > 0) {
      mbar_wait(&acc_done, 0, &err, 14);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < EC / 32; ++c) {
        uint32_t r[32];
        if constexpr (kDkdv) {
          tmem_ld32(tmem + lane_addr + C::T_ACC1 + part * EC + c * 32, r);
          tmem_ld_wait();
          if (row_ok) store_row32<TG>(o1 + c * 32, r, m1);
        }
        tmem_ld32(tmem + lane_addr + C::T_ACC2 + part * EC + c * 32, r);
        tmem_ld_wait();
        if (row_ok) store_row32<TG>(o2 + c * 32, r, m2);
      }
      tc_fence_before();
    } else if (row_ok) {
      if constexpr (kDkdv) zero_row(o1, EC);
      zero_row(o2, EC);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

}  // namespace nvfp4

extern "C" int nvfp4_bwd_fp4(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv, const uint8_t* ksc,
                             const uint8_t* vdnv, const uint8_t* vdsc, const uint8_t* donv,
                             const uint8_t* dosc, const uint8_t* dotnv, const uint8_t* dotsc,
                             const uint8_t* qtnv, const uint8_t* qtsc, const uint8_t* ktnv,
                             const uint8_t* ktsc, const float* lse, const float* delta,
                             const float* do_amax, const float* key_bias, const int32_t* seq_start,
                             const int32_t* seq_end, void* dq, void* dk, void* dv, int grad_dtype,
                             int64_t z, int64_t h, int64_t hk, int64_t s_q, int64_t s_kv,
                             int64_t sq_pad, int64_t skv_pad, int d, float scaling, int flags,
                             uint32_t seed, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_bwd_fp4: head dim must be 128 or 256");
  NVFP4_REQUIRE(z >= 1 && h >= 1 && hk >= 1 && h % hk == 0, "nvfp4_bwd_fp4: bad head counts");
  NVFP4_REQUIRE(s_q >= 1 && s_kv >= 1 && s_q < (1LL << 30) && s_kv < (1LL << 30), "nvfp4_bwd_fp4: bad sequence extents");
  NVFP4_REQUIRE(sq_pad % 128 == 0 && sq_pad >= s_q && skv_pad % 128 == 0 && skv_pad >= s_kv,
                "nvfp4_bwd_fp4: transposed packs must be padded to a multiple of 128 columns");
  NVFP4_REQUIRE(qnv && qsc && knv && ksc && vdnv && vdsc && donv && dosc && dotnv && dotsc && qtnv && qtsc && ktnv &&
                    ktsc && lse && delta && do_amax && dq && dk && dv,
                "nvfp4_bwd_fp4: null pointer");
  const bool varlen = seq_start != nullptr;
  NVFP4_REQUIRE(varlen == (seq_end != nullptr), "nvfp4_bwd_fp4: seq_start and seq_end go together");
  NVFP4_REQUIRE(!varlen || (z == 1 && s_q == s_kv), "nvfp4_bwd_fp4: varlen needs Z == 1 and Sq == Skv");
  NVFP4_REQUIRE(!(flags & NVFP4_FWD_CAUSAL) || varlen || s_kv >= s_q, "nvfp4_bwd_fp4: causal needs Skv >= Sq");
  NVFP4_REQUIRE((s_kv + 127) / 128 < 65536 && z * h < (1LL << 31) && (s_q + 127) / 128 < 65536,
                "nvfp4_bwd_fp4: grid too large");
  NVFP4_REQUIRE((((uintptr_t)qsc | (uintptr_t)ksc | (uintptr_t)vdsc | (uintptr_t)dosc | (uintptr_t)dotsc |
                  (uintptr_t)qtsc | (uintptr_t)ktsc) & 3) == 0,
                "nvfp4_bwd_fp4: scale tensors must be 4-byte aligned");
  const bool fp8 = (flags & NVFP4_BWD_MXFP8) != 0;
  NVFP4_REQUIRE(!fp8 || !(flags & (NVFP4_BWD_SR_DS_DK | NVFP4_BWD_SR_P_DV | NVFP4_BWD_SR_DS_DQ)),
                "nvfp4_bwd_fp4: the MXFP8 operands round to nearest only");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t zh = z * h, zhk = z * hk;
  const uint64_t pb = (uint64_t)d / 2;
  CUtensorMap t_q, t_k, t_vd, t_do, t_dot, t_qt, t_kt;
  int rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_q, qnv, pb, s_q, zh, pb, (uint64_t)s_q * pb, 128, "nvfp4_bwd_fp4(Q)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_k, knv, pb, s_kv, zhk, pb, (uint64_t)s_kv * pb, 128, "nvfp4_bwd_fp4(K)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_vd, vdnv, pb, s_kv, zhk, pb, (uint64_t)s_kv * pb, 128, "nvfp4_bwd_fp4(V)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_do, donv, pb, s_q, zh, pb, (uint64_t)s_q * pb, 128, "nvfp4_bwd_fp4(dO)"))) return rc;
  if (fp8) {      // transposed operands: one byte per element, 128-byte boxes
    if ((rc = make_tmap_u8_3d_sw128(&t_dot, dotnv, (uint64_t)sq_pad, d, zh, (uint64_t)sq_pad, (uint64_t)d * sq_pad, 128,
                                    "nvfp4_bwd_fp4(dO^T)"))) return rc;
    if ((rc = make_tmap_u8_3d_sw128(&t_qt, qtnv, (uint64_t)sq_pad, d, zh, (uint64_t)sq_pad, (uint64_t)d * sq_pad, 128,
                                    "nvfp4_bwd_fp4(Q^T)"))) return rc;
    if ((rc = make_tmap_u8_3d_sw128(&t_kt, ktnv, (uint64_t)skv_pad, d, zhk, (uint64_t)skv_pad, (uint64_t)d * skv_pad, 128,
                                    "nvfp4_bwd_fp4(K^T)"))) return rc;
  } else {
    if ((rc = make_tmap_u8_3d_sw64(&t_dot, dotnv, (uint64_t)sq_pad / 2, d, zh, (uint64_t)sq_pad / 2,
                                   (uint64_t)d * (sq_pad / 2), 128, "nvfp4_bwd_fp4(dO^T)"))) return rc;
    if ((rc = make_tmap_u8_3d_sw64(&t_qt, qtnv, (uint64_t)sq_pad / 2, d, zh, (uint64_t)sq_pad / 2,
                                   (uint64_t)d * (sq_pad / 2), 128, "nvfp4_bwd_fp4(Q^T)"))) return rc;
    if ((rc = make_tmap_u8_3d_sw64(&t_kt, ktnv, (uint64_t)skv_pad / 2, d, zhk, (uint64_t)skv_pad / 2,
                                   (uint64_t)d * (skv_pad / 2), 128, "nvfp4_bwd_fp4(K^T)"))) return rc;
  }
  B4Params p;
  p.lse = lse; p.delta = delta; p.amax = do_amax; p.bias = key_bias;
  p.seq_start = seq_start; p.seq_end = seq_end;
  p.h = (int)h; p.hk = (int)hk; p.g = (int)(h / hk); p.s_q = (int)s_q; p.s_kv = (int)s_kv;
  p.scaling = scaling; p.causal = (flags & NVFP4_FWD_CAUSAL) ? 1 : 0; p.status = status;
  p.seed = seed; p.sr_p = 0; p.sr_ds = 0;
  const unsigned halves = (unsigned)(d / 128);
  auto launch = [&](auto kdkdv, auto kdq, int smem, int threads) -> int {
    cudaError_t e = cudaFuncSetAttribute(kdkdv, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_fp4: smem attribute: %s", cudaGetErrorString(e));
    e = cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_fp4: smem attribute: %s", cudaGetErrorString(e));
    // dK / dV: rows = keys (K, V packs), columns = queries (Q, dO' packs; dO'^T, Q^T transposed packs)
    B4Params a = p;
    a.x1sc = ksc; a.x2sc = vdsc; a.y1sc = qsc; a.y2sc = dosc; a.t1sc = dotsc; a.t2sc = qtsc;
    a.out1 = dv; a.out2 = dk; a.c_pad = (int)sq_pad;
    a.sr_p = (flags & NVFP4_BWD_SR_P_DV) ? 1 : 0; a.sr_ds = (flags & NVFP4_BWD_SR_DS_DK) ? 1 : 0;
    dim3 g1((unsigned)zhk, (unsigned)((s_kv + 127) / 128), halves);
    kdkdv<<<g1, threads, smem, st>>>(t_k, t_vd, t_q, t_do, t_dot, t_qt, a);
    int r1 = launch_result("nvfp4_bwd_fp4(dkdv)");
    if (r1) return r1;
    // dQ: rows = queries (Q, dO' packs), columns = keys (K, V packs; K^T transposed pack)
    B4Params b = p;
    b.x1sc = qsc; b.x2sc = dosc; b.y1sc = ksc; b.y2sc = vdsc; b.t1sc = nullptr; b.t2sc = ktsc;
    b.out1 = nullptr; b.out2 = dq; b.c_pad = (int)skv_pad;
    b.sr_ds = (flags & NVFP4_BWD_SR_DS_DQ) ? 1 : 0;
    dim3 g2((unsigned)zh, (unsigned)((s_q + 127) / 128), halves);
    kdq<<<g2, threads, smem, st>>>(t_q, t_do, t_k, t_vd, t_kt, t_kt, b);
    return launch_result("nvfp4_bwd_fp4(dq)");
  };
  const bool any_sr = (flags & (NVFP4_BWD_SR_DS_DK | NVFP4_BWD_SR_P_DV | NVFP4_BWD_SR_DS_DQ)) != 0;
#define NVFP4_B4_LAUNCH(DD, TT)                                                                                   \
  (fp8      ? launch(bwd4_kernel<DD, true, TT, 2>, bwd4_kernel<DD, false, TT, 2>, B4Cfg<DD, true>::TOTAL,         \
                     B4Cfg<DD, true>::THREADS)                                                                    \
   : any_sr ? launch(bwd4_kernel<DD, true, TT, 1>, bwd4_kernel<DD, false, TT, 1>, B4Cfg<DD, false>::TOTAL,        \
                     B4Cfg<DD, false>::THREADS)                                                                   \
            : launch(bwd4_kernel<DD, true, TT, 0>, bwd4_kernel<DD, false, TT, 0>, B4Cfg<DD, false>::TOTAL,        \
                     B4Cfg<DD, false>::THREADS))
  if (d == 128) {
    switch (grad_dtype) {
      case NVFP4_DT_BF16: return NVFP4_B4_LAUNCH(128, __nv_bfloat16);
      case NVFP4_DT_FP16: return NVFP4_B4_LAUNCH(128, __half);
      case NVFP4_DT_FP32: return NVFP4_B4_LAUNCH(128, float);
      default: return fail(-1, "nvfp4_bwd_fp4: unknown grad dtype %d", grad_dtype);
    }
  }
  switch (grad_dtype) {
    case NVFP4_DT_BF16: return NVFP4_B4_LAUNCH(256, __nv_bfloat16);
    case NVFP4_DT_FP16: return NVFP4_B4_LAUNCH(256, __half);
    case NVFP4_DT_FP32: return NVFP4_B4_LAUNCH(256, float);
    default: return fail(-1, "nvfp4_bwd_fp4: unknown grad dtype %d", grad_dtype);
  }
#undef NVFP4_B4_LAUNCH
}
