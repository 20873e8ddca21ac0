// Backward of the NVFP4 flash attention with high-precision gradient GEMMs ("HP-grad-dots").
//
// S is recomputed with the same FP4 block-scaled MMA (and the same packs) as the forward, so
// P = exp(S*scale - LSE) is the forward's probability; every gradient GEMM then runs in bf16 on
// the exact (unquantised) operands with fp32 accumulation in TMEM:
//     dV += P^T dO      dP = dO V^T      dS = P o (dP - delta) * scale
//     dQ += dS K        dK += dS^T Q     delta = rowsum(dO o O)
// Two kernels, both tcgen05:
//   * bwd_dkdv_kernel -- one CTA per 128-key tile of a (batch, kv-head) unit, "keys on M": it
//     loops over 64-query tiles and over the G query heads that share the kv head, so dK and dV
//     are reduced over the GQA group inside the kernel and written once.
//   * bwd_dq_kernel   -- one CTA per 128-query tile of a head, loops over key tiles.
// A pre-pass (bwd_prep_kernel) writes delta and the bf16 transposes (Q^T, dO^T, K^T) so that
// every MMA operand is K-major in shared memory (128-byte swizzle, loaded by TMA).
// Causal masking is bottom-right aligned; packed varlen is block-diagonal with per-tile loop
// bounds from the sample boundaries.  Head dim 128.  Every barrier wait is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"

namespace nvfp4 {

constexpr int kBwdThreads = 256;  // warps: 0 TMA, 1 MMA, 2 scale/aux loader, 3 idle, 4-7 compute
constexpr float kBwdLog2e = 1.4426950408889634f;

__host__ __device__ inline uint32_t make_idesc_bf16(uint32_t m, uint32_t n) {
  uint32_t d = 0;
  d |= 1u << 4;   // accumulator: fp32
  d |= 1u << 7;   // A: bf16
  d |= 1u << 10;  // B: bf16
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
__device__ __forceinline__ float ex2_bwd(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// K-major bf16 tile, rows of 128 bytes (64 elements), 128-byte swizzle: descriptor for the MMA
// that consumes 16 elements starting at element k16*16 of the row.
__device__ __forceinline__ uint64_t desc_sw128(const void* tile, int k16) {
  return make_smem_desc(smem_u32(tile) + (k16 & 3) * 32, 16, 1024, 2);
}
__device__ __forceinline__ uint64_t desc_sw64(const void* tile, int k64) {
  return make_smem_desc(smem_u32(tile) + (k64 & 1) * 32, 16, 512, 4);
}

// ------------------------------------------------------------------------------------------
// Pre-pass: x [B, S, D] (strided rows, unit stride along D) -> xt [B, D, Sp] bf16 (transposed,
// zero padded to Sp), optionally xc [B, S, D] bf16 contiguous, optionally
// delta [B, S] = rowsum(x o y).  One block per 64 x 64 tile.
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) bwd_prep_kernel(const T* __restrict__ x, int64_t sxb1, int64_t sxb2,
                                                       int64_t sxs, int nb2, const T* __restrict__ y,
                                                       int64_t syb1, int64_t syb2, int64_t sys, int S, int Sp,
                                                       int D, __nv_bfloat16* __restrict__ xt,
                                                       __nv_bfloat16* __restrict__ xc,
                                                       float* __restrict__ delta) {
  __shared__ float tile[64][65];
  __shared__ float dpart[64][4];
  const int b = blockIdx.z, s0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
  const int b1 = b / nb2, b2 = b % nb2;
  const T* xb = x + b1 * sxb1 + b2 * sxb2;
  const T* yb = y ? (y + b1 * syb1 + b2 * syb2) : nullptr;
  const int tid = threadIdx.x;
  // load 64 rows x 64 cols: thread -> (row = tid / 4 + 0.., 16 cols)
  const int r = tid >> 2, c0 = (tid & 3) * 16;
  float dsum = 0.0f;
  if (s0 + r < S) {
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      const float v = to_f32<T>(xb[(int64_t)(s0 + r) * sxs + d0 + c0 + c]);
      tile[r][c0 + c] = v;
      if (yb) dsum += v * to_f32<T>(yb[(int64_t)(s0 + r) * sys + d0 + c0 + c]);
      if (xc) xc[((int64_t)b * S + s0 + r) * D + d0 + c0 + c] = __float2bfloat16_rn(v);
    }
  } else {
#pragma unroll
    for (int c = 0; c < 16; ++c) tile[r][c0 + c] = 0.0f;
  }
  if (delta) dpart[r][tid & 3] = dsum;
  __syncthreads();
  if (delta && tid < 64 && s0 + tid < S)
    atomicAdd(&delta[(int64_t)b * S + s0 + tid], dpart[tid][0] + dpart[tid][1] + dpart[tid][2] + dpart[tid][3]);
  if (xt) {
    // write transposed: thread -> (d = tid / 4, 16 consecutive s)
    const int d = tid >> 2, sc0 = (tid & 3) * 16;
#pragma unroll
    for (int c = 0; c < 16; ++c)
      if (s0 + sc0 + c < Sp) xt[((int64_t)b * D + d0 + d) * Sp + s0 + sc0 + c] = __float2bfloat16_rn(tile[sc0 + c][d]);
  }
}

struct BwdParams {
  const uint8_t* qsc;   // [ZH, Sq, 8]
  const uint8_t* ksc;   // [ZHk, Skv, 8]
  const float* lse;     // [ZH, Sq] natural log
  const float* delta;   // [ZH, Sq]
  const int32_t* seq_id;     // [S] or null (varlen)
  const int32_t* seq_start;  // [S] or null
  const int32_t* seq_end;    // [S] or null
  void* dq;             // [ZH, Sq, D]
  void* dk;             // [ZHk, Skv, D]
  void* dv;             // [ZHk, Skv, D]
  int h, hk, g;
  int s_q, s_kv;
  float scaling;
  int causal;
  int* status;
};

template <typename TG>
__device__ __forceinline__ void store_row128(TG* dst, const uint32_t (&r)[32], float mul) {
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

// ------------------------------------------------------------------------------------------
// dK / dV: one CTA per 128-key tile of a (batch, kv-head) unit.
// TMEM: S^T [0,64) | dP^T [64,128) | dV [128,256) | dK [256,384) | SFK [384,392) | SFQ [392,400)
// ------------------------------------------------------------------------------------------
struct DkdvSmem {
  static constexpr int KP = 8192;        // K pack tile, 128 keys x 64 B (sw64)
  static constexpr int KSF = 1024;       // K scale atoms (2 x 512)
  static constexpr int V = 32768;        // V bf16 [128 keys x 128 d] = 2 sub-tiles of 16 KB (sw128)
  static constexpr int PT = 16384;       // P^T bf16 [128 keys x 64 q] (sw128)
  static constexpr int DST = 16384;      // dS^T
  // per stage
  static constexpr int QP = 4096;        // Q pack tile, 64 queries x 64 B (sw64)
  static constexpr int QSF = 1024;       // Q scale atoms
  static constexpr int DO = 16384;       // dO bf16 [64 q x 128 d] = 2 sub-tiles of 8 KB
  static constexpr int DOT = 16384;      // dO^T bf16 [128 d x 64 q]
  static constexpr int QT = 16384;       // Q^T bf16 [128 d x 64 q]
  static constexpr int AUX = 1024;       // lse*log2e [64], delta [64], seq id [64], pad
  static constexpr int STAGE = QP + QSF + DO + DOT + QT + AUX;
  static constexpr int NSTAGE = 2;
  static constexpr int TOTAL = KP + KSF + V + PT + DST + NSTAGE * STAGE + 1024;
  // offsets inside a stage (128-byte-swizzled tiles first: they need 1 KB alignment)
  static constexpr int O_DO = 0, O_DOT = DO, O_QT = DO + DOT, O_QP = DO + DOT + QT, O_QSF = O_QP + QP,
                       O_AUX = O_QSF + QSF;
};

template <typename TG>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_kp, const __grid_constant__ CUtensorMap tm_qp,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_dot, const __grid_constant__ CUtensorMap tm_qt,
                const BwdParams p) {
  using L = DkdvSmem;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_v = smem;
  uint8_t* s_pt = s_v + L::V;
  uint8_t* s_dst = s_pt + L::PT;
  uint8_t* s_kp = s_dst + L::DST;
  uint8_t* s_stage = s_kp + L::KP;
  uint8_t* s_ksf = s_stage + L::NSTAGE * L::STAGE;

  __shared__ uint64_t full_tma[L::NSTAGE], full_aux[L::NSTAGE], empty[L::NSTAGE];
  __shared__ uint64_t kv_full, ksf_full, sdp_full, pds_full, acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int jt = blockIdx.x;           // key tile
  const int unit = blockIdx.y;         // z * hk + kh
  const int zi = unit / p.hk, kh = unit % p.hk;
  const int n0 = jt * 128;
  const int shift = p.s_kv - p.s_q;
  // 64-query tiles that can see a key of this tile
  int q_lo = 0, q_hi = p.s_q;
  if (p.causal) q_lo = max(0, n0 - shift);
  if (p.seq_id != nullptr) {
    q_lo = max(q_lo, (int)p.seq_start[min(n0, p.s_kv - 1)]);
    q_hi = min(q_hi, (int)p.seq_end[min(n0 + 127, p.s_kv - 1)]);
  }
  const int i_lo = q_lo / 64, i_hi = (q_hi + 63) / 64;
  const int n_i = max(i_hi - i_lo, 0);
  const int nstep = n_i * p.g;

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < L::NSTAGE; ++i) {
      mbar_init(&full_tma[i], 1);
      mbar_init(&full_aux[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&kv_full, 1);
    mbar_init(&ksf_full, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&pds_full, 4);
    mbar_init(&acc_done, 1);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  constexpr uint32_t T_ST = 0, T_DPT = 64, T_DV = 128, T_DK = 256, T_SFK = 384, T_SFQ = 392;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && nstep > 0) {
      mbar_expect_tx(&kv_full, L::KP + L::V);
      tma_load_3d(s_kp, &tm_kp, &kv_full, 0, n0, unit);
      tma_load_3d(s_v, &tm_v, &kv_full, 0, n0, unit);
      tma_load_3d(s_v + 16384, &tm_v, &kv_full, 64, n0, unit);
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE;
        const int gq = st / n_i, i = i_lo + st % n_i;
        const int zh = zi * p.h + kh * p.g + gq;
        if (st >= L::NSTAGE) mbar_wait(&empty[s], ((st / L::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_expect_tx(&full_tma[s], L::QP + L::DO + L::DOT + L::QT);
        tma_load_3d(sb + L::O_QP, &tm_qp, &full_tma[s], 0, i * 64, zh);
        tma_load_3d(sb + L::O_DO, &tm_do, &full_tma[s], 0, i * 64, zh);
        tma_load_3d(sb + L::O_DO + 8192, &tm_do, &full_tma[s], 64, i * 64, zh);
        tma_load_3d(sb + L::O_DOT, &tm_dot, &full_tma[s], i * 64, 0, zh);
        tma_load_3d(sb + L::O_QT, &tm_qt, &full_tma[s], i * 64, 0, zh);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale / aux loader
    if (nstep > 0) {
      // K scale atoms of this key tile (once)
      const uint8_t* ksrc = p.ksc + (int64_t)unit * p.s_kv * 8;
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = lane + 32 * r4;
        const bool ok = n0 + r < p.s_kv;
        const uint8_t* g = ksrc + (int64_t)(ok ? n0 + r : 0) * 8;
        cp_async_4(smem_u32(s_ksf) + sf_atom_offset(r, 0), g, ok ? 4u : 0u);
        cp_async_4(smem_u32(s_ksf) + 512 + sf_atom_offset(r, 0), g + 4, ok ? 4u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ksf_full);
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE;
        const int gq = st / n_i, i = i_lo + st % n_i;
        const int zh = zi * p.h + kh * p.g + gq;
        if (st >= L::NSTAGE) mbar_wait(&empty[s], ((st / L::NSTAGE) & 1) ^ 1, &err, 2);
        uint8_t* sb = s_stage + s * L::STAGE;
        const uint32_t qsf = smem_u32(sb + L::O_QSF);
        float* aux = reinterpret_cast<float*>(sb + L::O_AUX);
#pragma unroll
        for (int r2 = 0; r2 < 2; ++r2) {
          const int r = lane + 32 * r2;
          const int qi = i * 64 + r;
          const bool ok = qi < p.s_q;
          const uint8_t* g = p.qsc + ((int64_t)zh * p.s_q + (ok ? qi : 0)) * 8;
          cp_async_4(qsf + sf_atom_offset(r, 0), g, ok ? 4u : 0u);
          cp_async_4(qsf + 512 + sf_atom_offset(r, 0), g + 4, ok ? 4u : 0u);
          aux[r] = ok ? p.lse[(int64_t)zh * p.s_q + qi] * kBwdLog2e : INFINITY;   // masked rows: P = 0
          aux[64 + r] = ok ? p.delta[(int64_t)zh * p.s_q + qi] : 0.0f;
          reinterpret_cast<int32_t*>(aux)[128 + r] = (p.seq_id != nullptr && ok) ? p.seq_id[qi] : -1;
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
      const uint32_t id_s = make_idesc_nvfp4(128, 64);
      const uint32_t id_dp = make_idesc_bf16(128, 64);
      const uint32_t id_acc = make_idesc_bf16(128, 128);
      mbar_wait(&kv_full, 0, &err, 3);
      mbar_wait(&ksf_full, 0, &err, 4);
      tc_fence_after();
      tmem_cp_32x128b_warpx4(tmem + T_SFK, smem_u32(s_ksf));
      tmem_cp_32x128b_warpx4(tmem + T_SFK + 4, smem_u32(s_ksf + 512));
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE;
        const uint32_t ph = (st / L::NSTAGE) & 1;
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_wait(&full_tma[s], ph, &err, 5);
        mbar_wait(&full_aux[s], ph, &err, 6);
        // S^T / dP^T of the previous step must have been read, and its dV / dK MMAs issued
        if (st > 0) mbar_wait(&pds_full, (st - 1) & 1, &err, 7);
        tc_fence_after();
        if (st > 0) {
          // dV += P^T dO, dK += dS^T Q of the previous step
          const int sp = (st - 1) % L::NSTAGE;
          uint8_t* sbp = s_stage + sp * L::STAGE;
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + T_DV, desc_sw128(s_pt, k), desc_sw128(sbp + L::O_DOT, k), id_acc,
                      (st > 1 || k > 0) ? 1u : 0u);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem + T_DK, desc_sw128(s_dst, k), desc_sw128(sbp + L::O_QT, k),
                      id_acc, (st > 1 || k > 0) ? 1u : 0u);
          umma_commit(&empty[sp]);
          umma_commit(&acc_done);
        }
        tmem_cp_32x128b_warpx4(tmem + T_SFQ, smem_u32(sb + L::O_QSF));
        tmem_cp_32x128b_warpx4(tmem + T_SFQ + 4, smem_u32(sb + L::O_QSF + 512));
#pragma unroll
        for (int k = 0; k < 2; ++k)
          umma_nvfp4(tmem + T_ST, desc_sw64(s_kp, k), desc_sw64(sb + L::O_QP, k), id_s, tmem + T_SFK + k * 4,
                     tmem + T_SFQ + k * 4, k > 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tmem + T_DPT, desc_sw128(s_v + (k >> 2) * 16384, k),
                    desc_sw128(sb + L::O_DO + (k >> 2) * 8192, k), id_dp, k > 0);
        umma_commit(&sdp_full);
      }
      // tail: gradient GEMMs of the last step
      mbar_wait(&pds_full, (nstep - 1) & 1, &err, 8);
      tc_fence_after();
      {
        const int sp = (nstep - 1) % L::NSTAGE;
        uint8_t* sbp = s_stage + sp * L::STAGE;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem + T_DV, desc_sw128(s_pt, k), desc_sw128(sbp + L::O_DOT, k), id_acc,
                    (nstep > 1 || k > 0) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16(tmem + T_DK, desc_sw128(s_dst, k), desc_sw128(sbp + L::O_QT, k),
                    id_acc, (nstep > 1 || k > 0) ? 1u : 0u);
        umma_commit(&acc_done);
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ P^T / dS^T producers, epilogue
    const int wq = warp - 4;
    const int row = wq * 32 + lane;     // key within the tile
    const int key = n0 + row;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c2 = p.scaling * kBwdLog2e;
    const int key_seq = (p.seq_id != nullptr && key < p.s_kv) ? p.seq_id[key] : -1;
    for (int st = 0; st < nstep; ++st) {
      const int s = st % L::NSTAGE;
      const int i = i_lo + st % n_i;
      uint8_t* sb = s_stage + s * L::STAGE;
      const float* aux = reinterpret_cast<const float*>(sb + L::O_AUX);
      const int32_t* aux_seq = reinterpret_cast<const int32_t*>(aux) + 128;
      mbar_wait(&sdp_full, st & 1, &err, 9);
      tc_fence_after();
      // P^T / dS^T buffers are free once the previous step's gradient GEMMs have completed
      if (st > 0) mbar_wait(&acc_done, (st - 1) & 1, &err, 10);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld32(tmem + lane_addr + T_ST + c * 32, sr);
        tmem_ld32(tmem + lane_addr + T_DPT + c * 32, dr);
        tmem_ld_wait();
        uint32_t pw[16], dw[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float pv[2], dsv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int qc = c * 32 + e + u;
            const int qi = i * 64 + qc;
            bool ok = key < p.s_kv && qi < p.s_q;
            if (p.causal) ok = ok && (key <= qi + shift);
            if (p.seq_id != nullptr) ok = ok && (aux_seq[qc] == key_seq);
            const float pe = ok ? ex2_bwd(__uint_as_float(sr[e + u]) * c2 - aux[qc]) : 0.0f;
            pv[u] = pe;
            dsv[u] = pe * (__uint_as_float(dr[e + u]) - aux[64 + qc]);
          }
          const __nv_bfloat162 pb = __floats2bfloat162_rn(pv[0], pv[1]);
          const __nv_bfloat162 db = __floats2bfloat162_rn(dsv[0], dsv[1]);
          pw[e >> 1] = *reinterpret_cast<const uint32_t*>(&pb);
          dw[e >> 1] = *reinterpret_cast<const uint32_t*>(&db);
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4) {
          const uint32_t off = sw128_offset(row, c * 64 + v4 * 16);
          *reinterpret_cast<uint4*>(s_pt + off) = make_uint4(pw[4 * v4], pw[4 * v4 + 1], pw[4 * v4 + 2], pw[4 * v4 + 3]);
          *reinterpret_cast<uint4*>(s_dst + off) = make_uint4(dw[4 * v4], dw[4 * v4 + 1], dw[4 * v4 + 2], dw[4 * v4 + 3]);
        }
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full);
    }
    // ---- epilogue
    TG* dkrow = static_cast<TG*>(p.dk) + ((int64_t)unit * p.s_kv + key) * 128;
    TG* dvrow = static_cast<TG*>(p.dv) + ((int64_t)unit * p.s_kv + key) * 128;
    if (nstep > 0) {
      mbar_wait(&acc_done, (nstep - 1) & 1, &err, 11);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + T_DV + c * 32, r);
        tmem_ld_wait();
        if (key < p.s_kv) store_row128<TG>(dvrow + c * 32, r, 1.0f);
        tmem_ld32(tmem + lane_addr + T_DK + c * 32, r);
        tmem_ld_wait();
        if (key < p.s_kv) store_row128<TG>(dkrow + c * 32, r, p.scaling);
      }
      tc_fence_before();
    } else if (key < p.s_kv) {
      for (int e = 0; e < 128; ++e) { dkrow[e] = from_f32<TG>(0.0f); dvrow[e] = from_f32<TG>(0.0f); }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------
// dQ: one CTA per 128-query tile of a head, loops over 128-key tiles.
// TMEM: S [0,128) | dP [128,256) | dQ [256,384) | SFQ [384,392) | SFK [392,400)
// ------------------------------------------------------------------------------------------
struct DqSmem {
  static constexpr int QP = 8192;        // Q pack tile, 128 queries x 64 B
  static constexpr int QSF = 1024;
  static constexpr int DO = 32768;       // dO bf16 [128 q x 128 d] = 2 sub-tiles of 16 KB
  static constexpr int DS = 32768;       // dS bf16 [128 q x 128 keys] = 2 sub-tiles (keys 0-63 | 64-127)
  // per stage
  static constexpr int KP = 8192;
  static constexpr int KSF = 1024;
  static constexpr int V = 32768;        // V bf16 [128 keys x 128 d]
  static constexpr int KT = 32768;       // K^T bf16 [128 d x 128 keys] = 2 sub-tiles by key half
  static constexpr int AUX = 512;        // seq id of the 128 keys
  static constexpr int STAGE = KP + KSF + V + KT + AUX + 512;
  static constexpr int NSTAGE = 2;
  static constexpr int TOTAL = QP + QSF + DO + DS + NSTAGE * STAGE + 1024;
  static constexpr int O_V = 0, O_KT = V, O_KP = V + KT, O_KSF = O_KP + KP, O_AUX = O_KSF + KSF;
};

template <typename TG>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qp, const __grid_constant__ CUtensorMap tm_kp,
              const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ CUtensorMap tm_kt, const BwdParams p) {
  using L = DqSmem;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_do = smem;
  uint8_t* s_ds = s_do + L::DO;
  uint8_t* s_qp = s_ds + L::DS;
  uint8_t* s_stage = s_qp + L::QP;
  uint8_t* s_qsf = s_stage + L::NSTAGE * L::STAGE;

  __shared__ uint64_t full_tma[L::NSTAGE], full_aux[L::NSTAGE], empty[L::NSTAGE];
  __shared__ uint64_t q_full, qsf_full, sdp_full, ds_full, acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  __shared__ int s_lo_tile;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mblk = gridDim.y - 1 - blockIdx.y;
  const int zh = blockIdx.x;
  const int zi = zh / p.h, hi = zh % p.h;
  const int unit = zi * p.hk + hi / p.g;
  const int m0 = mblk * 128;
  const int shift = p.s_kv - p.s_q;
  int hi_key = p.s_kv;
  if (p.causal) hi_key = min(p.s_kv, m0 + 128 + shift);
  if (hi_key < 0) hi_key = 0;
  const int t_hi = (hi_key + 127) / 128;

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < L::NSTAGE; ++i) {
      mbar_init(&full_tma[i], 1);
      mbar_init(&full_aux[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&q_full, 1);
    mbar_init(&qsf_full, 1);
    mbar_init(&sdp_full, 1);
    mbar_init(&ds_full, 4);
    mbar_init(&acc_done, 1);
    mbar_fence_init();
    s_lo_tile = (p.seq_start != nullptr) ? (p.seq_start[min(m0, p.s_q - 1)] / 128) : 0;
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  const int t_lo = s_lo_tile;
  const int ntile = max(t_hi - t_lo, 0);
  constexpr uint32_t T_S = 0, T_DP = 128, T_DQ = 256, T_SFQ = 384, T_SFK = 392;

  if (warp == 0) {
    if (elect_one() && ntile > 0) {
      mbar_expect_tx(&q_full, L::QP + L::DO);
      tma_load_3d(s_qp, &tm_qp, &q_full, 0, m0, zh);
      tma_load_3d(s_do, &tm_do, &q_full, 0, m0, zh);
      tma_load_3d(s_do + 16384, &tm_do, &q_full, 64, m0, zh);
      for (int i = 0; i < ntile; ++i) {
        const int s = i % L::NSTAGE, t = t_lo + i;
        if (i >= L::NSTAGE) mbar_wait(&empty[s], ((i / L::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_expect_tx(&full_tma[s], L::KP + L::V + L::KT);
        tma_load_3d(sb + L::O_KP, &tm_kp, &full_tma[s], 0, t * 128, unit);
        tma_load_3d(sb + L::O_V, &tm_v, &full_tma[s], 0, t * 128, unit);
        tma_load_3d(sb + L::O_V + 16384, &tm_v, &full_tma[s], 64, t * 128, unit);
        tma_load_3d(sb + L::O_KT, &tm_kt, &full_tma[s], t * 128, 0, unit);
        tma_load_3d(sb + L::O_KT + 16384, &tm_kt, &full_tma[s], t * 128 + 64, 0, unit);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    if (ntile > 0) {
      const uint8_t* qsrc = p.qsc + (int64_t)zh * p.s_q * 8;
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = lane + 32 * r4;
        const bool ok = m0 + r < p.s_q;
        const uint8_t* g = qsrc + (int64_t)(ok ? m0 + r : 0) * 8;
        cp_async_4(smem_u32(s_qsf) + sf_atom_offset(r, 0), g, ok ? 4u : 0u);
        cp_async_4(smem_u32(s_qsf) + 512 + sf_atom_offset(r, 0), g + 4, ok ? 4u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&qsf_full);
      const uint8_t* ksrc = p.ksc + (int64_t)unit * p.s_kv * 8;
      for (int i = 0; i < ntile; ++i) {
        const int s = i % L::NSTAGE, t = t_lo + i;
        if (i >= L::NSTAGE) mbar_wait(&empty[s], ((i / L::NSTAGE) & 1) ^ 1, &err, 2);
        uint8_t* sb = s_stage + s * L::STAGE;
        const uint32_t ksf = smem_u32(sb + L::O_KSF);
        int32_t* aux_seq = reinterpret_cast<int32_t*>(sb + L::O_AUX);
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int r = lane + 32 * r4;
          const int key = t * 128 + r;
          const bool ok = key < p.s_kv;
          const uint8_t* g = ksrc + (int64_t)(ok ? key : 0) * 8;
          cp_async_4(ksf + sf_atom_offset(r, 0), g, ok ? 4u : 0u);
          cp_async_4(ksf + 512 + sf_atom_offset(r, 0), g + 4, ok ? 4u : 0u);
          aux_seq[r] = (p.seq_id != nullptr && ok) ? p.seq_id[key] : -1;
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_aux[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && ntile > 0) {
      const uint32_t id_s = make_idesc_nvfp4(128, 128);
      const uint32_t id_b = make_idesc_bf16(128, 128);
      mbar_wait(&q_full, 0, &err, 3);
      mbar_wait(&qsf_full, 0, &err, 4);
      tc_fence_after();
      tmem_cp_32x128b_warpx4(tmem + T_SFQ, smem_u32(s_qsf));
      tmem_cp_32x128b_warpx4(tmem + T_SFQ + 4, smem_u32(s_qsf + 512));
      auto grad_gemm = [&](int i) {   // dQ += dS K for tile i
        const int sp = i % L::NSTAGE;
        uint8_t* sbp = s_stage + sp * L::STAGE;
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tmem + T_DQ, desc_sw128(s_ds + (k >> 2) * 16384, k),
                    desc_sw128(sbp + L::O_KT + (k >> 2) * 16384, k), id_b, (i > 0 || k > 0) ? 1u : 0u);
      };
      for (int i = 0; i < ntile; ++i) {
        const int s = i % L::NSTAGE;
        const uint32_t ph = (i / L::NSTAGE) & 1;
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_wait(&full_tma[s], ph, &err, 5);
        mbar_wait(&full_aux[s], ph, &err, 6);
        if (i > 0) mbar_wait(&ds_full, (i - 1) & 1, &err, 7);
        tc_fence_after();
        if (i > 0) {
          grad_gemm(i - 1);
          umma_commit(&empty[(i - 1) % L::NSTAGE]);
          umma_commit(&acc_done);
        }
        tmem_cp_32x128b_warpx4(tmem + T_SFK, smem_u32(sb + L::O_KSF));
        tmem_cp_32x128b_warpx4(tmem + T_SFK + 4, smem_u32(sb + L::O_KSF + 512));
#pragma unroll
        for (int k = 0; k < 2; ++k)
          umma_nvfp4(tmem + T_S, desc_sw64(s_qp, k), desc_sw64(sb + L::O_KP, k), id_s, tmem + T_SFQ + k * 4,
                     tmem + T_SFK + k * 4, k > 0);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          umma_bf16(tmem + T_DP, desc_sw128(s_do + (k >> 2) * 16384, k),
                    desc_sw128(sb + L::O_V + (k >> 2) * 16384, k), id_b, k > 0);
        umma_commit(&sdp_full);
      }
      mbar_wait(&ds_full, (ntile - 1) & 1, &err, 8);
      tc_fence_after();
      grad_gemm(ntile - 1);
      umma_commit(&acc_done);
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int wq = warp - 4;
    const int row_in = wq * 32 + lane;
    const int row = m0 + row_in;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c2 = p.scaling * kBwdLog2e;
    const bool row_ok = row < p.s_q;
    const float lse2 = row_ok ? p.lse[(int64_t)zh * p.s_q + row] * kBwdLog2e : INFINITY;
    const float dlt = row_ok ? p.delta[(int64_t)zh * p.s_q + row] : 0.0f;
    const int my_seq = (p.seq_id != nullptr && row_ok) ? p.seq_id[row] : -1;
    const int my_limit = p.causal ? (row + shift) : (p.s_kv - 1);
    for (int i = 0; i < ntile; ++i) {
      const int s = i % L::NSTAGE, t = t_lo + i;
      uint8_t* sb = s_stage + s * L::STAGE;
      const int32_t* aux_seq = reinterpret_cast<const int32_t*>(sb + L::O_AUX);
      mbar_wait(&sdp_full, i & 1, &err, 9);
      tc_fence_after();
      if (i > 0) mbar_wait(&acc_done, (i - 1) & 1, &err, 10);
      const int lim = min(my_limit, p.s_kv - 1) - t * 128;   // visible keys of this row: [0, lim]
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t sr[32], dr[32];
        tmem_ld32(tmem + lane_addr + T_S + c * 32, sr);
        tmem_ld32(tmem + lane_addr + T_DP + c * 32, dr);
        tmem_ld_wait();
        uint32_t dw[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float dsv[2];
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int kc = c * 32 + e + u;
            bool ok = row_ok && kc <= lim;
            if (p.seq_id != nullptr) ok = ok && (aux_seq[kc] == my_seq);
            const float pe = ok ? ex2_bwd(__uint_as_float(sr[e + u]) * c2 - lse2) : 0.0f;
            dsv[u] = pe * (__uint_as_float(dr[e + u]) - dlt);
          }
          const __nv_bfloat162 db = __floats2bfloat162_rn(dsv[0], dsv[1]);
          dw[e >> 1] = *reinterpret_cast<const uint32_t*>(&db);
        }
#pragma unroll
        for (int v4 = 0; v4 < 4; ++v4)
          *reinterpret_cast<uint4*>(s_ds + (c >> 1) * 16384 + sw128_offset(row_in, (c & 1) * 64 + v4 * 16)) =
              make_uint4(dw[4 * v4], dw[4 * v4 + 1], dw[4 * v4 + 2], dw[4 * v4 + 3]);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full);
    }
    TG* dqrow = static_cast<TG*>(p.dq) + ((int64_t)zh * p.s_q + row) * 128;
    if (ntile > 0) {
      mbar_wait(&acc_done, (ntile - 1) & 1, &err, 11);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + T_DQ + c * 32, r);
        tmem_ld_wait();
        if (row_ok) store_row128<TG>(dqrow + c * 32, r, p.scaling);
      }
      tc_fence_before();
    } else if (row_ok) {
      for (int e = 0; e < 128; ++e) dqrow[e] = from_f32<TG>(0.0f);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// bf16 tensor [n2][n1][n0] with 128-byte swizzle, box [1][b1][64 elements]
inline int make_tmap_bf16_3d_sw128(CUtensorMap* m, const void* base, uint64_t n0, uint64_t n1, uint64_t n2,
                                   uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b1, const char* what) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(-1, "%s: cuTensorMapEncodeTiled is unavailable", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1_bytes & 15) || (s2_bytes & 15))
    return fail(-1, "%s: base and strides must be 16-byte aligned for TMA", what);
  cuuint64_t dims[3] = {n0, n1, n2};
  cuuint64_t strides[2] = {s1_bytes, s2_bytes};
  cuuint32_t box[3] = {64, b1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, es,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-1, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return 0;
}

template <typename T>
int prep_launch(const void* x, int64_t sxb1, int64_t sxb2, int64_t sxs, int nb1, int nb2, const void* y,
                int64_t syb1, int64_t syb2, int64_t sys, int S, int Sp, int D, __nv_bfloat16* xt,
                __nv_bfloat16* xc, float* delta, cudaStream_t st) {
  dim3 grid((unsigned)((Sp + 63) / 64), (unsigned)(D / 64), (unsigned)(nb1 * nb2));
  bwd_prep_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(x), sxb1, sxb2, sxs, nb2,
                                           static_cast<const T*>(y), syb1, syb2, sys, S, Sp, D, xt, xc, delta);
  return launch_result("nvfp4_bwd_prep");
}

}  // namespace nvfp4

extern "C" int nvfp4_bwd_prep(const void* x, int dtype, int64_t sxb1, int64_t sxb2, int64_t sxs,
                              int64_t nb1, int64_t nb2, const void* y, int64_t syb1, int64_t syb2,
                              int64_t sys, int64_t s, int64_t s_pad, int d, void* xt, void* xc,
                              float* delta, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(x != nullptr && (xt || xc || delta), "nvfp4_bwd_prep: nothing to do");
  NVFP4_REQUIRE(d % 64 == 0 && s >= 1 && s_pad >= s && s_pad % 8 == 0, "nvfp4_bwd_prep: bad extents");
  NVFP4_REQUIRE(delta == nullptr || y != nullptr, "nvfp4_bwd_prep: delta needs the second operand");
  NVFP4_REQUIRE(nb1 * nb2 < 65536, "nvfp4_bwd_prep: too many batch entries");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* t = static_cast<__nv_bfloat16*>(xt);
  auto* c = static_cast<__nv_bfloat16*>(xc);
  switch (dtype) {
    case NVFP4_DT_BF16:
      return prep_launch<__nv_bfloat16>(x, sxb1, sxb2, sxs, (int)nb1, (int)nb2, y, syb1, syb2, sys, (int)s,
                                        (int)s_pad, d, t, c, delta, st);
    case NVFP4_DT_FP16:
      return prep_launch<__half>(x, sxb1, sxb2, sxs, (int)nb1, (int)nb2, y, syb1, syb2, sys, (int)s, (int)s_pad,
                                 d, t, c, delta, st);
    case NVFP4_DT_FP32:
      return prep_launch<float>(x, sxb1, sxb2, sxs, (int)nb1, (int)nb2, y, syb1, syb2, sys, (int)s, (int)s_pad, d,
                                t, c, delta, st);
    default:
      return fail(-1, "nvfp4_bwd_prep: unknown dtype %d", dtype);
  }
}

extern "C" int nvfp4_bwd_hp(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv,
                            const uint8_t* ksc, const void* v_bf16, const void* do_bf16,
                            const void* qt_bf16, const void* dot_bf16, const void* kt_bf16,
                            const float* lse, const float* delta, const int32_t* seq_id,
                            const int32_t* seq_start, const int32_t* seq_end, void* dq, void* dk,
                            void* dv, int grad_dtype, int64_t z, int64_t h, int64_t hk, int64_t s_q,
                            int64_t s_kv, int64_t sq_pad, int64_t skv_pad, int d, float scaling,
                            int flags, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128, "nvfp4_bwd_hp: this build implements the backward for D = 128 only");
  NVFP4_REQUIRE(z >= 1 && h >= 1 && hk >= 1 && h % hk == 0, "nvfp4_bwd_hp: bad head counts");
  NVFP4_REQUIRE(s_q >= 1 && s_kv >= 1 && sq_pad >= s_q && skv_pad >= s_kv && sq_pad % 8 == 0 && skv_pad % 8 == 0,
                "nvfp4_bwd_hp: bad sequence extents");
  NVFP4_REQUIRE(qnv && qsc && knv && ksc && v_bf16 && do_bf16 && qt_bf16 && dot_bf16 && kt_bf16 && lse &&
                    delta && dq && dk && dv,
                "nvfp4_bwd_hp: null pointer");
  const bool varlen = seq_id != nullptr;
  NVFP4_REQUIRE(varlen == (seq_start != nullptr) && varlen == (seq_end != nullptr),
                "nvfp4_bwd_hp: the three varlen arrays go together");
  NVFP4_REQUIRE(!varlen || (z == 1 && s_q == s_kv), "nvfp4_bwd_hp: varlen needs Z == 1 and Sq == Skv");
  NVFP4_REQUIRE(z * hk < 65536 && z * h < (1LL << 31) && (s_q + 127) / 128 < 65536, "nvfp4_bwd_hp: grid too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t zh = z * h, zhk = z * hk;
  CUtensorMap t_qp64, t_qp128, t_kp, t_v, t_do64, t_do128, t_dot, t_qt, t_kt;
  int rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_qp64, qnv, 64, s_q, zh, 64, (uint64_t)s_q * 64, 64, "nvfp4_bwd_hp(Qp64)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_qp128, qnv, 64, s_q, zh, 64, (uint64_t)s_q * 64, 128, "nvfp4_bwd_hp(Qp128)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_kp, knv, 64, s_kv, zhk, 64, (uint64_t)s_kv * 64, 128, "nvfp4_bwd_hp(Kp)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_v, v_bf16, 128, s_kv, zhk, 256, (uint64_t)s_kv * 256, 128, "nvfp4_bwd_hp(V)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_do64, do_bf16, 128, s_q, zh, 256, (uint64_t)s_q * 256, 64, "nvfp4_bwd_hp(dO64)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_do128, do_bf16, 128, s_q, zh, 256, (uint64_t)s_q * 256, 128, "nvfp4_bwd_hp(dO128)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_dot, dot_bf16, sq_pad, 128, zh, (uint64_t)sq_pad * 2, (uint64_t)sq_pad * 256, 128, "nvfp4_bwd_hp(dO^T)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_qt, qt_bf16, sq_pad, 128, zh, (uint64_t)sq_pad * 2, (uint64_t)sq_pad * 256, 128, "nvfp4_bwd_hp(Q^T)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_kt, kt_bf16, skv_pad, 128, zhk, (uint64_t)skv_pad * 2, (uint64_t)skv_pad * 256, 128, "nvfp4_bwd_hp(K^T)"))) return rc;
  BwdParams p;
  p.qsc = qsc; p.ksc = ksc; p.lse = lse; p.delta = delta;
  p.seq_id = seq_id; p.seq_start = seq_start; p.seq_end = seq_end;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.h = (int)h; p.hk = (int)hk; p.g = (int)(h / hk); p.s_q = (int)s_q; p.s_kv = (int)s_kv;
  p.scaling = scaling; p.causal = (flags & NVFP4_FWD_CAUSAL) ? 1 : 0; p.status = status;
  auto launch = [&](auto kdkdv, auto kdq) -> int {
    cudaError_t e = cudaFuncSetAttribute(kdkdv, cudaFuncAttributeMaxDynamicSharedMemorySize, DkdvSmem::TOTAL);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_hp: smem attribute: %s", cudaGetErrorString(e));
    e = cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, DqSmem::TOTAL);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_hp: smem attribute: %s", cudaGetErrorString(e));
    dim3 g1((unsigned)((s_kv + 127) / 128), (unsigned)zhk);
    kdkdv<<<g1, kBwdThreads, DkdvSmem::TOTAL, st>>>(t_kp, t_qp64, t_v, t_do64, t_dot, t_qt, p);
    int r1 = launch_result("nvfp4_bwd_hp(dkdv)");
    if (r1) return r1;
    dim3 g2((unsigned)zh, (unsigned)((s_q + 127) / 128));
    kdq<<<g2, kBwdThreads, DqSmem::TOTAL, st>>>(t_qp128, t_kp, t_do128, t_v, t_kt, p);
    return launch_result("nvfp4_bwd_hp(dq)");
  };
  switch (grad_dtype) {
    case NVFP4_DT_BF16: return launch(bwd_dkdv_kernel<__nv_bfloat16>, bwd_dq_kernel<__nv_bfloat16>);
    case NVFP4_DT_FP16: return launch(bwd_dkdv_kernel<__half>, bwd_dq_kernel<__half>);
    case NVFP4_DT_FP32: return launch(bwd_dkdv_kernel<float>, bwd_dq_kernel<float>);
    default: return fail(-1, "nvfp4_bwd_hp: unknown grad dtype %d", grad_dtype);
  }
}
