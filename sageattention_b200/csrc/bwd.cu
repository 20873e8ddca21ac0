// Backward of the NVFP4 flash attention with high-precision gradient GEMMs, sm_100a.
//
//   S  = Q K^T           recomputed from the NVFP4 packs (kind::mxf4nvf4, as the forward)
//   P  = exp2(S * scaling * log2e - lse * log2e)      (lse saved by the forward)
//   dP = dO V^T                                        bf16 tcgen05, exact operands
//   dS = P o (dP - delta),  delta = rowsum(dO o O)
//   dV = P^T dO,  dK = scaling * dS^T Q,  dQ = scaling * dS K      bf16 tcgen05
//
// Two kernels, both deterministic (no atomics):
//   bwd_dkdv_kernel  one CTA per 128-key tile of a (batch, kv-head) unit; walks 64-query steps of
//                    every query head of the GQA group, so dK / dV are reduced over the group in
//                    TMEM and written once.
//   bwd_dq_kernel    one CTA per 128-query tile of a head; walks 64-key steps.
// Every bf16 operand is read from the row-major [rows, 128] tensors by TMA into 128-byte-swizzled
// tiles; the same tile serves as a K-major operand (contraction along D) and as an MN-major
// operand (contraction along the rows), so no transposed copies exist anywhere.
//
// Pipeline of one CTA (384 threads): warp 0 TMA producer, warp 1 MMA issuer, warp 2 scale-atom /
// row-statistics loader, warps 4-7 and 8-11 two softmax groups that alternate steps.  S has two
// TMEM slots, dP one (a group pulls it into registers and hands the slot back at once); P^T / dS^T
// are written back as bf16 pairs into the S slot they were computed from and enter the gradient
// GEMMs as TMEM A operands, so the probabilities never touch shared memory and the tensor pipe
// works on step t+1 while a group is still busy with step t.  Causal masking is bottom-right
// aligned; packed varlen is block-diagonal, expressed as a per-row visible range.  Head dim 128,
// or 256 as two 128-wide output halves per tile (both halves recompute S and dP).  Every barrier
// wait is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"
#include "common/bwd_util.cuh"

namespace nvfp4 {

constexpr int kBwdThreads = 384;
constexpr float kBwdLog2e = 1.4426950408889634f;
constexpr int kBwdPrefetch = 8;   // stage loads are prefetched into L2 this many steps ahead

// ------------------------------------------------------------------------------------------
// Pre-pass over rows of x [B1, B2, S, D] (strided, unit stride along D): optional contiguous
// bf16 copy xc [B1*B2, S, D] and optional delta [B1*B2, S] = rowsum(x o y).  Half a warp per row,
// 16 bytes per lane and load; with D = 128 and aligned rows a warp has eight rows in flight.
// ------------------------------------------------------------------------------------------
// eight consecutive elements from a 16-byte aligned address: the loads only (no alignment test, no
// conversion), so that a thread can issue several before it uses the first
template <typename T> struct PrepRaw { uint4 q[sizeof(T) / 2]; };
template <typename T>
__device__ __forceinline__ void prep_load(const T* src, PrepRaw<T>& r) {
#pragma unroll
  for (int i = 0; i < (int)sizeof(T) / 2; ++i) r.q[i] = __ldg(reinterpret_cast<const uint4*>(src) + i);
}
template <typename T>
__device__ __forceinline__ void prep_unpack(const PrepRaw<T>& r, float (&v)[8]) {
  const T* t = reinterpret_cast<const T*>(&r);
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = to_f32<T>(t[e]);
}

constexpr int kPrepRows = 4;   // rows per half-warp and trip on the aligned path

template <typename T>
__global__ void __launch_bounds__(256) bwd_prep_kernel(const T* __restrict__ x, int64_t sxb1, int64_t sxb2,
                                                       int64_t sxs, int nb2, const T* __restrict__ y,
                                                       int64_t syb1, int64_t syb2, int64_t sys, int S, int D,
                                                       int64_t rows, __nv_bfloat16* __restrict__ xc,
                                                       float* __restrict__ delta, float* __restrict__ amax,
                                                       int aligned) {
  const int lane = threadIdx.x & 31, l16 = lane & 15;
  float vmax = 0.0f;   // largest |x| this thread has seen (non-negative floats order like their bit patterns)
  // 32-bit divisions (the host keeps rows below 2^31): a 64-bit divide costs more instructions than
  // everything else a thread does for its 16 bytes
  auto row_ptrs = [&](int64_t row, const T*& xr, const T*& yr) {
    const uint32_t b = (uint32_t)row / (uint32_t)S;
    const int s = (int)((uint32_t)row - b * (uint32_t)S);
    const uint32_t b1 = b / (uint32_t)nb2, b2 = b - b1 * (uint32_t)nb2;
    xr = x + (int64_t)b1 * sxb1 + (int64_t)b2 * sxb2 + (int64_t)s * sxs;
    yr = y ? (y + (int64_t)b1 * syb1 + (int64_t)b2 * syb2 + (int64_t)s * sys) : nullptr;
  };
  if (aligned && D == 128) {
    // every row is 16 lanes x 16 bytes, all addresses 16-byte aligned: a warp takes 2 * kPrepRows
    // rows per trip and issues all their loads (x and y) before it reduces the first
    const int64_t base0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * (2 * kPrepRows);
    const int64_t step = (int64_t)gridDim.x * 16 * kPrepRows;
    for (int64_t base = base0; base < rows; base += step) {
      int64_t row[kPrepRows];
      bool live[kPrepRows];
      PrepRaw<T> rx[kPrepRows], ry[kPrepRows];
#pragma unroll
      for (int j = 0; j < kPrepRows; ++j) {
        const int64_t row0 = base + 2 * j + (lane >> 4);
        live[j] = row0 < rows;
        row[j] = live[j] ? row0 : rows - 1;
        const T *xr, *yr;
        row_ptrs(row[j], xr, yr);
        prep_load<T>(xr + l16 * 8, rx[j]);
        if (y) prep_load<T>(yr + l16 * 8, ry[j]);
      }
#pragma unroll
      for (int j = 0; j < kPrepRows; ++j) {
        float v[8], w8[8];
        prep_unpack<T>(rx[j], v);
        if (amax != nullptr && live[j]) {
#pragma unroll
          for (int e = 0; e < 8; ++e) vmax = fmaxf(vmax, fabsf(v[e]));
        }
        if (xc && live[j]) {
          uint4 w;
          w.x = pack_bf16x2(v[0], v[1]);
          w.y = pack_bf16x2(v[2], v[3]);
          w.z = pack_bf16x2(v[4], v[5]);
          w.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(xc + row[j] * D + l16 * 8) = w;
        }
        if (delta) {
          float acc = 0.0f;
          prep_unpack<T>(ry[j], w8);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc = fmaf(v[e], w8[e], acc);
#pragma unroll
          for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
          if (l16 == 0 && live[j]) delta[row[j]] = acc;
        }
      }
    }
  } else {
    const int64_t base0 = ((int64_t)blockIdx.x * 8 + (threadIdx.x >> 5)) * 2;
    const int64_t nhw = (int64_t)gridDim.x * 16;
    for (int64_t base = base0; base < rows; base += nhw) {    // both half-warps take every trip (shuffles)
      const int64_t row0 = base + (lane >> 4);
      const bool live = row0 < rows;
      const int64_t row = live ? row0 : rows - 1;
      const T *xr, *yr;
      row_ptrs(row, xr, yr);
      float acc = 0.0f;
      for (int c = l16 * 8; c < D; c += 128) {
        float v[8], w8[8];
        load8<T>(xr + c, v);
        if (amax != nullptr && live) {
#pragma unroll
          for (int e = 0; e < 8; ++e) vmax = fmaxf(vmax, fabsf(v[e]));
        }
        if (yr) {
          load8<T>(yr + c, w8);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc = fmaf(v[e], w8[e], acc);
        }
        if (xc && live) {
          uint4 w;
          w.x = pack_bf16x2(v[0], v[1]);
          w.y = pack_bf16x2(v[2], v[3]);
          w.z = pack_bf16x2(v[4], v[5]);
          w.w = pack_bf16x2(v[6], v[7]);
          *reinterpret_cast<uint4*>(xc + row * D + c) = w;
        }
      }
      if (delta) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (l16 == 0 && live) delta[row] = acc;
      }
    }
  }
  if (amax != nullptr) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    if (lane == 0 && vmax > 0.0f && vmax < INFINITY)
      atomicMax(reinterpret_cast<unsigned int*>(amax), __float_as_uint(vmax));
  }
}

struct BwdParams {
  const uint8_t* qsc;   // [ZH, Sq, 8]
  const uint8_t* ksc;   // [ZHk, Skv, 8]
  const float* lse;     // [ZH, Sq] natural log
  const float* delta;   // [ZH, Sq]
  const float* bias;    // [Z, Skv] additive key bias (after the scaling) or null
  const int32_t* seq_start;  // [S] or null (varlen)
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

// P for 32 columns of one accumulator row: exp2(s * c2 + offsets).  Per-column statistics (the
// dK/dV kernel): `nl` points at the raw lse of the 32 columns in shared memory and `nl_row` is a
// per-thread offset (the key's bias * log2e, or 0).  Per-row (the dQ kernel): `nl_row` is
// -lse*log2e of the row and `nl`, when not null, points at the raw key bias of the 32 columns.
// Columns outside [lo, hi) relative to the chunk's first column are masked when `masked`.
template <bool kPerColumn, bool kColumnBias = false>
__device__ __forceinline__ void prob_chunk(const uint32_t (&sr)[32], float (&pf)[32], float c2, const float* nl,
                                           float nl_row, bool masked, int lo, int hi) {
  const float2 c22 = make_float2(c2, c2);
  const float2 row2 = make_float2(nl_row, nl_row);
  const float2 ml2 = make_float2(kPerColumn ? -kBwdLog2e : kBwdLog2e, kPerColumn ? -kBwdLog2e : kBwdLog2e);
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    float2 n01 = row2, n23 = row2;
    if constexpr (kPerColumn || kColumnBias) {
      const float4 l4 = *reinterpret_cast<const float4*>(nl + e);
      n01 = __ffma2_rn(make_float2(l4.x, l4.y), ml2, row2);
      n23 = __ffma2_rn(make_float2(l4.z, l4.w), ml2, row2);
    }
    const float2 t0 = __ffma2_rn(make_float2(__uint_as_float(sr[e]), __uint_as_float(sr[e + 1])), c22, n01);
    const float2 t1 = __ffma2_rn(make_float2(__uint_as_float(sr[e + 2]), __uint_as_float(sr[e + 3])), c22, n23);
    pf[e] = ex2_bwd(t0.x);
    pf[e + 1] = ex2_bwd(t0.y);
    pf[e + 2] = ex2_bwd(t1.x);
    pf[e + 3] = ex2_bwd(t1.y);
  }
  if (masked) {
#pragma unroll
    for (int e = 0; e < 32; ++e) pf[e] = (e >= lo && e < hi) ? pf[e] : 0.0f;
  }
}
// dS = P o (dP - delta) for 32 columns, packed to bf16 pairs.  Per-column: `nd` points at the raw
// delta values; per-row: `nd_row` is -delta.
template <bool kPerColumn>
__device__ __forceinline__ void ds_chunk(const float (&pf)[32], const uint32_t (&dr)[32], uint32_t (&dw)[16],
                                         const float* nd, float nd_row) {
#pragma unroll
  for (int e = 0; e < 32; e += 4) {
    float2 a0, a1;
    const float2 d01 = make_float2(__uint_as_float(dr[e]), __uint_as_float(dr[e + 1]));
    const float2 d23 = make_float2(__uint_as_float(dr[e + 2]), __uint_as_float(dr[e + 3]));
    if constexpr (kPerColumn) {
      const float4 n4 = *reinterpret_cast<const float4*>(nd + e);
      const float2 m1 = make_float2(-1.0f, -1.0f);
      a0 = __ffma2_rn(make_float2(n4.x, n4.y), m1, d01);
      a1 = __ffma2_rn(make_float2(n4.z, n4.w), m1, d23);
    } else {
      a0 = __fadd2_rn(d01, make_float2(nd_row, nd_row));
      a1 = __fadd2_rn(d23, make_float2(nd_row, nd_row));
    }
    const float2 d0 = __fmul2_rn(make_float2(pf[e], pf[e + 1]), a0);
    const float2 d1 = __fmul2_rn(make_float2(pf[e + 2], pf[e + 3]), a1);
    dw[e >> 1] = pack_bf16x2(d0.x, d0.y);
    dw[(e >> 1) + 1] = pack_bf16x2(d1.x, d1.y);
  }
}
// ------------------------------------------------------------------------------------------
// dK / dV
// TMEM: dV [0,128) | dK [128,256) | S^T slots [256,320) [320,384) | dP^T [384,448) |
//       SFK [448, 448+D/16) | two SFQ slots of D/16 columns
// Head dim 256: the accumulators of a full tile would need all 512 columns, so blockIdx.z picks a
// 128-wide half of dV / dK; S^T and dP^T still contract over the whole head dim.
// A softmax group reads its S^T slot into registers and writes P^T and dS^T (bf16 pairs, 16
// columns per 32 queries each) back into the same slot: the gradient GEMMs take them as TMEM A
// operands.
// ------------------------------------------------------------------------------------------
template <int D>
struct DkdvSmem {
  static constexpr int DS = D / 64;      // 64-element (128-byte) sub-tiles of a bf16 row
  static constexpr int KSUB = D / 128;   // 64-byte sub-tiles of a pack row
  static constexpr int KB = D / 64;      // K = 64 block-scaled MMAs per S^T, scale atoms per tile
  static constexpr int V = DS * 16384;   // V bf16 [128 keys x D]
  static constexpr int KP = KSUB * 8192; // K pack tile, 128 keys x D/2 B (64-byte swizzle)
  static constexpr int KSF = KB * 512;   // K scale atoms
  // per stage: dO bf16 [64 q x D], the 128-wide half of Q bf16 [64 q x 128] (8 KB sub-tiles),
  // Q pack [64 q x D/2 B], Q scale atoms, lse [64] and delta [64]
  static constexpr int DO = DS * 8192, Q = 16384, QP = KSUB * 4096, QSF = KB * 512, AUX = 1024;
  static constexpr int O_DO = 0, O_Q = DO, O_QP = DO + Q, O_QSF = O_QP + QP, O_AUX = O_QSF + QSF;
  static constexpr int STAGE = DO + Q + QP + QSF + AUX;
  static constexpr int NSTAGE = D == 128 ? 4 : 2;
  static constexpr int TOTAL = V + KP + NSTAGE * STAGE + KSF + 1024;
  static_assert(STAGE % 1024 == 0 && (V + KP) % 1024 == 0, "128-byte-swizzled tiles need 1 KB alignment");
};

template <int D, typename TG>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_kp, const __grid_constant__ CUtensorMap tm_qp,
                const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                const __grid_constant__ CUtensorMap tm_q, const BwdParams p) {
  using L = DkdvSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_v = smem;
  uint8_t* s_kp = s_v + L::V;
  uint8_t* s_stage = s_kp + L::KP;
  uint8_t* s_ksf = s_stage + L::NSTAGE * L::STAGE;

  __shared__ uint64_t full_tma[L::NSTAGE], full_aux[L::NSTAGE], empty[L::NSTAGE];
  __shared__ uint64_t kv_full, ksf_full, s_full[2], dp_full, dp_free, pds_full[2], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int jt = blockIdx.y;           // key tile (low tiles have the most visible queries: first)
  const int unit = blockIdx.x;         // z * hk + kh
  const int half = blockIdx.z;         // 128-wide slice of the head dim owned by this CTA
  const int zi = unit / p.hk, kh = unit % p.hk;
  const int n0 = jt * 128;
  const int shift = p.s_kv - p.s_q;
  const bool varlen = p.seq_start != nullptr;
  // 64-query steps that can see a key of this tile
  int q_lo = 0, q_hi = p.s_q;
  if (p.causal) q_lo = max(0, n0 - shift);
  if (varlen) {
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
    mbar_init(&dp_full, 1);
    mbar_init(&dp_free, 8);
    mbar_init(&acc_done, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&pds_full[b], 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  constexpr uint32_t T_DV = 0, T_DK = 128, T_ST = 256, T_DPT = 384, T_SFK = 448, T_SFQ = T_SFK + L::KB * 4;
  constexpr uint32_t SFQ_SLOT = L::KB * 4;
  static_assert(T_SFQ + 2 * SFQ_SLOT <= 512, "TMEM budget");

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && nstep > 0) {
      mbar_expect_tx(&kv_full, L::KP + L::V);
#pragma unroll
      for (int c = 0; c < L::KSUB; ++c) tma_load_3d(s_kp + c * 8192, &tm_kp, &kv_full, c * 64, n0, unit);
#pragma unroll
      for (int c = 0; c < L::DS; ++c) tma_load_3d(s_v + c * 16384, &tm_v, &kv_full, c * 64, n0, unit);
      // L2 prefetch kBwdPrefetch steps ahead: co-resident CTAs walk the same query tiles in step,
      // so without it every stage load is a first touch that waits on HBM
      auto prefetch = [&](int t) {
        const int gq = t / n_i, i = i_lo + t % n_i;
        const int zh = zi * p.h + kh * p.g + gq;
#pragma unroll
        for (int c = 0; c < L::KSUB; ++c) tma_prefetch_3d(&tm_qp, c * 64, i * 64, zh);
#pragma unroll
        for (int c = 0; c < L::DS; ++c) tma_prefetch_3d(&tm_do, c * 64, i * 64, zh);
        tma_prefetch_3d(&tm_q, half * 128, i * 64, zh);
        tma_prefetch_3d(&tm_q, half * 128 + 64, i * 64, zh);
      };
      for (int t = L::NSTAGE; t < min(nstep, kBwdPrefetch); ++t) prefetch(t);
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE;
        const int gq = st / n_i, i = i_lo + st % n_i;
        const int zh = zi * p.h + kh * p.g + gq;
        if (st + kBwdPrefetch < nstep) prefetch(st + kBwdPrefetch);
        if (st >= L::NSTAGE) mbar_wait(&empty[s], ((st / L::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_expect_tx(&full_tma[s], L::QP + L::DO + L::Q);
#pragma unroll
        for (int c = 0; c < L::KSUB; ++c)
          tma_load_3d(sb + L::O_QP + c * 4096, &tm_qp, &full_tma[s], c * 64, i * 64, zh);
#pragma unroll
        for (int c = 0; c < L::DS; ++c)
          tma_load_3d(sb + L::O_DO + c * 8192, &tm_do, &full_tma[s], c * 64, i * 64, zh);
        tma_load_3d(sb + L::O_Q, &tm_q, &full_tma[s], half * 128, i * 64, zh);
        tma_load_3d(sb + L::O_Q + 8192, &tm_q, &full_tma[s], half * 128 + 64, i * 64, zh);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale atoms / row statistics
    if (nstep > 0) {
      const uint8_t* ksrc = p.ksc + (int64_t)unit * p.s_kv * (D / 16);
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = lane + 32 * r4;
        const bool ok = n0 + r < p.s_kv;
        const uint8_t* g = ksrc + (int64_t)(ok ? n0 + r : 0) * (D / 16);
#pragma unroll
        for (int c = 0; c < L::KB; ++c)
          cp_async_4(smem_u32(s_ksf) + c * 512 + sf_atom_offset(r, 0), g + 4 * c, ok ? 4u : 0u);
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
          const uint8_t* g = p.qsc + ((int64_t)zh * p.s_q + (ok ? qi : 0)) * (D / 16);
#pragma unroll
          for (int c = 0; c < L::KB; ++c) cp_async_4(qsf + c * 512 + sf_atom_offset(r, 0), g + 4 * c, ok ? 4u : 0u);
          // lse and delta land as they are (rows past the end read 0 and are masked by range)
          const int64_t gi = (int64_t)zh * p.s_q + (ok ? qi : 0);
          cp_async_4(smem_u32(aux + r), p.lse + gi, ok ? 4u : 0u);
          cp_async_4(smem_u32(aux + 64 + r), p.delta + gi, ok ? 4u : 0u);
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
      const uint32_t id_dp = make_idesc_bf16(128, 64, false);
      const uint32_t id_acc = make_idesc_bf16(128, 128, true);
      mbar_wait(&kv_full, 0, &err, 3);
      mbar_wait(&ksf_full, 0, &err, 4);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < L::KB; ++c) tmem_cp_32x128b_warpx4(tmem + T_SFK + 4 * c, smem_u32(s_ksf + c * 512));
      // descriptors: constant fields once, then only the 16-byte-unit address field moves
      const uint64_t b_v = desc_sw128(s_v, 0), b_kp = desc_sw64(s_kp, 0);
      const uint64_t b_do = desc_sw128(s_stage + L::O_DO, 0);
      const uint64_t b_do_mn = desc_sw128_mn(s_stage + L::O_DO + half * 16384, 0, 8192);   // this half's two sub-tiles
      const uint64_t b_q_mn = desc_sw128_mn(s_stage + L::O_Q, 0, 8192), b_qp = desc_sw64(s_stage + L::O_QP, 0);
      // dV += P^T dO and dK += dS^T Q of step t (operands: slot t&1, stage t%NSTAGE)
      auto grad_gemms = [&](int t) {
        const uint64_t so = (uint64_t)((t % L::NSTAGE) * (L::STAGE >> 4));
        // slot columns: [P^T q0-31 | dS^T q0-31 | P^T q32-63 | dS^T q32-63], 16 each
        const uint32_t a_pt = tmem + T_ST + (t & 1) * 64, a_dst = a_pt + 16;
        const uint64_t x_do = b_do_mn + so, x_q = b_q_mn + so;
        const uint32_t acc0 = t > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ta(tmem + T_DV, a_pt + (k >> 1) * 32 + (k & 1) * 8, x_do + 128 * k, id_acc, k > 0 ? 1u : acc0);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ta(tmem + T_DK, a_dst + (k >> 1) * 32 + (k & 1) * 8, x_q + 128 * k, id_acc, k > 0 ? 1u : acc0);
      };
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE, b = st & 1;
        const uint32_t ph = (st / L::NSTAGE) & 1;
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_wait(&full_tma[s], ph, &err, 5);
        mbar_wait(&full_aux[s], ph, &err, 6);
        tc_fence_after();
        // S^T slot b: its P^T / dS^T were consumed by the gradient GEMMs of step st-2, issued
        // earlier on this in-order pipe
#pragma unroll
        for (int c = 0; c < L::KB; ++c)
          tmem_cp_32x128b_warpx4(tmem + T_SFQ + b * SFQ_SLOT + 4 * c, smem_u32(sb + L::O_QSF + c * 512));
        const uint64_t so = (uint64_t)(s * (L::STAGE >> 4));
        const uint64_t x_qp = b_qp + so, x_do = b_do + so;
#pragma unroll
        for (int k = 0; k < L::KB; ++k)
          umma_nvfp4(tmem + T_ST + b * 64, b_kp + (k >> 1) * 512 + (k & 1) * 2, x_qp + (k >> 1) * 256 + (k & 1) * 2,
                     id_s, tmem + T_SFK + k * 4, tmem + T_SFQ + b * SFQ_SLOT + k * 4, k > 0);
        umma_commit(&s_full[b]);
        if (st > 0) {
          mbar_wait(&dp_free, (st - 1) & 1, &err, 7);
          tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + T_DPT, b_v + (k >> 2) * 1024 + (k & 3) * 2, x_do + (k >> 2) * 512 + (k & 3) * 2, id_dp,
                    k > 0);
        umma_commit(&dp_full);
        if (st > 0) {
          mbar_wait(&pds_full[b ^ 1], ((st - 1) >> 1) & 1, &err, 8);
          tc_fence_after();
          grad_gemms(st - 1);
          umma_commit(&empty[(st - 1) % L::NSTAGE]);
        }
      }
      mbar_wait(&pds_full[(nstep - 1) & 1], ((nstep - 1) >> 1) & 1, &err, 9);
      tc_fence_after();
      grad_gemms(nstep - 1);
      umma_commit(&acc_done);
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax groups, epilogue
    const int grp = (warp - 4) >> 2;
    const int wq = warp & 3;
    const int row = wq * 32 + lane;     // key within the tile
    const int key = n0 + row;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c2 = p.scaling * kBwdLog2e;
    // additive bias of this key, in the exponent's base-2 units (-inf masks the key)
    const float bk2 = (p.bias != nullptr && key < p.s_kv) ? p.bias[(int64_t)zi * p.s_kv + key] * kBwdLog2e : 0.0f;
    // visible queries of this key: [ql, qh)
    int ql = 0, qh = 0;
    if (key < p.s_kv) {
      ql = p.causal ? max(key - shift, 0) : 0;
      qh = p.s_q;
      if (varlen) {
        ql = max(ql, (int)p.seq_start[key]);
        qh = min(qh, (int)p.seq_end[key]);
      }
      qh = max(qh, ql);
    }
    // both groups work on every step: group g owns queries [32g, 32g+32) of the 64-query tile
    for (int st = 0; st < nstep; ++st) {
      const int s = st % L::NSTAGE, b = st & 1, k2 = st >> 1;
      const int q0 = (i_lo + st % n_i) * 64 + grp * 32;
      uint8_t* sb = s_stage + s * L::STAGE;
      const float* aux = reinterpret_cast<const float*>(sb + L::O_AUX) + grp * 32;
      const uint32_t slot = tmem + lane_addr + T_ST + b * 64 + grp * 32;
      const bool masked = !__all_sync(0xffffffffu, q0 >= ql && q0 + 32 <= qh);
      mbar_wait(&full_aux[s], (st / L::NSTAGE) & 1, &err, 10);
      mbar_wait(&s_full[b], k2 & 1, &err, 11);
      mbar_wait(&dp_full, st & 1, &err, 13);
      tc_fence_after();
      // dP^T first: the single dP^T slot goes back to the issuer before any arithmetic
      uint32_t dr[32], sr[32];
      tmem_ld32(tmem + lane_addr + T_DPT + grp * 32, dr);
      tmem_ld32(slot, sr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dp_free);
      // P^T -> 16 columns, dS^T -> the next 16, over the S^T columns just read
      {
        float pf[32];
        uint32_t w[16];
        prob_chunk<true>(sr, pf, c2, aux, bk2, masked, ql - q0, qh - q0);
#pragma unroll
        for (int e = 0; e < 16; ++e) w[e] = pack_bf16x2(pf[2 * e], pf[2 * e + 1]);
        tmem_st16(slot, w);
        ds_chunk<true>(pf, dr, w, aux + 64, 0.0f);
        tmem_st16(slot + 16, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pds_full[b]);
    }
    // ---- epilogue: group g writes gradient columns [64g, 64g+64)
    TG* dkrow = static_cast<TG*>(p.dk) + ((int64_t)unit * p.s_kv + key) * D + half * 128 + grp * 64;
    TG* dvrow = static_cast<TG*>(p.dv) + ((int64_t)unit * p.s_kv + key) * D + half * 128 + grp * 64;
    if (nstep > 0) {
      mbar_wait(&acc_done, 0, &err, 14);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + T_DV + grp * 64 + c * 32, r);
        tmem_ld_wait();
        if (key < p.s_kv) store_row32<TG>(dvrow + c * 32, r, 1.0f);
        tmem_ld32(tmem + lane_addr + T_DK + grp * 64 + c * 32, r);
        tmem_ld_wait();
        if (key < p.s_kv) store_row32<TG>(dkrow + c * 32, r, p.scaling);
      }
      tc_fence_before();
    } else if (key < p.s_kv) {
      zero_row(dkrow, 64);
      zero_row(dvrow, 64);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ------------------------------------------------------------------------------------------
// dQ
// TMEM: dQ [0,128) | S slots [128,192) [192,256) | dP [256,320) | SFQ [320, 320+D/16) |
//       two SFK slots of D/16 columns.  Head dim 256: blockIdx.z picks a 128-wide half of dQ.
// dS (bf16 pairs, 32 columns) is written back into the S slot it came from and feeds the dQ GEMM
// as a TMEM A operand.
// ------------------------------------------------------------------------------------------
template <int D>
struct DqSmem {
  static constexpr int DS = D / 64, KSUB = D / 128, KB = D / 64;
  static constexpr int DO = DS * 16384;    // dO bf16 [128 q x D] as 16 KB sub-tiles
  static constexpr int QP = KSUB * 8192;   // Q pack tile, 128 queries x D/2 B
  static constexpr int QSF = KB * 512;
  // per stage: V bf16 [64 keys x D] and the 128-wide half of K bf16 (8 KB sub-tiles), K pack
  // [64 keys x D/2 B], K scale atoms
  static constexpr int V = DS * 8192, K = 16384, KP = KSUB * 4096, KSF = KB * 512, AUX = 1024;
  static constexpr int O_V = 0, O_K = V, O_KP = V + K, O_KSF = O_KP + KP, O_AUX = O_KSF + KSF;   // AUX: key bias [64]
  static constexpr int STAGE = V + K + KP + KSF + AUX;
  static constexpr int NSTAGE = D == 128 ? 4 : 2;
  static constexpr int TOTAL = DO + QP + NSTAGE * STAGE + QSF + 1024;
  static_assert(STAGE % 1024 == 0 && (DO + QP) % 1024 == 0, "128-byte-swizzled tiles need 1 KB alignment");
};

template <int D, typename TG>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_qp, const __grid_constant__ CUtensorMap tm_kp,
              const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ CUtensorMap tm_k, const BwdParams p) {
  using L = DqSmem<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_do = smem;
  uint8_t* s_qp = s_do + L::DO;
  uint8_t* s_stage = s_qp + L::QP;
  uint8_t* s_qsf = s_stage + L::NSTAGE * L::STAGE;

  __shared__ uint64_t full_tma[L::NSTAGE], full_sf[L::NSTAGE], empty[L::NSTAGE];
  __shared__ uint64_t q_full, qsf_full, s_full[2], dp_full, dp_free, ds_full[2], acc_done;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mblk = gridDim.y - 1 - blockIdx.y;   // late query tiles see the most keys: first
  const int zh = blockIdx.x;
  const int half = blockIdx.z;         // 128-wide slice of the head dim owned by this CTA
  const int zi = zh / p.h, hi = zh % p.h;
  const int unit = zi * p.hk + hi / p.g;
  const int m0 = mblk * 128;
  const int shift = p.s_kv - p.s_q;
  const bool varlen = p.seq_start != nullptr;
  int k_lo = 0, k_hi = p.s_kv;
  if (p.causal) k_hi = max(0, min(p.s_kv, m0 + 128 + shift));
  if (varlen) {
    k_lo = p.seq_start[min(m0, p.s_q - 1)];
    k_hi = min(k_hi, (int)p.seq_end[min(m0 + 127, p.s_q - 1)]);
  }
  const int j_lo = k_lo / 64;
  const int nstep = max((k_hi + 63) / 64 - j_lo, 0);

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < L::NSTAGE; ++i) {
      mbar_init(&full_tma[i], 1);
      mbar_init(&full_sf[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(&q_full, 1);
    mbar_init(&qsf_full, 1);
    mbar_init(&dp_full, 1);
    mbar_init(&dp_free, 8);
    mbar_init(&acc_done, 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&ds_full[b], 8);
    }
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  constexpr uint32_t T_DQ = 0, T_S = 128, T_DP = 256, T_SFQ = 320, T_SFK = T_SFQ + L::KB * 4;
  constexpr uint32_t SFK_SLOT = L::KB * 4;

  if (warp == 0) {
    if (elect_one() && nstep > 0) {
      mbar_expect_tx(&q_full, L::QP + L::DO);
#pragma unroll
      for (int c = 0; c < L::KSUB; ++c) tma_load_3d(s_qp + c * 8192, &tm_qp, &q_full, c * 64, m0, zh);
#pragma unroll
      for (int c = 0; c < L::DS; ++c) tma_load_3d(s_do + c * 16384, &tm_do, &q_full, c * 64, m0, zh);
      auto prefetch = [&](int t) {
        const int key0 = (j_lo + t) * 64;
#pragma unroll
        for (int c = 0; c < L::KSUB; ++c) tma_prefetch_3d(&tm_kp, c * 64, key0, unit);
#pragma unroll
        for (int c = 0; c < L::DS; ++c) tma_prefetch_3d(&tm_v, c * 64, key0, unit);
        tma_prefetch_3d(&tm_k, half * 128, key0, unit);
        tma_prefetch_3d(&tm_k, half * 128 + 64, key0, unit);
      };
      for (int t = L::NSTAGE; t < min(nstep, kBwdPrefetch); ++t) prefetch(t);
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE, key0 = (j_lo + st) * 64;
        if (st + kBwdPrefetch < nstep) prefetch(st + kBwdPrefetch);
        if (st >= L::NSTAGE) mbar_wait(&empty[s], ((st / L::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_expect_tx(&full_tma[s], L::KP + L::V + L::K);
#pragma unroll
        for (int c = 0; c < L::KSUB; ++c)
          tma_load_3d(sb + L::O_KP + c * 4096, &tm_kp, &full_tma[s], c * 64, key0, unit);
#pragma unroll
        for (int c = 0; c < L::DS; ++c) tma_load_3d(sb + L::O_V + c * 8192, &tm_v, &full_tma[s], c * 64, key0, unit);
        tma_load_3d(sb + L::O_K, &tm_k, &full_tma[s], half * 128, key0, unit);
        tma_load_3d(sb + L::O_K + 8192, &tm_k, &full_tma[s], half * 128 + 64, key0, unit);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    if (nstep > 0) {
      const uint8_t* qsrc = p.qsc + (int64_t)zh * p.s_q * (D / 16);
#pragma unroll
      for (int r4 = 0; r4 < 4; ++r4) {
        const int r = lane + 32 * r4;
        const bool ok = m0 + r < p.s_q;
        const uint8_t* g = qsrc + (int64_t)(ok ? m0 + r : 0) * (D / 16);
#pragma unroll
        for (int c = 0; c < L::KB; ++c)
          cp_async_4(smem_u32(s_qsf) + c * 512 + sf_atom_offset(r, 0), g + 4 * c, ok ? 4u : 0u);
      }
      cp_async_commit();
      cp_async_wait<0>();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&qsf_full);
      const uint8_t* ksrc = p.ksc + (int64_t)unit * p.s_kv * (D / 16);
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE, key0 = (j_lo + st) * 64;
        if (st >= L::NSTAGE) mbar_wait(&empty[s], ((st / L::NSTAGE) & 1) ^ 1, &err, 2);
        const uint32_t ksf = smem_u32(s_stage + s * L::STAGE + L::O_KSF);
#pragma unroll
        for (int r2 = 0; r2 < 2; ++r2) {
          const int r = lane + 32 * r2;
          const int key = key0 + r;
          const bool ok = key < p.s_kv;
          const uint8_t* g = ksrc + (int64_t)(ok ? key : 0) * (D / 16);
#pragma unroll
          for (int c = 0; c < L::KB; ++c) cp_async_4(ksf + c * 512 + sf_atom_offset(r, 0), g + 4 * c, ok ? 4u : 0u);
          if (p.bias != nullptr)
            cp_async_4(smem_u32(s_stage + s * L::STAGE + L::O_AUX) + r * 4,
                       p.bias + (int64_t)zi * p.s_kv + (ok ? key : 0), ok ? 4u : 0u);
        }
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_sf[s]);
      }
    }
  } else if (warp == 1) {
    if (elect_one() && nstep > 0) {
      const uint32_t id_s = make_idesc_nvfp4(128, 64);
      const uint32_t id_dp = make_idesc_bf16(128, 64, false);
      const uint32_t id_acc = make_idesc_bf16(128, 128, true);
      mbar_wait(&q_full, 0, &err, 3);
      mbar_wait(&qsf_full, 0, &err, 4);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < L::KB; ++c) tmem_cp_32x128b_warpx4(tmem + T_SFQ + 4 * c, smem_u32(s_qsf + c * 512));
      const uint64_t b_do = desc_sw128(s_do, 0), b_qp = desc_sw64(s_qp, 0);
      const uint64_t b_v = desc_sw128(s_stage + L::O_V, 0), b_k_mn = desc_sw128_mn(s_stage + L::O_K, 0, 8192);
      const uint64_t b_kp = desc_sw64(s_stage + L::O_KP, 0);
      auto grad_gemm = [&](int t) {   // dQ += dS K of step t
        const uint32_t a_ds = tmem + T_S + (t & 1) * 64;
        const uint64_t x_k = b_k_mn + (uint64_t)((t % L::NSTAGE) * (L::STAGE >> 4));
        const uint32_t acc0 = t > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ta(tmem + T_DQ, a_ds + (k >> 1) * 32 + (k & 1) * 8, x_k + 128 * k, id_acc, k > 0 ? 1u : acc0);
      };
      for (int st = 0; st < nstep; ++st) {
        const int s = st % L::NSTAGE, b = st & 1;
        const uint32_t ph = (st / L::NSTAGE) & 1;
        uint8_t* sb = s_stage + s * L::STAGE;
        mbar_wait(&full_tma[s], ph, &err, 5);
        mbar_wait(&full_sf[s], ph, &err, 6);
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < L::KB; ++c)
          tmem_cp_32x128b_warpx4(tmem + T_SFK + b * SFK_SLOT + 4 * c, smem_u32(sb + L::O_KSF + c * 512));
        const uint64_t so = (uint64_t)(s * (L::STAGE >> 4));
        const uint64_t x_kp = b_kp + so, x_v = b_v + so;
#pragma unroll
        for (int k = 0; k < L::KB; ++k)
          umma_nvfp4(tmem + T_S + b * 64, b_qp + (k >> 1) * 512 + (k & 1) * 2, x_kp + (k >> 1) * 256 + (k & 1) * 2,
                     id_s, tmem + T_SFQ + k * 4, tmem + T_SFK + b * SFK_SLOT + k * 4, k > 0);
        umma_commit(&s_full[b]);
        if (st > 0) {
          mbar_wait(&dp_free, (st - 1) & 1, &err, 7);
          tc_fence_after();
        }
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16(tmem + T_DP, b_do + (k >> 2) * 1024 + (k & 3) * 2, x_v + (k >> 2) * 512 + (k & 3) * 2, id_dp,
                    k > 0);
        umma_commit(&dp_full);
        if (st > 0) {
          mbar_wait(&ds_full[b ^ 1], ((st - 1) >> 1) & 1, &err, 8);
          tc_fence_after();
          grad_gemm(st - 1);
          umma_commit(&empty[(st - 1) % L::NSTAGE]);
        }
      }
      mbar_wait(&ds_full[(nstep - 1) & 1], ((nstep - 1) >> 1) & 1, &err, 9);
      tc_fence_after();
      grad_gemm(nstep - 1);
      umma_commit(&acc_done);
    }
    __syncwarp();
  } else if (warp >= 4) {
    const int grp = (warp - 4) >> 2;
    const int wq = warp & 3;
    const int row_in = wq * 32 + lane;
    const int row = m0 + row_in;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const float c2 = p.scaling * kBwdLog2e;
    const bool row_ok = row < p.s_q;
    const float nl = row_ok ? -p.lse[(int64_t)zh * p.s_q + row] * kBwdLog2e : 0.0f;
    const float nd = row_ok ? -p.delta[(int64_t)zh * p.s_q + row] : 0.0f;
    // visible keys of this row: [kl, kh)
    int kl = 0, kh = 0;
    if (row_ok) {
      kh = p.causal ? min(p.s_kv, row + shift + 1) : p.s_kv;
      if (varlen) {
        kl = p.seq_start[row];
        kh = min(kh, (int)p.seq_end[row]);
      }
      kh = max(kh, kl);
    }
    // both groups work on every step: group g owns keys [32g, 32g+32) of the 64-key tile
    for (int st = 0; st < nstep; ++st) {
      const int b = st & 1, k2 = st >> 1;
      const int key0 = (j_lo + st) * 64 + grp * 32;
      const uint32_t slot = tmem + lane_addr + T_S + b * 64;
      const bool masked = !__all_sync(0xffffffffu, key0 >= kl && key0 + 32 <= kh);
      const float* kbias = nullptr;
      if (p.bias != nullptr) {      // the stage's key bias (landed with the scale atoms)
        const int sg = st % L::NSTAGE;
        mbar_wait(&full_sf[sg], (st / L::NSTAGE) & 1, &err, 10);
        kbias = reinterpret_cast<const float*>(s_stage + sg * L::STAGE + L::O_AUX) + grp * 32;
      }
      mbar_wait(&s_full[b], k2 & 1, &err, 11);
      mbar_wait(&dp_full, st & 1, &err, 13);
      tc_fence_after();
      uint32_t dr[32], sr[32];
      tmem_ld32(tmem + lane_addr + T_DP + grp * 32, dr);
      tmem_ld32(slot + grp * 32, sr);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&dp_free);
      {
        float pf[32];
        uint32_t w[16];
        if (kbias != nullptr) prob_chunk<false, true>(sr, pf, c2, kbias, nl, masked, kl - key0, kh - key0);
        else prob_chunk<false, false>(sr, pf, c2, nullptr, nl, masked, kl - key0, kh - key0);
        ds_chunk<false>(pf, dr, w, nullptr, nd);
        // dS of keys [32g, 32g+32) replaces the first 16 of the S columns this thread just read
        tmem_st16(slot + grp * 32, w);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ds_full[b]);
    }
    TG* dqrow = static_cast<TG*>(p.dq) + ((int64_t)zh * p.s_q + row) * D + half * 128 + grp * 64;
    if (nstep > 0) {
      mbar_wait(&acc_done, 0, &err, 14);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + T_DQ + grp * 64 + c * 32, r);
        tmem_ld_wait();
        if (row_ok) store_row32<TG>(dqrow + c * 32, r, p.scaling);
      }
      tc_fence_before();
    } else if (row_ok) {
      zero_row(dqrow, 64);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

template <typename T>
int prep_launch(const void* x, int64_t sxb1, int64_t sxb2, int64_t sxs, int64_t nb1, int64_t nb2, const void* y,
                int64_t syb1, int64_t syb2, int64_t sys, int S, int D, __nv_bfloat16* xc, float* delta,
                float* amax, cudaStream_t st) {
  const int64_t rows = nb1 * nb2 * S;
  if (rows >= (1LL << 31)) return fail(-1, "nvfp4_bwd_prep: more than 2^31 rows");
  auto al = [](const void* p, int64_t a, int64_t b, int64_t c) {
    return p == nullptr || ((reinterpret_cast<uintptr_t>(p) & 15) == 0 && (a * (int64_t)sizeof(T)) % 16 == 0 &&
                            (b * (int64_t)sizeof(T)) % 16 == 0 && (c * (int64_t)sizeof(T)) % 16 == 0);
  };
  const int aligned = al(x, sxb1, sxb2, sxs) && al(y, syb1, syb2, sys) && D == 128;
  const int64_t per_block = aligned ? 16 * kPrepRows : 16;
  const int64_t blocks = (rows + per_block - 1) / per_block;
  const unsigned grid = (unsigned)(blocks < 148 * 16 ? blocks : 148 * 16);
  bwd_prep_kernel<T><<<grid, 256, 0, st>>>(static_cast<const T*>(x), sxb1, sxb2, sxs, (int)nb2,
                                           static_cast<const T*>(y), syb1, syb2, sys, S, D, rows, xc, delta, amax,
                                           aligned);
  return launch_result("nvfp4_bwd_prep");
}

}  // namespace nvfp4

extern "C" int nvfp4_bwd_prep(const void* x, int dtype, int64_t sxb1, int64_t sxb2, int64_t sxs,
                              int64_t nb1, int64_t nb2, const void* y, int64_t syb1, int64_t syb2,
                              int64_t sys, int64_t s, int d, void* xc, float* delta, float* amax,
                              nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(x != nullptr && (xc || delta || amax), "nvfp4_bwd_prep: nothing to do");
  NVFP4_REQUIRE(d >= 8 && d % 8 == 0 && s >= 1 && nb1 >= 1 && nb2 >= 1, "nvfp4_bwd_prep: bad extents");
  NVFP4_REQUIRE(s < (1LL << 31), "nvfp4_bwd_prep: sequence too long");
  NVFP4_REQUIRE(delta == nullptr || y != nullptr, "nvfp4_bwd_prep: delta needs the second operand");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  auto* c = static_cast<__nv_bfloat16*>(xc);
  switch (dtype) {
    case NVFP4_DT_BF16:
      return prep_launch<__nv_bfloat16>(x, sxb1, sxb2, sxs, nb1, nb2, y, syb1, syb2, sys, (int)s, d, c, delta, amax, st);
    case NVFP4_DT_FP16:
      return prep_launch<__half>(x, sxb1, sxb2, sxs, nb1, nb2, y, syb1, syb2, sys, (int)s, d, c, delta, amax, st);
    case NVFP4_DT_FP32:
      return prep_launch<float>(x, sxb1, sxb2, sxs, nb1, nb2, y, syb1, syb2, sys, (int)s, d, c, delta, amax, st);
    default:
      return fail(-1, "nvfp4_bwd_prep: unknown dtype %d", dtype);
  }
}

extern "C" int nvfp4_bwd_hp(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv,
                            const uint8_t* ksc, const void* q_bf16, const void* k_bf16,
                            const void* v_bf16, const void* do_bf16, const float* lse,
                            const float* delta, const float* key_bias, const int32_t* seq_start,
                            const int32_t* seq_end, void* dq, void* dk, void* dv, int grad_dtype, int64_t z, int64_t h,
                            int64_t hk, int64_t s_q, int64_t s_kv, int d, float scaling, int flags,
                            int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_bwd_hp: head dim must be 128 or 256");
  NVFP4_REQUIRE(z >= 1 && h >= 1 && hk >= 1 && h % hk == 0, "nvfp4_bwd_hp: bad head counts");
  NVFP4_REQUIRE(s_q >= 1 && s_kv >= 1 && s_q < (1LL << 30) && s_kv < (1LL << 30), "nvfp4_bwd_hp: bad sequence extents");
  NVFP4_REQUIRE(qnv && qsc && knv && ksc && q_bf16 && k_bf16 && v_bf16 && do_bf16 && lse && delta && dq && dk && dv,
                "nvfp4_bwd_hp: null pointer");
  const bool varlen = seq_start != nullptr;
  NVFP4_REQUIRE(varlen == (seq_end != nullptr), "nvfp4_bwd_hp: seq_start and seq_end go together");
  NVFP4_REQUIRE(!varlen || (z == 1 && s_q == s_kv), "nvfp4_bwd_hp: varlen needs Z == 1 and Sq == Skv");
  NVFP4_REQUIRE(!(flags & NVFP4_FWD_CAUSAL) || varlen || s_kv >= s_q, "nvfp4_bwd_hp: causal needs Skv >= Sq");
  NVFP4_REQUIRE((s_kv + 127) / 128 < 65536 && z * h < (1LL << 31) && (s_q + 127) / 128 < 65536,
                "nvfp4_bwd_hp: grid too large");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t zh = z * h, zhk = z * hk;
  CUtensorMap t_qp64, t_qp128, t_kp64, t_kp128, t_v64, t_v128, t_do64, t_do128, t_q64, t_k64;
  int rc;
  const uint64_t pb = (uint64_t)d / 2, hb = (uint64_t)d * 2;   // bytes per pack row / bf16 row
  if ((rc = make_tmap_u8_3d_sw64(&t_qp64, qnv, pb, s_q, zh, pb, (uint64_t)s_q * pb, 64, "nvfp4_bwd_hp(Qp64)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_qp128, qnv, pb, s_q, zh, pb, (uint64_t)s_q * pb, 128, "nvfp4_bwd_hp(Qp128)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_kp64, knv, pb, s_kv, zhk, pb, (uint64_t)s_kv * pb, 64, "nvfp4_bwd_hp(Kp64)"))) return rc;
  if ((rc = make_tmap_u8_3d_sw64(&t_kp128, knv, pb, s_kv, zhk, pb, (uint64_t)s_kv * pb, 128, "nvfp4_bwd_hp(Kp128)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_v64, v_bf16, d, s_kv, zhk, hb, (uint64_t)s_kv * hb, 64, "nvfp4_bwd_hp(V64)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_v128, v_bf16, d, s_kv, zhk, hb, (uint64_t)s_kv * hb, 128, "nvfp4_bwd_hp(V128)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_do64, do_bf16, d, s_q, zh, hb, (uint64_t)s_q * hb, 64, "nvfp4_bwd_hp(dO64)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_do128, do_bf16, d, s_q, zh, hb, (uint64_t)s_q * hb, 128, "nvfp4_bwd_hp(dO128)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_q64, q_bf16, d, s_q, zh, hb, (uint64_t)s_q * hb, 64, "nvfp4_bwd_hp(Q64)"))) return rc;
  if ((rc = make_tmap_bf16_3d_sw128(&t_k64, k_bf16, d, s_kv, zhk, hb, (uint64_t)s_kv * hb, 64, "nvfp4_bwd_hp(K64)"))) return rc;
  BwdParams p;
  p.qsc = qsc; p.ksc = ksc; p.lse = lse; p.delta = delta; p.bias = key_bias;
  p.seq_start = seq_start; p.seq_end = seq_end;
  p.dq = dq; p.dk = dk; p.dv = dv;
  p.h = (int)h; p.hk = (int)hk; p.g = (int)(h / hk); p.s_q = (int)s_q; p.s_kv = (int)s_kv;
  p.scaling = scaling; p.causal = (flags & NVFP4_FWD_CAUSAL) ? 1 : 0; p.status = status;
  const unsigned halves = (unsigned)(d / 128);
  auto launch = [&](auto kdkdv, auto kdq, int smem_dkdv, int smem_dq) -> int {
    cudaError_t e = cudaFuncSetAttribute(kdkdv, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkdv);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_hp: smem attribute: %s", cudaGetErrorString(e));
    e = cudaFuncSetAttribute(kdq, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_bwd_hp: smem attribute: %s", cudaGetErrorString(e));
    dim3 g1((unsigned)zhk, (unsigned)((s_kv + 127) / 128), halves);
    kdkdv<<<g1, kBwdThreads, smem_dkdv, st>>>(t_kp128, t_qp64, t_v128, t_do64, t_q64, p);
    int r1 = launch_result("nvfp4_bwd_hp(dkdv)");
    if (r1) return r1;
    dim3 g2((unsigned)zh, (unsigned)((s_q + 127) / 128), halves);
    kdq<<<g2, kBwdThreads, smem_dq, st>>>(t_qp128, t_kp64, t_do128, t_v64, t_k64, p);
    return launch_result("nvfp4_bwd_hp(dq)");
  };
#define NVFP4_BWD_LAUNCH(DD, TT) \
  launch(bwd_dkdv_kernel<DD, TT>, bwd_dq_kernel<DD, TT>, DkdvSmem<DD>::TOTAL, DqSmem<DD>::TOTAL)
  if (d == 128) {
    switch (grad_dtype) {
      case NVFP4_DT_BF16: return NVFP4_BWD_LAUNCH(128, __nv_bfloat16);
      case NVFP4_DT_FP16: return NVFP4_BWD_LAUNCH(128, __half);
      case NVFP4_DT_FP32: return NVFP4_BWD_LAUNCH(128, float);
      default: return fail(-1, "nvfp4_bwd_hp: unknown grad dtype %d", grad_dtype);
    }
  }
  switch (grad_dtype) {
    case NVFP4_DT_BF16: return NVFP4_BWD_LAUNCH(256, __nv_bfloat16);
    case NVFP4_DT_FP16: return NVFP4_BWD_LAUNCH(256, __half);
    case NVFP4_DT_FP32: return NVFP4_BWD_LAUNCH(256, float);
    default: return fail(-1, "nvfp4_bwd_hp: unknown grad dtype %d", grad_dtype);
  }
#undef NVFP4_BWD_LAUNCH
}
