// NVFP4 flash-attention forward for sm_100a.
//
// One CTA owns a 128-row query tile of one (batch, head) and walks 128-key tiles:
//     S[128 x 128]  = Q_tile . K_tile^T        tcgen05.mma kind::mxf4nvf4, e4m3 scale per 16
//     P             = exp(S*scale - m) packed to NVFP4 per 16 keys (same scale rule as the packer)
//     O[128 x D]   += P . V_tile               same MMA kind, V held as V^T (packed along keys)
// Q/K/V^T nibble tiles arrive by TMA straight from the packed tensors; scale bytes are re-laid
// into the 32x16-byte form tcgen05.cp expects by two loader warps; S and O live in TMEM.  One
// thread owns a slice of one query row (one TMEM lane, 32 or 64 key columns), so the
// per-16-key P pack needs no cross-thread traffic.  The running maximum is exact (O is rescaled in TMEM whenever a row's maximum moves),
// which keeps the P quantisation decisions those of a plain 128-key tile walk.
//
// Warp roles (640 threads): 0 TMA producer, 1 QK^T issuer, 2 scale loader (+bias, +sample
// ids), 3 PV issuer, 4-19 softmax / correction / epilogue.  At D=128 the sixteen softmax warps
// form two groups that alternate key tiles; at D=256 (one S buffer) they share each tile.
// Every barrier wait is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"

namespace nvfp4 {

#ifndef NVFP4_FWD_NP
#define NVFP4_FWD_NP 4
#endif
constexpr int kFwdNP = NVFP4_FWD_NP;               // softmax threads per query row (D = 256 path)
constexpr int kFwdThreads = 128 + 128 * kFwdNP;
constexpr float kFwdLog2e = 1.4426950408889634f;

template <int D>
struct FwdCfg {
  static constexpr int KSUB = D / 128;  // 64-byte-wide sub-tiles of a Q/K row
  static constexpr int KB = D / 64;     // K=64 MMAs per QK tile
  static constexpr int NT = D / 128;    // 128-row pieces of the V^T tile (N of the PV MMA = D)
  static constexpr int NSBUF = (D == 128) ? 2 : 1;  // S / P buffers
  static constexpr int NSTAGE = (D == 128) ? 4 : 3;
  static constexpr int Q_BYTES = KSUB * 8192;
  static constexpr int K_BYTES = KSUB * 8192;
  static constexpr int V_BYTES = NT * 8192;
  static constexpr int KSF_BYTES = KB * 512;
  static constexpr int VSF_BYTES = 2 * NT * 512;  // [kb][nt]
  static constexpr int AUX_BYTES = 1024;          // 128 fp32 bias + 128 int32 sample ids
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + KSF_BYTES + VSF_BYTES + AUX_BYTES;
  static constexpr int QSF_BYTES = KB * 512;
  static constexpr int P_BYTES = 8192;
  static constexpr int PSF_BYTES = 1024;
  static constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + Q_BYTES + QSF_BYTES +
                                    NSBUF * (P_BYTES + PSF_BYTES) + 1024;
  // TMEM columns
  static constexpr int T_S = 0;                       // NSBUF x 128
  static constexpr int T_O = NSBUF * 128;             // D
  static constexpr int T_SFQ = T_O + D;               // KB * 4
  static constexpr int T_SFK = T_SFQ + KB * 4;        // 2 x KB * 4
  static constexpr int T_SFP = T_SFK + 2 * KB * 4;    // 2 x 8
  static constexpr int T_SFV = T_SFP + 16;            // 2 x (2 * NT * 4)
  static constexpr int T_END = T_SFV + 2 * 2 * NT * 4;
  static_assert(T_END <= 512, "TMEM budget exceeded");
};

struct FwdParams {
  const uint8_t* qsc;  // [ZH, Sq, D/16]
  const uint8_t* ksc;  // [ZHk, Skv, D/16]
  const uint8_t* vsc;  // [ZHk, D, s_pad/16]
  const float* bias;   // [Z, Skv] or null
  const int32_t* seq_id;     // [S] or null
  const int32_t* seq_start;  // [S] or null
  void* out;
  int64_t so_z, so_h, so_s;
  float* lse;  // [ZH, Sq] or null
  int h, hk, g;
  int s_q, s_kv, s_pad;
  float scaling;
  int causal;
  int* status;
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// kVarlen: packed rows with per-token sample ids (a separate instantiation keeps the dense kernel
// free of the sample tests).
// sample-id test: a compile-time yes in the varlen instantiation, the run-time test otherwise
#define FWD_HAS_SEQ (kVarlen || p.seq_id != nullptr)
template <int D, typename TO, bool kVarlen>
__global__ void __launch_bounds__(kFwdThreads, 1)
fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const FwdParams p) {
  using C = FwdCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_stage = smem;
  uint8_t* s_q = s_stage + C::NSTAGE * C::STAGE_BYTES;
  uint8_t* s_qsf = s_q + C::Q_BYTES;
  uint8_t* s_p = s_qsf + C::QSF_BYTES;
  uint8_t* s_psf = s_p + C::NSBUF * C::P_BYTES;

  __shared__ uint64_t full_kv[C::NSTAGE], full_sf[C::NSTAGE], empty[C::NSTAGE];
  __shared__ uint64_t s_full[2], s_free[2], p_full[2], pv_done[2], q_full, qsf_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  __shared__ int s_lo_tile;
  __shared__ float xmax[2][kFwdNP][128];
  __shared__ float xl[kFwdNP][128];
  __shared__ float m_row[2][128];
  __shared__ uint64_t m_ready[2];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // grid = (heads, query tiles): all heads of the heaviest (last) query tile are scheduled first,
  // so the kernel ends on the cheapest tiles instead of on a long straggler
  const int mblk = gridDim.y - 1 - blockIdx.y;
  const int zh = blockIdx.x;
  const int zi = zh / p.h, hi = zh % p.h;
  const int unit = zi * p.hk + hi / p.g;  // (batch, kv head)
  const int m0 = mblk * 128;
  const int shift = p.s_kv - p.s_q;  // bottom-right aligned causal offset

  // key-tile range of this query tile
  int hi_key = p.s_kv;
  if (p.causal) hi_key = min(p.s_kv, m0 + 128 + shift);
  if (hi_key < 0) hi_key = 0;
  const int t_hi = (hi_key + 127) / 128;

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(&full_kv[i], 1);
      mbar_init(&full_sf[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], C::NSBUF == 2 ? 256 : 128 * kFwdNP);
      mbar_init(&p_full[i], C::NSBUF == 2 ? 8 : 4 * kFwdNP);
      mbar_init(&pv_done[i], 1);
      mbar_init(&m_ready[i], 128);
    }
    mbar_init(&q_full, 1);
    mbar_init(&qsf_full, 4);
    mbar_fence_init();
    int lo = 0;
    if (FWD_HAS_SEQ) lo = (p.seq_start[min(m0, p.s_q - 1)] / 128) * 128;
    s_lo_tile = lo / 128;
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, 512);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;
  // varlen: rows of a tile are sorted by sample, so the first row has the earliest start
  const int t_lo = s_lo_tile;
  const int ntile = max(t_hi - t_lo, 0);

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && ntile > 0) {
      mbar_expect_tx(&q_full, C::Q_BYTES);
#pragma unroll
      for (int ks = 0; ks < C::KSUB; ++ks) tma_load_3d(s_q + ks * 8192, &tm_q, &q_full, ks * 64, m0, zh);
      for (int i = 0; i < ntile; ++i) {
        const int s = i % C::NSTAGE, t = t_lo + i;
        if (i >= C::NSTAGE) mbar_wait(&empty[s], ((i / C::NSTAGE) & 1) ^ 1, &err, 1);
        uint8_t* st = s_stage + s * C::STAGE_BYTES;
        mbar_expect_tx(&full_kv[s], C::K_BYTES + C::V_BYTES);
#pragma unroll
        for (int ks = 0; ks < C::KSUB; ++ks)
          tma_load_3d(st + ks * 8192, &tm_k, &full_kv[s], ks * 64, t * 128, unit);
#pragma unroll
        for (int nt = 0; nt < C::NT; ++nt)
          tma_load_3d(st + C::K_BYTES + nt * 8192, &tm_v, &full_kv[s], t * 64, nt * 128, unit);
      }
    }
    __syncwarp();
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale loader
    // K scales (+ key bias, sample ids) and V^T scales of a tile, re-laid into the 32 x 16-byte
    // atoms tcgen05.cp copies.  The next tile's bytes are fetched into registers one tile
    // ahead, so per tile the warp pays a shared-memory store, not a trip to L2.
    const uint8_t* ksrc = p.ksc + (int64_t)unit * p.s_kv * (D / 16);
    const uint8_t* vsrc = p.vsc + (int64_t)unit * D * (p.s_pad / 16);
    uint32_t kx[4][C::KB];
    float nb[4];
    int32_t ns[4];
    uint2 vx[D / 32];
    auto fetch = [&](int t) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int key = t * 128 + lane + 32 * j;
#pragma unroll
        for (int k = 0; k < C::KB; ++k) kx[j][k] = 0u;
        nb[j] = 0.0f;
        ns[j] = -1;
        if (key < p.s_kv) {
          const uint32_t* gsrc = reinterpret_cast<const uint32_t*>(ksrc + (int64_t)key * (D / 16));
#pragma unroll
          for (int k = 0; k < C::KB; ++k) kx[j][k] = __ldg(gsrc + k);
          if (p.bias != nullptr) nb[j] = __ldg(p.bias + (int64_t)zi * p.s_kv + key);
          if (FWD_HAS_SEQ) ns[j] = __ldg(p.seq_id + key);
        }
      }
#pragma unroll
      for (int j = 0; j < D / 32; ++j)
        vx[j] = __ldg(reinterpret_cast<const uint2*>(vsrc + (int64_t)(lane + 32 * j) * (p.s_pad / 16) + (int64_t)t * 8));
    };
    if (ntile > 0) fetch(t_lo);
    for (int i = 0; i < ntile; ++i) {
      const int s = i % C::NSTAGE;
      if (i >= C::NSTAGE) mbar_wait(&empty[s], ((i / C::NSTAGE) & 1) ^ 1, &err, 2);
      uint8_t* st = s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES;
      float* aux_bias = reinterpret_cast<float*>(st + C::KSF_BYTES + C::VSF_BYTES);
      int32_t* aux_seq = reinterpret_cast<int32_t*>(st + C::KSF_BYTES + C::VSF_BYTES + 512);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int r = lane + 32 * j;
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          *reinterpret_cast<uint32_t*>(st + k * 512 + sf_atom_offset(r, 0)) = kx[j][k];
        aux_bias[r] = nb[j];
        aux_seq[r] = ns[j];
      }
      uint8_t* dst = st + C::KSF_BYTES;
#pragma unroll
      for (int j = 0; j < D / 32; ++j) {
        const int dr = lane + 32 * j;
        const int nt = dr >> 7, r = dr & 127;
        *reinterpret_cast<uint32_t*>(dst + (0 * C::NT + nt) * 512 + sf_atom_offset(r, 0)) = vx[j].x;
        *reinterpret_cast<uint32_t*>(dst + (1 * C::NT + nt) * 512 + sf_atom_offset(r, 0)) = vx[j].y;
      }
      if (i + 1 < ntile) fetch(t_lo + i + 1);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_sf[s]);
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ QK^T issuer
    if (elect_one() && ntile > 0) {
      const uint32_t idesc_qk = make_idesc_nvfp4(128, 128);
      mbar_wait(&q_full, 0, &err, 3);
      mbar_wait(&qsf_full, 0, &err, 4);
      tc_fence_after();
#pragma unroll
      for (int k = 0; k < C::KB; ++k)
        tmem_cp_32x128b_warpx4(tmem + C::T_SFQ + k * 4, smem_u32(s_qsf + k * 512));
      for (int j = 0; j < ntile; ++j) {
        const int s = j % C::NSTAGE, b = j % C::NSBUF;
        const uint32_t ph = (j / C::NSTAGE) & 1;
        mbar_wait(&full_kv[s], ph, &err, 5);
        mbar_wait(&full_sf[s], ph, &err, 6);
        if (j >= C::NSBUF) mbar_spin_wait(&s_free[b], ((j / C::NSBUF) & 1) ^ 1, &err, 7);
        tc_fence_after();
        uint8_t* st = s_stage + s * C::STAGE_BYTES;
        const uint32_t sfk = tmem + C::T_SFK + (j & 1) * C::KB * 4;
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          tmem_cp_32x128b_warpx4(sfk + k * 4, smem_u32(st + C::K_BYTES + C::V_BYTES + k * 512));
#pragma unroll
        for (int k = 0; k < C::KB; ++k) {
          const uint64_t ad = make_smem_desc(smem_u32(s_q + (k >> 1) * 8192) + (k & 1) * 32, 16, 512, 4);
          const uint64_t bd = make_smem_desc(smem_u32(st + (k >> 1) * 8192) + (k & 1) * 32, 16, 512, 4);
          umma_nvfp4(tmem + C::T_S + b * 128, ad, bd, idesc_qk, tmem + C::T_SFQ + k * 4, sfk + k * 4,
                     k > 0);
        }
        umma_commit(&s_full[b]);
      }
    }
    __syncwarp();
  } else if (warp == 3) {
    // ------------------------------------------------------------------ PV issuer
    // A thread of its own, so a QK^T for tile i+2 is never queued behind the wait for P(i).
    if (elect_one() && ntile > 0) {
      const uint32_t idesc_pv = make_idesc_nvfp4(128, D);
      for (int i = 0; i < ntile; ++i) {
        const int s = i % C::NSTAGE, b = i % C::NSBUF;
        // the V tile and V scales of stage s landed before this tile's QK^T was issued, but this
        // thread has to observe them itself; it does so while P is still being written
        mbar_wait(&full_kv[s], (i / C::NSTAGE) & 1, &err, 15);
        mbar_wait(&full_sf[s], (i / C::NSTAGE) & 1, &err, 16);
        mbar_spin_wait(&p_full[b], (i / C::NSBUF) & 1, &err, 8);
        tc_fence_after();
        uint8_t* st = s_stage + s * C::STAGE_BYTES;
        const uint32_t sfp = tmem + C::T_SFP + (i & 1) * 8;
        const uint32_t sfv = tmem + C::T_SFV + (i & 1) * (2 * C::NT * 4);
#pragma unroll
        for (int k = 0; k < 2; ++k)
          tmem_cp_32x128b_warpx4(sfp + k * 4, smem_u32(s_psf + b * C::PSF_BYTES + k * 512));
#pragma unroll
        for (int k = 0; k < 2 * C::NT; ++k)
          tmem_cp_32x128b_warpx4(sfv + k * 4,
                                 smem_u32(st + C::K_BYTES + C::V_BYTES + C::KSF_BYTES + k * 512));
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const uint64_t ad = make_smem_desc(smem_u32(s_p + b * C::P_BYTES) + k * 32, 16, 512, 4);
          const uint64_t bd = make_smem_desc(smem_u32(st + C::K_BYTES) + k * 32, 16, 512, 4);
          umma_nvfp4(tmem + C::T_O, ad, bd, idesc_pv, sfp + k * 4, sfv + k * C::NT * 4,
                     (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&pv_done[b]);
        umma_commit(&empty[s]);
      }
    }
    __syncwarp();
  } else if (C::NSBUF == 2) {
    // ------------------------------------------------------------------ softmax / epilogue (D = 128)
    // Two groups of eight warps alternate key tiles (group g owns tiles g, g+2, ...), so while
    // one group sits in its exp/pack phase the other does its TMEM loads, row maxima,
    // barrier and O rescale: the phases of consecutive tiles overlap instead of adding up.
    // Within a group two threads share a query row (64 key columns each, handled as two
    // 32-column chunks to stay inside the register budget of a 640-thread CTA).  The running
    // maximum is handed from tile to tile through shared memory (m_row / m_ready), so it is
    // still the exact maximum of a sequential 128-key tile walk.
    const int sw = warp - 4;
    const int grp = sw >> 3;             // which tiles (parity)
    const int wq = sw & 3;               // TMEM lane quadrant
    const int half = (sw >> 2) & 1;      // which 64 key columns
    const int part = grp * 2 + half;     // 0..3: slice of O this thread stores in the epilogue
    const int row_in = wq * 32 + lane;
    const int row = m0 + row_in;
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    constexpr int OC = D / 4;            // O columns stored per thread in the epilogue
    constexpr int RC = D / 2;            // O columns rescaled per thread (two threads per row in a group)
    if (part == 0) {
      uint32_t wds[C::KB];
#pragma unroll
      for (int k = 0; k < C::KB; ++k) wds[k] = 0u;
      if (row < p.s_q) {
        const uint32_t* gsrc =
            reinterpret_cast<const uint32_t*>(p.qsc + ((int64_t)zh * p.s_q + row) * (D / 16));
#pragma unroll
        for (int k = 0; k < C::KB; ++k) wds[k] = __ldg(gsrc + k);
      }
#pragma unroll
      for (int k = 0; k < C::KB; ++k)
        *reinterpret_cast<uint32_t*>(s_qsf + k * 512 + sf_atom_offset(row_in, 0)) = wds[k];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&qsf_full);
    }
    const int my_seq = FWD_HAS_SEQ ? p.seq_id[min(row, p.s_q - 1)] : 0;
    // packed rows: when all 128 rows of this tile belong to one sample, key tiles that lie wholly
    // inside that sample need no per-element sample test
    const bool q_one_sample =
        FWD_HAS_SEQ && (p.seq_id[min(m0, p.s_q - 1)] == p.seq_id[min(m0 + 127, p.s_q - 1)]);
    const int my_limit = p.causal ? (row + shift) : (p.s_kv - 1);
    const float c2 = p.scaling * kFwdLog2e;
    const float inv_scaling = 1.0f / p.scaling;
    float m_own = -INFINITY, l_run = 0.0f;   // running max (log2 units) after this group's last tile
    const uint32_t xmax_s = smem_u32(&xmax[0][0][0]);
    const uint32_t mrow_s = smem_u32(&m_row[0][0]);

    for (int i = grp; i < ntile; i += 2) {
      const int b = i & 1, s = i % C::NSTAGE, t = t_lo + i;
      const int n0 = t * 128 + half * 64;
      const uint32_t s_addr = tmem + lane_addr + C::T_S + b * 128 + half * 64;
      bool tile_masked = (t * 128 + 127 > m0 + shift && p.causal) || (t * 128 + 128 > p.s_kv) ||
                         (p.bias != nullptr) || (!kVarlen && p.seq_id != nullptr);   // varlen: completed below
      const uint8_t* aux = s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES + C::KSF_BYTES +
                           C::VSF_BYTES;
      const float* aux_bias0 = reinterpret_cast<const float*>(aux);
      const int32_t* aux_seq0 = reinterpret_cast<const int32_t*>(aux + 512);
      // visible keys of this row inside the tile: columns [0, lim128] (causal + tail)
      const int lim128 = min(my_limit, p.s_kv - 1) - t * 128;
      auto mask_cols = [&](int col0, float (&sv)[32]) {   // col0: first key column inside the tile
        if (tile_masked) {
          if (p.bias != nullptr) {
#pragma unroll
            for (int e = 0; e < 32; ++e) sv[e] += aux_bias0[col0 + e] * inv_scaling;
          }
          if (FWD_HAS_SEQ) {
#pragma unroll
            for (int e = 0; e < 32; ++e) sv[e] = (aux_seq0[col0 + e] == my_seq) ? sv[e] : -INFINITY;
          }
#pragma unroll
          for (int e = 0; e < 32; ++e) sv[e] = (col0 + e <= lim128) ? sv[e] : -INFINITY;
        }
      };
      auto mask_chunk = [&](int c, float (&sv)[32]) { mask_cols(half * 64 + c * 32, sv); };
      auto load_chunk = [&](int c, float (&sv)[32]) {
        uint32_t r[32];
        tmem_ld32(s_addr + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) sv[e] = __uint_as_float(r[e]);
        mask_chunk(c, sv);
      };
      mbar_wait(&s_full[b], (i >> 1) & 1, &err, 9);
      tc_fence_after();
      if constexpr (kVarlen)   // keys are sorted by sample: first and last id equal => all equal
        tile_masked = tile_masked || !(q_one_sample && aux_seq0[0] == my_seq && aux_seq0[127] == my_seq);
      // ---- pass 1: maxima of the four 16-key groups of this thread's 64 columns, and their maximum
      float mx = -INFINITY;
      float gm[4];
      auto group_max = [&](int c, const float (&sv)[32]) {
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          float v = fmax3(sv[h2 * 16], sv[h2 * 16 + 1], sv[h2 * 16 + 2]);
#pragma unroll
          for (int e = 3; e < 15; e += 2) v = fmax3(v, sv[h2 * 16 + e], sv[h2 * 16 + e + 1]);
          gm[c * 2 + h2] = fmaxf(v, sv[h2 * 16 + 15]);
        }
        mx = fmax3(mx, gm[c * 2], gm[c * 2 + 1]);
      };
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float sv[32];
        load_chunk(c, sv);
        group_max(c, sv);
      }
      const uint32_t xb = (uint32_t)(((i >> 1) & 1) * 4 + grp * 2);
      sts_f32(xmax_s + ((xb + half) * 128 + row_in) * 4u, mx);
      named_bar_sync(1 + grp, 256);
      mx = fmaxf(mx, lds_f32(xmax_s + ((xb + (half ^ 1)) * 128 + row_in) * 4u));
      // ---- running maximum handed over from the tile before (owned by the other group)
      float m_prev = -INFINITY;
      if (i > 0) {
        mbar_wait(&m_ready[b ^ 1], ((i - 1) >> 1) & 1, &err, 13);
        m_prev = lds_f32(mrow_s + (uint32_t)((b ^ 1) * 128 + row_in) * 4u);
      }
      const float m_new = fmaxf(m_prev, mx * c2);
      if (half == 0) {
        sts_f32(mrow_s + (uint32_t)(b * 128 + row_in) * 4u, m_new);
        mbar_arrive(&m_ready[b]);
      }
      const float m_sf = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = ex2_approx(m_prev - m_sf);
      const bool changed = (m_new > m_prev) && (i > 0);
      l_run *= ex2_approx(m_own - m_sf);
      m_own = m_new;

      // Block scales of P ahead of the exponentials: ex2 is monotonic, so the largest probability
      // of a 16-key group is ex2 of its largest score -- the same bits as the maximum over the
      // sixteen results -- and the scale chain (e4m3 round, decode, reciprocal) leaves the
      // dependent path of the pack.
      uint32_t scw = 0u;
      float inv_g[4];
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        const float am = ex2_approx(fmaf(gm[g], c2, -m_sf));
        const float s32 = fminf(fmaxf(am * 0.16666667f, kScaleFloor), kScaleMax);
        uint16_t sb16;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sb16) : "f"(0.0f), "f"(s32));
        const uint32_t sb = sb16 & 0xFFu;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_g[g]) : "f"(e4m3_to_f32((uint8_t)sb)));
        scw |= sb << (8 * g);
      }
      // P buffer b must have been consumed by the PV of tile i - 2
      if (i >= 2) mbar_wait(&pv_done[b], ((i >> 1) & 1) ^ 1, &err, 10);
      const uint32_t pt = smem_u32(s_p + b * C::P_BYTES);
      const uint32_t psf = smem_u32(s_psf + b * C::PSF_BYTES);
      const float2 c22 = make_float2(c2, c2);
      const float2 nm2 = make_float2(-m_sf, -m_sf);
      float2 lsum4[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) lsum4[c] = make_float2(0.0f, 0.0f);
      // ---- pass 2: exp, row sum, NVFP4 pack of P (two 32-column chunks = four 16-key groups)
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = cc;
        float sv[32];
        load_chunk(c, sv);
        if (c == 1) {
          tc_fence_before();
          mbar_arrive(&s_free[b]);
        }
#pragma unroll
        for (int g2 = 0; g2 < 2; ++g2) {
          const int g = c * 2 + g2;
          const float2 inv2 = make_float2(inv_g[g], inv_g[g]);
          float2 y[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            const float2 t2 = __ffma2_rn(make_float2(sv[g2 * 16 + 2 * e], sv[g2 * 16 + 2 * e + 1]), c22, nm2);
            const float2 pe = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
            lsum4[g] = __fadd2_rn(lsum4[g], pe);
            y[e] = __fmul2_rn(pe, inv2);
          }
          const uint32_t lo = e2m1x8(y[0].x, y[0].y, y[1].x, y[1].y, y[2].x, y[2].y, y[3].x, y[3].y);
          const uint32_t hi2 = e2m1x8(y[4].x, y[4].y, y[5].x, y[5].y, y[6].x, y[6].y, y[7].x, y[7].y);
          sts_v2(pt + sw64_offset(row_in, (half * 4 + g) * 8), lo, hi2);
        }
      }
      sts_b32(psf + half * 512 + sf_atom_offset(row_in, 0), scw);
      {
        const float2 t01 = __fadd2_rn(lsum4[0], lsum4[1]), t23 = __fadd2_rn(lsum4[2], lsum4[3]);
        const float2 tt = __fadd2_rn(t01, t23);
        l_run += tt.x + tt.y;
      }
      if (__any_sync(0xffffffffu, changed)) {
        // O is rescaled (this thread: half of its row) once the PV of tile i - 1 has landed
        mbar_wait(&pv_done[b ^ 1], ((i - 1) >> 1) & 1, &err, 11);
        tc_fence_after();
        const float a = changed ? alpha : 1.0f;
        const float2 a2 = make_float2(a, a);
        {
#pragma unroll
          for (int c = 0; c < RC / 32; ++c) {
            uint32_t r[32];
            tmem_ld32(tmem + lane_addr + C::T_O + half * RC + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
              const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), a2);
              r[e] = __float_as_uint(v.x);
              r[e + 1] = __float_as_uint(v.y);
            }
            tmem_st32(tmem + lane_addr + C::T_O + half * RC + c * 32, r);
          }
        }
        tmem_st_wait();
        tc_fence_before();
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }

    // ---- epilogue: bring the four partial row sums to the final maximum, O / l -> out, LSE
    float m_fin = -INFINITY;
    if (ntile > 0) {
      const int last = ntile - 1;
      mbar_wait(&m_ready[last & 1], (last >> 1) & 1, &err, 14);
      m_fin = lds_f32(mrow_s + (uint32_t)((last & 1) * 128 + row_in) * 4u);
    }
    {
      const float m_sf = (m_fin == -INFINITY) ? 0.0f : m_fin;
      xl[part][row_in] = l_run * ex2_approx(m_own - m_sf);
    }
    named_bar_sync(3, 512);
    l_run = xl[0][row_in] + xl[1][row_in] + xl[2][row_in] + xl[3][row_in];
    TO* orow = nullptr;
    if (row < p.s_q)
      orow = static_cast<TO*>(p.out) + (int64_t)zi * p.so_z + (int64_t)hi * p.so_h +
             (int64_t)row * p.so_s + part * OC;
    if (ntile > 0) {
      const int last = ntile - 1;
      mbar_wait(&pv_done[last & 1], (last >> 1) & 1, &err, 12);
      tc_fence_after();
      float inv_l;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_l) : "f"((l_run == 0.0f) ? 1.0f : l_run));
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + C::T_O + part * OC + c * 32, r);
        tmem_ld_wait();
        if (orow != nullptr) {
          if constexpr (sizeof(TO) == 2) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const TO a0 = from_f32<TO>(__uint_as_float(r[2 * e]) * inv_l);
              const TO a1 = from_f32<TO>(__uint_as_float(r[2 * e + 1]) * inv_l);
              w[e] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a0)) |
                     ((uint32_t)(*reinterpret_cast<const uint16_t*>(&a1)) << 16);
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
          } else {
            float4* dst = reinterpret_cast<float4*>(orow + c * 32);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              dst[e] = make_float4(__uint_as_float(r[4 * e]) * inv_l, __uint_as_float(r[4 * e + 1]) * inv_l,
                                   __uint_as_float(r[4 * e + 2]) * inv_l, __uint_as_float(r[4 * e + 3]) * inv_l);
          }
        }
      }
      tc_fence_before();
    } else if (orow != nullptr) {
      for (int e = 0; e < OC; ++e) orow[e] = from_f32<TO>(0.0f);
    }
    if (p.lse != nullptr && row < p.s_q && part == 0) {
      const float l_safe = (l_run == 0.0f) ? 1.0f : l_run;
      const float m_f = (m_fin == -INFINITY) ? 0.0f : m_fin;
      p.lse[(int64_t)zh * p.s_q + row] = m_f * 0.6931471805599453f + logf(l_safe);
    }
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    // (D = 256: one S buffer.)  All sixteen softmax warps share each tile: NP threads per query
    // row, each owning 128/NP key columns; a row's threads exchange their partial maxima
    // through shared memory once per tile and rescale / store their own slice of O.
    const int sw = warp - 4;
    const int wq = sw & 3;               // TMEM lane quadrant
    const int half = sw >> 2;            // which slice of the tile's key columns (0 .. NP-1)
    constexpr int NP = kFwdNP;
    constexpr int CW = 128 / NP;         // key columns per thread
    constexpr int NG = CW / 16;          // 16-key groups per thread
    const int row_in = wq * 32 + lane;   // row within the query tile
    const int row = m0 + row_in;         // query index
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    constexpr int OC = D / kFwdNP;       // O columns owned by this thread
    if (half == 0) {
      // Q scale bytes -> A-operand scale atoms
      uint32_t wds[C::KB];
#pragma unroll
      for (int k = 0; k < C::KB; ++k) wds[k] = 0u;
      if (row < p.s_q) {
        const uint32_t* gsrc =
            reinterpret_cast<const uint32_t*>(p.qsc + ((int64_t)zh * p.s_q + row) * (D / 16));
#pragma unroll
        for (int k = 0; k < C::KB; ++k) wds[k] = __ldg(gsrc + k);
      }
#pragma unroll
      for (int k = 0; k < C::KB; ++k)
        *reinterpret_cast<uint32_t*>(s_qsf + k * 512 + sf_atom_offset(row_in, 0)) = wds[k];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&qsf_full);
    }
    const int my_seq = FWD_HAS_SEQ ? p.seq_id[min(row, p.s_q - 1)] : 0;
    const bool q_one_sample =
        FWD_HAS_SEQ && (p.seq_id[min(m0, p.s_q - 1)] == p.seq_id[min(m0 + 127, p.s_q - 1)]);
    const int my_limit = p.causal ? (row + shift) : (p.s_kv - 1);  // last visible key index
    const float c2 = p.scaling * kFwdLog2e;
    const float inv_scaling = 1.0f / p.scaling;
    float m_run = -INFINITY, l_run = 0.0f;   // m_run in log2 units
    const uint32_t xmax_s = smem_u32(&xmax[0][0][0]);

    for (int i = 0; i < ntile; ++i) {
      const int b = i % C::NSBUF, s = i % C::NSTAGE, t = t_lo + i;
      const int n0 = t * 128 + half * CW;
      mbar_wait(&s_full[b], (i / C::NSBUF) & 1, &err, 9);
      tc_fence_after();
      float sv[CW];
      {
        uint32_t r0[CW / 32][32];
#pragma unroll
        for (int c = 0; c < CW / 32; ++c) tmem_ld32(tmem + lane_addr + C::T_S + b * 128 + half * CW + c * 32, r0[c]);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < CW / 32; ++c)
#pragma unroll
          for (int e = 0; e < 32; ++e) sv[c * 32 + e] = __uint_as_float(r0[c][e]);
      }
      tc_fence_before();
      mbar_arrive(&s_free[b]);

      bool tile_masked = (t * 128 + 127 > m0 + shift && p.causal) || (t * 128 + 128 > p.s_kv) ||
                         (p.bias != nullptr) || (!kVarlen && p.seq_id != nullptr);
      {
        const int32_t* aux_seq0 = reinterpret_cast<const int32_t*>(
            s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES + C::KSF_BYTES + C::VSF_BYTES + 512);
        if constexpr (kVarlen)   // keys are sorted by sample: first and last id equal => all equal
          tile_masked = tile_masked || !(q_one_sample && aux_seq0[0] == my_seq && aux_seq0[127] == my_seq);
      }
      if (tile_masked) {
        const uint8_t* aux = s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES + C::KSF_BYTES +
                             C::VSF_BYTES;
        const float* aux_bias = reinterpret_cast<const float*>(aux) + half * CW;
        const int32_t* aux_seq = reinterpret_cast<const int32_t*>(aux + 512) + half * CW;
#pragma unroll
        for (int e = 0; e < CW; ++e) {
          float v = sv[e];
          if (p.bias != nullptr) v += aux_bias[e] * inv_scaling;
          const int key = n0 + e;
          bool ok = key <= my_limit && key < p.s_kv;
          if (FWD_HAS_SEQ) ok = ok && (aux_seq[e] == my_seq);
          sv[e] = ok ? v : -INFINITY;
        }
      }
      float mx;
      float m4[NG];                     // maxima of the thread's 16-key groups
      {
#pragma unroll
        for (int c = 0; c < NG; ++c) {
          float v = fmax3(sv[c * 16], sv[c * 16 + 1], sv[c * 16 + 2]);
#pragma unroll
          for (int e = 3; e < 15; e += 2) v = fmax3(v, sv[c * 16 + e], sv[c * 16 + e + 1]);
          m4[c] = fmaxf(v, sv[c * 16 + 15]);
        }
        mx = m4[0];
#pragma unroll
        for (int c = 1; c < NG; ++c) mx = fmaxf(mx, m4[c]);
      }
      sts_f32(xmax_s + (uint32_t)(((i & 1) * NP + half) * 128 + row_in) * 4u, mx);
      named_bar_sync(1, 128 * NP);
#pragma unroll
      for (int o = 1; o < NP; ++o)
        mx = fmaxf(mx, lds_f32(xmax_s + (uint32_t)(((i & 1) * NP + ((half + o) % NP)) * 128 + row_in) * 4u));
      const float m_new = fmaxf(m_run, mx * c2);
      const float m_sf = (m_new == -INFINITY) ? 0.0f : m_new;
      const float alpha = ex2_approx(m_run - m_sf);
      const bool changed = (m_new > m_run) && (i > 0);
      m_run = m_new;

      // P buffer b must have been consumed by the PV of tile i - NSBUF
      if (i >= C::NSBUF) mbar_wait(&pv_done[b], ((i / C::NSBUF) & 1) ^ 1, &err, 10);
      const uint32_t pt = smem_u32(s_p + b * C::P_BYTES);
      const uint32_t psf = smem_u32(s_psf + b * C::PSF_BYTES);
      float2 lsum4[NG];
#pragma unroll
      for (int c = 0; c < NG; ++c) lsum4[c] = make_float2(0.0f, 0.0f);
      uint32_t scw = 0u;
      const float2 c22 = make_float2(c2, c2);
      const float2 nm2 = make_float2(-m_sf, -m_sf);
      // block scales of P ahead of the exponentials (ex2 is monotonic: the largest probability of a
      // group is ex2 of its largest score), so the scale chain is off the dependent path of the pack
      float inv_g[NG];
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const float am = ex2_approx(fmaf(m4[g], c2, -m_sf));
        const float s32 = fminf(fmaxf(am * 0.16666667f, kScaleFloor), kScaleMax);
        uint16_t sb16;
        asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sb16) : "f"(0.0f), "f"(s32));
        const uint32_t sb = sb16 & 0xFFu;
        asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_g[g]) : "f"(e4m3_to_f32((uint8_t)sb)));
        scw |= sb << (8 * g);
      }
#pragma unroll
      for (int g = 0; g < NG; ++g) {
        const float2 inv2 = make_float2(inv_g[g], inv_g[g]);
        float2 y[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float2 t2 = __ffma2_rn(make_float2(sv[g * 16 + 2 * e], sv[g * 16 + 2 * e + 1]), c22, nm2);
          const float2 pe = make_float2(ex2_approx(t2.x), ex2_approx(t2.y));
          lsum4[g] = __fadd2_rn(lsum4[g], pe);
          y[e] = __fmul2_rn(pe, inv2);
        }
        const uint32_t lo = e2m1x8(y[0].x, y[0].y, y[1].x, y[1].y, y[2].x, y[2].y, y[3].x, y[3].y);
        const uint32_t hi2 = e2m1x8(y[4].x, y[4].y, y[5].x, y[5].y, y[6].x, y[6].y, y[7].x, y[7].y);
        sts_v2(pt + sw64_offset(row_in, (half * NG + g) * 8), lo, hi2);
      }
      // this thread's NG scale bytes: groups half*NG .. of the row's 8 (4 per K=64 atom)
      if constexpr (NG == 4) {
        sts_b32(psf + half * 512 + sf_atom_offset(row_in, 0), scw);
      } else {
        asm volatile("st.shared.b16 [%0], %1;" ::"r"(psf + (half >> 1) * 512 + sf_atom_offset(row_in, (half & 1) * 2)),
                     "h"((uint16_t)scw) : "memory");
      }
      {
        float2 tt = lsum4[0];
#pragma unroll
        for (int c = 1; c < NG; ++c) tt = __fadd2_rn(tt, lsum4[c]);
        l_run = l_run * alpha + (tt.x + tt.y);
      }

      if (__any_sync(0xffffffffu, changed)) {
        // this thread's slice of O is rescaled once the previous PV has landed
        const int pb = (i - 1) % C::NSBUF;
        mbar_wait(&pv_done[pb], ((i - 1) / C::NSBUF) & 1, &err, 11);
        tc_fence_after();
        const float a = changed ? alpha : 1.0f;
        const float2 a2 = make_float2(a, a);
#pragma unroll
        for (int c = 0; c < OC / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(tmem + lane_addr + C::T_O + half * OC + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[e]), __uint_as_float(r[e + 1])), a2);
            r[e] = __float_as_uint(v.x);
            r[e + 1] = __float_as_uint(v.y);
          }
          tmem_st32(tmem + lane_addr + C::T_O + half * OC + c * 32, r);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[b]);
    }

    // ---- epilogue: O / l -> out, LSE.  The row sum is the total of the NP slices.
    xl[half][row_in] = l_run;
    named_bar_sync(1, 128 * NP);
#pragma unroll
    for (int o = 1; o < NP; ++o) l_run += xl[(half + o) % NP][row_in];
    TO* orow = nullptr;
    if (row < p.s_q)
      orow = static_cast<TO*>(p.out) + (int64_t)zi * p.so_z + (int64_t)hi * p.so_h +
             (int64_t)row * p.so_s + half * OC;
    if (ntile > 0) {
      const int last = ntile - 1;
      mbar_wait(&pv_done[last % C::NSBUF], (last / C::NSBUF) & 1, &err, 12);
      tc_fence_after();
      float inv_l;
      asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv_l) : "f"((l_run == 0.0f) ? 1.0f : l_run));
#pragma unroll
      for (int c = 0; c < OC / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(tmem + lane_addr + C::T_O + half * OC + c * 32, r);
        tmem_ld_wait();
        if (orow != nullptr) {
          if constexpr (sizeof(TO) == 2) {
            uint32_t w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const TO a0 = from_f32<TO>(__uint_as_float(r[2 * e]) * inv_l);
              const TO a1 = from_f32<TO>(__uint_as_float(r[2 * e + 1]) * inv_l);
              w[e] = (uint32_t)(*reinterpret_cast<const uint16_t*>(&a0)) |
                     ((uint32_t)(*reinterpret_cast<const uint16_t*>(&a1)) << 16);
            }
            uint4* dst = reinterpret_cast<uint4*>(orow + c * 32);
#pragma unroll
            for (int e = 0; e < 4; ++e) dst[e] = make_uint4(w[4 * e], w[4 * e + 1], w[4 * e + 2], w[4 * e + 3]);
          } else {
            float4* dst = reinterpret_cast<float4*>(orow + c * 32);
#pragma unroll
            for (int e = 0; e < 8; ++e)
              dst[e] = make_float4(__uint_as_float(r[4 * e]) * inv_l, __uint_as_float(r[4 * e + 1]) * inv_l,
                                   __uint_as_float(r[4 * e + 2]) * inv_l, __uint_as_float(r[4 * e + 3]) * inv_l);
          }
        }
      }
      tc_fence_before();
    } else if (orow != nullptr) {
      for (int e = 0; e < OC; ++e) orow[e] = from_f32<TO>(0.0f);
    }
    if (p.lse != nullptr && row < p.s_q && half == 0) {
      const float l_safe = (l_run == 0.0f) ? 1.0f : l_run;
      const float m_fin = (m_run == -INFINITY) ? 0.0f : m_run;
      p.lse[(int64_t)zh * p.s_q + row] = m_fin * 0.6931471805599453f + logf(l_safe);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, 512);
}

#undef FWD_HAS_SEQ
template <int D, typename TO>
int fwd_launch(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
               const FwdParams& p, int64_t zh, cudaStream_t st) {
  using C = FwdCfg<D>;
  auto kern = (p.seq_id != nullptr) ? fwd_kernel<D, TO, true> : fwd_kernel<D, TO, false>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES);
  if (e != cudaSuccess) return fail((int)e, "nvfp4_fwd: smem attribute: %s", cudaGetErrorString(e));
  dim3 grid((unsigned)zh, (unsigned)((p.s_q + 127) / 128));
  kern<<<grid, kFwdThreads, C::SMEM_BYTES, st>>>(tq, tk, tv, p);
  return launch_result("nvfp4_fwd");
}

}  // namespace nvfp4

extern "C" int nvfp4_fwd(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv,
                         const uint8_t* ksc, const uint8_t* vnv, const uint8_t* vsc,
                         const float* bias, const int32_t* seq_id, const int32_t* seq_start,
                         void* out, int out_dtype, int64_t so_z, int64_t so_h, int64_t so_s,
                         float* lse, int64_t z, int64_t h, int64_t hk, int64_t s_q, int64_t s_kv,
                         int64_t s_pad, int d, float scaling, int flags, int* status,
                         nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_fwd: D must be 128 or 256");
  NVFP4_REQUIRE(z >= 1 && h >= 1 && hk >= 1 && h % hk == 0, "nvfp4_fwd: bad head counts");
  NVFP4_REQUIRE(s_q >= 1 && s_kv >= 1, "nvfp4_fwd: empty sequence");
  NVFP4_REQUIRE(s_pad % 128 == 0 && s_pad >= s_kv, "nvfp4_fwd: s_pad must be a multiple of 128 >= s_kv");
  NVFP4_REQUIRE(qnv && qsc && knv && ksc && vnv && vsc && out, "nvfp4_fwd: null pointer");
  NVFP4_REQUIRE((seq_id == nullptr) == (seq_start == nullptr), "nvfp4_fwd: seq_id/seq_start go together");
  NVFP4_REQUIRE(seq_id == nullptr || (z == 1 && s_q == s_kv), "nvfp4_fwd: varlen needs Z == 1 and Sq == Skv");
  NVFP4_REQUIRE((s_q + 127) / 128 < 65536, "nvfp4_fwd: too many query tiles");
  NVFP4_REQUIRE(s_q < (1LL << 30) && s_kv < (1LL << 30), "nvfp4_fwd: sequence too long");
  const size_t esz = out_dtype == NVFP4_DT_FP32 ? 4 : 2;
  NVFP4_REQUIRE(((uintptr_t)out % 16) == 0 && (so_z * esz) % 16 == 0 && (so_h * esz) % 16 == 0 &&
                    (so_s * esz) % 16 == 0,
                "nvfp4_fwd: out must be 16-byte aligned with 16-byte-multiple strides");
  NVFP4_REQUIRE(((uintptr_t)qsc % 4) == 0 && ((uintptr_t)ksc % 4) == 0 && ((uintptr_t)vsc % 8) == 0,
                "nvfp4_fwd: scale tensors must be aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t zh = z * h, zhk = z * hk;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_u8_3d_sw64(&tq, qnv, d / 2, s_q, zh, d / 2, (uint64_t)s_q * (d / 2), 128, "nvfp4_fwd(Q)");
  if (rc) return rc;
  rc = make_tmap_u8_3d_sw64(&tk, knv, d / 2, s_kv, zhk, d / 2, (uint64_t)s_kv * (d / 2), 128, "nvfp4_fwd(K)");
  if (rc) return rc;
  rc = make_tmap_u8_3d_sw64(&tv, vnv, s_pad / 2, d, zhk, s_pad / 2, (uint64_t)d * (s_pad / 2), 128, "nvfp4_fwd(V)");
  if (rc) return rc;
  FwdParams p;
  p.qsc = qsc; p.ksc = ksc; p.vsc = vsc; p.bias = bias; p.seq_id = seq_id; p.seq_start = seq_start;
  p.out = out; p.so_z = so_z; p.so_h = so_h; p.so_s = so_s; p.lse = lse;
  p.h = (int)h; p.hk = (int)hk; p.g = (int)(h / hk);
  p.s_q = (int)s_q; p.s_kv = (int)s_kv; p.s_pad = (int)s_pad;
  p.scaling = scaling; p.causal = (flags & NVFP4_FWD_CAUSAL) ? 1 : 0; p.status = status;
#define NVFP4_FWD(DD, T) return fwd_launch<DD, T>(tq, tk, tv, p, zh, st)
  if (d == 128) {
    switch (out_dtype) {
      case NVFP4_DT_BF16: NVFP4_FWD(128, __nv_bfloat16);
      case NVFP4_DT_FP16: NVFP4_FWD(128, __half);
      case NVFP4_DT_FP32: NVFP4_FWD(128, float);
    }
  } else {
    switch (out_dtype) {
      case NVFP4_DT_BF16: NVFP4_FWD(256, __nv_bfloat16);
      case NVFP4_DT_FP16: NVFP4_FWD(256, __half);
      case NVFP4_DT_FP32: NVFP4_FWD(256, float);
    }
  }
#undef NVFP4_FWD
  return fail(-1, "nvfp4_fwd: unknown out dtype %d", out_dtype);
}
