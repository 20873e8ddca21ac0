// Split-K decode over an NVFP4 KV cache, read in place through its strides.
//
// The step is HBM-bound: per (batch, kv-head) unit it streams S*(D/2 + D/16) bytes of K and
// D*(Sp/2 + Sp/16) bytes of V^T once.  The kernel is persistent (one CTA per SM) and walks work
// items (unit, key range); each 128-key tile is fetched by TMA straight from the cache into a
// multi-stage shared-memory ring and consumed by tcgen05 block-scaled MMAs in the
// "keys on the M axis" orientation, so the cache layout is the operand layout:
//     S^T[128 keys x 16] = K_tile[128 x D] . Q^T           (A = K tile, B = the G<=16 query rows)
//     O^T[D x 16]       += V^T_tile[D x 128] . P^T          (A = V^T tile, B = P packed along keys)
// Scale bytes are re-laid into the 32x16-byte form tcgen05.cp expects by two loader warps.
// Softmax runs with one thread per key (TMEM lane); P is packed to NVFP4 per 16 keys with the
// same scale rule as the packer.  Each work item writes un-normalised (acc, m, l) partials; a
// second small kernel combines them exactly and emits the output and its log-sum-exp.
//
// Warp roles (256 threads): 0 TMA producer, 1 MMA issuer, 2 K-scale loader, 3 V-scale loader,
// 4-7 softmax / correction / epilogue.  Every barrier wait is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"

namespace nvfp4 {

constexpr float kLog2e = 1.4426950408889634f;
constexpr int kDecodeThreads = 256;

template <int D>
struct DecodeCfg {
  static constexpr int KSUB = D / 128;   // 64-byte-wide sub-tiles of a K row
  static constexpr int KB = D / 64;      // K=64 MMAs per QK tile
  static constexpr int MT = D / 128;     // 128-row M tiles of V^T
  static constexpr int K_BYTES = KSUB * 8192;
  static constexpr int V_BYTES = MT * 8192;
  static constexpr int KSF_BYTES = KB * 512;
  static constexpr int VSF_BYTES = MT * 2 * 512;
  static constexpr int STAGE_BYTES = K_BYTES + V_BYTES + KSF_BYTES + VSF_BYTES;
  static constexpr int NSTAGE = (D == 128) ? 8 : 5;
  static constexpr int Q_BYTES = KSUB * 1024;     // 16 rows x 64 B per sub-tile
  static constexpr int QSF_BYTES = KB * 512;
  static constexpr int P_BYTES = 1024;            // 16 rows x 64 B
  static constexpr int PSF_BYTES = 2 * 512;
  static constexpr int SMEM_BYTES =
      NSTAGE * STAGE_BYTES + Q_BYTES + QSF_BYTES + 2 * P_BYTES + 2 * PSF_BYTES + 1024;
  // TMEM columns
  static constexpr int T_ST = 0;      // 2 x 16
  static constexpr int T_OT = 32;     // MT x 16
  static constexpr int T_SFK = 64;    // 2 x 16
  static constexpr int T_SFQ = 96;    // 16
  static constexpr int T_SFV = 112;   // 2 x 16
  static constexpr int T_SFP = 144;   // 2 x 8
  static constexpr int T_COLS = 256;
};

struct DecodeParams {
  const void* q;
  int64_t s_qz, s_qh;
  const uint8_t* ksc;
  int64_t ksc_unit;
  const uint8_t* vsc;
  int64_t vsc_unit, vsc_row;
  int hk, g;
  int64_t s_kv;
  float scaling;
  int nsplit;
  int chunk_tiles;
  int ntiles;
  int64_t nitems;
  float* ws_acc;  // [nitems][16][D]
  float* ws_m;    // [nitems][16]
  float* ws_l;    // [nitems][16]
  int* status;
};

template <int D, typename TQ, int NQ>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const DecodeParams p) {
  using C = DecodeCfg<D>;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_stage = smem;
  uint8_t* s_q = s_stage + C::NSTAGE * C::STAGE_BYTES;
  uint8_t* s_qsf = s_q + C::Q_BYTES;
  uint8_t* s_p = s_qsf + C::QSF_BYTES;
  uint8_t* s_psf = s_p + 2 * C::P_BYTES;

  __shared__ uint64_t full_kv[C::NSTAGE], full_sf[C::NSTAGE], empty[C::NSTAGE];
  __shared__ uint64_t s_full[2], s_free[2], p_full[2], pv_done[2], q_full;
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  __shared__ float xch[2][4][16];
  __shared__ float lred[4][16];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(&full_kv[i], 1);
      mbar_init(&full_sf[i], 2);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 4);
      mbar_init(&pv_done[i], 1);
    }
    mbar_init(&q_full, 4);
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(&tmem_base_s, C::T_COLS);
  // zero the operand buffers that are only partly rewritten (rows >= G stay zero)
  for (int i = tid; i < (C::Q_BYTES + C::QSF_BYTES + 2 * C::P_BYTES + 2 * C::PSF_BYTES) / 4;
       i += kDecodeThreads)
    reinterpret_cast<uint32_t*>(s_q)[i] = 0u;
  fence_proxy_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_s;

  auto item_range = [&](int64_t w, int& unit, int& t0, int& t1) {
    unit = (int)(w / p.nsplit);
    const int split = (int)(w % p.nsplit);
    t0 = split * p.chunk_tiles;
    t1 = min(t0 + p.chunk_tiles, p.ntiles);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      for (int64_t w = blockIdx.x; w < p.nitems; w += gridDim.x) {
        int unit, t0, t1;
        item_range(w, unit, t0, t1);
        for (int t = t0; t < t1; ++t, ++it) {
          const int s = it % C::NSTAGE;
          if (it >= (uint32_t)C::NSTAGE) mbar_wait(&empty[s], ((it / C::NSTAGE) & 1) ^ 1, &err, 1);
          uint8_t* st = s_stage + s * C::STAGE_BYTES;
          mbar_expect_tx(&full_kv[s], C::K_BYTES + C::V_BYTES);
#pragma unroll
          for (int ks = 0; ks < C::KSUB; ++ks)
            tma_load_3d(st + ks * 8192, &tm_k, &full_kv[s], ks * 64, t * 128, unit);
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt)
            tma_load_3d(st + C::K_BYTES + mt * 8192, &tm_v, &full_kv[s], t * 64, mt * 128, unit);
        }
      }
    }
    __syncwarp();
  } else if (warp == 2 || warp == 3) {
    // ------------------------------------------------------------------ scale loaders
    uint32_t it = 0;
    for (int64_t w = blockIdx.x; w < p.nitems; w += gridDim.x) {
      int unit, t0, t1;
      item_range(w, unit, t0, t1);
      for (int t = t0; t < t1; ++t, ++it) {
        const int s = it % C::NSTAGE;
        if (it >= (uint32_t)C::NSTAGE) mbar_wait(&empty[s], ((it / C::NSTAGE) & 1) ^ 1, &err, 2);
        uint8_t* st = s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES;
        if (warp == 2) {
          const uint8_t* src = p.ksc + (int64_t)unit * p.ksc_unit;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int r = lane + 32 * j;
            const int64_t key = (int64_t)t * 128 + r;
            uint32_t wds[C::KB];
#pragma unroll
            for (int k = 0; k < C::KB; ++k) wds[k] = 0u;
            if (key < p.s_kv) {
              const uint32_t* g = reinterpret_cast<const uint32_t*>(src + key * (D / 16));
#pragma unroll
              for (int k = 0; k < C::KB; ++k) wds[k] = __ldg(g + k);
            }
#pragma unroll
            for (int k = 0; k < C::KB; ++k)
              *reinterpret_cast<uint32_t*>(st + k * 512 + sf_atom_offset(r, 0)) = wds[k];
          }
        } else {
          const uint8_t* src = p.vsc + (int64_t)unit * p.vsc_unit + (int64_t)t * 8;
          uint8_t* dst = st + C::KSF_BYTES;
#pragma unroll
          for (int j = 0; j < D / 32; ++j) {
            const int dr = lane + 32 * j;
            const uint2 v = __ldg(reinterpret_cast<const uint2*>(src + (int64_t)dr * p.vsc_row));
            const int mt = dr >> 7, r = dr & 127;
            *reinterpret_cast<uint32_t*>(dst + (mt * 2 + 0) * 512 + sf_atom_offset(r, 0)) = v.x;
            *reinterpret_cast<uint32_t*>(dst + (mt * 2 + 1) * 512 + sf_atom_offset(r, 0)) = v.y;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_sf[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_nvfp4(128, 16);
      uint32_t it = 0, item_idx = 0;
      auto issue_qk = [&](uint32_t j) {
        const int s = j % C::NSTAGE, b = j & 1;
        const uint32_t ph = (j / C::NSTAGE) & 1;
        mbar_wait(&full_kv[s], ph, &err, 3);
        mbar_wait(&full_sf[s], ph, &err, 4);
        if (j >= 2) mbar_wait(&s_free[b], ((j >> 1) & 1) ^ 1, &err, 5);
        tc_fence_after();
        uint8_t* st = s_stage + s * C::STAGE_BYTES;
        const uint32_t sfk = tmem + C::T_SFK + b * 16;
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          tmem_cp_32x128b_warpx4(sfk + k * 4, smem_u32(st + C::K_BYTES + C::V_BYTES + k * 512));
#pragma unroll
        for (int k = 0; k < C::KB; ++k) {
          const uint64_t ad = make_smem_desc(smem_u32(st + (k >> 1) * 8192) + (k & 1) * 32, 16, 512, 4);
          const uint64_t bd = make_smem_desc(smem_u32(s_q + (k >> 1) * 1024) + (k & 1) * 32, 16, 512, 4);
          umma_nvfp4(tmem + C::T_ST + b * 16, ad, bd, idesc, sfk + k * 4, tmem + C::T_SFQ + k * 4,
                     k > 0);
        }
        umma_commit(&s_full[b]);
      };
      for (int64_t w = blockIdx.x; w < p.nitems; w += gridDim.x, ++item_idx) {
        int unit, t0, t1;
        item_range(w, unit, t0, t1);
        const int ntile = t1 - t0;
        mbar_wait(&q_full, item_idx & 1, &err, 6);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          tmem_cp_32x128b_warpx4(tmem + C::T_SFQ + k * 4, smem_u32(s_qsf + k * 512));
        issue_qk(it);
        for (int i = 0; i < ntile; ++i, ++it) {
          if (i + 1 < ntile) issue_qk(it + 1);
          const int s = it % C::NSTAGE, b = it & 1;
          mbar_wait(&p_full[b], (it >> 1) & 1, &err, 7);
          tc_fence_after();
          uint8_t* st = s_stage + s * C::STAGE_BYTES;
          const uint32_t sfv = tmem + C::T_SFV + b * 16, sfp = tmem + C::T_SFP + b * 8;
#pragma unroll
          for (int k = 0; k < C::MT * 2; ++k)
            tmem_cp_32x128b_warpx4(sfv + k * 4,
                                   smem_u32(st + C::K_BYTES + C::V_BYTES + C::KSF_BYTES + k * 512));
#pragma unroll
          for (int k = 0; k < 2; ++k)
            tmem_cp_32x128b_warpx4(sfp + k * 4, smem_u32(s_psf + b * C::PSF_BYTES + k * 512));
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const uint64_t ad =
                  make_smem_desc(smem_u32(st + C::K_BYTES + mt * 8192) + k * 32, 16, 512, 4);
              const uint64_t bd = make_smem_desc(smem_u32(s_p + b * C::P_BYTES) + k * 32, 16, 512, 4);
              umma_nvfp4(tmem + C::T_OT + mt * 16, ad, bd, idesc, sfv + (mt * 2 + k) * 4, sfp + k * 4,
                         (i > 0 || k > 0) ? 1u : 0u);
            }
          }
          umma_commit(&pv_done[b]);
          umma_commit(&empty[s]);
        }
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / epilogue
    const int wq = warp - 4;               // TMEM lane quadrant
    const int ts = tid - 128;              // 0..127 = key lane within a tile / d row in epilogue
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    const TQ* qbase = static_cast<const TQ*>(p.q);
    uint32_t it = 0;
    for (int64_t w = blockIdx.x; w < p.nitems; w += gridDim.x) {
      int unit, t0, t1;
      item_range(w, unit, t0, t1);
      const int zi = unit / p.hk, kh = unit % p.hk;
      // ---- quantise the G query rows of this kv head into the B operand of QK
      for (int i = ts; i < p.g * (D / 16); i += 128) {
        const int qr = i / (D / 16), gi = i % (D / 16);
        const TQ* src = qbase + zi * p.s_qz + (int64_t)(kh * p.g + qr) * p.s_qh + gi * 16;
        float v[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) v[e] = to_f32<TQ>(src[e]);
        uint32_t lo, hi;
        const uint8_t sb = pack_group16(v, lo, hi);
        *reinterpret_cast<uint2*>(s_q + (gi >> 3) * 1024 + sw64_offset(qr, (gi & 7) * 8)) =
            make_uint2(lo, hi);
        s_qsf[(gi >> 2) * 512 + sf_atom_offset(qr, gi & 3)] = sb;
      }
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full);

      float m_run[NQ], l_run[NQ];
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) { m_run[qi] = -INFINITY; l_run[qi] = 0.0f; }

      for (int t = t0; t < t1; ++t, ++it) {
        const int b = it & 1;
        mbar_wait(&s_full[b], (it >> 1) & 1, &err, 8);
        tc_fence_after();
        uint32_t r[16];
        tmem_ld16(tmem + lane_addr + C::T_ST + b * 16, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_free[b]);
        const bool valid = ((int64_t)t * 128 + ts) < p.s_kv;
        float sv[NQ], mx[NQ];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          sv[qi] = (valid && qi < p.g) ? __uint_as_float(r[qi]) * p.scaling : -INFINITY;
          float v = sv[qi];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
          mx[qi] = v;
        }
        if (lane == 0) {
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) xch[b][wq][qi] = mx[qi];
        }
        named_bar_sync(1, 128);
        bool need = false;
        float alpha[NQ], pv[NQ];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          const float mt_ = fmaxf(fmaxf(xch[b][0][qi], xch[b][1][qi]), fmaxf(xch[b][2][qi], xch[b][3][qi]));
          const float m_new = fmaxf(m_run[qi], mt_);
          const float m_sf = (m_new == -INFINITY) ? 0.0f : m_new;
          alpha[qi] = exp2f((m_run[qi] - m_sf) * kLog2e);
          pv[qi] = exp2f((sv[qi] - m_sf) * kLog2e);
          need = need || (m_new > m_run[qi]);
          l_run[qi] = l_run[qi] * alpha[qi] + pv[qi];
          m_run[qi] = m_new;
        }
        need = need && (t > t0);
        if (it >= 2) mbar_wait(&pv_done[b], ((it >> 1) & 1) ^ 1, &err, 9);
        // ---- pack P along keys (16 consecutive lanes = one group)
        uint8_t* pt = s_p + b * C::P_BYTES;
        uint8_t* psf = s_psf + b * C::PSF_BYTES;
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          if (qi < p.g) {
            float am = pv[qi];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            const uint8_t sb = scale_byte_from_amax(am);
            const float y = __fdiv_rn(pv[qi], e4m3_to_f32(sb));
            const float yn = __shfl_xor_sync(0xffffffffu, y, 1);
            if ((lane & 1) == 0) {
              uint16_t byte;
              asm("{\n\t.reg .b8 t;\n\tcvt.rn.satfinite.e2m1x2.f32 t, %1, %2;\n\tcvt.u16.u8 %0, t;\n\t}\n"
                  : "=h"(byte)
                  : "f"(yn), "f"(y));
              pt[sw64_offset(qi, ts >> 1)] = (uint8_t)byte;
            }
            if ((lane & 15) == 0) {
              const int gi = ts >> 4;
              psf[(gi >> 2) * 512 + sf_atom_offset(qi, gi & 3)] = sb;
            }
          }
        }
        if (need) {
          // PV of the previous tile must have landed before O^T is rescaled
          mbar_wait(&pv_done[b ^ 1], ((it - 1) >> 1) & 1, &err, 10);
          tc_fence_after();
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt) {
            uint32_t o[16];
            tmem_ld16(tmem + lane_addr + C::T_OT + mt * 16, o);
            tmem_ld_wait();
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi) o[qi] = __float_as_uint(__uint_as_float(o[qi]) * alpha[qi]);
            tmem_st16(tmem + lane_addr + C::T_OT + mt * 16, o);
          }
          tmem_st_wait();
          tc_fence_before();
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[b]);
      }
      // ---- item epilogue: un-normalised partials
      {
        const uint32_t last = it - 1;
        mbar_wait(&pv_done[last & 1], (last >> 1) & 1, &err, 11);
        tc_fence_after();
        float* acc = p.ws_acc + w * 16 * D;
#pragma unroll
        for (int mt = 0; mt < C::MT; ++mt) {
          uint32_t o[16];
          tmem_ld16(tmem + lane_addr + C::T_OT + mt * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi)
            if (qi < p.g) acc[qi * D + mt * 128 + ts] = __uint_as_float(o[qi]);
        }
        tc_fence_before();
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          float v = l_run[qi];
#pragma unroll
          for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
          if (lane == 0) lred[wq][qi] = v;
        }
        named_bar_sync(1, 128);
        if (ts < p.g) {
          float lsum = 0.0f, mfin = -INFINITY;
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi)
            if (qi == ts) { lsum = lred[0][qi] + lred[1][qi] + lred[2][qi] + lred[3][qi]; mfin = m_run[qi]; }
          p.ws_m[w * 16 + ts] = mfin;
          p.ws_l[w * 16 + ts] = lsum;
        }
        named_bar_sync(1, 128);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && err != 0 && p.status != nullptr) atomicExch(p.status, err);
  if (warp == 1) tmem_dealloc(tmem, C::T_COLS);
}

// Exact combine of the per-split partials (one block per (unit, query row), D threads).
template <typename TQ>
__global__ void decode_combine_kernel(const float* __restrict__ ws_acc,
                                      const float* __restrict__ ws_m,
                                      const float* __restrict__ ws_l, int nsplit, int hk, int g, int d,
                                      TQ* __restrict__ out, float* __restrict__ lse) {
  const int unit = blockIdx.x / g, qi = blockIdx.x % g;
  const int t = threadIdx.x;
  float gm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) gm = fmaxf(gm, ws_m[((int64_t)unit * nsplit + s) * 16 + qi]);
  float acc = 0.0f, den = 0.0f;
  for (int s = 0; s < nsplit; ++s) {
    const int64_t w = (int64_t)unit * nsplit + s;
    const float ms = ws_m[w * 16 + qi];
    const float f = (ms == -INFINITY) ? 0.0f : expf(ms - gm);
    acc += f * ws_acc[(w * 16 + qi) * d + t];
    den += f * ws_l[w * 16 + qi];
  }
  if (den == 0.0f) den = 1.0f;
  const int zi = unit / hk, kh = unit % hk;
  const int64_t row = (int64_t)zi * hk * g + kh * g + qi;
  out[row * d + t] = from_f32<TQ>(acc / den);
  if (lse != nullptr && t == 0) lse[row] = gm + logf(den);
}

template <int D, typename TQ>
int decode_launch(const CUtensorMap& tm_k, const CUtensorMap& tm_v, const DecodeParams& p,
                  int64_t zhk, void* out, float* lse, int sm_count, cudaStream_t st) {
  using C = DecodeCfg<D>;
  const int grid = (int)std::min<int64_t>(p.nitems, sm_count);
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_decode: smem attribute: %s", cudaGetErrorString(e));
    kern<<<grid, kDecodeThreads, C::SMEM_BYTES, st>>>(tm_k, tm_v, p);
    return launch_result("nvfp4_decode");
  };
  int rc;
  if (p.g <= 4) rc = launch(decode_kernel<D, TQ, 4>);
  else if (p.g <= 8) rc = launch(decode_kernel<D, TQ, 8>);
  else rc = launch(decode_kernel<D, TQ, 16>);
  if (rc) return rc;
  decode_combine_kernel<TQ><<<(unsigned)(zhk * p.g), D, 0, st>>>(
      p.ws_acc, p.ws_m, p.ws_l, p.nsplit, p.hk, p.g, D, static_cast<TQ*>(out), lse);
  return launch_result("nvfp4_decode(combine)");
}

}  // namespace nvfp4

extern "C" int nvfp4_decode_plan(int64_t s_kv, int64_t zhk, int d, int sm_count, int* nsplit,
                                 int64_t* split_kv, size_t* workspace_bytes) {
  using namespace nvfp4;
  NVFP4_REQUIRE(s_kv >= 1 && zhk >= 1, "nvfp4_decode_plan: s_kv and zhk must be positive");
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_decode_plan: D must be 128 or 256");
  if (sm_count <= 0) sm_count = 148;
  const int64_t tiles = (s_kv + 127) / 128;
  // about eight work items per SM keeps the persistent CTAs balanced; no item under 4 tiles
  int64_t want = (8LL * sm_count + zhk - 1) / zhk;
  want = std::max<int64_t>(1, std::min<int64_t>(want, std::max<int64_t>(1, tiles / 4)));
  const int64_t chunk = (tiles + want - 1) / want;
  const int64_t ns = (tiles + chunk - 1) / chunk;
  if (nsplit) *nsplit = (int)ns;
  if (split_kv) *split_kv = chunk * 128;
  if (workspace_bytes) *workspace_bytes = (size_t)(zhk * ns) * (size_t)(16 * d + 32) * sizeof(float);
  return 0;
}

extern "C" int nvfp4_decode(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh,
                            const uint8_t* knv, int64_t knv_unit, const uint8_t* ksc,
                            int64_t ksc_unit, const uint8_t* vnv, int64_t vnv_unit, int64_t vnv_row,
                            const uint8_t* vsc, int64_t vsc_unit, int64_t vsc_row, int64_t z,
                            int64_t hk, int g, int d, int64_t s_kv, float scaling, void* out,
                            float* lse, void* workspace, size_t workspace_bytes, int nsplit,
                            int64_t split_kv, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_decode: D must be 128 or 256");
  NVFP4_REQUIRE(g >= 1 && g <= 16, "nvfp4_decode: GQA group %d must be <= 16", g);
  NVFP4_REQUIRE(z >= 1 && hk >= 1 && s_kv >= 1, "nvfp4_decode: empty problem");
  NVFP4_REQUIRE(q && knv && ksc && vnv && vsc && out && workspace, "nvfp4_decode: null pointer");
  NVFP4_REQUIRE(nsplit >= 1 && split_kv >= 128 && split_kv % 128 == 0,
                "nvfp4_decode: split_kv must be a positive multiple of 128");
  NVFP4_REQUIRE((int64_t)nsplit * split_kv >= s_kv && (int64_t)(nsplit - 1) * split_kv < s_kv,
                "nvfp4_decode: nsplit * split_kv does not cover s_kv exactly");
  const int64_t zhk = z * hk;
  const size_t need = (size_t)(zhk * nsplit) * (size_t)(16 * d + 32) * sizeof(float);
  NVFP4_REQUIRE(workspace_bytes >= need, "nvfp4_decode: workspace too small (%zu < %zu)",
                workspace_bytes, need);
  NVFP4_REQUIRE(((uintptr_t)workspace & 15) == 0, "nvfp4_decode: workspace must be 16-byte aligned");
  NVFP4_REQUIRE(((uintptr_t)ksc % (d / 16)) == 0 && ksc_unit % (d / 16) == 0,
                "nvfp4_decode: K scales must be aligned to a row (%d bytes)", d / 16);
  NVFP4_REQUIRE(((uintptr_t)vsc & 7) == 0 && vsc_unit % 8 == 0 && vsc_row % 8 == 0,
                "nvfp4_decode: V scales must be 8-byte aligned");
  const int64_t s_pad = (s_kv + 127) / 128 * 128;
  NVFP4_REQUIRE(vnv_row * 2 >= s_pad && vsc_row * 16 >= s_pad,
                "nvfp4_decode: V^T rows shorter than the padded key axis");
  cudaStream_t st = static_cast<cudaStream_t>(stream);

  CUtensorMap tm_k, tm_v;
  int rc = make_tmap_u8_3d_sw64(&tm_k, knv, (uint64_t)d / 2, (uint64_t)s_kv, (uint64_t)zhk,
                                (uint64_t)d / 2, (uint64_t)knv_unit, 128, "nvfp4_decode(K)");
  if (rc) return rc;
  rc = make_tmap_u8_3d_sw64(&tm_v, vnv, (uint64_t)s_pad / 2, (uint64_t)d, (uint64_t)zhk,
                            (uint64_t)vnv_row, (uint64_t)vnv_unit, 128, "nvfp4_decode(V)");
  if (rc) return rc;

  int dev = 0, sm_count = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (sm_count <= 0) return fail(-1, "nvfp4_decode: no CUDA device");

  DecodeParams p;
  p.q = q; p.s_qz = s_qz; p.s_qh = s_qh;
  p.ksc = ksc; p.ksc_unit = ksc_unit;
  p.vsc = vsc; p.vsc_unit = vsc_unit; p.vsc_row = vsc_row;
  p.hk = (int)hk; p.g = g; p.s_kv = s_kv; p.scaling = scaling;
  p.nsplit = nsplit; p.chunk_tiles = (int)(split_kv / 128); p.ntiles = (int)((s_kv + 127) / 128);
  p.nitems = zhk * nsplit;
  float* ws = static_cast<float*>(workspace);
  p.ws_acc = ws;
  p.ws_m = ws + p.nitems * 16 * d;
  p.ws_l = p.ws_m + p.nitems * 16;
  p.status = status;

#define NVFP4_DECODE(DD, T) return decode_launch<DD, T>(tm_k, tm_v, p, zhk, out, lse, sm_count, st)
  if (d == 128) {
    switch (q_dtype) {
      case NVFP4_DT_BF16: NVFP4_DECODE(128, __nv_bfloat16);
      case NVFP4_DT_FP16: NVFP4_DECODE(128, __half);
      case NVFP4_DT_FP32: NVFP4_DECODE(128, float);
    }
  } else {
    switch (q_dtype) {
      case NVFP4_DT_BF16: NVFP4_DECODE(256, __nv_bfloat16);
      case NVFP4_DT_FP16: NVFP4_DECODE(256, __half);
      case NVFP4_DT_FP32: NVFP4_DECODE(256, float);
    }
  }
#undef NVFP4_DECODE
  return fail(-1, "nvfp4_decode: unknown dtype %d", q_dtype);
}

// ---------------------------------------------------------------------------------------------
// Decode without any allocation by the caller or the library.
//
// Some hosts of this library cannot hand it scratch memory: a serving runtime that carved up the
// whole device into its own pools at start-up and forbids later cudaMalloc calls (every byte is
// accounted for, and an allocation at request time could fail or stall the device), or a plugin
// loaded by a process whose allocator the plugin must not touch.  For those callers the split-K
// partials live in a fixed array that is part of the library image on every GPU that loads it.
// ---------------------------------------------------------------------------------------------
namespace nvfp4 {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;  // 16 MiB per GPU, held until exit

// In host code this name is only a handle for cudaGetSymbolAddress, never a device address.
static __device__ __align__(256) unsigned char g_decode_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static void* g_static_scratch_ptr[kMaxDevices] = {nullptr};

// Device address of the static scratch on the CURRENT device; looked up once per device.
static int static_scratch_address(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "nvfp4_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(-1, "nvfp4_decode_static: device index %d out of range", dev);
  if (g_static_scratch_ptr[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_decode_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(e != cudaSuccess ? (int)e : -1, "nvfp4_decode_static: cudaGetSymbolAddress: %s",
                  cudaGetErrorString(e));
    g_static_scratch_ptr[dev] = ptr;
  }
  *out = g_static_scratch_ptr[dev];
  return 0;
}

}  // namespace nvfp4

extern "C" size_t nvfp4_decode_static_capacity(void) { return nvfp4::kStaticScratchBytes; }

extern "C" int nvfp4_decode_static(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh,
                                   const uint8_t* knv, int64_t knv_unit, const uint8_t* ksc,
                                   int64_t ksc_unit, const uint8_t* vnv, int64_t vnv_unit,
                                   int64_t vnv_row, const uint8_t* vsc, int64_t vsc_unit,
                                   int64_t vsc_row, int64_t z, int64_t hk, int g, int d,
                                   int64_t s_kv, float scaling, void* out, float* lse, int nsplit,
                                   int64_t split_kv, int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_decode_static: D must be 128 or 256");
  NVFP4_REQUIRE(z >= 1 && hk >= 1 && nsplit >= 1, "nvfp4_decode_static: empty problem");
  const size_t need = (size_t)(z * hk) * (size_t)nsplit * (size_t)(16 * d + 32) * sizeof(float);
  if (need > kStaticScratchBytes)
    return fail(-1,
                "nvfp4_decode_static: this problem needs %zu bytes of split-K scratch but the static "
                "array holds %zu; use fewer splits (larger split_kv) or nvfp4_decode with a workspace",
                need, kStaticScratchBytes);
  void* ws = nullptr;
  const int rc = static_scratch_address(&ws);
  if (rc) return rc;
  return nvfp4_decode(q, q_dtype, s_qz, s_qh, knv, knv_unit, ksc, ksc_unit, vnv, vnv_unit, vnv_row,
                      vsc, vsc_unit, vsc_row, z, hk, g, d, s_kv, scaling, out, lse, ws,
                      kStaticScratchBytes, nsplit, split_kv, status, stream);
}
