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
// Warp roles (384 threads): 0 TMA producer, 1 QK^T issuer, 2 scale loader, 3 PV issuer,
// 4-11 softmax / accumulate / epilogue (two groups splitting each round's tiles).  Every barrier
// wait is bounded.
#include "common/abi.cuh"
#include "common/fp4.cuh"
#include "common/sm100.cuh"
#include "common/tma_host.cuh"

namespace nvfp4 {

constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float ex2f_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
constexpr int kDecodeThreads = 384;

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
  static constexpr int NSTAGE = (D == 128) ? 10 : 5;
  static constexpr int STMAX = (D == 128) ? 4 : 2;  // key tiles per softmax round ("super-tile")
  static constexpr int Q_BYTES = KSUB * 1024;     // 16 rows x 64 B per sub-tile
  static constexpr int QSF_BYTES = KB * 512;
  static constexpr int P_BYTES = 1024;            // 16 rows x 64 B per tile
  static constexpr int PSF_BYTES = 2 * 512;       // per tile
  static constexpr int MERGE_BYTES = 16 * D * 4;   // one group's O^T partial at the item end
  static constexpr int PBUF_BYTES = 2 * STMAX * (P_BYTES + PSF_BYTES);
  static constexpr int SSC_BYTES = 16 * 1024;      // scores of one round, [tile][head][128 keys] fp32
  // the merge buffer reuses the P tiles, which are idle once an item's last PV has completed
  static constexpr int SMEM_BYTES = NSTAGE * STAGE_BYTES + 2 * (Q_BYTES + QSF_BYTES) +
                                    (PBUF_BYTES > MERGE_BYTES ? PBUF_BYTES : MERGE_BYTES) + SSC_BYTES + 1024;
  // TMEM columns: [buffer][tile of the super-tile][...]
  static constexpr int T_ST = 0;                              // 2 x STMAX x 16
  static constexpr int T_OT = T_ST + 2 * STMAX * 16;          // 2 x STMAX x MT x 16
  static constexpr int T_SFK = T_OT + 2 * STMAX * MT * 16;    // 2 x STMAX x KB*4
  static constexpr int T_SFV = T_SFK + 2 * STMAX * KB * 4;    // 2 x STMAX x MT*8
  static constexpr int T_SFP = T_SFV + 2 * STMAX * MT * 8;    // 2 x STMAX x 8
  static constexpr int T_SFQ = T_SFP + 2 * STMAX * 8;         // 2 x KB*4 (one per work-item parity)
  static constexpr int T_END = T_SFQ + 2 * KB * 4;
  static constexpr int T_COLS = 512;
  static_assert(T_END <= T_COLS, "TMEM budget exceeded");
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
  // balanced mode: CTA b owns the global tiles [b*T/G, (b+1)*T/G) of the unit-major tile list
  // (T = units * ntiles); its work items are the pieces of the units that range touches
  int balanced;
  int64_t total_tiles;
  int maxseg;     // partial slots reserved per CTA
  float* ws_acc;  // [slots][16][D]
  float* ws_m;    // [nitems][16]
  float* ws_l;    // [nitems][16]
  int64_t extra_base;   // first of the partial slots appended by another kernel (n_extra per unit)
  int n_extra;
  int* status;
};

// The kernel amortises its per-tile latencies (barrier round trips, cross-lane reductions) by
// treating ST consecutive 128-key tiles as one softmax round: ST QK^T products land in ST
// S^T accumulators, one pass of the softmax warps turns them into ST packed P tiles (the
// running maximum still advances tile by tile, exactly as in a sequential walk), and each
// tile's P.V goes to a FRESH O^T accumulator in TMEM.  The softmax threads (one per head-dim
// row in this role) fold those ST accumulators into registers one round later with the exact
// weights exp(m_tile - m_now), so O is never rescaled in TMEM.
template <int D, typename TQ, int NQ>
__global__ void __launch_bounds__(kDecodeThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
              const __grid_constant__ CUtensorMap tm_vpf, const __grid_constant__ CUtensorMap tm_vpf4,
              const DecodeParams p) {
  using C = DecodeCfg<D>;
  constexpr int ST = (NQ == 16 && C::STMAX > 2) ? 2 : C::STMAX;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* s_stage = smem;
  // the quantised query rows are double buffered by work-item parity: item n+1's are prepared
  // while item n runs, so the QK^T issuer walks into the next item without draining the pipeline
  uint8_t* s_q = s_stage + C::NSTAGE * C::STAGE_BYTES;    // [2][Q_BYTES]
  uint8_t* s_qsf = s_q + 2 * C::Q_BYTES;                  // [2][QSF_BYTES]
  uint8_t* s_p = s_qsf + 2 * C::QSF_BYTES;                // [2][STMAX][P_BYTES]
  uint8_t* s_psf = s_p + 2 * C::STMAX * C::P_BYTES;       // [2][STMAX][PSF_BYTES]
  float* s_merge = reinterpret_cast<float*>(s_p);          // [16][D], only at the end of an item
  float* ssc = reinterpret_cast<float*>(s_p + (C::PBUF_BYTES > C::MERGE_BYTES ? C::PBUF_BYTES : C::MERGE_BYTES));

  __shared__ uint64_t full_kv[C::NSTAGE], full_sf[C::NSTAGE], empty[C::NSTAGE];
  __shared__ uint64_t s_full[2], s_free[2], p_full[2], o_full[2], q_full[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int err;
  __shared__ float xch[C::STMAX][16];      // tile maxima of the current round, per head
  __shared__ float lred[C::STMAX][16];     // row sums at the end of an item, per tile slot and head

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // work items of this CTA: i = 0 .. my_items-1
  const int64_t nctas = gridDim.x;
  int64_t bal_start = 0, bal_end = 0;
  int bal_u0 = 0, my_items = 0;
  if (p.balanced) {
    bal_start = (int64_t)blockIdx.x * p.total_tiles / nctas;
    bal_end = (int64_t)(blockIdx.x + 1) * p.total_tiles / nctas;
    bal_u0 = (int)(bal_start / p.ntiles);
    my_items = bal_end > bal_start ? (int)((bal_end - 1) / p.ntiles) - bal_u0 + 1 : 0;
  } else if ((int64_t)blockIdx.x < p.nitems) {
    my_items = (int)((p.nitems - blockIdx.x + nctas - 1) / nctas);
  }
  auto item_at = [&](int i, int& unit, int& t0, int& t1) {
    if (p.balanced) {
      unit = bal_u0 + i;
      const int64_t base = (int64_t)unit * p.ntiles;
      t0 = (int)(max(bal_start, base) - base);
      t1 = (int)(min(bal_end, base + p.ntiles) - base);
    } else {
      const int64_t w = blockIdx.x + (int64_t)i * nctas;
      unit = (int)(w / p.nsplit);
      const int split = (int)(w % p.nsplit);
      t0 = split * p.chunk_tiles;
      t1 = min(t0 + p.chunk_tiles, p.ntiles);
    }
  };
  auto slot_at = [&](int i) -> int64_t {
    return p.balanced ? (int64_t)blockIdx.x * p.maxseg + i : blockIdx.x + (int64_t)i * nctas;
  };

  // Before anything else: ask L2 for the scale bytes of this CTA's first tiles.  They are the
  // scattered first touches of the kernel (one 128-byte line per V^T row, a few KB of K scales), and
  // their DRAM latency otherwise sits in front of the very first MMA.
  if (my_items > 0) {
    int unit, t0, t1;
    item_at(0, unit, t0, t1);
    if (tid < D) {                      // V^T scale row `tid`: the line holding tiles t0 .. t0 + 15
      prefetch_l2(p.vsc + (int64_t)unit * p.vsc_unit + (int64_t)tid * p.vsc_row + (int64_t)t0 * 8);
    } else {                            // K scales: contiguous, 128 * D/16 bytes per tile
      const int64_t line = tid - D;
      const int64_t off = (int64_t)t0 * 128 * (D / 16) + line * 128;
      const int64_t end = min((int64_t)min(t1, t0 + 8) * 128, p.s_kv) * (D / 16);
      if (off < end) prefetch_l2(p.ksc + (int64_t)unit * p.ksc_unit + off);
    }
  }

  if (tid == 0) {
    err = 0;
    for (int i = 0; i < C::NSTAGE; ++i) {
      mbar_init(&full_kv[i], 1);
      mbar_init(&full_sf[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_free[i], 256);
      mbar_init(&p_full[i], 8);
      mbar_init(&o_full[i], 1);
      mbar_init(&q_full[i], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  // The TMA producer (warp 0) and the scale loader (warp 2) need nothing but the barriers and the
  // stage buffers: they start streaming now, while the other warps allocate TMEM and clear the
  // operand buffers behind a barrier of their own.
  uint32_t tmem = 0;
  if (warp != 0 && warp != 2) {
    if (warp == 1) tmem_alloc(&tmem_base_s, C::T_COLS);
    // zero the operand buffers that are only partly rewritten (rows >= G stay zero)
    const int zt = warp == 1 ? lane : (warp == 3 ? 32 + lane : tid - 64);     // 0 .. 319
    for (int i = zt; i < (2 * (C::Q_BYTES + C::QSF_BYTES) + 2 * C::STMAX * (C::P_BYTES + C::PSF_BYTES)) / 4;
         i += kDecodeThreads - 64)
      reinterpret_cast<uint32_t*>(s_q)[i] = 0u;
    fence_proxy_async_smem();
    tc_fence_before();
    named_bar_sync(5, kDecodeThreads - 64);
    tc_fence_after();
    tmem = tmem_base_s;
  }

  // quantise the G query rows of item `wi`'s kv head into the B operand of QK^T, buffer `qb`
  // (called by the 32 lanes of the QK^T issuer's warp, one work item ahead of the MMAs)
  const TQ* qbase = static_cast<const TQ*>(p.q);
  auto prep_q = [&](int wi, int qb) {
    int unit_q, t0q, t1q;
    item_at(wi, unit_q, t0q, t1q);
    const int zq = unit_q / p.hk, khq = unit_q % p.hk;
    uint8_t* dq = s_q + qb * C::Q_BYTES;
    uint8_t* dsf = s_qsf + qb * C::QSF_BYTES;
    for (int i = lane; i < p.g * (D / 16); i += 32) {
      const int qr = i / (D / 16), gi = i % (D / 16);
      const TQ* src = qbase + zq * p.s_qz + (int64_t)(khq * p.g + qr) * p.s_qh + gi * 16;
      float v[16];
#pragma unroll
      for (int e = 0; e < 16; ++e) v[e] = to_f32<TQ>(src[e]);
      uint32_t lo, hi;
      const uint8_t sb = pack_group16(v, lo, hi);
      *reinterpret_cast<uint2*>(dq + (gi >> 3) * 1024 + sw64_offset(qr, (gi & 7) * 8)) = make_uint2(lo, hi);
      dsf[(gi >> 2) * 512 + sf_atom_offset(qr, gi & 3)] = sb;
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) mbar_arrive(&q_full[qb]);
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      for (int wi = 0; wi < my_items; ++wi) {
        int unit, t0, t1;
        item_at(wi, unit, t0, t1);
        for (int t = t0; t < t1; ++t, ++it) {
          // V^T rows are D separate strips in memory and a 128-key tile touches only 64 bytes of
          // each; 1 KB per strip (16 tiles) is pulled into L2 one 16-tile block ahead so DRAM sees
          // long bursts.  The pull is spread over the tiles of the block before it (8 strips per
          // tile): a whole block at once, from every CTA in step, stalls the demand loads behind it.
          const int j = t - t0;
          // 8 strips (rows rows8 .. rows8+7 of every 128-row piece) of the block of <= 16 tiles that
          // starts at tile tb and must not reach past tile te: 1 KB boxes for whole blocks, 256-byte
          // boxes for a clipped tail, so nothing beyond the work item is read from DRAM
          auto pull = [&](int un, int tb, int te, int rows8) {
            const int nt = min(16, te - tb);
            if (nt <= 0) return;
#pragma unroll
            for (int mt = 0; mt < C::MT; ++mt) {
              if (nt == 16) {
                tma_prefetch_3d(&tm_vpf, tb * 16, mt * 128 + rows8, un);
              } else {
                for (int q4 = 0; q4 * 4 < nt; ++q4) tma_prefetch_3d(&tm_vpf4, (tb + q4 * 4) * 16, mt * 128 + rows8, un);
              }
            }
          };
          if (j == 0 && (wi == 0 || t1 - t0 < 16)) {
#pragma unroll 1
            for (int r = 0; r < 16; ++r) pull(unit, t0, t1, r * 8);
          }
          pull(unit, t0 + ((j >> 4) + 1) * 16, t1, (j & 15) * 8);      // the next block of this item
          // the first block of this CTA's NEXT work item, a whole item ahead: its first tiles would
          // otherwise be 128 scattered 64-byte first touches each, ~15k clocks of DRAM latency
          if (j < 16 && wi + 1 < my_items) {
            int unit_n, t0n, t1n;
            item_at(wi + 1, unit_n, t0n, t1n);
            pull(unit_n, t0n, t1n, j * 8);
          }
          const int s = it % C::NSTAGE;
          if (it >= (uint32_t)C::NSTAGE) mbar_spin_wait(&empty[s], ((it / C::NSTAGE) & 1) ^ 1, &err, 1);
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
  } else if (warp == 2) {
    // ------------------------------------------------------------------ scale loader
    // K and V^T scale bytes go straight from global memory into the 32 x 16-byte atoms that
    // tcgen05.cp copies, with per-thread 4-byte cp.async (no registers, no stall on the load):
    // the copies of tile n are issued as soon as its stage is free, and the stage is published
    // kLag tiles later, once cp.async.wait_group says they have landed.
    constexpr int kLag = 3;
    uint32_t it = 0, published = 0;   // tiles [published, it) have copies in flight
    auto publish = [&](uint32_t n) {
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(&full_sf[n % C::NSTAGE]);
    };
    for (int wi = 0; wi < my_items; ++wi) {
      int unit, t0, t1;
      item_at(wi, unit, t0, t1);
      const uint8_t* ksrc = p.ksc + (int64_t)unit * p.ksc_unit;
      const uint8_t* vsrc = p.vsc + (int64_t)unit * p.vsc_unit;
      for (int t = t0; t < t1; ++t, ++it) {
        const int s = it % C::NSTAGE;
        if (it >= (uint32_t)C::NSTAGE) {
          const uint32_t par = ((it / C::NSTAGE) & 1) ^ 1;
          if (!mbar_test_wait(&empty[s], par)) {
            // about to block on a full ring: publish everything in flight first
            cp_async_wait<0>();
            for (; published < it; ++published) publish(published);
            mbar_wait(&empty[s], par, &err, 2);
          }
        }
        const uint32_t st = smem_u32(s_stage + s * C::STAGE_BYTES + C::K_BYTES + C::V_BYTES);
#pragma unroll
        for (int r4 = 0; r4 < 4; ++r4) {
          const int r = lane + 32 * r4;
          const int64_t key = (int64_t)t * 128 + r;
          const bool ok = key < p.s_kv;
          const uint8_t* g = ksrc + (ok ? key : 0) * (D / 16);
#pragma unroll
          for (int k = 0; k < C::KB; ++k)
            cp_async_4(st + k * 512 + sf_atom_offset(r, 0), g + 4 * k, ok ? 4u : 0u);
        }
#pragma unroll
        for (int r8 = 0; r8 < D / 32; ++r8) {
          const int dr = lane + 32 * r8;
          const int mt = dr >> 7, r = dr & 127;
          const uint8_t* g = vsrc + (int64_t)dr * p.vsc_row + (int64_t)t * 8;
          cp_async_4_l2line(st + C::KSF_BYTES + (mt * 2 + 0) * 512 + sf_atom_offset(r, 0), g, 4u);
          cp_async_4_l2line(st + C::KSF_BYTES + (mt * 2 + 1) * 512 + sf_atom_offset(r, 0), g + 4, 4u);
        }
        cp_async_commit();
        if (it + 1 - published > (uint32_t)kLag) {
          cp_async_wait<kLag>();
          publish(published++);
        }
      }
    }
    // drain
    cp_async_wait<0>();
    for (; published < it; ++published) publish(published);
  } else if (warp == 1) {
    // ------------------------------------------------------------------ QK^T issuer (+ query prep)
    const bool leader = elect_one();
    const uint32_t idesc = make_idesc_nvfp4(128, 16);
    uint32_t it_w = 0, su_w = 0, item_idx = 0;   // warp-uniform: tiles and rounds issued before this item
    if (my_items > 0) prep_q(0, 0);
    for (int wi = 0; wi < my_items; ++wi, ++item_idx) {
      // the whole warp quantises the NEXT item's query rows into the other buffer; that buffer's
      // last readers are the QK^T MMAs of the previous item, complete once its last s_full fired
      if (wi + 1 < my_items) {
        if (item_idx > 0) mbar_wait(&s_full[(su_w - 1) & 1], ((su_w - 1) >> 1) & 1, &err, 12);
        prep_q(wi + 1, (int)((item_idx + 1) & 1));
      }
      int unit, t0, t1;
      item_at(wi, unit, t0, t1);
      if (leader) {
        uint32_t it = it_w, su = su_w;      // the leader's running counters for this item
        const int qb = item_idx & 1;
        mbar_wait(&q_full[qb], (item_idx >> 1) & 1, &err, 6);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < C::KB; ++k)
          tmem_cp_32x128b_warpx4(tmem + C::T_SFQ + qb * C::KB * 4 + k * 4,
                                 smem_u32(s_qsf + qb * C::QSF_BYTES + k * 512));
        for (int ts0 = t0; ts0 < t1; ts0 += ST, ++su) {
          const int b = su & 1;
          const int nt = min(ST, t1 - ts0);
          if (su >= 2) {
            mbar_spin_wait(&s_free[b], ((su >> 1) & 1) ^ 1, &err, 5);
            // the V-scale TMEM slots of buffer b are rewritten below: the PV of round su - 2 must be done
            mbar_spin_wait(&o_full[b], ((su >> 1) & 1) ^ 1, &err, 11);
          }
          for (int j = 0; j < nt; ++j, ++it) {
            const int s = it % C::NSTAGE;
            const uint32_t ph = (it / C::NSTAGE) & 1;
            mbar_spin_wait(&full_kv[s], ph, &err, 3);
            mbar_spin_wait(&full_sf[s], ph, &err, 4);
            tc_fence_after();
            uint8_t* st = s_stage + s * C::STAGE_BYTES;
            const uint32_t sfk = tmem + C::T_SFK + (b * C::STMAX + j) * C::KB * 4;
#pragma unroll
            for (int k = 0; k < C::KB; ++k)
              tmem_cp_32x128b_warpx4(sfk + k * 4, smem_u32(st + C::K_BYTES + C::V_BYTES + k * 512));
            // the V^T scales of this tile go to TMEM now as well, off the PV issuer's critical path
            // (slot (b, j) was last read by the PV of round su - 2, complete before s_free fired)
            const uint32_t sfv = tmem + C::T_SFV + (b * C::STMAX + j) * C::MT * 8;
#pragma unroll
            for (int k = 0; k < C::MT * 2; ++k)
              tmem_cp_32x128b_warpx4(sfv + k * 4,
                                     smem_u32(st + C::K_BYTES + C::V_BYTES + C::KSF_BYTES + k * 512));
#pragma unroll
            for (int k = 0; k < C::KB; ++k) {
              const uint64_t ad = make_smem_desc(smem_u32(st + (k >> 1) * 8192) + (k & 1) * 32, 16, 512, 4);
              const uint64_t bd =
                  make_smem_desc(smem_u32(s_q + qb * C::Q_BYTES + (k >> 1) * 1024) + (k & 1) * 32, 16, 512, 4);
              umma_nvfp4(tmem + C::T_ST + (b * C::STMAX + j) * 16, ad, bd, idesc, sfk + k * 4,
                         tmem + C::T_SFQ + qb * C::KB * 4 + k * 4, k > 0);
            }
          }
          umma_commit(&s_full[b]);
        }
      }
      it_w += (uint32_t)(t1 - t0);
      su_w += (uint32_t)((t1 - t0 + ST - 1) / ST);
      __syncwarp();
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ PV issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_nvfp4(128, 16);
      uint32_t it = 0, su = 0;
      for (int wi = 0; wi < my_items; ++wi) {
        int unit, t0, t1;
        item_at(wi, unit, t0, t1);
        for (int ts0 = t0; ts0 < t1; ts0 += ST, ++su) {
          const int b = su & 1;
          const int nt = min(ST, t1 - ts0);
          mbar_spin_wait(&p_full[b], (su >> 1) & 1, &err, 7);
          tc_fence_after();
          for (int j = 0; j < nt; ++j, ++it) {
            // V^T tile and scales of stage s were observed by the QK^T issuer before S^T of this
            // round was produced, and P arrived after the softmax warps saw that S^T
            const int s = it % C::NSTAGE;
            uint8_t* st = s_stage + s * C::STAGE_BYTES;
            const uint32_t sfv = tmem + C::T_SFV + (b * C::STMAX + j) * C::MT * 8;
            const uint32_t sfp = tmem + C::T_SFP + (b * C::STMAX + j) * 8;
#pragma unroll
            for (int k = 0; k < 2; ++k)
              tmem_cp_32x128b_warpx4(sfp + k * 4,
                                     smem_u32(s_psf + (b * C::STMAX + j) * C::PSF_BYTES + k * 512));
#pragma unroll
            for (int mt = 0; mt < C::MT; ++mt) {
#pragma unroll
              for (int k = 0; k < 2; ++k) {
                const uint64_t ad =
                    make_smem_desc(smem_u32(st + C::K_BYTES + mt * 8192) + k * 32, 16, 512, 4);
                const uint64_t bd = make_smem_desc(
                    smem_u32(s_p + (b * C::STMAX + j) * C::P_BYTES) + k * 32, 16, 512, 4);
                umma_nvfp4(tmem + C::T_OT + ((b * C::STMAX + j) * C::MT + mt) * 16, ad, bd, idesc,
                           sfv + (mt * 2 + k) * 4, sfp + k * 4, k > 0 ? 1u : 0u);
              }
            }
            umma_commit(&empty[s]);
          }
          umma_commit(&o_full[b]);
        }
      }
    }
    __syncwarp();
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax / accumulate / epilogue
    // Two groups of four warps split every round by tiles (group g owns tiles g*TPG ..), so each
    // SM sub-partition has two warps to overlap latencies with and each thread carries half the
    // state.  All threads see every tile maximum, so the running maximum is the same sequential
    // one in both groups; their O^T / row-sum partials are merged at the end of the item.
    constexpr int TPG = ST / 2;            // tiles per group and round
    const int sw = warp - 4;
    const int grp = sw >> 2;
    const int wq = sw & 3;                 // TMEM lane quadrant
    const int ts = (tid - 128) & 127;      // key lane within a tile (softmax) / d row (accumulate)
    const int tall = tid - 128;            // 0..255
    // pack role: thread `tall` owns (tile ij, head ih, 16-key group ig) of every round
    constexpr int kItems = ST * NQ * 8;
    static_assert(kItems <= 256, "one pack item per softmax thread");
    const bool it_on = tall < kItems;
    const int ig = tall & 7, ih = (tall >> 3) % NQ, ij = tall / (8 * NQ);
    const uint32_t lane_addr = (uint32_t)(wq * 32) << 16;
    uint32_t su = 0;
    for (int wi = 0; wi < my_items; ++wi) {
      int unit, t0, t1;
      item_at(wi, unit, t0, t1);
      float m_run[NQ];                        // running max of every head (all threads agree)
      float o_run[C::MT][NQ], m_acc[NQ];      // d-row role: accumulated O^T, the max it refers to
      float w_prev[TPG][NQ], m_end_prev[NQ];  // weights of the round whose PV is still in flight
      float m_it = -INFINITY, l_it = 0.0f;    // pack role: running max of this thread's head, its part of the row sum
#pragma unroll
      for (int qi = 0; qi < NQ; ++qi) {
        m_run[qi] = -INFINITY; m_acc[qi] = -INFINITY; m_end_prev[qi] = -INFINITY;
#pragma unroll
        for (int mt = 0; mt < C::MT; ++mt) o_run[mt][qi] = 0.0f;
#pragma unroll
        for (int jj = 0; jj < TPG; ++jj) w_prev[jj][qi] = 0.0f;
      }
      // fold this group's fresh accumulators of round `sv` (buffer bb, nt tiles) into o_run
      auto accumulate = [&](uint32_t sv, int nt) {
        const int bb = sv & 1;
        mbar_wait(&o_full[bb], (sv >> 1) & 1, &err, 10);
        tc_fence_after();
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          const float me = m_end_prev[qi];
          const float sc = (me == -INFINITY) ? 0.0f : ex2f_fast((m_acc[qi] - me) * kLog2e);
          m_acc[qi] = me;
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt) o_run[mt][qi] *= sc;
        }
        uint32_t o[TPG][C::MT][16];
#pragma unroll
        for (int jj = 0; jj < TPG; ++jj)
          if (grp * TPG + jj < nt) {
#pragma unroll
            for (int mt = 0; mt < C::MT; ++mt)
              tmem_ld16(tmem + lane_addr + C::T_OT + ((bb * C::STMAX + grp * TPG + jj) * C::MT + mt) * 16,
                        o[jj][mt]);
          }
        tmem_ld_wait();
#pragma unroll
        for (int jj = 0; jj < TPG; ++jj)
          if (grp * TPG + jj < nt) {
#pragma unroll
            for (int mt = 0; mt < C::MT; ++mt)
#pragma unroll
              for (int qi = 0; qi < NQ; ++qi) o_run[mt][qi] += w_prev[jj][qi] * __uint_as_float(o[jj][mt][qi]);
          }
        tc_fence_before();
      };

      int nt_prev = 0;
      bool have_prev = false;
      for (int ts0 = t0; ts0 < t1; ts0 += ST, ++su) {
        const int b = su & 1;
        const int nt = min(ST, t1 - ts0);
        mbar_wait(&s_full[b], (su >> 1) & 1, &err, 8);
        tc_fence_after();
        // ---- key-lane role: this thread's key of each of its group's tiles, every head, goes to
        // the exchange buffer [tile][head][key] (keys permuted within their 16-group so that both
        // these stores and the 16-byte reads below are free of bank conflicts)
        {
          uint32_t r[TPG][16];
#pragma unroll
          for (int jj = 0; jj < TPG; ++jj)
            if (grp * TPG + jj < nt)
              tmem_ld16(tmem + lane_addr + C::T_ST + (b * C::STMAX + grp * TPG + jj) * 16, r[jj]);
          tmem_ld_wait();
          const int kg = ts >> 4, kc = (ts >> 2) & 3, ke = ts & 3;
          const int kpos = kg * 16 + ((kc ^ (kg >> 1)) & 3) * 4 + ke;
#pragma unroll
          for (int jj = 0; jj < TPG; ++jj) {
            const int j = grp * TPG + jj;
            if (j < nt) {
              const bool valid = ((int64_t)(ts0 + j) * 128 + ts) < p.s_kv;
#pragma unroll
              for (int qi = 0; qi < NQ; ++qi)
                ssc[(j * NQ + qi) * 128 + kpos] =
                    (valid && qi < p.g) ? __uint_as_float(r[jj][qi]) * p.scaling : -INFINITY;
            }
          }
        }
        tc_fence_before();
        mbar_arrive(&s_free[b]);
        named_bar_sync(1, 256);
        // ---- pack role: thread = (tile ij, head ih, 16-key group ig) of the round; its sixteen
        // scores are thread-local from here on
        float sc16[16];
        float mx16 = -INFINITY;
        if (it_on && ij < nt) {
          const float* src = ssc + (ij * NQ + ih) * 128 + ig * 16;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            const float4 v = *reinterpret_cast<const float4*>(src + ((c ^ (ig >> 1)) & 3) * 4);
            sc16[4 * c] = v.x; sc16[4 * c + 1] = v.y; sc16[4 * c + 2] = v.z; sc16[4 * c + 3] = v.w;
          }
#pragma unroll
          for (int e = 0; e < 16; ++e) mx16 = fmaxf(mx16, sc16[e]);
        } else {
#pragma unroll
          for (int e = 0; e < 16; ++e) sc16[e] = -INFINITY;
        }
        {
          float tm = mx16;      // maximum of the tile for this head: the eight groups sit in adjacent lanes
          tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 1));
          tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 2));
          tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, 4));
          if (it_on && ig == 0) xch[ij][ih] = tm;
        }
        named_bar_sync(1, 256);
        // running maximum advances tile by tile; weights bring each tile to the round's end
        float w_cur[TPG][NQ];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          float m = m_run[qi];
          float m_mine[TPG];
#pragma unroll
          for (int j = 0; j < ST; ++j) {
            m = (j < nt) ? fmaxf(m, xch[j][qi]) : m;
            if (j / TPG == grp) m_mine[j % TPG] = m;
          }
          m_run[qi] = m;
          const float m_sf = (m == -INFINITY) ? 0.0f : m;
#pragma unroll
          for (int jj = 0; jj < TPG; ++jj)
            w_cur[jj][qi] = (m_mine[jj] == -INFINITY) ? 0.0f : ex2f_fast((m_mine[jj] - m_sf) * kLog2e);
        }
        // the previous round's PV has had a whole round to finish: fold it into registers now,
        // which also frees its P buffers for rewriting
        if (have_prev) accumulate(su - 1, nt_prev);
        if (it_on) {
          // this thread's tile maximum and the round's final one, for its head
          float mj = m_it, mend = m_it;
#pragma unroll
          for (int j = 0; j < ST; ++j) {
            if (j < nt) {
              mend = fmaxf(mend, xch[j][ih]);
              if (j <= ij) mj = mend;
            }
          }
          const float mend_sf = (mend == -INFINITY) ? 0.0f : mend;
          l_it *= ex2f_fast((m_it - mend_sf) * kLog2e);
          m_it = mend;
          if (ij < nt && ih < p.g) {
            const float mj_sf = (mj == -INFINITY) ? 0.0f : mj;
            const float wj = (mj == -INFINITY) ? 0.0f : ex2f_fast((mj_sf - mend_sf) * kLog2e);
            float pv[16], psum = 0.0f;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              pv[e] = ex2f_fast((sc16[e] - mj_sf) * kLog2e);
              psum += pv[e];
            }
            l_it = fmaf(psum, wj, l_it);
            // NVFP4 pack of the sixteen probabilities: ex2 is monotonic, so the exponential of the
            // group's largest score is the group's largest probability
            const float am = ex2f_fast((mx16 - mj_sf) * kLog2e);
            const float s32 = fminf(fmaxf(am * 0.16666667f, kScaleFloor), kScaleMax);
            uint16_t sb16;
            asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(sb16) : "f"(0.0f), "f"(s32));
            float inv;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(e4m3_to_f32((uint8_t)(sb16 & 0xFFu))));
            const uint32_t lo = e2m1x8(pv[0] * inv, pv[1] * inv, pv[2] * inv, pv[3] * inv, pv[4] * inv, pv[5] * inv,
                                       pv[6] * inv, pv[7] * inv);
            const uint32_t hi = e2m1x8(pv[8] * inv, pv[9] * inv, pv[10] * inv, pv[11] * inv, pv[12] * inv,
                                       pv[13] * inv, pv[14] * inv, pv[15] * inv);
            const uint32_t pt = smem_u32(s_p + (b * C::STMAX + ij) * C::P_BYTES);
            const uint32_t psf = smem_u32(s_psf + (b * C::STMAX + ij) * C::PSF_BYTES);
            sts_v2(pt + sw64_offset(ih, ig * 8), lo, hi);
            asm volatile("st.shared.u8 [%0], %1;" ::"r"(psf + (ig >> 2) * 512 + sf_atom_offset(ih, ig & 3)),
                         "h"((uint16_t)(sb16 & 0xFFu)) : "memory");
          }
        }
#pragma unroll
        for (int jj = 0; jj < TPG; ++jj)
#pragma unroll
          for (int qi = 0; qi < NQ; ++qi) w_prev[jj][qi] = w_cur[jj][qi];
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) m_end_prev[qi] = m_run[qi];
        nt_prev = nt;
        have_prev = true;
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&p_full[b]);
      }
      // ---- item epilogue: fold the last round, merge the two groups, write un-normalised partials
      if (have_prev) accumulate(su - 1, nt_prev);
      {
        // bring this group's accumulator to the final running maximum
#pragma unroll
        for (int qi = 0; qi < NQ; ++qi) {
          const float mf = m_run[qi];
          const float sc = (mf == -INFINITY || m_acc[qi] == -INFINITY) ? 0.0f
                                                                        : ex2f_fast((m_acc[qi] - mf) * kLog2e);
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt) o_run[mt][qi] *= sc;
        }
        if (grp == 1) {
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt)
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi) s_merge[qi * D + mt * 128 + ts] = o_run[mt][qi];
        }
        {
          // row sums: the eight groups of a (tile slot, head) sit in adjacent lanes
          float v = it_on ? l_it : 0.0f;
          v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          v += __shfl_xor_sync(0xffffffffu, v, 4);
          if (it_on && ig == 0) lred[ij][ih] = v;
        }
        named_bar_sync(1, 256);
        if (grp == 0) {
          const int64_t w = slot_at(wi);
          float* acc = p.ws_acc + w * 16 * D;
#pragma unroll
          for (int mt = 0; mt < C::MT; ++mt)
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi)
              if (qi < p.g) acc[qi * D + mt * 128 + ts] = o_run[mt][qi] + s_merge[qi * D + mt * 128 + ts];
          if (ts < p.g) {
            float lsum = 0.0f, mfin = -INFINITY;
#pragma unroll
            for (int qi = 0; qi < NQ; ++qi)
              if (qi == ts) {
#pragma unroll
                for (int ww = 0; ww < ST; ++ww) lsum += lred[ww][qi];
                mfin = m_run[qi];
              }
            p.ws_m[w * 16 + ts] = mfin;
            p.ws_l[w * 16 + ts] = lsum;
          }
        }
        // no barrier here: the merge buffer (= the P tiles) and lred are next written after the
        // max-exchange barrier of the next item's first round, which these reads precede in
        // program order; the kernel's final __syncthreads covers the last item
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
                                      const float* __restrict__ ws_l, int nsplit, int64_t extra_base,
                                      int n_extra, int hk, int g, int d,
                                      TQ* __restrict__ out, float* __restrict__ lse) {
  const int unit = blockIdx.x / g, qi = blockIdx.x % g;
  const int t = threadIdx.x;
  float gm = -INFINITY;
  for (int s = 0; s < nsplit; ++s) gm = fmaxf(gm, ws_m[((int64_t)unit * nsplit + s) * 16 + qi]);
  // partials appended by another kernel over further keys of the unit (a high-precision window)
  for (int e = 0; e < n_extra; ++e) gm = fmaxf(gm, ws_m[(extra_base + (int64_t)unit * n_extra + e) * 16 + qi]);
  float acc = 0.0f, den = 0.0f;
  for (int s = 0; s < nsplit + n_extra; ++s) {
    const int64_t w = s < nsplit ? (int64_t)unit * nsplit + s : extra_base + (int64_t)unit * n_extra + (s - nsplit);
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

// The same for the balanced decomposition: the partials of a unit are the pieces written by the
// CTAs whose tile ranges reach into it.
template <typename TQ>
__global__ void decode_combine_balanced_kernel(const float* __restrict__ ws_acc,
                                               const float* __restrict__ ws_m,
                                               const float* __restrict__ ws_l, int64_t total_tiles,
                                               int ntiles, int nctas, int maxseg, int64_t extra_base,
                                               int n_extra, int hk, int g, int d,
                                               TQ* __restrict__ out, float* __restrict__ lse) {
  const int unit = blockIdx.x / g, qi = blockIdx.x % g;
  const int t = threadIdx.x;
  const int64_t x0 = (int64_t)unit * ntiles, x1 = x0 + ntiles;
  int64_t b0 = x0 * nctas / total_tiles;      // the CTA whose range contains tile x0
  while (b0 + 1 < nctas && (b0 + 1) * total_tiles / nctas <= x0) ++b0;
  while (b0 > 0 && b0 * total_tiles / nctas > x0) --b0;
  float gm = -INFINITY;
  for (int64_t b = b0; b < nctas && b * total_tiles / nctas < x1; ++b) {
    const int64_t st = b * total_tiles / nctas, en = (b + 1) * total_tiles / nctas;
    if (en <= st || en <= x0) continue;
    const int64_t w = b * maxseg + (unit - st / ntiles);
    gm = fmaxf(gm, ws_m[w * 16 + qi]);
  }
  for (int e = 0; e < n_extra; ++e) gm = fmaxf(gm, ws_m[(extra_base + (int64_t)unit * n_extra + e) * 16 + qi]);
  float acc = 0.0f, den = 0.0f;
  for (int e = 0; e < n_extra; ++e) {
    const int64_t w = extra_base + (int64_t)unit * n_extra + e;
    const float ms = ws_m[w * 16 + qi];
    const float f = (ms == -INFINITY) ? 0.0f : expf(ms - gm);
    acc += f * ws_acc[(w * 16 + qi) * d + t];
    den += f * ws_l[w * 16 + qi];
  }
  for (int64_t b = b0; b < nctas && b * total_tiles / nctas < x1; ++b) {
    const int64_t st = b * total_tiles / nctas, en = (b + 1) * total_tiles / nctas;
    if (en <= st || en <= x0) continue;
    const int64_t w = b * maxseg + (unit - st / ntiles);
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

// Balanced decomposition: CTAs and partial slots per CTA for `zhk` units of `ntiles` tiles.
inline void decode_balanced_geometry(int64_t zhk, int64_t ntiles, int sm_count, int* nctas, int* maxseg) {
  const int64_t total = zhk * ntiles;
  const int64_t g = std::max<int64_t>(1, std::min<int64_t>(sm_count, total / 4 > 0 ? total / 4 : 1));
  const int64_t per = (total + g - 1) / g;
  *nctas = (int)g;
  *maxseg = (int)((per + ntiles - 2) / ntiles + 1);
}

template <int D, typename TQ>
int decode_launch(const CUtensorMap& tm_k, const CUtensorMap& tm_v, const CUtensorMap& tm_vpf,
                  const CUtensorMap& tm_vpf4,
                  const DecodeParams& p,
                  int64_t zhk, void* out, float* lse, int sm_count, cudaStream_t st) {
  using C = DecodeCfg<D>;
  int grid = (int)std::min<int64_t>(p.nitems, sm_count);
  if (p.balanced) {
    int ms;
    decode_balanced_geometry(zhk, p.ntiles, sm_count, &grid, &ms);
  }
  auto launch = [&](auto kern) -> int {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         C::SMEM_BYTES);
    if (e != cudaSuccess) return fail((int)e, "nvfp4_decode: smem attribute: %s", cudaGetErrorString(e));
    kern<<<grid, kDecodeThreads, C::SMEM_BYTES, st>>>(tm_k, tm_v, tm_vpf, tm_vpf4, p);
    return launch_result("nvfp4_decode");
  };
  int rc;
  if (p.g <= 4) rc = launch(decode_kernel<D, TQ, 4>);
  else if (p.g <= 8) rc = launch(decode_kernel<D, TQ, 8>);
  else rc = launch(decode_kernel<D, TQ, 16>);
  if (rc) return rc;
  if (p.balanced)
    decode_combine_balanced_kernel<TQ><<<(unsigned)(zhk * p.g), D, 0, st>>>(
        p.ws_acc, p.ws_m, p.ws_l, p.total_tiles, p.ntiles, grid, p.maxseg, p.extra_base, p.n_extra, p.hk, p.g, D,
        static_cast<TQ*>(out), lse);
  else
    decode_combine_kernel<TQ><<<(unsigned)(zhk * p.g), D, 0, st>>>(
        p.ws_acc, p.ws_m, p.ws_l, p.nsplit, p.extra_base, p.n_extra, p.hk, p.g, D, static_cast<TQ*>(out), lse);
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
  // Persistent CTAs take work items round-robin, so the step costs
  //     waves * (tiles_per_item * t_tile + t_item),  waves = ceil(zhk * nsplit / sm_count):
  // few splits leave SMs idle in the last wave, many splits pay the per-item pipeline drain
  // (measured on B200: about 6 tile times per item).  Pick the split count that minimises it; no
  // item under 4 tiles.
  const int64_t max_split = std::max<int64_t>(1, std::min<int64_t>(tiles / 4, 64));
  int64_t best_chunk = tiles;
  double best_cost = 1e300;
  for (int64_t want = 1; want <= max_split; ++want) {
    const int64_t c = (tiles + want - 1) / want;
    const int64_t n = (tiles + c - 1) / c;
    const int64_t waves = (zhk * n + sm_count - 1) / sm_count;
    const double cost = (double)waves * ((double)c + 6.0);
    if (cost < best_cost - 1e-9) { best_cost = cost; best_chunk = c; }
  }
  const int64_t chunk = best_chunk;
  int64_t ns = (tiles + chunk - 1) / chunk;
  size_t bytes = (size_t)(zhk * ns) * (size_t)(16 * d + 32) * sizeof(float);
  // balanced decomposition (nsplit = 0): every CTA streams an equal share of the unit-major tile
  // list and a unit's partials are the pieces of the CTAs that touch it
  int bg, bm;
  decode_balanced_geometry(zhk, tiles, sm_count, &bg, &bm);
  const double per = (double)((zhk * tiles + bg - 1) / bg);
  const double bal_cost = per + 6.0 * (1.0 + per / (double)tiles);
  int64_t kv = chunk * 128;
  if (bal_cost < best_cost) {
    ns = 0;
    kv = 0;
    bytes = (size_t)bg * (size_t)bm * (size_t)(16 * d + 32) * sizeof(float);
  }
  if (nsplit) *nsplit = (int)ns;
  if (split_kv) *split_kv = kv;
  if (workspace_bytes) *workspace_bytes = bytes;
  return 0;
}

extern "C" int nvfp4_decode(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh,
                            const uint8_t* knv, int64_t knv_unit, const uint8_t* ksc,
                            int64_t ksc_unit, const uint8_t* vnv, int64_t vnv_unit, int64_t vnv_row,
                            const uint8_t* vsc, int64_t vsc_unit, int64_t vsc_row, int64_t z,
                            int64_t hk, int g, int d, int64_t s_kv, float scaling, void* out,
                            float* lse, void* workspace, size_t workspace_bytes, int nsplit,
                            int64_t split_kv, int* status, nvfp4_stream_t stream) {
  return nvfp4_decode_hybrid(q, q_dtype, s_qz, s_qh, knv, knv_unit, ksc, ksc_unit, vnv, vnv_unit, vnv_row, vsc,
                             vsc_unit, vsc_row, z, hk, g, d, s_kv, scaling, out, lse, workspace, workspace_bytes,
                             nsplit, split_kv, 0, status, stream);
}

extern "C" int nvfp4_decode_hybrid(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh,
                                   const uint8_t* knv, int64_t knv_unit, const uint8_t* ksc,
                                   int64_t ksc_unit, const uint8_t* vnv, int64_t vnv_unit,
                                   int64_t vnv_row, const uint8_t* vsc, int64_t vsc_unit,
                                   int64_t vsc_row, int64_t z, int64_t hk, int g, int d, int64_t s_kv,
                                   float scaling, void* out, float* lse, void* workspace,
                                   size_t workspace_bytes, int nsplit, int64_t split_kv, int n_extra,
                                   int* status, nvfp4_stream_t stream) {
  using namespace nvfp4;
  NVFP4_REQUIRE(n_extra >= 0 && n_extra <= 64, "nvfp4_decode: extra partials per unit must be in [0, 64]");
  NVFP4_REQUIRE(d == 128 || d == 256, "nvfp4_decode: D must be 128 or 256");
  NVFP4_REQUIRE(g >= 1 && g <= 16, "nvfp4_decode: GQA group %d must be <= 16", g);
  NVFP4_REQUIRE(z >= 1 && hk >= 1 && s_kv >= 1, "nvfp4_decode: empty problem");
  NVFP4_REQUIRE(q && knv && ksc && vnv && vsc && out && workspace, "nvfp4_decode: null pointer");
  const bool balanced = nsplit == 0;   // balanced decomposition chosen by nvfp4_decode_plan
  NVFP4_REQUIRE(balanced || (nsplit >= 1 && split_kv >= 128 && split_kv % 128 == 0),
                "nvfp4_decode: split_kv must be a positive multiple of 128");
  NVFP4_REQUIRE(balanced ||
                    ((int64_t)nsplit * split_kv >= s_kv && (int64_t)(nsplit - 1) * split_kv < s_kv),
                "nvfp4_decode: nsplit * split_kv does not cover s_kv exactly");
  const int64_t zhk = z * hk;
  int dev = 0, sm_count = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
  if (sm_count <= 0) return fail(-1, "nvfp4_decode: no CUDA device");
  int bal_ctas = 0, bal_maxseg = 0;
  decode_balanced_geometry(zhk, (s_kv + 127) / 128, sm_count, &bal_ctas, &bal_maxseg);
  const int64_t own_slots = balanced ? (int64_t)bal_ctas * bal_maxseg : zhk * nsplit;
  const int64_t slots = own_slots + zhk * n_extra;      // the caller's extra partials follow the kernel's own
  const size_t need = (size_t)slots * (size_t)(16 * d + 32) * sizeof(float);
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

  CUtensorMap tm_k, tm_v, tm_vpf, tm_vpf4;
  int rc = make_tmap_u8_3d_sw64(&tm_k, knv, (uint64_t)d / 2, (uint64_t)s_kv, (uint64_t)zhk,
                                (uint64_t)d / 2, (uint64_t)knv_unit, 128, "nvfp4_decode(K)");
  if (rc) return rc;
  rc = make_tmap_u8_3d_sw64(&tm_v, vnv, (uint64_t)s_pad / 2, (uint64_t)d, (uint64_t)zhk,
                            (uint64_t)vnv_row, (uint64_t)vnv_unit, 128, "nvfp4_decode(V)");
  if (rc) return rc;

  rc = make_tmap_u32_3d_prefetch(&tm_vpf, vnv, (uint64_t)s_pad / 2, (uint64_t)d, (uint64_t)zhk,
                                 (uint64_t)vnv_row, (uint64_t)vnv_unit,
                                 (uint32_t)std::min<uint64_t>(256, (uint64_t)s_pad / 8), 8,
                                 "nvfp4_decode(V prefetch)");
  if (rc) return rc;
  rc = make_tmap_u32_3d_prefetch(&tm_vpf4, vnv, (uint64_t)s_pad / 2, (uint64_t)d, (uint64_t)zhk,
                                 (uint64_t)vnv_row, (uint64_t)vnv_unit,
                                 (uint32_t)std::min<uint64_t>(64, (uint64_t)s_pad / 8), 8,
                                 "nvfp4_decode(V prefetch, tail)");
  if (rc) return rc;

  DecodeParams p;
  p.q = q; p.s_qz = s_qz; p.s_qh = s_qh;
  p.ksc = ksc; p.ksc_unit = ksc_unit;
  p.vsc = vsc; p.vsc_unit = vsc_unit; p.vsc_row = vsc_row;
  p.hk = (int)hk; p.g = g; p.s_kv = s_kv; p.scaling = scaling;
  p.nsplit = balanced ? 1 : nsplit; p.chunk_tiles = (int)(split_kv / 128); p.ntiles = (int)((s_kv + 127) / 128);
  p.nitems = balanced ? 0 : zhk * nsplit;
  p.balanced = balanced ? 1 : 0;
  p.total_tiles = zhk * p.ntiles;
  p.maxseg = bal_maxseg;
  float* ws = static_cast<float*>(workspace);
  p.ws_acc = ws;
  p.ws_m = ws + slots * 16 * d;
  p.ws_l = p.ws_m + slots * 16;
  p.extra_base = own_slots;
  p.n_extra = n_extra;
  p.status = status;

#define NVFP4_DECODE(DD, T) return decode_launch<DD, T>(tm_k, tm_v, tm_vpf, tm_vpf4, p, zhk, out, lse, sm_count, st)
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
  NVFP4_REQUIRE(z >= 1 && hk >= 1 && nsplit >= 0 && s_kv >= 1, "nvfp4_decode_static: empty problem");
  size_t slots = (size_t)(z * hk) * (size_t)nsplit;
  if (nsplit == 0) {   // balanced decomposition
    int dev = 0, sm_count = 0, bc = 0, bm = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
    decode_balanced_geometry(z * hk, (s_kv + 127) / 128, sm_count > 0 ? sm_count : 148, &bc, &bm);
    slots = (size_t)bc * (size_t)bm;
  }
  const size_t need = slots * (size_t)(16 * d + 32) * sizeof(float);
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
