// Thin inline-PTX layer for sm_100a: mbarrier, TMA (cp.async.bulk.tensor), tcgen05
// (TMEM allocation, block-scaled MMA, tcgen05.cp/ld/st, commit) and descriptor builders.
//
// Every wait in this file is BOUNDED: a wait that exceeds its iteration budget records a
// status word and returns false instead of spinning forever, and once a CTA has recorded an
// error all of its later waits return immediately, so a protocol bug ends the kernel in
// milliseconds with a readable status instead of hanging the device.
#pragma once
#include <cuda_runtime.h>
#include <cuda.h>
#include <stdint.h>

namespace nvfp4 {

// ---------------------------------------------------------------------------------------
// status codes written by kernels into their device status word (0 = ok)
// ---------------------------------------------------------------------------------------
enum : int {
  KSTAT_OK = 0,
  KSTAT_WAIT_TIMEOUT = 0x100,  // | site id
};

#ifndef NVFP4_WAIT_SPINS
#define NVFP4_WAIT_SPINS (1u << 20)
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(pred));
  return pred != 0;
}

// ------------------------------------------------------------------ mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One potentially-blocking probe: the hardware may park the thread until the phase completes or
// the hint (ns) runs out, so a waiting warp costs few issue slots.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(2000u)
      : "memory");
  return ok != 0;
}

// Non-blocking probe (cheap when the phase has already completed).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait with an explicit probe budget. `err` is a CTA-shared int (0 = healthy). Returns
// false on timeout, after recording KSTAT_WAIT_TIMEOUT | site in `err`.
__device__ __forceinline__ bool mbar_wait_n(uint64_t* bar, uint32_t parity, volatile int* err,
                                            int site, uint32_t spins) {
  if (mbar_test_wait(bar, parity)) return true;
  if (mbar_try_wait(bar, parity)) return true;
  if (*err) return false;
  for (uint32_t i = 0; i < spins; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*err) return false;
  }
  *err = KSTAT_WAIT_TIMEOUT | site;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* err,
                                          int site) {
  return mbar_wait_n(bar, parity, err, site, NVFP4_WAIT_SPINS);
}

// Bounded wait that polls without parking the thread: lowest wake-up latency, meant for a lone
// elected thread (an MMA issuer) whose reaction time is on the critical path.
__device__ __forceinline__ bool mbar_spin_wait(uint64_t* bar, uint32_t parity, volatile int* err,
                                               int site) {
  for (uint32_t i = 0; i < (NVFP4_WAIT_SPINS << 4); ++i) {
    if (mbar_test_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *err) return false;
  }
  *err = KSTAT_WAIT_TIMEOUT | site;
  return false;
}

// barrier among a subset of warps (id 1..15, nthreads multiple of 32)
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// generic-proxy writes (st.shared) -> visible to the async proxy (TMA / tcgen05 reads of smem)
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// shared-memory accesses by 32-bit shared address (keeps them out of the generic path)
__device__ __forceinline__ void sts_v2(uint32_t saddr, uint32_t a, uint32_t b) {
  asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(saddr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void sts_b32(uint32_t saddr, uint32_t a) {
  asm volatile("st.shared.b32 [%0], %1;" ::"r"(saddr), "r"(a) : "memory");
}
__device__ __forceinline__ void sts_f32(uint32_t saddr, float a) {
  asm volatile("st.shared.f32 [%0], %1;" ::"r"(saddr), "f"(a) : "memory");
}
__device__ __forceinline__ float lds_f32(uint32_t saddr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(saddr) : "memory");
  return v;
}

// ------------------------------------------------------------------ TMA
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0,
                                            int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, "
      "%4, %5}], [%2];" ::"r"(smem_u32(dst)),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

// L2 prefetch of a tensor-map box (no shared memory, no barrier).
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* m, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(c0), "r"(c1), "r"(c2)
               : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void* p) {
  asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}

// Per-thread asynchronous 4-byte global -> shared copy; src_bytes = 0 zero-fills.
__device__ __forceinline__ void cp_async_4(uint32_t saddr, const void* gptr, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(saddr), "l"(gptr), "r"(src_bytes)
               : "memory");
}
// The same with a hint that L2 should fetch the whole 128-byte line: for scattered small reads
// whose neighbours in the line are wanted a few tiles later (strided scale bytes).
__device__ __forceinline__ void cp_async_4_l2line(uint32_t saddr, const void* gptr, uint32_t src_bytes) {
  asm volatile("cp.async.ca.shared.global.L2::128B [%0], [%1], 4, %2;" ::"r"(saddr), "l"(gptr),
               "r"(src_bytes)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// ------------------------------------------------------------------ TMEM management
// Must be executed by one full warp. ncols: power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ------------------------------------------------------------------ descriptors
// Shared-memory matrix descriptor, K-major operand, 16-byte units.
//   swizzle_code: 0 none, 2 = 128B, 4 = 64B, 6 = 32B.
//   sbo_bytes: distance between consecutive 8-row groups.
__host__ __device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes,
                                                            uint32_t swizzle_code) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;  // descriptor version for sm_100
  d |= (uint64_t)(swizzle_code & 7) << 61;
  return d;
}

// Instruction descriptor (upper 32 bits of the i-desc operand) for
// kind::mxf4nvf4, e2m1 x e2m1, ue4m3 scales per 16, fp32 accumulate, both operands K-major.
__host__ __device__ __forceinline__ uint32_t make_idesc_nvfp4(uint32_t m, uint32_t n) {
  uint32_t d = 0;
  d |= 1u << 7;          // A format: e2m1
  d |= 1u << 10;         // B format: e2m1
  d |= (n >> 3) << 17;   // N / 8
  d |= 0u << 23;         // scale format: ue4m3
  d |= (m >> 4) << 24;   // M / 16
  return d;              // sf ids 0, K = 64
}

// D[tmem] (+)= A[smem] * B[smem]^T with block scales held in TMEM. One thread issues.
__device__ __forceinline__ void umma_nvfp4(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                           uint32_t idesc, uint32_t sfa_tmem, uint32_t sfb_tmem,
                                           uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], "
      "p;\n\t}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
      : "memory");
}

// All tcgen05 async ops issued so far by this thread arrive (once) on `bar` when complete.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
          smem_u32(bar))
      : "memory");
}

// smem (32 rows x 16 bytes, rows 16 B apart) -> TMEM (32 lanes x 4 columns, replicated to the
// four 32-lane sub-partitions). One thread issues. Used for block-scale factors.
__device__ __forceinline__ void tmem_cp_32x128b_warpx4(uint32_t taddr, uint32_t saddr) {
  uint64_t desc = make_smem_desc(saddr, 0, 128, 0);
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(desc)
               : "memory");
}

// ------------------------------------------------------------------ TMEM <-> registers
// 32 lanes x 32 consecutive 32-bit columns; thread t of the warp gets lane (base_lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(
          taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
      "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]),
      "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
      "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------ operand layouts in smem
// Byte offset of (row, byte-in-row) inside a K-major tile whose rows are 64 bytes wide and
// stored with the 64-byte swizzle (8-row x 64 B = 512 B repeating pattern; tile base 512 B
// aligned): the 16-byte chunk index is XORed with bits [1,3) of the row.
__device__ __forceinline__ uint32_t sw64_offset(uint32_t row, uint32_t byte_in_row) {
  uint32_t chunk = byte_in_row >> 4;
  return row * 64u + (((chunk ^ (row >> 1)) & 3u) << 4) + (byte_in_row & 15u);
}
// Same for 128-byte rows with the 128-byte swizzle (8 x 128 B = 1 KB pattern, base 1 KB aligned).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t byte_in_row) {
  uint32_t chunk = byte_in_row >> 4;
  return row * 128u + (((chunk ^ row) & 7u) << 4) + (byte_in_row & 15u);
}
// Block-scale "atom" consumed by tcgen05.cp 32x128b.warpx4: 128 rows x 4 scale bytes (one
// K=64 MMA) stored as 32 x 16 B; row r, scale k sits at (r % 32) * 16 + (r / 32) * 4 + k.
__device__ __forceinline__ uint32_t sf_atom_offset(uint32_t row, uint32_t k) {
  return (row & 31u) * 16u + (row >> 5) * 4u + k;
}

}  // namespace nvfp4
