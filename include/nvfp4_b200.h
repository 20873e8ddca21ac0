/*
 * nvfp4_b200 -- C ABI of the B200 (sm_100a) NVFP4 flash-attention kernels.
 *
 * This is the drop-in boundary for the `sageattention.nvfp4` path of thad0ctor/SageAttention.
 * The reference has no FFI of its own (it launches Triton kernels from Python); every entry
 * point below replaces one Triton launch site and cites it as `file:line` inside the reference
 * project.  A host binding passes raw device pointers, element/byte strides and the CUDA stream
 * to enqueue on; no entry point allocates memory, synchronises, or throws.
 *
 * Return value: 0 on success; < 0 for an invalid argument (text in nvfp4_last_error()); > 0 is a
 * cudaError_t from a launch.  Kernels that wait on hardware barriers bound every wait and report
 * a non-zero word through the `status` pointer instead of hanging.
 *
 * Packed layouts (identical to the reference, flash.py:363-419 and kv_cache.py:6-7):
 *   along-D pack    nib [B, rows, D/2] uint8, sc [B, rows, D/16] e4m3 bytes
 *   V^T pack        nib [B, D, Sp/2]  uint8, sc [B, D, Sp/16]  e4m3 bytes, Sp = keys padded to 128
 *   byte j of a row = code[2j] | code[2j+1] << 4, codes are e2m1 with sign in bit 3.
 */
#ifndef NVFP4_B200_H_
#define NVFP4_B200_H_

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* element types of high-precision tensors */
#define NVFP4_DT_BF16 0
#define NVFP4_DT_FP16 1
#define NVFP4_DT_FP32 2

/* flags of nvfp4_fwd */
#define NVFP4_FWD_CAUSAL 1
/* nvfp4_bwd_fp4 only: stochastic rounding of an in-kernel gradient-operand pack (fp4_legacy) */
#define NVFP4_BWD_SR_DS_DK 16  /* dS^T, the operand of dK  (`stochastic_rounding`)            */
#define NVFP4_BWD_SR_P_DV 32   /* P^T,  the operand of dV  (`backward_p_dv_stochastic_rounding`) */
#define NVFP4_BWD_SR_DS_DQ 64  /* dS,   the operand of dQ  (`backward_ds_dq_stochastic_rounding`) */
/* nvfp4_bwd_fp4 only: the transposed packs (dotnv, qtnv, ktnv) are MXFP8 and the in-kernel gradient
 * operands are packed as MXFP8 ("fp8_rownorm") */
#define NVFP4_BWD_MXFP8 128
/* nvfp4_pack_dual sr_flags */
#define NVFP4_PACK_SR_ALONG_D 1
#define NVFP4_PACK_SR_ALONG_S 2

typedef void* nvfp4_stream_t; /* a cudaStream_t */

/* Library identification; bumps when a signature changes. */
int nvfp4_abi_version(void);

/* Text of the last error returned on the calling thread ("" if none). */
const char* nvfp4_last_error(void);

/*
 * NVFP4 pack of a strided [B, R, K] view along K: per 16 elements
 * amax -> e4m3(clamp(amax / 6, 2^-9, 448)) -> IEEE divide -> e2m1 RTNE, saturating.
 * Replaces `_quant_nvfp4` / `_quant_nvfp4_kernel` (sageattention/nvfp4/flash.py:310-419); the
 * reference's `transpose=True` (V^T) is expressed by passing sxr = 1 and sxk = the key stride.
 * Elements at contraction index >= k_read read as +0.0; groups up to k_pad are written
 * (k_pad % 16 == 0, k_pad >= k_read).  x strides are in elements, output strides in bytes; output
 * rows are contiguous (k_pad/2 and k_pad/16 bytes).
 */
int nvfp4_pack(const void* x, int dtype, int64_t B, int64_t R, int64_t k_read, int64_t k_pad,
               int64_t sxb, int64_t sxr, int64_t sxk, uint8_t* nib, int64_t snb, int64_t snr,
               uint8_t* sc, int64_t ssb, int64_t ssr, nvfp4_stream_t stream);

/*
 * V projection with the pack as its epilogue (the "v_proj epilogue" producer asked for in
 * flash.py:10-13, 2812-2821; the reference itself ships no such kernel): V = X W^T (+ bias) on the
 * tensor cores (tcgen05.mma kind::f16, fp32 accumulate), rounded once to the operand dtype, and
 * written as the V^T pack along the keys -- vnv [z*hk, d, s_pad/2], vsc [z*hk, d, s_pad/16],
 * tokens >= s packed as +0.0 -- and, when v_out is given, as the 16-bit V [z, s, hk*d] itself
 * (element strides svb, svs; unit stride along the features).  The packed bytes equal nvfp4_pack
 * of that V.  x [z, s, hidden] (element strides sxb, sxs, multiples of 8; unit stride along
 * hidden), w [hk*d, hidden] contiguous, bias [hk*d] or NULL, all bf16 or all fp16; hidden % 8 == 0,
 * s_pad % 16 == 0.
 */
int nvfp4_vproj_pack(const void* x, const void* w, const void* bias, int dtype, int64_t z, int64_t s,
                     int64_t hidden, int64_t hk, int d, int64_t sxb, int64_t sxs, int64_t s_pad,
                     uint8_t* vnv, uint8_t* vsc, void* v_out, int64_t svb, int64_t svs, int* status,
                     nvfp4_stream_t stream);

/*
 * Both packs of x [B, S, d] (element strides sxb, sxs; unit stride along d) from ONE read: along d
 * (dnib [B, S, d/2], dsc [B, S, d/16]) and along S as the transposed layout (tnib [B, d, s_pad/2],
 * tsc [B, d, s_pad/16], tokens >= S read as +0.0).  All four outputs contiguous.  Replaces
 * `_quant_nvfp4_dual` / `_quant_nvfp4_dual_kernel` (flash.py:434-561); bytes equal two nvfp4_pack
 * calls.  d % 16 == 0, s_pad % 16 == 0, s_pad >= S.  With `prescale_amax` (a device float holding
 * max|x|, e.g. from nvfp4_bwd_prep) every element is first divided by the smallest power of two
 * >= that value (exact), so the packed tensor is x / 2^e with 0.5 < max|.| <= 1 -- the global
 * normalisation of dO in the all-FP4 backward; NULL packs x itself.  sr_flags
 * (NVFP4_PACK_SR_ALONG_D | NVFP4_PACK_SR_ALONG_S) round that output's e2m1 codes stochastically
 * from (seed, position) instead of to nearest (scale bytes unchanged): the dO / dO^T packs of the
 * fp4_legacy backward (`SR_DO` / `SR_DOT`, flash.py:1352-1394).
 */
int nvfp4_pack_dual(const void* x, int dtype, int64_t B, int64_t S, int d, int64_t s_pad,
                    int64_t sxb, int64_t sxs, const float* prescale_amax, int sr_flags,
                    uint32_t seed, uint8_t* dnib, uint8_t* dsc, uint8_t* tnib, uint8_t* tsc,
                    nvfp4_stream_t stream);

/*
 * MXFP8 pack along the tokens: x [B, S, d] (element strides sxb, sxs; unit stride along d) ->
 * e4m3 bytes out [B, d, s_pad] and e8m0 scale bytes sc [B, d, s_pad/32], one scale per 32 tokens
 * (tokens >= S read as +0.0).  The rule of `_pack_mxfp8_along_k` (flash.py:243-257): e = the smallest
 * integer with amax / 2^e <= 448 (amax floored at 1e-30), bytes = e4m3 RTNE of x / 2^e, scale =
 * e + 127.  s_pad % 32 == 0.  `prescale_amax` as in nvfp4_pack_dual.  Feeds nvfp4_bwd_fp4 with
 * NVFP4_BWD_MXFP8 (which wants s_pad % 128 == 0).
 */
int nvfp4_pack_mx8_t(const void* x, int dtype, int64_t B, int64_t S, int d, int64_t s_pad, int64_t sxb,
                     int64_t sxs, const float* prescale_amax, uint8_t* out, uint8_t* sc,
                     nvfp4_stream_t stream);

/*
 * Forward pre-pack in ONE launch: Q [bq, s_q, d] and K [bk, s_kv, d] along d, V [bk, s_kv, d] along
 * the keys as V^T padded to s_pad.  Replaces `_quant_qkv_fwd` / `_quant_qkv_fwd_kernel`
 * (flash.py:579-732).  Inputs have unit stride along d and element strides (batch, row) as given;
 * outputs are contiguous in the layouts of nvfp4_pack.  Bytes equal three nvfp4_pack calls.
 */
int nvfp4_pack_qkv(const void* q, const void* k, const void* v, int dtype, int64_t bq, int64_t bk,
                   int64_t s_q, int64_t s_kv, int64_t s_pad, int d, int64_t sqb, int64_t sqr,
                   int64_t skb, int64_t skr, int64_t svb, int64_t svk, uint8_t* qnv, uint8_t* qsc,
                   uint8_t* knv, uint8_t* ksc, uint8_t* vnv, uint8_t* vsc, nvfp4_stream_t stream);

/*
 * Rotary position embedding fused into the packer: y = rope(x) is rounded once to the input dtype
 * and packed along D exactly as nvfp4_pack would pack it, without y ever reaching HBM.  The
 * reference names this fused producer as the condition for an end-to-end win of its pre-packed
 * entry points (`q_packs` / `k_packs`, flash.py:10-13, 2812-2821) and leaves it to the caller.
 *   x [B, R, d]: element strides sxb, sxr, unit stride along d; d a power of two >= 32.
 *   cos_tab / sin_tab [P, d/2] fp32; row r uses position positions[r] (int32, may be NULL) or
 *   pos0 + r.  Half-split convention: y[i] = x[i] cos[i] - x[i + d/2] sin[i] (i < d/2),
 *   y[i] = x[i] cos[i - d/2] + x[i - d/2] sin[i - d/2] (i >= d/2).
 *   out_nib / out_sc as for nvfp4_pack (byte strides; nibble rows 8-byte aligned).
 */
int nvfp4_rope_pack(const void* x, int dtype, int64_t B, int64_t R, int d, int64_t sxb, int64_t sxr,
                    const float* cos_tab, const float* sin_tab, const int32_t* positions,
                    int64_t pos0, uint8_t* out_nib, int64_t snb, int64_t snr, uint8_t* out_sc,
                    int64_t ssb, int64_t ssr, nvfp4_stream_t stream);

/*
 * One decode-step append into an NVFP4 KV cache, one launch, no host synchronisation.
 * Replaces NVFP4KVCache.append (sageattention/nvfp4/kv_cache.py:228-257): packs the new K row
 * along D into position `pos`; stores the new V token into slot pos % 16 of the partial-group
 * buffer (zeroing the buffer first when the slot is 0) and re-packs that 16-key group of V^T;
 * optionally writes the token into the recent-window rings at slot pos % ring_cap.
 * k_new / v_new: [ZHk, D] rows with element stride s_new between units.  Cache strides in bytes
 * per (z,hk) unit: knv rows are D/2 bytes, ksc rows D/16, vnv rows `vnv_row` bytes, vsc rows
 * `vsc_row` bytes.  partial: [ZHk, 16, D] in `dtype`.  ring_k / ring_v may be NULL.
 */
int nvfp4_kv_append(const void* k_new, const void* v_new, int dtype, int64_t s_new, int64_t zhk,
                    int d, int64_t pos, uint8_t* knv, int64_t knv_unit, uint8_t* ksc,
                    int64_t ksc_unit, uint8_t* vnv, int64_t vnv_unit, int64_t vnv_row, uint8_t* vsc,
                    int64_t vsc_unit, int64_t vsc_row, void* partial, void* ring_k, void* ring_v,
                    int64_t ring_cap, nvfp4_stream_t stream);

/*
 * Split-K decode plan for a cache of s_kv keys and zhk (batch x kv-head) units: how many
 * splits the decode kernel will use, keys per split (a multiple of 128) and the scratch bytes it
 * needs.  Replaces the heuristic of `_decode_compute` (flash.py:3255-3266), sized for the
 * device's SM count instead of a fixed 256 programs: the split count minimises
 * waves x (tiles per item + per-item drain).  When it is cheaper still, the plan is the balanced
 * decomposition, reported as *nsplit = 0, *split_kv = 0: every persistent CTA streams an equal
 * share of the unit-major list of 128-key tiles, so a unit may be cut anywhere and its partials
 * are the pieces of the CTAs that touch it (exact combine as for fixed splits).
 */
int nvfp4_decode_plan(int64_t s_kv, int64_t zhk, int d, int sm_count, int* nsplit,
                      int64_t* split_kv, size_t* workspace_bytes);

/*
 * Decode attention of one query token per head against a packed cache, reading the cache in
 * place through its strides.  Replaces `nvfp4_flash_decode_prequant` + `_flash_decode_kernel` +
 * `_flash_decode_combine_kernel` (flash.py:3031-3342) and the LSE recovery of
 * `_decode_prequant_with_lse` (kv_cache.py:32-97).
 *   q        [Z, H, D] high precision (`q_dtype`), s_qz / s_qh element strides; the G = H / Hk
 *            query heads of a kv head are quantised to NVFP4 in the kernel prologue.
 *   knv/ksc  [ZHk, >= s_kv, D/2 | D/16], unit strides in bytes (rows contiguous).
 *   vnv/vsc  [ZHk, D, >= s_pad/2 | s_pad/16], unit and row strides in bytes; s_pad = s_kv rounded
 *            up to 128.  Key groups beyond s_kv must hold zero nibbles (any scale byte).
 *   out      [Z, H, D] in `q_dtype`, contiguous.  lse: [Z, H] fp32 or NULL.
 *   workspace: >= workspace_bytes from nvfp4_decode_plan(nsplit as planned), 16-byte aligned.
 *   nsplit / split_kv: as planned, or any explicit fixed split (nsplit * split_kv covering s_kv);
 *            nsplit = 0 selects the balanced decomposition.
 *   status   device int, written non-zero if a bounded wait expired; may be NULL.
 */
int nvfp4_decode(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh, const uint8_t* knv,
                 int64_t knv_unit, const uint8_t* ksc, int64_t ksc_unit, const uint8_t* vnv,
                 int64_t vnv_unit, int64_t vnv_row, const uint8_t* vsc, int64_t vsc_unit,
                 int64_t vsc_row, int64_t z, int64_t hk, int g, int d, int64_t s_kv, float scaling,
                 void* out, float* lse, void* workspace, size_t workspace_bytes, int nsplit,
                 int64_t split_kv, int* status, nvfp4_stream_t stream);

/*
 * nvfp4_decode for callers that cannot provide scratch memory.  (No counterpart in the
 * reference: its decode allocates its split-K partials with torch on every call.)
 *
 * Who needs it: a host that pre-partitioned the GPU into its own pools and forbids allocation
 * at request time (an inference server with a fixed memory plan, a plugin inside a process
 * whose allocator it must not touch).  The split-K partials live in a 16 MiB array that is part
 * of the library image, so every GPU that loads the library holds those 16 MiB until the
 * process exits.  Arguments are those of nvfp4_decode without the workspace; inputs and
 * outputs are still the caller's.  The call allocates nothing (no cudaMalloc / cudaFree, no
 * allocating library routine).
 *
 *  - Limit: Z*Hk*nsplit*(16*D + 32)*4 bytes must fit in nvfp4_decode_static_capacity()
 *    (16 MiB); larger problems are rejected with a message -- pass a larger split_kv (fewer
 *    splits) or use nvfp4_decode.
 *  - The first call on each device looks up the array's device address (with that device
 *    current); make that first call before any stream capture begins.
 *  - All calls on a device share the one array.  The kernel overwrites every partial it later
 *    reads, so nothing has to be cleared between calls, but two calls whose kernels overlap on
 *    the GPU (different streams) race on it: serialise them.
 */
size_t nvfp4_decode_static_capacity(void);
int nvfp4_decode_static(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh, const uint8_t* knv,
                        int64_t knv_unit, const uint8_t* ksc, int64_t ksc_unit, const uint8_t* vnv,
                        int64_t vnv_unit, int64_t vnv_row, const uint8_t* vsc, int64_t vsc_unit,
                        int64_t vsc_row, int64_t z, int64_t hk, int g, int d, int64_t s_kv,
                        float scaling, void* out, float* lse, int nsplit, int64_t split_kv,
                        int* status, nvfp4_stream_t stream);

/*
 * Hybrid decode in two calls, replacing the torch code of `NVFP4KVCache.hybrid_decode`
 * (kv_cache.py:293-351: FP4 prefix decode, bf16 window attention, log-sum-exp merge).
 *
 * nvfp4_window_partials: exact attention of one query token per head over `count` high-precision
 * ring keys (layout as nvfp4_window_attention), cut into `pieces` key ranges; block (unit, piece)
 * writes its UN-normalised result (sum exp(s - m) v, m, sum exp(s - m)) as split-K partial slot
 * extra_base + unit * pieces + piece of `workspace`, whose layout is that of nvfp4_decode with
 * `total_slots` slots: acc [total_slots][16][d], then m [total_slots][16], then l.
 *
 * nvfp4_decode_hybrid: nvfp4_decode over the FP4 prefix whose final combine also merges `n_extra`
 * such partials per unit (they follow the kernel's own slots: extra_base = own slots, total_slots =
 * own slots + Z*Hk*n_extra; workspace_bytes must cover them).  out / lse are the attention over
 * prefix and window together, written once in the query dtype.
 */
int nvfp4_window_partials(const void* q, int dtype, int64_t s_qz, int64_t s_qh, const void* rk,
                          const void* rv, int64_t z, int64_t hk, int g, int d, int64_t ring_cap,
                          int64_t first_pos, int64_t count, float scaling, int pieces,
                          void* workspace, int64_t total_slots, int64_t extra_base,
                          nvfp4_stream_t stream);
int nvfp4_decode_hybrid(const void* q, int q_dtype, int64_t s_qz, int64_t s_qh, const uint8_t* knv,
                        int64_t knv_unit, const uint8_t* ksc, int64_t ksc_unit, const uint8_t* vnv,
                        int64_t vnv_unit, int64_t vnv_row, const uint8_t* vsc, int64_t vsc_unit,
                        int64_t vsc_row, int64_t z, int64_t hk, int g, int d, int64_t s_kv,
                        float scaling, void* out, float* lse, void* workspace,
                        size_t workspace_bytes, int nsplit, int64_t split_kv, int n_extra,
                        int* status, nvfp4_stream_t stream);

/*
 * Exact merge of two attention results over disjoint key sets from their log-sum-exps:
 * out = (e^{lse1-m} o1 + e^{lse2-m} o2) / (e^{lse1-m} + e^{lse2-m}).  Replaces the torch
 * expressions of NVFP4KVCache.hybrid_decode (kv_cache.py:346-351).  o1,o2,out: [rows, d] in
 * `dtype`; lse1,lse2: [rows] fp32; lse_out [rows] fp32 receives the merged log-sum-exp
 * m + log(e^{lse1-m} + e^{lse2-m}) (rows where both inputs are -inf stay -inf and get a zero
 * output row) or is NULL.
 */
int nvfp4_lse_merge(const void* o1, const float* lse1, const void* o2, const float* lse2,
                    void* out, float* lse_out, int dtype, int64_t rows, int d,
                    nvfp4_stream_t stream);

/*
 * Exact attention of one query token per head over a short high-precision window held in ring
 * buffers (the "recent" side of hybrid decode, kv_cache.py:321-335).  rk/rv: [Z, Hk, ring_cap, D]
 * contiguous in `dtype`; keys are absolute positions [first_pos, first_pos + count) found at slot
 * pos % ring_cap.  out: [Z, H, D] fp32, lse: [Z, H] fp32.
 */
int nvfp4_window_attention(const void* q, int dtype, int64_t s_qz, int64_t s_qh, const void* rk,
                           const void* rv, int64_t z, int64_t hk, int g, int d, int64_t ring_cap,
                           int64_t first_pos, int64_t count, float scaling, float* out, float* lse,
                           nvfp4_stream_t stream);

/*
 * Flash-attention forward over packed operands.  Replaces `_flash_fwd_kernel` and its host
 * drivers `_run_flash_packed` / `nvfp4_flash_attention_packed` (flash.py:739-933, 2560-2766).
 *   qnv/qsc  [Z*H,  s_q,  D/2 | D/16]  contiguous
 *   knv/ksc  [Z*Hk, s_kv, D/2 | D/16]  contiguous
 *   vnv/vsc  [Z*Hk, D, s_pad/2 | s_pad/16] contiguous, s_pad % 128 == 0, s_pad >= s_kv
 *   bias     [Z, s_kv] fp32 additive key bias (may hold -inf) or NULL
 *   seq_id / seq_start: [s_q] int32 per-token sample index / first token of the sample (varlen,
 *            requires Z == 1 and s_q == s_kv) or NULL
 *   out      element strides (so_z, so_h, so_s), unit stride along D, in `out_dtype`
 *            ("zhsd": so_z = H*S*D, so_h = S*D, so_s = D; "zshd": so_z = S*H*D, so_h = D,
 *            so_s = H*D)
 *   lse      [Z*H, s_q] fp32 natural-log LSE or NULL
 *   flags    NVFP4_FWD_CAUSAL: key j visible to query i iff j <= i + (s_kv - s_q)
 *   status   device int, written non-zero if a bounded wait expired; may be NULL.
 */
int nvfp4_fwd(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv, const uint8_t* ksc,
              const uint8_t* vnv, const uint8_t* vsc, const float* bias, const int32_t* seq_id,
              const int32_t* seq_start, void* out, int out_dtype, int64_t so_z, int64_t so_h,
              int64_t so_s, float* lse, int64_t z, int64_t h, int64_t hk, int64_t s_q, int64_t s_kv,
              int64_t s_pad, int d, float scaling, int flags, int* status, nvfp4_stream_t stream);

/*
 * Backward pre-pass over x [nb1, nb2, s, d] (element strides sxb1, sxb2, sxs; unit stride along
 * d): writes either or both of xc [nb1*nb2, s, d] (contiguous bf16 copy) and delta [nb1*nb2, s] =
 * rowsum(x o y) (y has its own strides, same dtype as x); with `amax` (one device float the
 * caller zeroed) also max|x| over the whole tensor by atomic maximum, which the all-FP4 backward
 * turns into its global power-of-two pre-scale of dO.  Replaces the delta part of
 * `_flash_bwd_packprep_kernel` (flash.py:1175-1403).  nb1 * nb2 * s < 2^31 rows.
 */
int nvfp4_bwd_prep(const void* x, int dtype, int64_t sxb1, int64_t sxb2, int64_t sxs, int64_t nb1,
                   int64_t nb2, const void* y, int64_t syb1, int64_t syb2, int64_t sys, int64_t s,
                   int d, void* xc, float* delta, float* amax, nvfp4_stream_t stream);

/*
 * Backward with high-precision gradient GEMMs: dQ, dK, dV of the forward above.  Replaces
 * `_run_bwd_hp` and its kernels `_flash_bwd_dkdv_hp_kernel` / `_flash_bwd_dq_hp_kernel`
 * (flash.py:2008-2399, 3459-3805): S is recomputed from the NVFP4 packs of Q and K, P uses the
 * forward's LSE, dP / dV / dK / dQ are bf16 GEMMs on the exact operands; dK and dV are reduced
 * over the GQA group inside the kernel.  No atomics: results are run-to-run identical.
 *   qnv/qsc, knv/ksc   packs of Q [Z*H, s_q, .] and K [Z*Hk, s_kv, .] along D (as for nvfp4_fwd)
 *   q_bf16, do_bf16 [Z*H, s_q, D];  k_bf16, v_bf16 [Z*Hk, s_kv, D]      contiguous bf16
 *   lse, delta [Z*H, s_q] fp32;  key_bias [Z, s_kv] fp32 additive key bias of the forward or NULL
 *   (flash.py:2098-2100; -inf masks a key);  seq_start / seq_end [s] int32 (packed varlen) or both NULL
 *   dq [Z*H, s_q, D], dk, dv [Z*Hk, s_kv, D] contiguous in `grad_dtype`
 * flags: NVFP4_FWD_CAUSAL.  D is 128 or 256 (256: two 128-wide output halves per tile).
 */
int nvfp4_bwd_hp(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv, const uint8_t* ksc,
                 const void* q_bf16, const void* k_bf16, const void* v_bf16, const void* do_bf16,
                 const float* lse, const float* delta, const float* key_bias,
                 const int32_t* seq_start, const int32_t* seq_end, void* dq, void* dk, void* dv,
                 int grad_dtype, int64_t z,
                 int64_t h, int64_t hk, int64_t s_q, int64_t s_kv, int d, float scaling, int flags,
                 int* status, nvfp4_stream_t stream);

/*
 * Backward with ALL GEMMs in NVFP4 (the "fp4_rownorm" mode).  Replaces `_run_bwd` and its kernels
 * `_flash_bwd_dkdv_kernel` / `_flash_bwd_dq_kernel` (flash.py:1559-1995, 3811-4265); the pre-pass
 * packs (`_flash_bwd_packprep_kernel`, `_flash_bwd_kprep_kernel`, flash.py:1175-1538) are made with
 * nvfp4_bwd_prep (delta, max|dO|), nvfp4_pack_dual (dO with the power-of-two pre-scale) and
 * nvfp4_pack.  S and dP are block-scaled FP4 products of along-D packs; P and dS are packed along
 * the contraction axis inside the kernels and multiplied with the transposed packs.  The
 * reference keeps operand scales in range with a per-row rms factor recomputed every tile
 * (flash.py:184-228); here the factors are constant while a tile accumulates (dO / 2^e globally,
 * P * 2^11, dS * 2^9), so dK / dV / dQ accumulate in tensor memory and dK / dV are reduced over
 * the GQA group in the kernel.  No atomics.
 *   qnv/qsc, knv/ksc     packs of Q [Z*H, s_q, .] and K [Z*Hk, s_kv, .] along D (the forward's)
 *   vdnv/vdsc            V [Z*Hk, s_kv, .] packed along D
 *   donv/dosc            dO / 2^e [Z*H, s_q, .] along D;  dotnv/dotsc its transpose [Z*H, D, sq_pad/2 | /16]
 *   qtnv/qtsc            Q^T [Z*H, D, sq_pad/2 | /16];  ktnv/ktsc  K^T [Z*Hk, D, skv_pad/2 | /16]
 *   lse, delta [Z*H, s_q] fp32 (delta in units of dO);  do_amax: device float, max|dO| (2^e is the
 *   smallest power of two >= it);  key_bias [Z, s_kv] or NULL;  seq_start / seq_end [s] or NULL
 *   dq [Z*H, s_q, D], dk, dv [Z*Hk, s_kv, D] contiguous in `grad_dtype`
 * sq_pad / skv_pad: multiples of 128.  flags: NVFP4_FWD_CAUSAL | NVFP4_BWD_SR_*.  D is 128 or 256.
 * With NVFP4_BWD_MXFP8 (the "fp8_rownorm" mode, flash.py:243-257, 3889-3896) the operands of the three
 * gradient GEMMs are MXFP8 -- e4m3 bytes with one e8m0 scale per 32 (tcgen05.mma kind::mxf8f6f4) --
 * while S and dP stay NVFP4 products of the along-D packs: dotnv [Z*H, D, sq_pad], qtnv [Z*H, D,
 * sq_pad], ktnv [Z*Hk, D, skv_pad] are then byte tensors from nvfp4_pack_mx8_t with scales
 * [.., D, pad/32], and P^T, dS^T, dS are packed as MXFP8 inside the kernels.
 * The NVFP4_BWD_SR_* bits (the "fp4_legacy" mode's knobs, flash.py:161-176, 4102-4256) make the
 * e2m1 convert of that in-kernel pack stochastic (cvt.rs: a value goes to one of its two e2m1
 * neighbours with probability proportional to the distance to the other, so the packed operand is
 * unbiased); the random bits are a counter-based hash of (seed, tensor, row, column), so a launch
 * is reproducible from its seed.  The reference draws philox numbers per tile offset; the streams
 * differ, the distribution of the rounding does not.
 */
int nvfp4_bwd_fp4(const uint8_t* qnv, const uint8_t* qsc, const uint8_t* knv, const uint8_t* ksc,
                  const uint8_t* vdnv, const uint8_t* vdsc, const uint8_t* donv, const uint8_t* dosc,
                  const uint8_t* dotnv, const uint8_t* dotsc, const uint8_t* qtnv,
                  const uint8_t* qtsc, const uint8_t* ktnv, const uint8_t* ktsc, const float* lse,
                  const float* delta, const float* do_amax, const float* key_bias,
                  const int32_t* seq_start, const int32_t* seq_end, void* dq, void* dk, void* dv,
                  int grad_dtype, int64_t z, int64_t h, int64_t hk, int64_t s_q, int64_t s_kv,
                  int64_t sq_pad, int64_t skv_pad, int d, float scaling, int flags, uint32_t seed,
                  int* status, nvfp4_stream_t stream);

/*
 * Measured pipe rates (no counterpart in the reference): launches a resident-operand micro-kernel
 * on every SM -- what = 0: tcgen05.mma kind::mxf4nvf4 M128 N128 K64; 1: kind::f16 (bf16) M128 N128
 * K16; 2: ex2.approx.f32; 3: cvt e2m1x2; 4: fma.f32; 5: ex2 + cvt e2m1x2 pairs; 6: cvt e4m3x2.f32;
 * 7: cvt f16x2.e4m3x2 -- `iters` operations per issuing thread, and
 * stores the work of one launch in *work_per_launch (FLOP for 0/1, thread-instructions for 2-4).
 * The caller times the launch with CUDA events; the result is the roofline denominator benchmarks
 * of this library quote.  `sink` is one device float (never written in practice).
 */
int nvfp4_peak_probe(int what, int iters, double* work_per_launch, float* sink, int* status,
                     nvfp4_stream_t stream);

/*
 * Self-test of the failure-detection path (no counterpart in the reference, whose kernels have no
 * device-side waits): one small kernel waits on a barrier that is never completed, with a budget of
 * `spins` probes, gives up, and writes KSTAT_WAIT_TIMEOUT (0x100) | site to *status exactly as a
 * production kernel would.  Nothing asynchronous is in flight and nothing traps: the kernel ends
 * by itself in well under a millisecond and the context stays usable.
 */
int nvfp4_selftest_wait_timeout(int site, unsigned spins, int* status, nvfp4_stream_t stream);

#ifdef __cplusplus
}
#endif

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#endif /* NVFP4_B200_H_ */
