// Host-side construction of TMA tensor maps.  The driver entry point is resolved at run time so
// the library loads (and exports its symbols) on machines without a CUDA driver.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include "abi.cuh"

namespace nvfp4 {

typedef CUresult (*TensorMapEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                           const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                           const cuuint32_t*, CUtensorMapInterleave,
                                           CUtensorMapSwizzle, CUtensorMapL2promotion,
                                           CUtensorMapFloatOOBfill);

inline TensorMapEncodeTiledFn tensor_map_encoder() {
  static TensorMapEncodeTiledFn fn = []() -> TensorMapEncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess)
      return nullptr;
    return reinterpret_cast<TensorMapEncodeTiledFn>(p);
  }();
  return fn;
}

// Byte tensor [n2][n1][n0] (n0 innermost, contiguous) with byte strides s1, s2 (multiples of 16),
// box [1][b1][b0] with b0 == 64 bytes and the 64-byte shared-memory swizzle; out-of-range
// coordinates read as zero.
inline int make_tmap_u8_3d_sw64(CUtensorMap* m, const void* base, uint64_t n0, uint64_t n1,
                                uint64_t n2, uint64_t s1, uint64_t s2, uint32_t b1,
                                const char* what) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(-1, "%s: cuTensorMapEncodeTiled is unavailable", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 & 15) || (s2 & 15))
    return fail(-1, "%s: base and strides must be 16-byte aligned for TMA", what);
  cuuint64_t dims[3] = {n0, n1, n2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {64, b1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                   es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-1, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return 0;
}

// Map used only for L2 prefetch of wide row segments: the same bytes seen as 32-bit words,
// [n2][n1][n0w] with a box of [1][b1][b0w] words (b0w <= 256, i.e. up to 1 KB per row), no swizzle.
inline int make_tmap_u32_3d_prefetch(CUtensorMap* m, const void* base, uint64_t n0_bytes,
                                     uint64_t n1, uint64_t n2, uint64_t s1, uint64_t s2,
                                     uint32_t b0_words, uint32_t b1, const char* what) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(-1, "%s: cuTensorMapEncodeTiled is unavailable", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 & 15) || (s2 & 15) || (n0_bytes & 3))
    return fail(-1, "%s: base and strides must be 16-byte aligned for TMA", what);
  cuuint64_t dims[3] = {n0_bytes / 4, n1, n2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {b0_words, b1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 3, const_cast<void*>(base), dims, strides, box,
                   es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-1, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return 0;
}

// Byte tensor as make_tmap_u8_3d_sw64, with rows of 128 bytes per box and the 128-byte swizzle.
inline int make_tmap_u8_3d_sw128(CUtensorMap* m, const void* base, uint64_t n0, uint64_t n1,
                                 uint64_t n2, uint64_t s1, uint64_t s2, uint32_t b1,
                                 const char* what) {
  TensorMapEncodeTiledFn enc = tensor_map_encoder();
  if (!enc) return fail(-1, "%s: cuTensorMapEncodeTiled is unavailable", what);
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (s1 & 15) || (s2 & 15))
    return fail(-1, "%s: base and strides must be 16-byte aligned for TMA", what);
  cuuint64_t dims[3] = {n0, n1, n2};
  cuuint64_t strides[2] = {s1, s2};
  cuuint32_t box[3] = {128, b1, 1};
  cuuint32_t es[3] = {1, 1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box,
                   es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(-1, "%s: cuTensorMapEncodeTiled failed with %d", what, (int)r);
  return 0;
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

}  // namespace nvfp4
