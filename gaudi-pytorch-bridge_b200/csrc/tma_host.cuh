// Host-side construction of TMA tensor maps (cuTensorMapEncodeTiled through the runtime's
// driver entry-point query, so the library does not link against libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "b200q.h"

namespace b200q {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static std::atomic<EncodeTiledFn> fn{nullptr};
  EncodeTiledFn f = fn.load(std::memory_order_acquire);
  if (f) return f;
  void* sym = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
      qres == cudaDriverEntryPointSuccess && sym) {
    f = reinterpret_cast<EncodeTiledFn>(sym);
    fn.store(f, std::memory_order_release);
  }
  return f;
}

// Row-major matrix [rows][inner] of elements of elem_bytes, row stride ld_bytes; box = box_inner x box_rows
// elements.  Out-of-range parts of a box read as zero.
inline int make_tma_map_2d(CUtensorMap* map, const void* base, CUtensorMapDataType dtype, int elem_bytes,
                           int64_t inner, int64_t rows, int64_t ld_bytes, int box_inner, int box_rows,
                           CUtensorMapSwizzle swizzle) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return B200Q_ERR_CUDA;
  (void)elem_bytes;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld_bytes};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, dtype, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? B200Q_OK : B200Q_ERR_CUDA;
}

}  // namespace b200q
