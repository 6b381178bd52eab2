// Host-side construction of TMA tensor maps. The driver entry point is resolved at run time
// through the CUDA runtime, so the library links against nothing but cudart.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace ft {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// 2-D row-major tensor [rows][cols] of `elt_bytes`-wide elements with a row pitch of
// `ld_elems` elements; box = [box_rows][box_cols]. Returns 0 on success.
inline int make_tmap_2d(CUtensorMap* tm, const void* base, int elt_bytes, uint64_t rows,
                        uint64_t cols, uint64_t ld_elems, uint32_t box_rows, uint32_t box_cols,
                        CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  CUtensorMapDataType dt = elt_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elt_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_elems * static_cast<uint64_t>(elt_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr,
            "[forgetrain_b200] cuTensorMapEncodeTiled failed (%d): base=%p elt=%d rows=%llu "
            "cols=%llu ld=%llu box=%ux%u\n",
            (int)r, base, elt_bytes, (unsigned long long)rows, (unsigned long long)cols,
            (unsigned long long)ld_elems, box_rows, box_cols);
    return -2;
  }
  return 0;
}

// 3-D tensor [d2][d1][d0] (d0 contiguous) with pitches in elements.
inline int make_tmap_3d(CUtensorMap* tm, const void* base, int elt_bytes, uint64_t d0, uint64_t d1,
                        uint64_t d2, uint64_t ld1_elems, uint64_t ld2_elems, uint32_t b0,
                        uint32_t b1, uint32_t b2, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_tiled();
  if (!fn) return -1;
  CUtensorMapDataType dt = elt_bytes == 2   ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elt_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                            : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {ld1_elems * static_cast<uint64_t>(elt_bytes),
                           ld2_elems * static_cast<uint64_t>(elt_bytes)};
  cuuint32_t box[3] = {b0, b1, b2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[forgetrain_b200] cuTensorMapEncodeTiled(3d) failed (%d)\n", (int)r);
    return -2;
  }
  return 0;
}

}  // namespace ft
