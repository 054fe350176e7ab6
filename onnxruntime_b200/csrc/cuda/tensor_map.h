// Host helper: build a 2-D TMA descriptor (CUtensorMap) for a row-major matrix
// with a 128-byte-swizzled box.  The driver entry point is looked up through
// the runtime so the library needs no link-time dependency on libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace ortb200 {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_encodeTiled>(ptr);
    }
  }
  return fn;
}

// inner = number of elements along the contiguous dimension, rows = number of rows,
// pitch_bytes = distance between rows (multiple of 16), box = {box_inner, box_rows}.
// box_inner * elem_bytes must be <= 128 for the 128-byte swizzle.
inline int make_tensor_map_2d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                              int64_t inner, int64_t rows, int64_t pitch_bytes, int box_inner, int box_rows,
                              CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch_bytes & 15)) return -2;
  if (box_rows > 256 || box_inner * elem_bytes > 128) return -3;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(pitch_bytes)};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

// 3-D variant: dims {inner, rows, planes}; strides for rows and planes in bytes.
inline int make_tensor_map_3d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                              int64_t inner, int64_t rows, int64_t planes, int64_t row_pitch_bytes,
                              int64_t plane_pitch_bytes, int box_inner, int box_rows,
                              CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_pitch_bytes & 15) || (plane_pitch_bytes & 15)) return -2;
  if (box_rows > 256 || box_inner * elem_bytes > 128) return -3;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(row_pitch_bytes), static_cast<cuuint64_t>(plane_pitch_bytes)};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

// 4-D variant: dims {d0 (contiguous), d1, d2, d3} with byte strides for d1..d3; box {box0, box1, 1, 1}.
inline int make_tensor_map_4d(CUtensorMap* out, const void* base, CUtensorMapDataType dt, int elem_bytes,
                              const int64_t dims_in[4], const int64_t strides_bytes[3], int box0, int box1,
                              CUtensorMapSwizzle swz = CU_TENSOR_MAP_SWIZZLE_128B) {
  PFN_encodeTiled fn = get_encode_fn();
  if (!fn) return -1;
  if (reinterpret_cast<uintptr_t>(base) & 15) return -2;
  for (int i = 0; i < 3; ++i)
    if (strides_bytes[i] & 15) return -2;
  if (box1 > 256 || box0 * elem_bytes > 128) return -3;
  cuuint64_t dims[4], strides[3];
  for (int i = 0; i < 4; ++i) dims[i] = static_cast<cuuint64_t>(dims_in[i]);
  for (int i = 0; i < 3; ++i) strides[i] = static_cast<cuuint64_t>(strides_bytes[i]);
  cuuint32_t box[4] = {static_cast<cuuint32_t>(box0), static_cast<cuuint32_t>(box1), 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = fn(out, dt, 4, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

}  // namespace ortb200
