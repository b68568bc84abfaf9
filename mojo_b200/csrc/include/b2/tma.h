// Host-side construction of TMA tensor maps without linking libcuda: the encoder is fetched from the
// driver through the runtime (`cudaGetDriverEntryPoint`), so the library loads on machines without a GPU.
#pragma once
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace b2 {

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TensorMapEncodeFn tensor_map_encoder() {
  static TensorMapEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<TensorMapEncodeFn>(p);
  }();
  return fn;
}

// Row-major matrix [rows, cols] with `row_stride_bytes` between rows; box = [box_rows, box_cols].
// Requirements (checked here, because a violation only shows up as a device fault): base 16-byte aligned,
// stride multiple of 16 bytes, box_cols * elem_size multiple of 16 bytes and <= the swizzle span.
inline bool make_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elem_size, const void* base, uint64_t rows,
                         uint64_t cols, uint64_t row_stride_bytes, uint32_t box_rows, uint32_t box_cols,
                         CUtensorMapSwizzle swizzle) {
  auto enc = tensor_map_encoder();
  if (enc == nullptr) return false;
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0 || (row_stride_bytes & 15u) != 0) return false;
  if ((static_cast<uint64_t>(box_cols) * elem_size) % 16 != 0 || box_rows > 256 || box_cols > 256) return false;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

}  // namespace b2
