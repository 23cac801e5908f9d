// Host-side TMA descriptor construction. cuTensorMapEncodeTiled is fetched from the driver at run time
// so that the extension has no link-time dependency on libcuda (it must import on a machine without a GPU).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdexcept>
#include <string>

namespace pfb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres);
    if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !ptr)
      throw std::runtime_error("cuTensorMapEncodeTiled is not available from the CUDA driver");
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// cuTensorMapEncodeTiled needs a current driver context in the calling thread. Threads created by the autograd
// engine may not have one yet; a no-op runtime call binds the device's primary context to the thread.
inline void ensure_context() {
  static thread_local int bound_device = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (bound_device != dev) {
    cudaFree(nullptr);
    bound_device = dev;
  }
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-sized elements; box = [box_rows, box_cols];
// 128-byte swizzle needs box_cols * elem_bytes == 128.
inline CUtensorMap make_tma_2d(const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t rows,
                               uint64_t cols, uint64_t row_stride_elems, uint32_t box_rows, uint32_t box_cols,
                               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  CUtensorMap m;
  ensure_context();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((strides[0] & 15) != 0) throw std::runtime_error("TMA row stride must be a multiple of 16 bytes");
  CUresult r = get_encode_tiled()(&m, dtype, 2, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return m;
}

inline CUtensorMap make_tma_3d(const void* base, CUtensorMapDataType dtype, int elem_bytes, uint64_t d2, uint64_t d1,
                               uint64_t d0, uint64_t stride2_elems, uint64_t stride1_elems, uint32_t box2,
                               uint32_t box1, uint32_t box0,
                               CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_128B) {
  CUtensorMap m;
  ensure_context();
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_elems * static_cast<uint64_t>(elem_bytes),
                           stride2_elems * static_cast<uint64_t>(elem_bytes)};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) throw std::runtime_error("TMA base must be 16-byte aligned");
  if ((strides[0] & 15) != 0 || (strides[1] & 15) != 0)
    throw std::runtime_error("TMA strides must be multiples of 16 bytes");
  CUresult r = get_encode_tiled()(&m, dtype, 3, const_cast<void*>(base), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed with code " + std::to_string(r));
  return m;
}

}  // namespace pfb
