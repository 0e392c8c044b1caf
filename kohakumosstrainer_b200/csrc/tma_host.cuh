// Host helpers to encode TMA tensor maps without linking libcuda: the driver entry point is
// resolved through the runtime once per process.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace kmoss {

typedef CUresult (*TmaEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                     const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                     CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline TmaEncodeTiledFn tma_encode_fn() {
  static TmaEncodeTiledFn fn = []() -> TmaEncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    if (q != cudaDriverEntryPointSuccess) return nullptr;
    return reinterpret_cast<TmaEncodeTiledFn>(ptr);
  }();
  return fn;
}

// The encode call is a driver API and needs the device's primary context current on the
// calling thread; autograd runs backward on threads where no runtime call may have bound it yet.
inline void tma_bind_context() {
  thread_local bool bound = false;
  if (!bound) {
    cudaFree(nullptr);
    bound = true;
  }
}

// Row-major 2-D bf16 matrix [rows, cols], row stride `ld` elements, 128-byte swizzle,
// box = [box_rows, 64 columns]. Out-of-range rows / columns read as zero.
inline bool tma_map_bf16_sw128(CUtensorMap* map, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                               uint32_t box_rows) {
  TmaEncodeTiledFn fn = tma_encode_fn();
  if (fn == nullptr) return false;
  tma_bind_context();
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    fprintf(stderr, "tensor map encode failed (%d): base=%p rows=%llu cols=%llu ld=%llu box_rows=%u\n", (int)r, base,
            (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld, box_rows);
  return r == CUDA_SUCCESS;
}

}  // namespace kmoss
