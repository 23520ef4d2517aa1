// Host-side helpers shared by the launchers: TMA descriptor creation through
// the driver entry point (no link-time dependency on libcuda), SM count cache.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cudaTypedefs.h>
#include <stdint.h>
#include <stdio.h>

namespace dsb {

inline PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) !=
            cudaSuccess ||
        q != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(ptr);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major matrix: `inner` contiguous elements per
// row, `outer` rows, `ld` elements between rows.  128-byte swizzle, zero fill.
// Requirements (checked): base 16-byte aligned, ld*2 a multiple of 16 bytes,
// box_inner == 64 (one swizzle row).
inline int make_tmap_bf16(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer,
                          uint64_t ld, uint32_t box_inner, uint32_t box_outer) {
  auto enc = tensor_map_encoder();
  if (enc == nullptr) return 1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ((ld * 2) & 15) != 0 || box_inner != 64 ||
      box_outer > 256)
    return 2;
  cuuint64_t dims[2] = {inner, outer};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_inner, box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3;
}

// Output tensor map for the epilogue stagers: a row-major [rows, cols] matrix
// of bf16 (elem_bytes 2) or fp32 (4); box = 128 bytes x 32 rows, 128B swizzle.
inline int make_out_tmap(CUtensorMap* map, void* ptr, uint64_t rows, uint64_t cols, uint64_t ld,
                         int elem_bytes) {
  auto enc = tensor_map_encoder();
  if (enc == nullptr) return 1;
  if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0 || ((ld * elem_bytes) & 15) != 0) return 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), 32};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                   2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : 3;
}

inline int sm_count() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (n <= 0) n = 148;
  }
  return n;
}

}  // namespace dsb
