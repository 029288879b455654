// Host-side helpers shared by every translation unit of the native library:
// TMA descriptor encoding through the driver entry point (no link-time libcuda dependency),
// launch error reporting, and the C ABI export macro.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define CSB_API extern "C" __attribute__((visibility("default")))

// Error codes returned by the C entry points (negative = host-side refusal, positive = cudaError).
enum : int {
  CSB_ERR_BAD_ARG = -1,
  CSB_ERR_NO_DRIVER_SYMBOL = -2,
  CSB_ERR_TENSORMAP = -3,
  CSB_ERR_TOO_LARGE = -4,
};

namespace csb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult q;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || !p) return nullptr;
  fn = reinterpret_cast<EncodeTiledFn>(p);
  return fn;
}

// Row-major 2-D bf16 tensor [rows][cols] with leading dimension ld (elements); box = box_cols x box_rows,
// 128-byte swizzle (box_cols * 2 bytes must be 128).
inline int make_tmap_2d_bf16(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld,
                             uint32_t box_cols, uint32_t box_rows, CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return CSB_ERR_NO_DRIVER_SYMBOL;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[cornstarch_b200] cuTensorMapEncodeTiled failed: %d (base=%p rows=%llu cols=%llu ld=%llu)\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return CSB_ERR_TENSORMAP;
  }
  return 0;
}

// Row-major 2-D tensor of 2- or 4-byte elements (bf16 / fp32) for epilogue stores: box_cols * elem_bytes must be 128.
inline int make_tmap_2d_out(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, int fp32,
                            uint32_t box_cols, uint32_t box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return CSB_ERR_NO_DRIVER_SYMBOL;
  const uint64_t eb = fp32 ? 4 : 2;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * eb};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, fp32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                  const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[cornstarch_b200] cuTensorMapEncodeTiled(out) failed: %d (base=%p rows=%llu cols=%llu ld=%llu)\n",
            (int)r, base, (unsigned long long)rows, (unsigned long long)cols, (unsigned long long)ld);
    return CSB_ERR_TENSORMAP;
  }
  return 0;
}

// General N-d bf16 tensor map (dims/strides innermost first; strides in BYTES for dims 1..n-1).
inline int make_tmap_nd_bf16(CUtensorMap* out, const void* base, int nd, const uint64_t* dims_in,
                             const uint64_t* strides_bytes, const uint32_t* box_in,
                             CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_128B) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return CSB_ERR_NO_DRIVER_SYMBOL;
  cuuint64_t dims[5];
  cuuint64_t strides[4];
  cuuint32_t box[5];
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < nd; ++i) { dims[i] = dims_in[i]; box[i] = box_in[i]; }
  for (int i = 0; i + 1 < nd; ++i) strides[i] = strides_bytes[i];
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, nd, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[cornstarch_b200] cuTensorMapEncodeTiled(nd=%d) failed: %d\n", nd, (int)r);
    return CSB_ERR_TENSORMAP;
  }
  return 0;
}

// General N-d fp32 tensor map without swizzle (rows of the staged tile are plain row-major in shared memory).
inline int make_tmap_nd_f32(CUtensorMap* out, const void* base, int nd, const uint64_t* dims_in,
                            const uint64_t* strides_bytes, const uint32_t* box_in) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return CSB_ERR_NO_DRIVER_SYMBOL;
  cuuint64_t dims[5];
  cuuint64_t strides[4];
  cuuint32_t box[5];
  cuuint32_t estr[5] = {1, 1, 1, 1, 1};
  for (int i = 0; i < nd; ++i) { dims[i] = dims_in[i]; box[i] = box_in[i]; }
  for (int i = 0; i + 1 < nd; ++i) strides[i] = strides_bytes[i];
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, nd, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "[cornstarch_b200] cuTensorMapEncodeTiled(f32, nd=%d) failed: %d\n", nd, (int)r);
    return CSB_ERR_TENSORMAP;
  }
  return 0;
}

inline int launch_result() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    fprintf(stderr, "[cornstarch_b200] kernel launch failed: %s\n", cudaGetErrorString(e));
    return (int)e;
  }
  return 0;
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

}  // namespace csb
