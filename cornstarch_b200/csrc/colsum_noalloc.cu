// csb_colsum_noalloc: the column sum of csb_colsum with its scratch buffer kept inside the library.
// See no_alloc.h for who needs this and for the rules of use.
#include "no_alloc.h"

#include "host.h"
#include "ptx.cuh"

namespace csb {

// Per-block partial sums: [parts][H] floats, parts <= MAX_PARTS, H <= MAX_H.  One array per device
// that loads the library; shared by every call on that device.
static __device__ __align__(256) float g_colsum_scratch[CSB_COLSUM_NOALLOC_MAX_PARTS * CSB_COLSUM_NOALLOC_MAX_H];

// Each thread owns 8 consecutive columns; blocks stride over the rows and write one partial row each.
// Every slot [blockIdx.x][0..H) is written before the second kernel reads it, so the array never has
// to be cleared between calls.
__global__ void __launch_bounds__(256) colsum_noalloc_partial_kernel(const __nv_bfloat16* __restrict__ x,
                                                                    float* __restrict__ partial, int rows, int H) {
  const int nvec = H / 8;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
      const uint4 u = *reinterpret_cast<const uint4*>(x + static_cast<size_t>(r) * H + c * 8);
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 t = __bfloat1622float2(h[j]);
        acc[2 * j] += t.x;
        acc[2 * j + 1] += t.y;
      }
    }
    float* p = partial + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = acc[j];
  }
}

__global__ void colsum_noalloc_reduce_kernel(const float* __restrict__ partial, void* __restrict__ out, int nparts,
                                             int H, int out_fp32, int accumulate) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= H) return;
  float s = 0.f;
  for (int r = 0; r < nparts; ++r) s += partial[static_cast<size_t>(r) * H + c];
  if (out_fp32) {
    float* o = reinterpret_cast<float*>(out);
    o[c] = accumulate ? o[c] + s : s;
  } else {
    __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
    o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
  }
}

constexpr int MAX_DEVICES = 64;
static float* g_scratch_addr[MAX_DEVICES] = {nullptr};

// Device address of the scratch array on the current device.  In host code the array's name is only a
// stand-in for the symbol, not a device pointer, so it is resolved once per device and cached.
static int scratch_for_current_device(float** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= MAX_DEVICES) return CSB_ERR_BAD_ARG;
  if (g_scratch_addr[dev] == nullptr) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_colsum_scratch);
    if (e != cudaSuccess) {
      fprintf(stderr, "[cornstarch_b200] csb_colsum_noalloc: cudaGetSymbolAddress failed: %s\n", cudaGetErrorString(e));
      return (int)e;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return 0;
}

}  // namespace csb

extern "C" __attribute__((visibility("default"))) int csb_colsum_noalloc(const void* x, void* out, int out_fp32,
                                                                          int accumulate, int rows, int H,
                                                                          void* stream) {
  using namespace csb;
  if (x == nullptr || out == nullptr || rows <= 0 || H <= 0 || (H % 8) != 0) return CSB_ERR_BAD_ARG;
  // x is read with 16-byte loads, out with its element size: a misaligned pointer would fault on the GPU
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return CSB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(out) & (out_fp32 ? 3 : 1)) != 0) return CSB_ERR_BAD_ARG;
  if (H > CSB_COLSUM_NOALLOC_MAX_H) {
    fprintf(stderr,
            "[cornstarch_b200] csb_colsum_noalloc: H=%d exceeds the built-in scratch (max %d columns); "
            "use csb_colsum with a caller-provided buffer instead\n",
            H, CSB_COLSUM_NOALLOC_MAX_H);
    return CSB_ERR_TOO_LARGE;
  }
  float* scratch = nullptr;
  int r = scratch_for_current_device(&scratch);
  if (r) return r;
  int parts = sm_count() * 2;
  if (parts > CSB_COLSUM_NOALLOC_MAX_PARTS) parts = CSB_COLSUM_NOALLOC_MAX_PARTS;
  if (parts > rows) parts = rows;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  colsum_noalloc_partial_kernel<<<parts, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), scratch, rows, H);
  if (int e = launch_result()) return e;
  colsum_noalloc_reduce_kernel<<<(H + 255) / 256, 256, 0, s>>>(scratch, out, parts, H, out_fp32, accumulate);
  return launch_result();
}
