// RMSNorm / LayerNorm forward + backward with the residual add fused in (sm_100a, HBM-bound).
//
//   forward :  h = x (+ res);  y = norm(h) * w (+ b);   writes y, (h if res given), per-row stats
//   backward:  dx = dnorm(dy) (+ dres);  dw/db partials per CTA, reduced by a second kernel
//
// One CTA handles rows in a grid-stride loop with the row held in registers (H <= 8192), 16-byte
// vector loads, fp32 math.  Replaces apex FusedRMSNorm/FusedLayerNorm reached through
// cornstarch/shardformer/policies/llama.py:252-275 and the eager HF norms.
#include "host.h"
#include "ptx.cuh"

namespace csb {

constexpr int NORM_THREADS = 256;
constexpr int NORM_MAX_VEC = 4;  // 256 threads * 8 elems * 4 = 8192 max hidden

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum(float v, float* sh) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) sh[w] = v;
  __syncthreads();
  float t = (l < (blockDim.x >> 5)) ? sh[l] : 0.f;
  t = warp_sum(t);
  return t;
}

struct Vec8 {
  float f[8];
};
__device__ __forceinline__ Vec8 load8(const __nv_bfloat16* p) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  Vec8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    v.f[2 * i] = t.x;
    v.f[2 * i + 1] = t.y;
  }
  return v;
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const Vec8& v) {
  uint4 u;
  u.x = pack_bf16x2(v.f[0], v.f[1]);
  u.y = pack_bf16x2(v.f[2], v.f[3]);
  u.z = pack_bf16x2(v.f[4], v.f[5]);
  u.w = pack_bf16x2(v.f[6], v.f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}

// IS_LN: LayerNorm (mean subtraction + bias) else RMSNorm.  w_offset: Gemma-style (1 + w).
template <bool IS_LN>
__global__ void __launch_bounds__(NORM_THREADS)
norm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ b,
                __nv_bfloat16* __restrict__ y, __nv_bfloat16* __restrict__ h_out, float* __restrict__ mean_out,
                float* __restrict__ rstd_out, int rows, int H, float eps, float w_offset) {
  __shared__ float sh[32];
  const int nvec = H / 8;
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    Vec8 v[NORM_MAX_VEC];
    float s = 0.f, ss = 0.f;
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        v[i] = load8(x + base + c * 8);
        if (res) {
          Vec8 r = load8(res + base + c * 8);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i].f[j] += r.f[j];
        }
        if (h_out) {
          // the residual stream is stored in bf16; normalise the rounded value so that the
          // backward (which re-reads h) sees exactly what the forward normalised
          store8(h_out + base + c * 8, v[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) v[i].f[j] = __bfloat162float(__float2bfloat16(v[i].f[j]));
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          s += v[i].f[j];
          ss += v[i].f[j] * v[i].f[j];
        }
      }
    }
    float mean = 0.f;
    if (IS_LN) {
      mean = block_sum(s, sh) / H;
      // two-pass variance on the register-resident row
      float d2 = 0.f;
#pragma unroll
      for (int i = 0; i < NORM_MAX_VEC; ++i) {
        const int c = threadIdx.x + i * NORM_THREADS;
        if (c < nvec) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            float d = v[i].f[j] - mean;
            d2 += d * d;
          }
        }
      }
      ss = d2;
    }
    const float var = block_sum(ss, sh) / H;
    const float rstd = rsqrtf(var + eps);
    if (threadIdx.x == 0) {
      if (IS_LN && mean_out) mean_out[row] = mean;
      rstd_out[row] = rstd;
    }
#pragma unroll
    for (int i = 0; i < NORM_MAX_VEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        Vec8 wv = load8(w + c * 8);
        Vec8 o;
        if (IS_LN && b) {
          Vec8 bv = load8(b + c * 8);
#pragma unroll
          for (int j = 0; j < 8; ++j) o.f[j] = (v[i].f[j] - mean) * rstd * (wv.f[j] + w_offset) + bv.f[j];
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) o.f[j] = (v[i].f[j] - mean) * rstd * (wv.f[j] + w_offset);
        }
        store8(y + base + c * 8, o);
      }
    }
  }
}

__device__ __forceinline__ Vec8 unpack8(const uint4& u) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
  Vec8 v;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    v.f[2 * i] = t.x;
    v.f[2 * i + 1] = t.y;
  }
  return v;
}

// dx = rstd * (g - xhat * mean(g*xhat) [- mean(g)])  with g = dy * w;  dw += dy * xhat;  db += dy
// NVEC = 16-byte vectors per thread (H <= NVEC * 2048).  The raw vectors of the CTA's next row are fetched before the
// current row is reduced, so that loads stay in flight across the block-wide reduction.
template <bool IS_LN, int NVEC>
__global__ void __launch_bounds__(NORM_THREADS)
norm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ h,
                const __nv_bfloat16* __restrict__ w, const float* __restrict__ mean_in,
                const float* __restrict__ rstd_in, const __nv_bfloat16* __restrict__ dres,
                __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial, float* __restrict__ db_partial,
                int rows, int H, float w_offset) {
  __shared__ float sh[32];
  const int nvec = H / 8;
  float dw_acc[NVEC][8];
  float db_acc[NVEC][8];
#pragma unroll
  for (int i = 0; i < NVEC; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      dw_acc[i][j] = 0.f;
      db_acc[i][j] = 0.f;
    }
  Vec8 wv[NVEC];
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      wv[i] = load8(w + c * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) wv[i].f[j] += w_offset;
    }
  }
  uint4 n_dy[NVEC], n_h[NVEC], n_dr[NVEC];
  auto fetch = [&](int row) {
    const size_t base = static_cast<size_t>(row) * H;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        n_dy[i] = __ldcs(reinterpret_cast<const uint4*>(dy + base + c * 8));
        n_h[i] = __ldcs(reinterpret_cast<const uint4*>(h + base + c * 8));
        if (dres) n_dr[i] = __ldcs(reinterpret_cast<const uint4*>(dres + base + c * 8));
      }
    }
  };
  if (blockIdx.x < rows) fetch(blockIdx.x);
  for (int row = blockIdx.x; row < rows; row += gridDim.x) {
    const size_t base = static_cast<size_t>(row) * H;
    uint4 c_dy[NVEC], c_h[NVEC], c_dr[NVEC];
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      c_dy[i] = n_dy[i];
      c_h[i] = n_h[i];
      c_dr[i] = n_dr[i];
    }
    if (row + (int)gridDim.x < rows) fetch(row + gridDim.x);
    const float mean = IS_LN ? mean_in[row] : 0.f;
    const float rstd = rstd_in[row];
    Vec8 g[NVEC], xh[NVEC];
    float s1 = 0.f, s2 = 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        const Vec8 d = unpack8(c_dy[i]);
        const Vec8 hv = unpack8(c_h[i]);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          xh[i].f[j] = (hv.f[j] - mean) * rstd;
          g[i].f[j] = d.f[j] * wv[i].f[j];
          s1 += g[i].f[j] * xh[i].f[j];
          s2 += g[i].f[j];
          dw_acc[i][j] += d.f[j] * xh[i].f[j];
          db_acc[i][j] += d.f[j];
        }
      }
    }
    const float m1 = block_sum(s1, sh) / H;
    const float m2 = IS_LN ? block_sum(s2, sh) / H : 0.f;
#pragma unroll
    for (int i = 0; i < NVEC; ++i) {
      const int c = threadIdx.x + i * NORM_THREADS;
      if (c < nvec) {
        Vec8 o;
#pragma unroll
        for (int j = 0; j < 8; ++j) o.f[j] = rstd * (g[i].f[j] - xh[i].f[j] * m1 - m2);
        if (dres) {
          const Vec8 r = unpack8(c_dr[i]);
#pragma unroll
          for (int j = 0; j < 8; ++j) o.f[j] += r.f[j];
        }
        store8(dx + base + c * 8, o);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < NVEC; ++i) {
    const int c = threadIdx.x + i * NORM_THREADS;
    if (c < nvec) {
      float* pw = dw_partial + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
      for (int j = 0; j < 8; ++j) pw[j] = dw_acc[i][j];
      if (IS_LN && db_partial) {
        float* pb = db_partial + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
        for (int j = 0; j < 8; ++j) pb[j] = db_acc[i][j];
      }
    }
  }
}

// out[c] (+)= sum_r partial[r][c]; out is fp32 (main-grad accumulation) or bf16.
// One CTA = 32 columns x 8 row groups: every warp reads 128 contiguous bytes of a row, the 8 groups are summed in
// shared memory (a column-per-thread loop over all rows left the partial buffer to 16 CTAs).
__global__ void __launch_bounds__(256) reduce_partials_kernel(const float* __restrict__ partial, void* __restrict__ out,
                                                              int nparts, int H, int out_fp32, int accumulate) {
  __shared__ float sh[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < H)
    for (int r = ty; r < nparts; r += 8) s += partial[static_cast<size_t>(r) * H + c];
  sh[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < H) {
#pragma unroll
    for (int k = 1; k < 8; ++k) s += sh[k][tx];
    if (out_fp32) {
      float* o = reinterpret_cast<float*>(out);
      o[c] = accumulate ? o[c] + s : s;
    } else {
      __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
      o[c] = __float2bfloat16(accumulate ? __bfloat162float(o[c]) + s : s);
    }
  }
}

// Column sum of a bf16 matrix [rows][H] (bias gradients): partial per CTA then reduce_partials.
__global__ void __launch_bounds__(256) colsum_partial_kernel(const __nv_bfloat16* __restrict__ x,
                                                            float* __restrict__ partial, int rows, int H) {
  // each thread owns 8 consecutive columns; CTAs stride over rows
  const int nvec = H / 8;
  for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = blockIdx.x; r < rows; r += gridDim.x) {
      Vec8 v = load8(x + static_cast<size_t>(r) * H + c * 8);
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] += v.f[j];
    }
    float* p = partial + static_cast<size_t>(blockIdx.x) * H + c * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = acc[j];
  }
}

}  // namespace csb

using namespace csb;

static int norm_grid(int rows) {
  int g = sm_count() * 4;
  return rows < g ? rows : g;
}

// Number of fp32 rows the caller must provide in the dw/db partial buffers for a given row count.
CSB_API int csb_norm_bwd_parts(int rows) { return norm_grid(rows); }

CSB_API int csb_norm_fwd(int is_layernorm, const void* x, const void* res, const void* w, const void* b, void* y,
                         void* h_out, float* mean, float* rstd, int rows, int H, float eps, float w_offset,
                         void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * 8 * NORM_MAX_VEC || rows <= 0) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  auto X = reinterpret_cast<const __nv_bfloat16*>(x);
  auto R = reinterpret_cast<const __nv_bfloat16*>(res);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto B = reinterpret_cast<const __nv_bfloat16*>(b);
  auto Y = reinterpret_cast<__nv_bfloat16*>(y);
  auto Ho = reinterpret_cast<__nv_bfloat16*>(h_out);
  if (is_layernorm)
    norm_fwd_kernel<true><<<norm_grid(rows), NORM_THREADS, 0, s>>>(X, R, W, B, Y, Ho, mean, rstd, rows, H, eps, w_offset);
  else
    norm_fwd_kernel<false><<<norm_grid(rows), NORM_THREADS, 0, s>>>(X, R, W, B, Y, Ho, mean, rstd, rows, H, eps, w_offset);
  return launch_result();
}

// dw_out/db_out: final gradient tensors (fp32 or bf16 by *_fp32 flag), accumulated into when accumulate=1.
CSB_API int csb_norm_bwd(int is_layernorm, const void* dy, const void* h, const void* w, const float* mean,
                         const float* rstd, const void* dres, void* dx, float* dw_partial, float* db_partial,
                         void* dw_out, void* db_out, int grads_fp32, int accumulate, int rows, int H,
                         float w_offset, void* stream) {
  if (H % 8 != 0 || H > NORM_THREADS * 8 * NORM_MAX_VEC || rows <= 0) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = norm_grid(rows);
  auto DY = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto Hh = reinterpret_cast<const __nv_bfloat16*>(h);
  auto W = reinterpret_cast<const __nv_bfloat16*>(w);
  auto DR = reinterpret_cast<const __nv_bfloat16*>(dres);
  auto DX = reinterpret_cast<__nv_bfloat16*>(dx);
#define CSB_NORM_BWD(LN, NV) \
  norm_bwd_kernel<LN, NV><<<grid, NORM_THREADS, 0, s>>>(DY, Hh, W, mean, rstd, DR, DX, dw_partial, db_partial, rows, H, w_offset)
  const int nv = H <= 2048 ? 1 : (H <= 4096 ? 2 : 4);
  if (is_layernorm) {
    if (nv == 1) CSB_NORM_BWD(true, 1); else if (nv == 2) CSB_NORM_BWD(true, 2); else CSB_NORM_BWD(true, 4);
  } else {
    if (nv == 1) CSB_NORM_BWD(false, 1); else if (nv == 2) CSB_NORM_BWD(false, 2); else CSB_NORM_BWD(false, 4);
  }
#undef CSB_NORM_BWD
  int r = launch_result();
  if (r) return r;
  if (dw_out) reduce_partials_kernel<<<(H + 31) / 32, 256, 0, s>>>(dw_partial, dw_out, grid, H, grads_fp32, accumulate);
  if (is_layernorm && db_out && db_partial)
    reduce_partials_kernel<<<(H + 31) / 32, 256, 0, s>>>(db_partial, db_out, grid, H, grads_fp32, accumulate);
  return launch_result();
}

// Bias gradient: out[H] (+)= column sums of dy[rows][H].  `partial` needs csb_colsum_parts() * H floats.
CSB_API int csb_colsum_parts(int rows) {
  int g = sm_count() * 2;
  return rows < g ? rows : g;
}
CSB_API int csb_colsum(const void* x, float* partial, void* out, int out_fp32, int accumulate, int rows, int H,
                       void* stream) {
  if (H % 8 != 0 || rows <= 0) return CSB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0) return CSB_ERR_BAD_ARG;  // 16-byte loads
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = csb_colsum_parts(rows);
  colsum_partial_kernel<<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(x), partial, rows, H);
  if (int e = launch_result()) return e;
  reduce_partials_kernel<<<(H + 31) / 32, 256, 0, s>>>(partial, out, grid, H, out_fp32, accumulate);
  return launch_result();
}
