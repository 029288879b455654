// HBM-bound fused elementwise kernels for sm_100a: RoPE, SwiGLU/GeGLU, GELU, fused AdamW,
// gradient norm / clip scale, (vocab-parallel) cross-entropy, embedding + modality merge.
// All use 16-byte vector accesses and fp32 math; none allocates.
//
// They replace the eager PyTorch elementwise ops the reference runs through HF modules
// (apply_rotary_pos_emb, SiLU*up, GELU, masked_scatter merge at
// cornstarch/models/multimodal_language_model/modeling_multimodal_language_model.py:930-936,
// cross-entropy) and torch.optim.Adam(fused=True)
// (examples/distributed/run_vlm_hybrid.py:167-169).
#include "host.h"
#include "ptx.cuh"

namespace csb {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// ------------------------------------------------------------------------------------ RoPE
// In place on the first `n_heads` heads of each token row of a [T][row_stride] buffer (the fused
// q|k|v projection output): rotate-half convention, cos/sin tables fp32 [max_pos][D/2].
// sign = +1 forward, -1 backward (the transpose of a rotation).
__global__ void rope_kernel(__nv_bfloat16* __restrict__ buf, const float* __restrict__ cos_t,
                            const float* __restrict__ sin_t, const int* __restrict__ pos_ids, long T, int S,
                            int row_stride, int n_heads, int D, int rot_dim, float sign, int table_rows) {
  const int half = rot_dim / 2;
  const int vec_per_head = half / 8;
  const long total = T * n_heads * vec_per_head;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int vc = i % vec_per_head;
    const long th = i / vec_per_head;
    const int hd = th % n_heads;
    const long t = th / n_heads;
    const int pos = pos_ids ? pos_ids[t] : static_cast<int>(t % S);
    if (!CSB_IN_BOUNDS(pos, table_rows, BND_ROPE_POS)) continue;
    __nv_bfloat16* p = buf + t * row_stride + hd * D + vc * 8;
    uint4 u1 = *reinterpret_cast<uint4*>(p);
    uint4 u2 = *reinterpret_cast<uint4*>(p + half);
    float x1[8], x2[8], o1[8], o2[8];
    unpack8(u1, x1);
    unpack8(u2, x2);
    const float* c = cos_t + static_cast<size_t>(pos) * half + vc * 8;
    const float* s = sin_t + static_cast<size_t>(pos) * half + vc * 8;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float cs = c[j], sn = sign * s[j];
      o1[j] = x1[j] * cs - x2[j] * sn;
      o2[j] = x2[j] * cs + x1[j] * sn;
    }
    *reinterpret_cast<uint4*>(p) = pack8(o1);
    *reinterpret_cast<uint4*>(p + half) = pack8(o2);
  }
}

// ------------------------------------------------------------------------------------ gated MLP activation
__device__ __forceinline__ float act_fwd(float g, int act) {
  if (act == 0) return g / (1.f + __expf(-g));  // silu
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;  // gelu_tanh
  return 0.5f * g * (1.f + tanhf(k0 * (g + k1 * g * g * g)));
}
__device__ __forceinline__ float act_bwd(float g, int act) {
  if (act == 0) {
    const float sg = 1.f / (1.f + __expf(-g));
    return sg * (1.f + g * (1.f - sg));
  }
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  const float t = tanhf(k0 * (g + k1 * g * g * g));
  return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * k0 * (1.f + 3.f * k1 * g * g);
}

// gu: [T][2I] (gate | up), y: [T][I].   y = act(gate) * up
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ gu, __nv_bfloat16* __restrict__ y, long T, int I,
                               int act) {
  const int vec = I / 8;
  const long total = T * vec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec;
    const int c = (i % vec) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + t * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c), u);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = act_fwd(g[j], act) * u[j];
    *reinterpret_cast<uint4*>(y + t * I + c) = pack8(o);
  }
}
// dgu: [T][2I] <- (dy * up * act'(gate) | dy * act(gate))
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ gu, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dgu, long T, int I, int act) {
  const int vec = I / 8;
  const long total = T * vec;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec;
    const int c = (i % vec) * 8;
    float g[8], u[8], d[8], og[8], ou[8];
    unpack8(*reinterpret_cast<const uint4*>(gu + t * 2 * I + c), g);
    unpack8(*reinterpret_cast<const uint4*>(gu + t * 2 * I + I + c), u);
    unpack8(*reinterpret_cast<const uint4*>(dy + t * I + c), d);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      og[j] = d[j] * u[j] * act_bwd(g[j], act);
      ou[j] = d[j] * act_fwd(g[j], act);
    }
    *reinterpret_cast<uint4*>(dgu + t * 2 * I + c) = pack8(og);
    *reinterpret_cast<uint4*>(dgu + t * 2 * I + I + c) = pack8(ou);
  }
}

// ------------------------------------------------------------------------------------ GELU (plain MLPs)
// kind: 1 = tanh approximation, 2 = erf (exact), 3 = quick_gelu x*sigmoid(1.702x), 4 = silu
__device__ __forceinline__ float gelu_f(float x, int kind) {
  if (kind == 1) return act_fwd(x, 1);
  if (kind == 2) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  if (kind == 3) return x / (1.f + __expf(-1.702f * x));
  return x / (1.f + __expf(-x));
}
__device__ __forceinline__ float gelu_df(float x, int kind) {
  if (kind == 1) return act_bwd(x, 1);
  if (kind == 2) {
    const float cdf = 0.5f * (1.f + erff(x * 0.70710678118654752f));
    const float pdf = 0.3989422804014327f * __expf(-0.5f * x * x);
    return cdf + x * pdf;
  }
  if (kind == 3) {
    const float s = 1.f / (1.f + __expf(-1.702f * x));
    return s + 1.702f * x * s * (1.f - s);
  }
  return act_bwd(x, 0);
}
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long n8, int kind) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float f[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = gelu_f(f[j], kind);
    reinterpret_cast<uint4*>(y)[i] = pack8(o);
  }
}
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, long n8, int kind) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float f[8], d[8], o[8];
    unpack8(reinterpret_cast<const uint4*>(x)[i], f);
    unpack8(reinterpret_cast<const uint4*>(dy)[i], d);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = d[j] * gelu_df(f[j], kind);
    reinterpret_cast<uint4*>(dx)[i] = pack8(o);
  }
}

// ------------------------------------------------------------------------------------ fused AdamW
// One pass over a flat shard: fp32 master/exp_avg/exp_avg_sq, bf16 (or fp32) grads, bf16 params.
// grad_scale (device scalar, optional) carries 1/loss_scale * clip factor; `skip` (device int,
// optional) non-zero turns the whole update into a no-op (inf/nan step under dynamic loss scaling).
constexpr int ADAMW_UNROLL = 4;
// SPLIT: the fp32 master weight is not stored as such.  Its upper half is the bf16 parameter itself (rounded half away
// from zero, so that the remainder always fits), its lower half a signed 16-bit remainder in `master_v` (an int16 array):
// master bits = (bf16 bits << 16) + remainder, exactly.  Same update, 2 bytes per parameter less.
template <typename GradT, bool SPLIT>
__global__ void __launch_bounds__(256)
adamw_kernel(__nv_bfloat16* __restrict__ param, void* __restrict__ master_v, float* __restrict__ m,
             float* __restrict__ v, GradT* __restrict__ grad, long n, float lr, float b1, float b2,
             float eps, float wd, float bc1, float bc2, const float* __restrict__ grad_scale,
             const int* __restrict__ skip, int zero_grad) {
  if (skip && *skip) return;
  float* __restrict__ master = reinterpret_cast<float*>(master_v);
  uint2* __restrict__ resid = reinterpret_cast<uint2*>(master_v);  // 4 x int16 per vector
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float inv_bc1 = 1.f / bc1, inv_bc2 = 1.f / bc2, decay = 1.f - lr * wd;
  const long n4 = n / 4;
  // A CTA works on ADAMW_UNROLL consecutive chunks of blockDim vectors per pass; all loads of a pass are issued before the
  // first use, which is what keeps enough bytes in flight (one vector per thread left HBM at a third of its bandwidth).
  // Every element is read once and written once: streaming (evict-first) accesses keep the L2 out of the way.
  const long pass = (long)blockDim.x * ADAMW_UNROLL;
  for (long base = blockIdx.x * pass; base < n4; base += (long)gridDim.x * pass) {
    float4 w[ADAMW_UNROLL], mm[ADAMW_UNROLL], vv[ADAMW_UNROLL];
    float g[ADAMW_UNROLL][4];
#pragma unroll
    for (int u = 0; u < ADAMW_UNROLL; ++u) {
      const long i = base + u * blockDim.x + threadIdx.x;
      if (i < n4) {
        if constexpr (SPLIT) {
          const uint2 pb = __ldcs(reinterpret_cast<const uint2*>(param) + i);
          const uint2 rb = __ldcs(resid + i);
          const uint32_t hi[4] = {pb.x & 0xffffu, pb.x >> 16, pb.y & 0xffffu, pb.y >> 16};
          const uint32_t lo[4] = {rb.x & 0xffffu, rb.x >> 16, rb.y & 0xffffu, rb.y >> 16};
          float f[4];
#pragma unroll
          for (int j = 0; j < 4; ++j)
            f[j] = __uint_as_float((hi[j] << 16) + static_cast<uint32_t>(static_cast<int32_t>(static_cast<int16_t>(lo[j]))));
          w[u] = make_float4(f[0], f[1], f[2], f[3]);
        } else {
          w[u] = __ldcs(reinterpret_cast<const float4*>(master) + i);
        }
        mm[u] = __ldcs(reinterpret_cast<const float4*>(m) + i);
        vv[u] = __ldcs(reinterpret_cast<const float4*>(v) + i);
        if constexpr (sizeof(GradT) == 4) {
          const float4 gg = __ldcs(reinterpret_cast<const float4*>(grad) + i);
          g[u][0] = gg.x; g[u][1] = gg.y; g[u][2] = gg.z; g[u][3] = gg.w;
        } else {
          uint2 gg = __ldcs(reinterpret_cast<const uint2*>(grad) + i);
          const float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&gg.x));
          const float2 b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&gg.y));
          g[u][0] = a.x; g[u][1] = a.y; g[u][2] = b.x; g[u][3] = b.y;
        }
      }
    }
#pragma unroll
    for (int u = 0; u < ADAMW_UNROLL; ++u) {
      const long i = base + u * blockDim.x + threadIdx.x;
      if (i >= n4) continue;
      float wv[4] = {w[u].x, w[u].y, w[u].z, w[u].w}, mv[4] = {mm[u].x, mm[u].y, mm[u].z, mm[u].w};
      float sv[4] = {vv[u].x, vv[u].y, vv[u].z, vv[u].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float gj = g[u][j] * gs;
        mv[j] = b1 * mv[j] + (1.f - b1) * gj;
        sv[j] = b2 * sv[j] + (1.f - b2) * gj * gj;
        const float denom = sqrtf(sv[j] * inv_bc2) + eps;
        wv[j] = wv[j] * decay - lr * (mv[j] * inv_bc1) / denom;
      }
      __stcs(reinterpret_cast<float4*>(m) + i, make_float4(mv[0], mv[1], mv[2], mv[3]));
      __stcs(reinterpret_cast<float4*>(v) + i, make_float4(sv[0], sv[1], sv[2], sv[3]));
      uint2 o;
      if constexpr (SPLIT) {
        uint32_t hb[4], lb[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t bits = __float_as_uint(wv[j]);
          hb[j] = (bits + 0x8000u) >> 16;  // round half away from zero: the remainder is in [-32768, 32767]
          lb[j] = (bits - (hb[j] << 16)) & 0xffffu;
        }
        o.x = hb[0] | (hb[1] << 16);
        o.y = hb[2] | (hb[3] << 16);
        __stcs(resid + i, make_uint2(lb[0] | (lb[1] << 16), lb[2] | (lb[3] << 16)));
      } else {
        __stcs(reinterpret_cast<float4*>(master) + i, make_float4(wv[0], wv[1], wv[2], wv[3]));
        o.x = pack_bf16x2(wv[0], wv[1]);
        o.y = pack_bf16x2(wv[2], wv[3]);
      }
      reinterpret_cast<uint2*>(param)[i] = o;
      if (zero_grad) {
        if constexpr (sizeof(GradT) == 4) __stcs(reinterpret_cast<float4*>(grad) + i, make_float4(0.f, 0.f, 0.f, 0.f));
        else __stcs(reinterpret_cast<uint2*>(grad) + i, make_uint2(0u, 0u));
      }
    }
  }
}

// sum of squares of a flat gradient buffer -> out[0] (atomic add of per-CTA sums; caller zeroes out).
template <typename GradT>
__global__ void sumsq_kernel(const GradT* __restrict__ g, long n, float* __restrict__ out, float* __restrict__ scratch) {
  float acc = 0.f;
  // 16-byte streaming loads, two per thread and pass (the base pointer is 16-byte aligned: arena slices and torch
  // allocations are); the tail that does not fill a vector is read element-wise
  constexpr int PER = 16 / sizeof(GradT);
  const long nvec = n / PER;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < nvec; i += 2 * stride) {
    uint4 u0 = __ldcs(reinterpret_cast<const uint4*>(g) + i);
    uint4 u1 = make_uint4(0u, 0u, 0u, 0u);
    if (i + stride < nvec) u1 = __ldcs(reinterpret_cast<const uint4*>(g) + i + stride);
    const uint32_t w[8] = {u0.x, u0.y, u0.z, u0.w, u1.x, u1.y, u1.z, u1.w};
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if constexpr (sizeof(GradT) == 4) {
        const float x = __uint_as_float(w[k]);
        acc += x * x;
      } else {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
        acc += f.x * f.x + f.y * f.y;
      }
    }
  }
  for (long i = nvec * PER + blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += stride) {
    float x;
    if constexpr (sizeof(GradT) == 4) x = g[i]; else x = __bfloat162float(g[i]);
    acc += x * x;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  __shared__ float sh[32];
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) sh[w] = acc;
  __syncthreads();
  if (w == 0) {
    float t = (l < (blockDim.x >> 5)) ? sh[l] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    // The block sums are added in block order by whichever block finishes last (scratch[0] is the ticket counter,
    // scratch[1 + b] block b's sum): the result does not depend on the order in which the blocks ran, so data-parallel
    // replicas that hold the same gradients compute the same norm, bit for bit.
    __shared__ bool last;
    if (l == 0) {
      scratch[1 + blockIdx.x] = t;
      __threadfence();
      const unsigned ticket = atomicAdd(reinterpret_cast<unsigned*>(scratch), 1u);
      last = ticket == gridDim.x - 1;
    }
    __syncwarp();
    if (last) {
      __threadfence();
      float tot = 0.f;
      for (unsigned b = l; b < gridDim.x; b += 32) tot += __ldcg(scratch + 1 + b);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
      if (l == 0) {
        *out += tot;  // launches that add into the same `out` are ordered by their stream
        *reinterpret_cast<unsigned*>(scratch) = 0u;
      }
    }
  }
}
// scale_out = inv_loss_scale * min(1, max_norm / (sqrt(sumsq) * inv_loss_scale + 1e-6)); skip = !finite.
// `status` (optional) is the device's bounded-wait status word: when a wait ran out earlier in the step the sums this
// step produced are incomplete, so the update is skipped as well (the host raises at its next status poll).
__global__ void clip_scale_kernel(const float* __restrict__ sumsq, float max_norm, float inv_loss_scale,
                                  float* __restrict__ scale_out, float* __restrict__ norm_out, int* __restrict__ skip,
                                  const int* __restrict__ status) {
  const float norm = sqrtf(*sumsq) * inv_loss_scale;
  float s = inv_loss_scale;
  if (max_norm > 0.f) s *= fminf(1.f, max_norm / (norm + 1e-6f));
  *scale_out = s;
  if (norm_out) *norm_out = norm;
  if (skip) *skip = (isfinite(norm) && (status == nullptr || *status == 0)) ? 0 : 1;
}

// ------------------------------------------------------------------------------------ cross entropy
// Pass 1 (per row): local max, sum of exp(x - max), and the logit at the label if the label falls in
// [vocab_start, vocab_start + V).  Under tensor parallelism the three vectors are all-reduced
// (max; then rescaled sum; sum) across the vocab shards before pass 2.
__global__ void __launch_bounds__(512) ce_stats_kernel(const __nv_bfloat16* __restrict__ logits, long ld,
                                                       const long* __restrict__ labels, int V, int vocab_start,
                                                       float* __restrict__ row_max, float* __restrict__ row_sum,
                                                       float* __restrict__ tgt_logit, long rows) {
  __shared__ float sh_m[16], sh_s[16];
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* x = logits + row * ld;
    float mx = -INFINITY, sm = 0.f;
    const int nvec = V / 8;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + c * 8), f);
      float lm = f[0];
#pragma unroll
      for (int j = 1; j < 8; ++j) lm = fmaxf(lm, f[j]);
      if (lm > mx) {
        sm *= __expf(mx - lm);
        mx = lm;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) sm += __expf(f[j] - mx);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) {
      const float f = __bfloat162float(x[c]);
      if (f > mx) {
        sm *= __expf(mx - f);
        mx = f;
      }
      sm += __expf(f - mx);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float om = __shfl_xor_sync(0xffffffffu, mx, o);
      const float os = __shfl_xor_sync(0xffffffffu, sm, o);
      const float nm = fmaxf(mx, om);
      sm = (nm == -INFINITY) ? 0.f : sm * __expf(mx - nm) + os * __expf(om - nm);
      mx = nm;
    }
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();
    if (l == 0) {
      sh_m[w] = mx;
      sh_s[w] = sm;
    }
    __syncthreads();
    if (w == 0) {
      const int nw = blockDim.x >> 5;
      mx = l < nw ? sh_m[l] : -INFINITY;
      sm = l < nw ? sh_s[l] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float om = __shfl_xor_sync(0xffffffffu, mx, o);
        const float os = __shfl_xor_sync(0xffffffffu, sm, o);
        const float nm = fmaxf(mx, om);
        sm = (nm == -INFINITY) ? 0.f : sm * __expf(mx - nm) + os * __expf(om - nm);
        mx = nm;
      }
      if (l == 0) {
        row_max[row] = mx;
        row_sum[row] = sm;
        const long lab = labels[row] - vocab_start;
        tgt_logit[row] = (lab >= 0 && lab < V) ? __bfloat162float(x[lab]) : 0.f;
      }
    }
  }
}
// Pass 2: loss[row] = log(sum) + max - tgt (0 for ignored rows); logits <- (softmax - onehot) * scale
// in place, where scale = *grad_scale (device scalar, e.g. 1 / number of valid tokens).
__global__ void __launch_bounds__(512) ce_grad_kernel(__nv_bfloat16* __restrict__ logits, long ld,
                                                      const long* __restrict__ labels, int V, int vocab_start,
                                                      const float* __restrict__ row_max,
                                                      const float* __restrict__ row_sum,
                                                      const float* __restrict__ tgt_logit, float* __restrict__ loss,
                                                      const float* __restrict__ grad_scale, long ignore_index,
                                                      long rows) {
  const float gs = grad_scale ? *grad_scale : 1.f;
  for (long row = blockIdx.x; row < rows; row += gridDim.x) {
    __nv_bfloat16* x = logits + row * ld;
    const long label = labels[row];
    const bool ignored = (label == ignore_index);
    const float mx = row_max[row];
    const float inv = 1.f / row_sum[row];
    if (threadIdx.x == 0 && loss) loss[row] = ignored ? 0.f : (logf(row_sum[row]) + mx - tgt_logit[row]);
    const long lab = label - vocab_start;
    const float s = ignored ? 0.f : gs;
    const int nvec = V / 8;
    for (int c = threadIdx.x; c < nvec; c += blockDim.x) {
      float f[8];
      unpack8(*reinterpret_cast<const uint4*>(x + c * 8), f);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float p = __expf(f[j] - mx) * inv;
        if (c * 8 + j == lab) p -= 1.f;
        f[j] = p * s;
      }
      *reinterpret_cast<uint4*>(x + c * 8) = pack8(f);
    }
    for (int c = nvec * 8 + threadIdx.x; c < V; c += blockDim.x) {
      float p = __expf(__bfloat162float(x[c]) - mx) * inv;
      if (c == lab) p -= 1.f;
      x[c] = __float2bfloat16(p * s);
    }
  }
}

// ------------------------------------------------------------------------------------ embedding + modality merge
// out[t] = src[t] >= 0 ? embed[src[t]] : feats[-src[t] - 1]
__global__ void gather_merge_kernel(const __nv_bfloat16* __restrict__ embed, const __nv_bfloat16* __restrict__ feats,
                                    const int* __restrict__ src, __nv_bfloat16* __restrict__ out, long T, int H,
                                    long n_embed, long n_feats) {
  const int vec = H / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < T * vec; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec;
    const int c = (i % vec) * 8;
    const int s = src[t];
    if (s >= 0 ? !CSB_IN_BOUNDS(s, n_embed, BND_EMBED_ROW) : !CSB_IN_BOUNDS(-(long)s - 1, n_feats, BND_FEAT_ROW)) continue;
    const __nv_bfloat16* p = s >= 0 ? embed + static_cast<size_t>(s) * H : feats + static_cast<size_t>(-s - 1) * H;
    *reinterpret_cast<uint4*>(out + t * H + c) = *reinterpret_cast<const uint4*>(p + c);
  }
}
// d_embed[src[t]] += dout[t] (atomics; several tokens may share an id), d_feats[-src-1] = dout[t]
template <typename GradT>
__global__ void scatter_merge_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const int* __restrict__ src,
                                         GradT* __restrict__ d_embed, __nv_bfloat16* __restrict__ d_feats, long T,
                                         int H, long n_embed, long n_feats) {
  const int vec = H / 8;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < T * vec; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec;
    const int c = (i % vec) * 8;
    const int s = src[t];
    if (s >= 0 ? !CSB_IN_BOUNDS(s, n_embed, BND_EMBED_ROW) : !CSB_IN_BOUNDS(-(long)s - 1, n_feats, BND_FEAT_ROW)) continue;
    const uint4 u = *reinterpret_cast<const uint4*>(dout + t * H + c);
    if (s < 0) {
      if (d_feats) *reinterpret_cast<uint4*>(d_feats + static_cast<size_t>(-s - 1) * H + c) = u;
    } else if (d_embed) {
      GradT* p = d_embed + static_cast<size_t>(s) * H + c;
      if constexpr (sizeof(GradT) == 4) {
        float f[8];
        unpack8(u, f);
#pragma unroll
        for (int j = 0; j < 8; ++j) atomicAdd(p + j, f[j]);
      } else {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) atomicAdd(reinterpret_cast<__nv_bfloat162*>(p) + j, h[j]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------ misc
// out[i] = a[i] + b[i]  (bf16; residual adds that are not followed by a norm)
__global__ void add_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                           __nv_bfloat16* __restrict__ out, long n8) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float x[8], y[8];
    unpack8(reinterpret_cast<const uint4*>(a)[i], x);
    unpack8(reinterpret_cast<const uint4*>(b)[i], y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] += y[j];
    reinterpret_cast<uint4*>(out)[i] = pack8(x);
  }
}

}  // namespace csb

using namespace csb;

static inline int ew_grid(long work, int threads) {
  long g = (work + threads - 1) / threads;
  long cap = (long)sm_count() * 16;
  return (int)(g < cap ? (g > 0 ? g : 1) : cap);
}

// table_rows: rows of the cos / sin tables (what positions are checked against in the bounds-checked build).
CSB_API int csb_rope(void* buf, const float* cos_t, const float* sin_t, const int* pos_ids, long T, int S,
                     int row_stride, int n_heads, int D, int rot_dim, float sign, int table_rows, void* stream) {
  if (rot_dim % 16 != 0 || rot_dim > D || (row_stride % 8) || (D % 8)) return CSB_ERR_BAD_ARG;
  if (pos_ids == nullptr && S > table_rows) return CSB_ERR_BAD_ARG;  // implicit positions 0..S-1 must fit the tables
  const long work = T * n_heads * (rot_dim / 16);
  rope_kernel<<<ew_grid(work, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(buf), cos_t, sin_t, pos_ids, T, S, row_stride, n_heads, D, rot_dim, sign, table_rows);
  return launch_result();
}

CSB_API int csb_glu_fwd(const void* gu, void* y, long T, int I, int act, void* stream) {
  if (I % 8) return CSB_ERR_BAD_ARG;
  glu_fwd_kernel<<<ew_grid(T * (I / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<__nv_bfloat16*>(y), T, I, act);
  return launch_result();
}
CSB_API int csb_glu_bwd(const void* gu, const void* dy, void* dgu, long T, int I, int act, void* stream) {
  if (I % 8) return CSB_ERR_BAD_ARG;
  glu_bwd_kernel<<<ew_grid(T * (I / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(gu), reinterpret_cast<const __nv_bfloat16*>(dy),
      reinterpret_cast<__nv_bfloat16*>(dgu), T, I, act);
  return launch_result();
}
CSB_API int csb_act_fwd(const void* x, void* y, long n, int kind, void* stream) {
  if (n % 8) return CSB_ERR_BAD_ARG;
  act_fwd_kernel<<<ew_grid(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<__nv_bfloat16*>(y), n / 8, kind);
  return launch_result();
}
CSB_API int csb_act_bwd(const void* x, const void* dy, void* dx, long n, int kind, void* stream) {
  if (n % 8) return CSB_ERR_BAD_ARG;
  act_bwd_kernel<<<ew_grid(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), reinterpret_cast<const __nv_bfloat16*>(dy),
      reinterpret_cast<__nv_bfloat16*>(dx), n / 8, kind);
  return launch_result();
}
CSB_API int csb_add(const void* a, const void* b, void* out, long n, void* stream) {
  if (n % 8) return CSB_ERR_BAD_ARG;
  add_kernel<<<ew_grid(n / 8, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(a), reinterpret_cast<const __nv_bfloat16*>(b),
      reinterpret_cast<__nv_bfloat16*>(out), n / 8);
  return launch_result();
}

CSB_API int csb_adamw(void* param, float* master, float* m, float* v, void* grad, int grad_fp32, long n, float lr,
                      float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
                      const int* skip, int zero_grad, void* stream) {
  if (n % 4) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = ew_grid(n / 4 / ADAMW_UNROLL + 1, 256);
  if (grad_fp32)
    adamw_kernel<float, false><<<grid, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(param), master, m, v,
                                                    reinterpret_cast<float*>(grad), n, lr, b1, b2, eps, wd, bc1, bc2,
                                                    grad_scale, skip, zero_grad);
  else
    adamw_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(param), master, m, v,
                                                            reinterpret_cast<__nv_bfloat16*>(grad), n, lr, b1, b2, eps,
                                                            wd, bc1, bc2, grad_scale, skip, zero_grad);
  return launch_result();
}
// Same update with the master weight kept as bf16 parameter + int16 remainder (`resid`, n entries, zero when the master
// equals the parameter).
CSB_API int csb_adamw_split(void* param, short* resid, float* m, float* v, void* grad, int grad_fp32, long n, float lr,
                            float b1, float b2, float eps, float wd, float bc1, float bc2, const float* grad_scale,
                            const int* skip, int zero_grad, void* stream) {
  if (n % 4) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = ew_grid(n / 4 / ADAMW_UNROLL + 1, 256);
  if (grad_fp32)
    adamw_kernel<float, true><<<grid, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(param), resid, m, v,
                                                   reinterpret_cast<float*>(grad), n, lr, b1, b2, eps, wd, bc1, bc2,
                                                   grad_scale, skip, zero_grad);
  else
    adamw_kernel<__nv_bfloat16, true><<<grid, 256, 0, s>>>(reinterpret_cast<__nv_bfloat16*>(param), resid, m, v,
                                                           reinterpret_cast<__nv_bfloat16*>(grad), n, lr, b1, b2, eps,
                                                           wd, bc1, bc2, grad_scale, skip, zero_grad);
  return launch_result();
}
// Adds the sum of squares of g[0..n) to *out.  `scratch`: scratch_elems floats of device memory owned by the caller (zero
// before the first call; the kernel leaves its ticket counter at zero again), used by one launch at a time.
CSB_API int csb_sumsq(const void* g, int grad_fp32, long n, float* out, float* scratch, int scratch_elems, void* stream) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (scratch == nullptr || scratch_elems < 2) return CSB_ERR_BAD_ARG;
  int grid = ew_grid(n / 16 + 1, 512);
  if (grid > scratch_elems - 1) grid = scratch_elems - 1;
  if (grad_fp32)
    sumsq_kernel<float><<<grid, 512, 0, s>>>(reinterpret_cast<const float*>(g), n, out, scratch);
  else
    sumsq_kernel<__nv_bfloat16><<<grid, 512, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(g), n, out, scratch);
  return launch_result();
}
CSB_API int csb_clip_scale(const float* sumsq, float max_norm, float inv_loss_scale, float* scale_out,
                           float* norm_out, int* skip, const int* status, void* stream) {
  clip_scale_kernel<<<1, 1, 0, reinterpret_cast<cudaStream_t>(stream)>>>(sumsq, max_norm, inv_loss_scale, scale_out,
                                                                          norm_out, skip, status);
  return launch_result();
}

CSB_API int csb_ce_stats(const void* logits, long ld, const long* labels, int V, int vocab_start, float* row_max,
                         float* row_sum, float* tgt_logit, long rows, void* stream) {
  if (ld % 8) return CSB_ERR_BAD_ARG;
  const int grid = rows < (long)sm_count() * 4 ? (int)rows : sm_count() * 4;
  ce_stats_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(logits), ld, labels, V, vocab_start, row_max, row_sum, tgt_logit, rows);
  return launch_result();
}
CSB_API int csb_ce_grad(void* logits, long ld, const long* labels, int V, int vocab_start, const float* row_max,
                        const float* row_sum, const float* tgt_logit, float* loss, const float* grad_scale,
                        long ignore_index, long rows, void* stream) {
  if (ld % 8) return CSB_ERR_BAD_ARG;
  const int grid = rows < (long)sm_count() * 4 ? (int)rows : sm_count() * 4;
  ce_grad_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(logits), ld, labels, V, vocab_start, row_max, row_sum, tgt_logit, loss,
      grad_scale, ignore_index, rows);
  return launch_result();
}

// n_embed / n_feats: rows of the embedding table and of the feature matrix (what the indices in src are checked against
// in the bounds-checked build).
CSB_API int csb_gather_merge(const void* embed, const void* feats, const int* src, void* out, long T, int H,
                             long n_embed, long n_feats, void* stream) {
  if (H % 8) return CSB_ERR_BAD_ARG;
  gather_merge_kernel<<<ew_grid(T * (H / 8), 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(embed), reinterpret_cast<const __nv_bfloat16*>(feats), src,
      reinterpret_cast<__nv_bfloat16*>(out), T, H, n_embed, n_feats);
  return launch_result();
}
CSB_API int csb_scatter_merge_bwd(const void* dout, const int* src, void* d_embed, int embed_fp32, void* d_feats,
                                  long T, int H, long n_embed, long n_feats, void* stream) {
  if (H % 8) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int grid = ew_grid(T * (H / 8), 256);
  if (embed_fp32)
    scatter_merge_bwd_kernel<float><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dout), src,
                                                         reinterpret_cast<float*>(d_embed),
                                                         reinterpret_cast<__nv_bfloat16*>(d_feats), T, H, n_embed, n_feats);
  else
    scatter_merge_bwd_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(dout), src,
                                                                 reinterpret_cast<__nv_bfloat16*>(d_embed),
                                                                 reinterpret_cast<__nv_bfloat16*>(d_feats), T, H, n_embed, n_feats);
  return launch_result();
}

CSB_BOUNDS_STATUS_GETTER(elementwise)
