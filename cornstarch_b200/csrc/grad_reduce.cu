// Data-parallel gradient reduction over NVLink peer memory, fused with the averaging scale (and the bf16 cast).
//
// Every rank keeps its flat gradient buffer in peer-mapped memory.  One kernel per rank does a two-shot all-reduce:
// rank r owns the r-th slice of the buffer, PULLS that slice from every peer (plain 16-byte loads through the peer
// mapping), sums in fp32, multiplies by `scale` (1/dp for a mean) and PUSHES the bf16 result into every rank's
// buffer (or only its own: reduce-scatter, which is what ZeRO-1 needs).  Nobody else touches slice r in between, so
// the only synchronisation is "all gradients are complete" before and "all slices were pushed" after, both as
// monotonic counters written with system-scope release stores and awaited with bounded spins.
//
// Replaces the per-parameter `dist.all_reduce(grad); grad.div_(dp)` loop of the reference
// (cornstarch/plugin/multimodal_parallel_plugin/multimodal_parallel_plugin.py:362-384).
#include "host.h"
#include "kv_segments.h"
#include "ptx.cuh"

namespace csb {

struct GradReduceParams {
  __nv_bfloat16* buf[CSB_MAX_SEG];  // every rank's flat gradient buffer (peer-mapped), same length
  int world, rank;
  long n8;              // number of 16-byte vectors in the buffer
  float scale;
  int all_reduce;       // 1: push the result to every rank; 0: keep it in the own buffer only (reduce-scatter)
  const int* ready;     // local int[world]: rank r's counter >= ready_value once its gradients are complete
  int ready_value;
  int* status;
};

__global__ void __launch_bounds__(512) grad_reduce_kernel(const GradReduceParams p) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < p.world && ok; ++r)
      if (r != p.rank && !wait_peer_flag(p.ready + r, p.ready_value)) ok = 0;
    if (!ok) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
    ok_s = ok;
  }
  __syncthreads();
  if (!ok_s) return;
  // slice of this rank: vectors [lo, hi)
  const long per = (p.n8 + p.world - 1) / p.world;
  const long lo = per * p.rank;
  const long hi = lo + per < p.n8 ? lo + per : p.n8;
  for (long i = lo + blockIdx.x * (long)blockDim.x + threadIdx.x; i < hi; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int rr = 0; rr < CSB_MAX_SEG; ++rr) {
      if (rr >= p.world) break;
      const int r = (p.rank + rr) % p.world;  // start with the own copy, spread the peers over the links
      const uint4 u = reinterpret_cast<const uint4*>(p.buf[r])[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0] * p.scale, acc[1] * p.scale);
    o.y = pack_bf16x2(acc[2] * p.scale, acc[3] * p.scale);
    o.z = pack_bf16x2(acc[4] * p.scale, acc[5] * p.scale);
    o.w = pack_bf16x2(acc[6] * p.scale, acc[7] * p.scale);
    if (p.all_reduce) {
#pragma unroll
      for (int rr = 0; rr < CSB_MAX_SEG; ++rr) {
        if (rr >= p.world) break;
        const int r = (p.rank + rr) % p.world;
        reinterpret_cast<uint4*>(p.buf[r])[i] = o;
      }
    } else {
      reinterpret_cast<uint4*>(p.buf[p.rank])[i] = o;
    }
  }
}

}  // namespace csb

using namespace csb;

// bufs: host array of `world` device pointers (entry r = rank r's gradient buffer, peer-mapped; entry `rank` is local);
// n: bf16 elements (multiple of 8).  `ready`: local int[world] counters, awaited until >= ready_value.
CSB_API int csb_grad_reduce(void* const* bufs, int world, int rank, long n, float scale, int all_reduce, const int* ready,
                            int ready_value, int max_ctas, int* status, void* stream) {
  if (world < 1 || world > CSB_MAX_SEG || rank < 0 || rank >= world || (n % 8)) return CSB_ERR_BAD_ARG;
  GradReduceParams p;
  for (int r = 0; r < CSB_MAX_SEG; ++r) p.buf[r] = reinterpret_cast<__nv_bfloat16*>(bufs[r < world ? r : 0]);
  p.world = world; p.rank = rank; p.n8 = n / 8; p.scale = scale; p.all_reduce = all_reduce;
  p.ready = ready; p.ready_value = ready_value; p.status = status;
  const long per = (p.n8 + world - 1) / world;
  long blocks = (per + 511) / 512;
  const long cap = max_ctas > 0 ? max_ctas : (long)sm_count() * 2;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  grad_reduce_kernel<<<(unsigned)blocks, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return launch_result();
}

CSB_WAIT_LIMIT_SETTER(grad_reduce)
