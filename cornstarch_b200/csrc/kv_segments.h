// K/V given as up to eight segments: the gathered key/value sequence of context parallelism, where segment r is
// rank r's shard and lives in rank r's memory (peer-mapped).  Segments are padded to whole 128-row tiles in the
// gathered index space; bits / positions / tile classes are indexed in that padded space.
#pragma once
#include <cuda.h>
#include <stdint.h>

#include "ptx.cuh"

#define CSB_MAX_SEG 8

// Host-side description (plain C layout, filled by the caller).
struct CsbKvSegments {
  int n_seg;
  int my_seg;             // segment in this GPU's own memory (never waited for); -1 = none
  int rows[CSB_MAX_SEG];  // valid rows per segment
  const void* k[CSB_MAX_SEG];
  const void* v[CSB_MAX_SEG];
  long k_stride_s[CSB_MAX_SEG], k_stride_b[CSB_MAX_SEG], v_stride_s[CSB_MAX_SEG], v_stride_b[CSB_MAX_SEG];
  const int* ready_flags;  // int[n_seg] in local memory: peer r stores its event counter here once its K/V are staged
  int ready_value;         // loads from segment r wait until ready_flags[r] >= ready_value
  // backward: where the dK / dV tiles of segment r go (the owner's inbox slot of this rank)
  void* dk[CSB_MAX_SEG];
  void* dv[CSB_MAX_SEG];
  long dk_stride_s[CSB_MAX_SEG], dk_stride_b[CSB_MAX_SEG], dv_stride_s[CSB_MAX_SEG], dv_stride_b[CSB_MAX_SEG];
  // forward, optional: the first pull_ctas thread blocks of the kernel copy every remote segment's K / V once into
  // this GPU's memory (pull_k[r] / pull_v[r], laid out like k[r] / v[r]) and all query tiles read the local copies,
  // so a remote tile crosses NVLink once instead of once per query tile that needs it.  0 = read k[r] / v[r] directly.
  int pull_ctas;
  void* pull_k[CSB_MAX_SEG];
  void* pull_v[CSB_MAX_SEG];
  long pull_elems[CSB_MAX_SEG];  // bf16 elements to copy per tensor of segment r (a multiple of 8)
  int* pulled;                   // int[n_seg], local: every pulling block adds 1 when it finished segment r
  int pull_target;               // pulled[r] reaches this once segment r is complete for this call
};

namespace csb {

struct KvMaps {
  CUtensorMap k[CSB_MAX_SEG];
  CUtensorMap v[CSB_MAX_SEG];
};

struct SegInfo {
  int n_seg, my_seg;
  int tile_start[CSB_MAX_SEG + 1];  // first gathered tile of each segment; [n_seg] = number of tiles
  int rows[CSB_MAX_SEG];
  const int* ready_flags;
  int ready_value;
  int pull_ctas;
  const uint4* pull_src_k[CSB_MAX_SEG];
  const uint4* pull_src_v[CSB_MAX_SEG];
  uint4* pull_dst_k[CSB_MAX_SEG];
  uint4* pull_dst_v[CSB_MAX_SEG];
  long pull_vecs[CSB_MAX_SEG];
  int* pulled;
  int pull_target;
};

__device__ __forceinline__ int seg_of_tile(const SegInfo& s, int j) {
  int r = 0;
  while (r + 1 < s.n_seg && j >= s.tile_start[r + 1]) ++r;
  return r;
}

// Bounded wait for a peer's "K/V staged" counter (written with a system-scope release store).
__device__ __forceinline__ bool wait_peer_flag(const int* flag, int value) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= value) return true;
    if ((i & 63u) == 63u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_limit_ns()) return false;
    }
  }
  return false;
}

// Bounded wait for a counter that other thread blocks of this GPU advance with a release.
__device__ __forceinline__ bool wait_local_count(const int* counter, int value) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
    if (v >= value) return true;
    if ((i & 63u) == 63u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_limit_ns()) return false;
    }
  }
  return false;
}

// One pulling thread block: copies its share of every remote segment (next rank first) from the peer's staging
// buffer into the local copy and counts the segment as done.  Returns false when a peer's counter never arrived.
__device__ __forceinline__ bool pull_remote_segments(const SegInfo& s, int block, int n_blocks, int* ok_smem) {
  const long stride = (long)n_blocks * blockDim.x;
  for (int d = 1; d < s.n_seg; ++d) {
    const int r = (s.my_seg + d) % s.n_seg;
    if (threadIdx.x == 0) *ok_smem = wait_peer_flag(s.ready_flags + r, s.ready_value) ? 1 : 0;
    __syncthreads();
    const bool ok = *ok_smem != 0;
    __syncthreads();
    if (!ok) return false;
    const long n = s.pull_vecs[r];
#pragma unroll 1
    for (int t = 0; t < 2; ++t) {
      const uint4* __restrict__ src = t ? s.pull_src_v[r] : s.pull_src_k[r];
      uint4* __restrict__ dst = t ? s.pull_dst_v[r] : s.pull_dst_k[r];
      for (long i = (long)block * blockDim.x + threadIdx.x; i < n; i += 4 * stride) {
        uint4 x[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * stride < n) x[u] = __ldcg(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (i + u * stride < n) dst[i + u * stride] = x[u];
      }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(s.pulled + r) : "memory");
  }
  return true;
}

inline void fill_seg_info(SegInfo* s, const CsbKvSegments* g, int tile_rows) {
  s->n_seg = g->n_seg;
  s->my_seg = g->my_seg;
  int t = 0;
  for (int r = 0; r < CSB_MAX_SEG; ++r) {
    s->tile_start[r] = t;
    s->rows[r] = r < g->n_seg ? g->rows[r] : 0;
    if (r < g->n_seg) t += (g->rows[r] + tile_rows - 1) / tile_rows;
  }
  s->tile_start[CSB_MAX_SEG] = t;
  for (int r = g->n_seg; r <= CSB_MAX_SEG; ++r) s->tile_start[r] = t;
  s->ready_flags = g->ready_flags;
  s->ready_value = g->ready_value;
  const bool pull = g->pull_ctas > 0 && g->n_seg > 1 && g->ready_flags != nullptr && g->pulled != nullptr &&
                    g->my_seg >= 0 && g->my_seg < g->n_seg;
  s->pull_ctas = pull ? g->pull_ctas : 0;
  s->pulled = g->pulled;
  s->pull_target = g->pull_target;
  for (int r = 0; r < CSB_MAX_SEG; ++r) {
    const bool on = pull && r < g->n_seg && r != g->my_seg;
    s->pull_src_k[r] = on ? reinterpret_cast<const uint4*>(g->k[r]) : nullptr;
    s->pull_src_v[r] = on ? reinterpret_cast<const uint4*>(g->v[r]) : nullptr;
    s->pull_dst_k[r] = on ? reinterpret_cast<uint4*>(g->pull_k[r]) : nullptr;
    s->pull_dst_v[r] = on ? reinterpret_cast<uint4*>(g->pull_v[r]) : nullptr;
    s->pull_vecs[r] = on ? g->pull_elems[r] / 8 : 0;
  }
}

}  // namespace csb
