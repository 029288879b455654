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
      else if (now - t0 > CSB_WAIT_NS) return false;
    }
  }
  return false;
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
}

}  // namespace csb
