// Expert-parallel token exchange by direct stores into the peers' memory (dispatch and combine of a MoE layer).
//
// The rows a rank sends are grouped by destination rank; row i of the send order is `src[index[i]]` (dispatch: the
// gather of the tokens by sorted (token, k) pair is fused into the copy) or `src[i]` (combine: expert outputs are
// already contiguous).  Destination d receives them at `dst[d] + (i - seg_start[d]) * H`, where `dst[d]` already points
// at this rank's region inside d's peer-mapped receive buffer (regions are laid out by source rank from the gathered
// count matrix).  16-byte stores, one row per warp pass; nothing waits inside this kernel: ordering is by the event
// counters around it (csb_cp_wait before: the slot is free; csb_cp_signal after: the rows have landed).
//
// The reference has no expert parallelism; this replaces the NCCL all_to_all the baseline path of this package uses.
#include "host.h"
#include "kv_segments.h"
#include "ptx.cuh"

namespace csb {

struct MoePushParams {
  const __nv_bfloat16* src;
  const int* index;  // may be null
  __nv_bfloat16* dst[CSB_MAX_SEG];
  int seg_start[CSB_MAX_SEG + 1];
  int world, H8;  // H8 = row length in 16-byte vectors
  long n_rows;
  long src_rows;  // rows of src (what index[] is checked against in the bounds-checked build)
};

__global__ void __launch_bounds__(256) moe_push_kernel(const MoePushParams p) {
  const int lane = threadIdx.x & 31;
  const long warp = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const long n_warps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long i = warp; i < p.n_rows; i += n_warps) {
    int d = 0;
    while (d + 1 < p.world && i >= p.seg_start[d + 1]) ++d;
    const long srow = p.index ? p.index[i] : i;
    if (!CSB_IN_BOUNDS(srow, p.src_rows, BND_MOE_SRC_ROW)) continue;
    const uint4* s = reinterpret_cast<const uint4*>(p.src) + srow * p.H8;
    uint4* t = reinterpret_cast<uint4*>(p.dst[d]) + (i - p.seg_start[d]) * (long)p.H8;
    for (int c = lane; c < p.H8; c += 32) t[c] = s[c];
  }
}

}  // namespace csb

using namespace csb;

// src: bf16 [*, H]; index: int32[n_rows] or null; seg_start: host int[world + 1] (rows per destination, prefix sums);
// dst: host array of `world` device pointers.  H must be a multiple of 8.
CSB_API int csb_moe_push(const void* src, const int* index, long n_rows, int H, const int* seg_start, void* const* dst,
                         int world, long src_rows, void* stream) {
  if (world < 1 || world > CSB_MAX_SEG || (H % 8)) return CSB_ERR_BAD_ARG;
  if (n_rows <= 0) return 0;
  MoePushParams p;
  p.src = reinterpret_cast<const __nv_bfloat16*>(src);
  p.index = index;
  for (int r = 0; r < CSB_MAX_SEG; ++r) p.dst[r] = reinterpret_cast<__nv_bfloat16*>(dst[r < world ? r : 0]);
  for (int r = 0; r <= CSB_MAX_SEG; ++r) p.seg_start[r] = seg_start[r <= world ? r : world];
  p.world = world; p.H8 = H / 8; p.n_rows = n_rows; p.src_rows = src_rows;
  long blocks = (n_rows + 7) / 8;  // 8 warps per block, one row per warp pass
  const long cap = (long)sm_count() * 8;
  if (blocks > cap) blocks = cap;
  moe_push_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return launch_result();
}

CSB_BOUNDS_STATUS_GETTER(moe_dispatch)
