// Bitfield attention-mask construction on the device: one int64 per token from the token ids.
//
//   modality mode : a placeholder token of modality i carries bit (i + 1); every other token is text and carries the
//                   text bits (bit 0 and bit 62) plus every modality bit; padded positions are 0.
//   instance mode : every contiguous run of placeholder tokens (one image, one audio clip) gets its own bit,
//                   (run index mod 61) + 1, for masks where an instance attends inside itself only; text carries bit 0,
//                   bit 62 and all 61 instance bits.
//
// One thread block per batch row.  The instance mode needs the running count of run starts along the row: an
// inclusive scan per 1024-token chunk (warp shuffles + one shared-memory pass) with the carry kept in a register.
//
// Replaces the chain of torch.where / cumsum launches that builds the same masks on the host side of the reference
// (cornstarch/kernel/interface.py:13-30 and the instance variant used with prefix-causal masks).
#include "host.h"

namespace csb {

constexpr int MB_THREADS = 1024;
constexpr int MB_MAX_IDS = 61;

struct MaskBuildParams {
  const long* ids;         // [B][S]
  const uint8_t* padding;  // [B][S] (nonzero = real token) or null
  long* out;               // [B][S]
  int S;
  int n_ids;
  long token_ids[MB_MAX_IDS];
  int instance_mode;
};

__global__ void __launch_bounds__(MB_THREADS) mask_build_kernel(const MaskBuildParams p) {
  __shared__ int warp_sums[MB_THREADS / 32];
  __shared__ int chunk_total;
  const long row = blockIdx.x;
  const long* ids = p.ids + row * p.S;
  const uint8_t* pad = p.padding ? p.padding + row * p.S : nullptr;
  long* out = p.out + row * p.S;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long text = (1L << 62) | 1L;
  if (p.instance_mode) text |= ((1L << MB_MAX_IDS) - 1L) << 1;
  else
    for (int i = 0; i < p.n_ids; ++i) text |= 1L << (i + 1);
  int carry = 0;  // run starts before this chunk
  for (int base = 0; base < p.S; base += MB_THREADS) {
    const int s = base + threadIdx.x;
    const bool in = s < p.S;
    const long id = in ? ids[s] : -1;
    int which = -1;
    for (int i = 0; i < p.n_ids; ++i)
      if (id == p.token_ids[i]) which = i;
    const bool modal = in && which >= 0;
    long bits;
    if (!p.instance_mode) {
      bits = modal ? (1L << (which + 1)) : text;
    } else {
      // a run starts at a placeholder whose predecessor is not a placeholder of the same id
      const long prev = (s > 0 && in) ? ids[s - 1] : -1;
      const int start = (modal && prev != id) ? 1 : 0;
      int x = start;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (lane == 31) warp_sums[warp] = x;
      __syncthreads();
      if (warp == 0) {
        int w = warp_sums[lane];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, w, o);
          if (lane >= o) w += y;
        }
        warp_sums[lane] = w;
        if (lane == 31) chunk_total = w;
      }
      __syncthreads();
      const int incl = carry + x + (warp > 0 ? warp_sums[warp - 1] : 0);  // run starts up to and including s
      carry += chunk_total;
      __syncthreads();  // warp_sums / chunk_total are rewritten by the next chunk
      bits = modal ? (1L << (((incl - 1) % MB_MAX_IDS) + 1)) : text;
    }
    if (in) out[s] = (pad && pad[s] == 0) ? 0L : bits;
  }
}

}  // namespace csb

using namespace csb;

// ids: int64 [B][S]; token_ids: host array of n_ids placeholder ids (n_ids <= 61); padding: uint8 / bool [B][S] or null;
// out: int64 [B][S].  instance_mode = 0: one bit per modality (order of token_ids); 1: one bit per contiguous run.
CSB_API int csb_bitfield_mask(const long* ids, const long* token_ids, int n_ids, const void* padding, long* out, int B, int S,
                              int instance_mode, void* stream) {
  if (n_ids < 0 || n_ids > MB_MAX_IDS || B <= 0 || S <= 0) return CSB_ERR_BAD_ARG;
  MaskBuildParams p;
  p.ids = ids; p.padding = reinterpret_cast<const uint8_t*>(padding); p.out = out; p.S = S; p.n_ids = n_ids;
  for (int i = 0; i < MB_MAX_IDS; ++i) p.token_ids[i] = i < n_ids ? token_ids[i] : -1;
  p.instance_mode = instance_mode;
  mask_build_kernel<<<B, MB_THREADS, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  return launch_result();
}
