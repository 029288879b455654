// Micro-benchmark of tcgen05.mma issue: cycles per 128 x N x 16 MMA when one warp issues a long run of them while the
// other eight warps of the thread block are idle or execute dense independent FMAs (what softmax / epilogue warps do).
//
// Two issue forms are compared: a single lane inside a divergent branch (`if (lane == 0)`), and the whole converged warp
// walking the code with one elected lane issuing (umma_f16_w).  Measured on B200: next to busy warps the first form needs
// 104 cycles per MMA whatever N is, the second 67 (N = 128, the rate of the tensor pipe) / 54 (N = 64); with idle
// neighbours both reach the pipe's rate (48.5 / 64.4 / 127.7 cycles for N = 64 / 128 / 256).  This is why every MMA warp
// of this library uses the second form.  `python -m cornstarch_b200.utils.kernel_probe mma_issue` prints the table.
//
// No counterpart in the reference (it has no tensor-core code of its own).
#include "host.h"
#include "ptx.cuh"

namespace csb {

template <int N, bool WHOLE_WARP>
__global__ void __launch_bounds__(320, 1) mma_issue_probe_kernel(long long* out, int reps, int busy_neighbours) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bar;
  __shared__ uint32_t slot;
  __shared__ volatile int stop;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    stop = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 96 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;  // finite operands
  fence_proxy_async_smem();
  if (warp == 1) {
    tmem_alloc(&slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tb = slot;
  if (warp == 0 && (WHOLE_WARP || lane == 0)) {
    const uint32_t idesc = make_idesc_bf16(128, N, 0, 0);
    const uint64_t a_desc = make_desc_kmajor_sw128(smem_u32(smem));          // A: 128 rows x 128 bf16 (two 16 KB chunks)
    const uint64_t b_desc = make_desc_kmajor_sw128(smem_u32(smem + 32768));  // B: up to 256 rows x 128 bf16 (two 32 KB chunks)
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t a_off = static_cast<uint64_t>(((kk >> 2) * 16384 + (kk & 3) * 32) >> 4);
        const uint64_t b_off = static_cast<uint64_t>(((kk >> 2) * 32768 + (kk & 3) * 32) >> 4);
        if (WHOLE_WARP) umma_f16_w(tb, a_desc + a_off, b_desc + b_off, idesc, 1u);
        else umma_f16(tb, a_desc + a_off, b_desc + b_off, idesc, 1u);
      }
    }
    const long long t1 = clock64();
    if (WHOLE_WARP) umma_commit_w(&bar);
    else umma_commit(&bar);
    const bool ok = mbar_wait(&bar, 0);
    const long long t2 = clock64();
    if (lane == 0) {
      out[0] = t1 - t0;  // until the last MMA was accepted
      out[1] = t2 - t0;  // until all of them have retired
      out[2] = ok ? 1 : 0;
      stop = 1;
    }
  } else if (warp >= 2 && busy_neighbours) {
    float a[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) a[i] = threadIdx.x + i;
    int guard = 0;
    while (!stop && guard < 4000000) {  // bounded: ends by itself even if the issuing warp never reports
      ++guard;
#pragma unroll 1
      for (int rr = 0; rr < 16; ++rr) {
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] = fmaf(a[i], 1.0001f, 0.5f);
      }
    }
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc += a[i];
    if (acc == 12345.f) out[3] = 1;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tb, 512);
  }
}

template <int N, bool WW>
static int run_probe(long long* out, int reps, int busy, cudaStream_t s) {
  auto k = mma_issue_probe_kernel<N, WW>;
  cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
  if (e != cudaSuccess) return (int)e;
  k<<<1, 320, 100 * 1024, s>>>(out, reps, busy);
  return launch_result();
}

}  // namespace csb

// out: device long long[4]: cycles until the last of reps * 8 MMAs (128 x tile_n x 16, bf16) was issued, cycles until all
// retired, 1 if the bounded wait succeeded.  whole_warp: 0 = one lane in a divergent branch, 1 = converged warp + elected lane.
CSB_API int csb_mma_issue_probe(int tile_n, int whole_warp, int busy_neighbours, int reps, long long* out, void* stream) {
  using namespace csb;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (reps < 1 || reps > 4096) return CSB_ERR_BAD_ARG;
  switch (tile_n * 2 + (whole_warp ? 1 : 0)) {
    case 64 * 2: return run_probe<64, false>(out, reps, busy_neighbours, s);
    case 64 * 2 + 1: return run_probe<64, true>(out, reps, busy_neighbours, s);
    case 128 * 2: return run_probe<128, false>(out, reps, busy_neighbours, s);
    case 128 * 2 + 1: return run_probe<128, true>(out, reps, busy_neighbours, s);
    case 256 * 2: return run_probe<256, false>(out, reps, busy_neighbours, s);
    case 256 * 2 + 1: return run_probe<256, true>(out, reps, busy_neighbours, s);
    default: return CSB_ERR_BAD_ARG;
  }
}
