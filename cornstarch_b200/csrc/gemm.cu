// bf16 GEMM for sm_100a: persistent, warp-specialised, tcgen05.mma with TMEM accumulators,
// operands staged by (non-multicast) TMA with 128-byte swizzle.
//
//   C[M,N] (+)= act( A[M,K] * B[N,K]^T + bias[N] )
//
// Each operand may be "K-major" (row = M/N index, K contiguous) or "MN-major" (row = K index,
// M/N contiguous), so the three GEMMs of a linear layer run without any transpose pass:
//   y  = x  * W^T        A = x  (K-major)    B = W  (K-major)
//   dx = dy * W          A = dy (K-major)    B = W  (MN-major: rows are the contraction index)
//   dW = dy^T * x        A = dy (MN-major)   B = x  (MN-major)
//
// Roles per CTA (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner,
// warps 2..5 = epilogue (TMEM -> registers -> global).  The accumulator is double-buffered in
// TMEM (2 x BN columns) so the epilogue of tile i overlaps the main loop of tile i+1.
//
// This file replaces the cuBLAS calls behind nn.Linear / Linear1D_Col / Linear1D_Row in the
// reference (cornstarch/shardformer/policies/llama.py:192-249).
#include "host.h"
#include "ptx.cuh"

namespace csb {

constexpr int BM = 128;
constexpr int BK = 64;  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

enum Act : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_GELU_ERF = 2, ACT_SILU = 3 };

struct GemmParams {
  void* C;
  const void* bias;  // bf16 [N] or null
  int M, N, K;
  int ldc;
  int out_fp32;
  int accumulate;  // C += result (read-modify-write in the epilogue)
  int act;
  int num_m_blocks, num_n_blocks, num_k_blocks;
  int* status;
  // ---- fused all-reduce through peer memory (ar_world > 1): the epilogue publishes this rank's partial
  // tile in its own staging buffer and raises a per-tile flag on every rank; reducer CTAs of the same
  // launch sum the partial tiles of all ranks (peer loads over NVLink) into C as tiles become ready.
  int ar_world, ar_rank, ar_epoch, n_gemm_ctas, ar_max_tiles;
  __nv_bfloat16* ar_part[8];   // staging buffer [M][N] of every rank (index = rank), peer-mapped
  int* ar_flags[8];            // flag array [world][max_tiles] of every rank, peer-mapped
};

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_OFFSET = STAGES * STAGE_BYTES;
  // full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2], tmem_addr, abort
  static constexpr int TOTAL = BAR_OFFSET + (2 * STAGES + 4) * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;  // slack for 1024-byte alignment
};

__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t phase, volatile int* abort_flag) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
    if (mbar_try_wait(bar, phase)) return true;
    if ((i & 511u) == 511u) {
      if (*abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > CSB_WAIT_NS) return false;
    }
  }
  return false;
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  constexpr int GROUP_M = 8;
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

__device__ __forceinline__ float apply_act(float x, int act) {
  switch (act) {
    case ACT_GELU_TANH: {
      const float k0 = 0.7978845608028654f, k1 = 0.044715f;
      float t = tanhf(k0 * (x + k1 * x * x * x));
      return 0.5f * x * (1.f + t);
    }
    case ACT_GELU_ERF:
      return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case ACT_SILU:
      return x / (1.f + __expf(-x));
    default:
      return x;
  }
}

// Reducer CTAs of a fused GEMM + all-reduce launch: for every output tile (strided over the reducer
// CTAs) wait (bounded) until each rank has raised the tile's flag for this epoch, then add up the
// partial tiles of all ranks, read straight from their staging buffers, and store the sum into C.
template <int BN>
__device__ void ar_reducer(const GemmParams& p, int num_tiles, int rid, int nred) {
  __shared__ int s_ok;
  const int tid = threadIdx.x;
  for (int tile = rid; tile < num_tiles; tile += nred) {
    if (tid == 0) s_ok = 1;
    __syncthreads();
    if (tid < p.ar_world) {
      const int* flag = p.ar_flags[p.ar_rank] + tid * p.ar_max_tiles + tile;
      uint64_t t0 = 0;
      bool seen = false;
      for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
        int v;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (v >= p.ar_epoch) { seen = true; break; }
        if ((i & 255u) == 255u) {
          const uint64_t now = global_timer_ns();
          if (t0 == 0) t0 = now;
          else if (now - t0 > CSB_WAIT_NS) break;
        }
      }
      if (!seen) {
        atomicExch(p.status, ST_TIMEOUT_PEER_FLAG);
        s_ok = 0;
      }
    }
    __syncthreads();
    if (!s_ok) return;  // a peer never delivered: leave the rest of C untouched, the status word says why
    int m_blk, n_blk;
    tile_coords(tile, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
    const int row0 = m_blk * BM, col0 = n_blk * BN;
    const int rows = min(BM, p.M - row0), cols = min(BN, p.N - col0);
    const int vec_per_row = (cols + 7) / 8;
    for (int i = tid; i < rows * vec_per_row; i += blockDim.x) {
      const int r = i / vec_per_row, c = (i % vec_per_row) * 8;
      const size_t off = static_cast<size_t>(row0 + r) * p.N + col0 + c;
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (c + 8 <= cols) {
        for (int src = 0; src < p.ar_world; ++src) {
          const uint4 u = *reinterpret_cast<const uint4*>(p.ar_part[src] + off);
          const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(h[j]);
            acc[2 * j] += f.x;
            acc[2 * j + 1] += f.y;
          }
        }
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row0 + r) * p.ldc + col0 + c;
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        *reinterpret_cast<uint4*>(dst) = o;
      } else {
        for (int j = 0; c + j < cols; ++j) {
          float a = 0.f;
          for (int src = 0; src < p.ar_world; ++src) a += __bfloat162float(p.ar_part[src][off + j]);
          reinterpret_cast<__nv_bfloat16*>(p.C)[static_cast<size_t>(row0 + r) * p.ldc + col0 + c + j] = __float2bfloat16(a);
        }
      }
    }
    __syncthreads();
  }
}

template <int BN, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const GemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + L::STAGES;
  uint64_t* tmem_full = empty_bar + L::STAGES;
  uint64_t* tmem_empty = tmem_full + 2;
  uint32_t* tmem_addr_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_addr_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_blocks * p.num_n_blocks;

  if (p.ar_world > 1 && static_cast<int>(blockIdx.x) >= p.n_gemm_ctas) {
    ar_reducer<BN>(p, num_tiles, blockIdx.x - p.n_gemm_ctas, gridDim.x - p.n_gemm_ctas);
    return;
  }
  const int gemm_ctas = p.ar_world > 1 ? p.n_gemm_ctas : static_cast<int>(gridDim.x);

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_addr_slot, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_addr_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gemm_ctas) {
        int m_blk, n_blk;
        tile_coords(tile, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
        for (int kb = 0; kb < p.num_k_blocks; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!wait_or_abort(&empty_bar[s], ph ^ 1, abort_flag)) {
            atomicExch(p.status, ST_TIMEOUT_EMPTY);
            *abort_flag = 1;
            ok = false;
            break;
          }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (64 * BK * 2), &tma_a, &full_bar[s], m_blk * BM + j * 64, kb * BK);
          } else {
            tma_load_2d(sa, &tma_a, &full_bar[s], kb * BK, m_blk * BM);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (64 * BK * 2), &tma_b, &full_bar[s], n_blk * BN + j * 64, kb * BK);
          } else {
            tma_load_2d(sb, &tma_b, &full_bar[s], kb * BK, n_blk * BN);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gemm_ctas, ++local_tile) {
        const uint32_t acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!wait_or_abort(&tmem_empty[acc], acc_ph ^ 1, abort_flag)) {
          atomicExch(p.status, ST_TIMEOUT_TMEM_EMPTY);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < p.num_k_blocks; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!wait_or_abort(&full_bar[s], ph, abort_flag)) {
            atomicExch(p.status, ST_TIMEOUT_FULL);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          const uint64_t adesc = A_MN ? make_desc_mnmajor_sw128(sa, 64 * BK * 2) : make_desc_kmajor_sw128(sa);
          const uint64_t bdesc = B_MN ? make_desc_mnmajor_sw128(sb, 64 * BK * 2) : make_desc_kmajor_sw128(sb);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 16 elements = 32 bytes along the swizzled row; MN-major: 16 rows of 128 bytes.
            const uint64_t a_adv = A_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : (uint64_t)((k * UMMA_K * 2) >> 4);
            const uint64_t b_adv = B_MN ? (uint64_t)((k * UMMA_K * 128) >> 4) : (uint64_t)((k * UMMA_K * 2) >> 4);
            umma_f16(d_tmem, adesc + a_adv, bdesc + b_adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // smem slot is free once these MMAs retire
        }
        if (ok) umma_commit(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gemm_ctas, ++local_tile) {
      int m_blk, n_blk;
      tile_coords(tile, p.num_m_blocks, p.num_n_blocks, m_blk, n_blk);
      const uint32_t acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      if (!wait_or_abort(&tmem_full[acc], acc_ph, abort_flag)) {
        if (lane == 0) atomicExch(p.status, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      const int row = m_blk * BM + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(quarter * 32) << 16);
      const bool vec_ok = ((p.ar_world > 1 ? p.N : p.ldc) & 7) == 0;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(t_row + c * 32, v);
        tmem_ld_wait();
        const int col0 = n_blk * BN + c * 32;
        if (row < p.M && col0 < p.N) {
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (p.bias) {
            const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (col0 + j < p.N) f[j] += __bfloat162float(b[j]);
          }
          if (p.act != ACT_NONE) {
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = apply_act(f[j], p.act);
          }
          const bool full = (col0 + 32 <= p.N);
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && (p.ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(f[j], f[j + 1], f[j + 2], f[j + 3]);
                if (p.accumulate) {
                  float4 old = *reinterpret_cast<float4*>(dst + j);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = p.accumulate ? dst[j] + f[j] : f[j];
            }
          } else {
            __nv_bfloat16* dst = (p.ar_world > 1)
                                     ? p.ar_part[p.ar_rank] + static_cast<size_t>(row) * p.N + col0
                                     : reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
            if (full && vec_ok) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                if (p.accumulate) {
                  uint4 old = *reinterpret_cast<uint4*>(dst + j);
                  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float2 of = __bfloat1622float2(o2[q]);
                    f[j + 2 * q] += of.x;
                    f[j + 2 * q + 1] += of.y;
                  }
                }
                uint4 o;
                o.x = pack_bf16x2(f[j], f[j + 1]);
                o.y = pack_bf16x2(f[j + 2], f[j + 3]);
                o.z = pack_bf16x2(f[j + 4], f[j + 5]);
                o.w = pack_bf16x2(f[j + 6], f[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < p.N; ++j) {
                float x = f[j];
                if (p.accumulate) x += __bfloat162float(dst[j]);
                dst[j] = __float2bfloat16(x);
              }
            }
          }
        }
      }
      tc_fence_before();
      mbar_arrive(&tmem_empty[acc]);
      if (p.ar_world > 1) {
        // all 128 epilogue threads have written their rows of the partial tile: publish it
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (warp == 2 && lane < p.ar_world) {
          __threadfence_system();
          int* flag = p.ar_flags[lane] + p.ar_rank * p.ar_max_tiles + tile;
          asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(flag), "r"(p.ar_epoch) : "memory");
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool A_MN, bool B_MN>
static int launch_gemm(const void* A, const void* B, const GemmParams& p, int lda, int ldb, int max_ctas,
                       cudaStream_t stream) {
  CUtensorMap ta, tb;
  int r;
  if (A_MN)
    r = make_tmap_2d_bf16(&ta, A, p.K, p.M, lda, 64, BK);
  else
    r = make_tmap_2d_bf16(&ta, A, p.M, p.K, lda, BK, BM);
  if (r) return r;
  if (B_MN)
    r = make_tmap_2d_bf16(&tb, B, p.K, p.N, ldb, 64, BK);
  else
    r = make_tmap_2d_bf16(&tb, B, p.N, p.K, ldb, BK, BN);
  if (r) return r;
  using L = SmemLayout<BN>;
  auto kfn = gemm_bf16_kernel<BN, A_MN, B_MN>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  int tiles = p.num_m_blocks * p.num_n_blocks;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  GemmParams q = p;
  if (q.ar_world > 1) {
    // reducer CTAs ride in the same launch; every CTA must be resident at once (1 CTA per SM)
    int nred = q.n_gemm_ctas > 0 ? q.n_gemm_ctas : 16;  // on entry n_gemm_ctas carries the requested reducer count
    if (nred > sm_count() / 2) nred = sm_count() / 2;
    int ngemm = sm_count() - nred;
    if (ngemm > tiles) ngemm = tiles;
    if (max_ctas > 0 && ngemm > max_ctas) ngemm = max_ctas;
    q.n_gemm_ctas = ngemm;
    grid = ngemm + nred;
  }
  kfn<<<grid, 192, L::DYN_BYTES, stream>>>(ta, tb, q);
  return launch_result();
}

}  // namespace csb

// C[M,N] (+)= act(op(A) * op(B)^T + bias).  a_mn_major=0: A is [M][K] with row stride lda;
// a_mn_major=1: A is [K][M] with row stride lda.  Same for B with N in place of M.
// Leading dimensions are in elements and must be multiples of 8 (16-byte TMA strides).
// `status` is a device int that receives a non-zero code if a bounded wait ran out.
CSB_API int csb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int lda,
                          int ldb, int ldc, int a_mn_major, int b_mn_major, int out_fp32, int accumulate, int act,
                          int tile_n, int max_ctas, int* status, void* stream) {
  using namespace csb;
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7)) return CSB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return CSB_ERR_BAD_ARG;
  int bn = tile_n;
  if (bn != 128 && bn != 256) {
    // 256-wide tiles halve the A re-reads; fall back to 128 when N is small or the tile count is low.
    long t256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    bn = (N >= 256 && t256 >= sm_count()) ? 256 : 128;
  }
  GemmParams p;
  p.C = C;
  p.bias = bias;
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.act = act;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.num_k_blocks = (K + BK - 1) / BK;
  p.status = status;
  p.ar_world = 1; p.ar_rank = 0; p.ar_epoch = 0; p.n_gemm_ctas = 0; p.ar_max_tiles = 0;
  for (int i = 0; i < 8; ++i) { p.ar_part[i] = nullptr; p.ar_flags[i] = nullptr; }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CSB_DISPATCH(BNV)                                                                       \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BNV, false, false>(A, B, p, lda, ldb, max_ctas, s); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BNV, false, true>(A, B, p, lda, ldb, max_ctas, s);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BNV, true, false>(A, B, p, lda, ldb, max_ctas, s);   \
  return launch_gemm<BNV, true, true>(A, B, p, lda, ldb, max_ctas, s);
  if (bn == 256) { CSB_DISPATCH(256) }
  CSB_DISPATCH(128)
#undef CSB_DISPATCH
}


// Fused GEMM + all-reduce across `world` ranks through peer-mapped memory:
//   C = sum over ranks of op(A_rank) * op(B_rank)^T      (bf16 out, every rank ends with the full sum)
// part_ptrs[r]  : staging buffer of rank r (>= M*N bf16), flags_ptrs[r]: int32 [world][max_tiles] of rank r;
// both arrays hold `world` device pointers valid on THIS rank (own buffer + peer mappings).
// epoch must grow by one per call on a given (staging, flags) pair and be the same on all ranks; callers
// alternate between two pairs so that a rank never overwrites a partial tile a slower peer still reads.
CSB_API int csb_gemm_allreduce_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                    int a_mn_major, int b_mn_major, int world, int rank, void* const* part_ptrs,
                                    void* const* flags_ptrs, int max_tiles, int epoch, int n_reducers, int tile_n,
                                    int* status, void* stream) {
  using namespace csb;
  if (M <= 0 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) || (N & 7) || world < 2 || world > 8) return CSB_ERR_BAD_ARG;
  int bn = (tile_n == 128 || tile_n == 256) ? tile_n : ((N >= 256) ? 256 : 128);
  GemmParams p;
  p.C = C; p.bias = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.out_fp32 = 0; p.accumulate = 0; p.act = 0;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.num_k_blocks = (K + BK - 1) / BK;
  if (p.num_m_blocks * p.num_n_blocks > max_tiles) return CSB_ERR_TOO_LARGE;
  p.status = status;
  p.ar_world = world; p.ar_rank = rank; p.ar_epoch = epoch; p.n_gemm_ctas = n_reducers; p.ar_max_tiles = max_tiles;
  for (int i = 0; i < 8; ++i) {
    p.ar_part[i] = i < world ? reinterpret_cast<__nv_bfloat16*>(part_ptrs[i]) : nullptr;
    p.ar_flags[i] = i < world ? reinterpret_cast<int*>(flags_ptrs[i]) : nullptr;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CSB_DISPATCH_AR(BNV)                                                                       \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BNV, false, false>(A, B, p, lda, ldb, 0, s); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BNV, false, true>(A, B, p, lda, ldb, 0, s);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BNV, true, false>(A, B, p, lda, ldb, 0, s);   \
  return launch_gemm<BNV, true, true>(A, B, p, lda, ldb, 0, s);
  if (bn == 256) { CSB_DISPATCH_AR(256) }
  CSB_DISPATCH_AR(128)
#undef CSB_DISPATCH_AR
}
