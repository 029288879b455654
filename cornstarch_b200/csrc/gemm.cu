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
#include <stdlib.h>

#include "host.h"
#include "ptx.cuh"

#ifndef CSB_GEMM_DEFAULT_CG
#define CSB_GEMM_DEFAULT_CG 2
#endif

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
  int tma_epi;  // epilogue through shared memory + TMA stores (needs a 16-byte aligned C with 16-byte row pitch)
  // ---- fused all-reduce through peer memory (ar_world > 1).  Tile rows are owned by ranks in contiguous
  // ranges; every rank walks the ranges starting after its own and ends with its own.  For a tile it does
  // not own, the epilogue PUSHES the bf16 partial into its slot of the owner's inbox (posted NVLink
  // stores) and bumps an arrival counter there.  For a tile it owns, the epilogue waits (bounded) for the
  // peers' partials, adds them to its TMEM accumulator in registers, stores the sum into C and pushes it
  // into the `final` buffer of every peer.  No extra CTAs, no extra pass over the local partial.
  int ar_world, ar_rank;
  int ar_base;                 // value of every arrival counter of this context before this call
  long ar_slot_elems;          // elements per inbox slot
  __nv_bfloat16* ar_inbox[8];  // inbox of every rank (peer-mapped): [world slots][M][N]; slot s = partial of rank s
  __nv_bfloat16* ar_final[8];  // final buffer [M][N] of every rank (peer-mapped): rows owned by others land here
  int* ar_cnt_part[8];         // per rank: int32 [world][512 tile rows], bumped by the sender of a partial tile
  int* ar_cnt_final[8];        // per rank: int32 [world][512 tile rows], bumped by the owner after pushing a final tile
  // Reduce-scatter form of the above (ar_scatter = 1): the owner keeps the sum of its rows and nothing is pushed back;
  // C then holds ONLY the owner's rows, stored from row 0 (ar_row_offset = first owned row).
  int ar_scatter;
  int ar_row_offset;
  // ---- fused all-gather of A (ag_world > 1): A is sharded by rows over the ranks (contiguous ranges of 128-row tile
  // rows, range r on rank r, as above).  The first ag_pull_ctas thread blocks copy every shard - the peers' through
  // their peer mappings, once - into the local full-size A that the tensor map covers; the other blocks compute tiles,
  // own rows first, and wait (bounded) for a range's copy before they load its first tile.
  int ag_world, ag_rank, ag_pull_ctas;
  const uint4* ag_src[8];   // shard of every rank (peer-mapped; [rows of range r][K] bf16, row pitch K)
  uint4* ag_dst;            // local full A [M][K], row pitch K
  const int* ag_ready;      // local int[world]: rank r's counter >= ag_ready_value once its shard is staged
  int ag_ready_value;
  int* ag_pulled;           // local int[world]: every pulling block adds 1 per finished range
  int ag_pull_target;       // ag_pulled[r] reaches this once range r is complete for this call
  // ---- grouped form (group_rows > 0): rows [g * group_rows, (g + 1) * group_rows) of A and C belong to group g and are
  // multiplied with that group's own B (the local experts of a MoE layer in ONE launch).  group_rows is a multiple of
  // the tile height, so a tile never straddles two groups; the B tensor maps travel in EpiMaps (see group_b_map).
  int group_rows;
};

constexpr int AR_MAX_ROWS = 512;

__host__ __device__ __forceinline__ int ar_range_start(int range, int num_m, int world) {
  return static_cast<int>((static_cast<long>(range) * num_m) / world);
}
__host__ __device__ __forceinline__ int ar_owner(int m_blk, int num_m, int world) {
  int o = static_cast<int>((static_cast<long>(m_blk) * world) / num_m);
  while (o + 1 < world && ar_range_start(o + 1, num_m, world) <= m_blk) ++o;
  while (o > 0 && ar_range_start(o, num_m, world) > m_blk) --o;
  return o;
}

// CG = CTAs per MMA (tcgen05 cta_group): 1 = every thread block computes its own 128 x BN tile; 2 = a cluster of two
// thread blocks computes one 256 x BN tile: each block stages its own 128 rows of A and HALF of the B tile (BN / 2
// rows), the leader block issues the MMAs, which read both blocks' shared memory and write both blocks' tensor memory.
template <int BN, int CG = 1>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = (BN / CG) * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (CG == 2) ? 6 : ((BN == 256) ? 4 : 6);
  static constexpr int EPI_OFFSET = STAGES * STAGE_BYTES;  // two 16 KB output slabs (128 rows x 128 B, swizzled)
  static constexpr int EPI_SLAB_BYTES = 128 * 128;
  static constexpr int BAR_OFFSET = EPI_OFFSET + 2 * EPI_SLAB_BYTES;
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
      else if (now - t0 > wait_limit_ns()) return false;
    }
  }
  return false;
}

// Tiles are walked in groups of GROUP_M tile rows (all columns of a group before the next group), so that the thread
// blocks running at one time share few rows of A and few columns of B (L2 reuse).  16 rows of 128 measured 2.7 % faster
// than 8 at 8192 x 8192 x 4096 with one thread block per tile; pairs (rows of 256) keep 8.
template <int GROUP_M>
__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_blk, int& n_blk) {
  const int per_group = GROUP_M * num_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gsz = min(num_m - first_m, GROUP_M);
  const int in_group = tile - group * per_group;
  m_blk = first_m + in_group % gsz;
  n_blk = in_group / gsz;
}

// Rotated order for the fused all-reduce: the tile-row index is shifted so that a rank starts with the
// rows owned by the next rank and finishes with its own.
template <int GROUP_M>
__device__ __forceinline__ void tile_coords_rot(int tile, int num_m, int num_n, int rot, int& m_blk, int& n_blk) {
  tile_coords<GROUP_M>(tile, num_m, num_n, m_blk, n_blk);
  m_blk += rot;
  if (m_blk >= num_m) m_blk -= num_m;
}

__device__ __forceinline__ bool spin_until_ge(const int* addr, int target) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    if (v >= target) return true;
    if ((i & 63u) == 63u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_limit_ns()) return false;
    }
  }
  return false;
}

__device__ __forceinline__ bool spin_local_ge(const int* addr, int target) {
  uint64_t t0 = 0;
  for (uint32_t i = 0; i < CSB_SPIN_LIMIT; ++i) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
    if (v >= target) return true;
    if ((i & 63u) == 63u) {
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > wait_limit_ns()) return false;
    }
  }
  return false;
}

// One pulling thread block of the fused all-gather.  One thread moves the block's share of every peer's shard from the
// peer-mapped source into the local full-size A with bulk copies through a ring of shared-memory stages: the loads of
// PULL_STAGES - 1 chunks are in flight while one chunk is written out, so a handful of blocks keep enough bytes on NVLink
// to fill it.  Each finished range is counted.  The tiles of the own rows read the own shard in place; the caller copies
// that shard into the full A (a local copy, outside this kernel).
constexpr int PULL_CHUNK = 16384;
constexpr int PULL_STAGES = 8;
__device__ __forceinline__ bool ag_pull(const GemmParams& p, int block, int n_blocks, uint8_t* stage_smem) {
  __shared__ uint64_t pull_bar[PULL_STAGES];
  if (threadIdx.x != 0) return true;
  for (int s = 0; s < PULL_STAGES; ++s) mbar_init(&pull_bar[s], 1);
  mbar_fence_init();
  const long row_bytes = (long)p.K * 2;
  uint32_t used = 0;  // chunks that went through the ring so far (stage = used % PULL_STAGES, phase from used / PULL_STAGES)
  for (int d = 1; d < p.ag_world; ++d) {
    const int r = (p.ag_rank + d) % p.ag_world;
    if (!spin_until_ge(p.ag_ready + r, p.ag_ready_value)) return false;
    const long row0 = (long)ar_range_start(r, p.num_m_blocks, p.ag_world) * BM;
    long row1 = (long)ar_range_start(r + 1, p.num_m_blocks, p.ag_world) * BM;
    if (row1 > p.M) row1 = p.M;
    const long n = (row1 - row0) * row_bytes;
    const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ag_src[r]);
    uint8_t* dst = reinterpret_cast<uint8_t*>(p.ag_dst) + row0 * row_bytes;
    const long n_chunks = (n + PULL_CHUNK - 1) / PULL_CHUNK;
    const long mine = block < n_chunks ? (n_chunks - block + n_blocks - 1) / n_blocks : 0;  // chunks block, block + n_blocks, ...
    auto chunk_bytes = [&](long j) -> uint32_t {
      const long off = (block + j * n_blocks) * (long)PULL_CHUNK;
      return (uint32_t)(n - off < PULL_CHUNK ? n - off : PULL_CHUNK);
    };
    auto load = [&](long j) {
      const uint32_t st = (used + (uint32_t)j) % PULL_STAGES;
      const long off = (block + j * n_blocks) * (long)PULL_CHUNK;
      mbar_expect_tx(&pull_bar[st], chunk_bytes(j));
      bulk_load_g2s(stage_smem + st * PULL_CHUNK, src + off, chunk_bytes(j), &pull_bar[st]);
    };
    for (long j = 0; j < mine && j < PULL_STAGES - 1; ++j) load(j);
    for (long j = 0; j < mine; ++j) {
      const uint32_t u = used + (uint32_t)j;
      if (!mbar_wait(&pull_bar[u % PULL_STAGES], (u / PULL_STAGES) & 1)) {
        tma_store_wait<0>();
        return false;
      }
      const long off = (block + j * n_blocks) * (long)PULL_CHUNK;
      bulk_store_s2g(dst + off, stage_smem + (u % PULL_STAGES) * PULL_CHUNK, chunk_bytes(j));
      tma_store_commit();
      // the stage that the next load overwrites was read by the store before this one
      tma_store_wait_read<1>();
      if (j + PULL_STAGES - 1 < mine) load(j + PULL_STAGES - 1);
    }
    used += (uint32_t)mine;
    tma_store_wait<0>();  // the writes of this range are complete
    __threadfence();
    asm volatile("red.release.gpu.global.add.s32 [%0], 1;" ::"l"(p.ag_pulled + r) : "memory");
  }
  return true;
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

// Tensor maps of the output side: C itself and, for the fused all-reduce, this rank's slot in every
// rank's inbox and every rank's final buffer (128-byte swizzled boxes of 128 rows x 128 bytes).
struct EpiMaps {
  CUtensorMap a_own;  // fused all-gather: this rank's own shard of A, read in place by the tiles of the own rows
  CUtensorMap c;
  CUtensorMap inbox[8];
  CUtensorMap fin[8];
};

// The grouped form never runs together with the fused all-reduce, so its per-group B maps use the sixteen slots of the
// all-reduce maps: the kernel's parameter block keeps its size.
constexpr int MAX_GROUPS = 16;
__host__ __device__ __forceinline__ const CUtensorMap* group_b_map(const EpiMaps& m, int g) {
  return g < 8 ? &m.inbox[g] : &m.fin[g - 8];
}

// Epilogue of one tile through shared memory: every thread owns one accumulator row; 128-byte row pieces
// (64 bf16 or 32 fp32 columns) are staged in a swizzled slab and written with ONE TMA store per slab and
// destination, so global and NVLink writes are full 128-byte lines.  `accumulate` uses the TMA reduce-add.
// Arrive on an accumulator-drained barrier: the block's own, or (second block of a pair) the leader's.
__device__ __forceinline__ void arrive_tmem_empty(uint64_t* bar, bool remote_leader) {
  if (remote_leader) mbar_arrive_cluster(bar, 0);
  else mbar_arrive(bar);
}

template <int BN, int EPI_OFF_BYTES_SLAB = 128 * 128>
__device__ __forceinline__ void epilogue_tile_tma(const GemmParams& p, const EpiMaps& maps, uint8_t* epi_smem,
                                                  uint32_t t_row, int m_blk, int n_blk, int quarter, int lane, int warp,
                                                  uint32_t& slab_ctr, uint64_t* tmem_empty_bar, bool ar, int owner,
                                                  bool mine, bool remote_leader = false) {
  const int r = quarter * 32 + lane;
  const int row = m_blk * BM + r;
  const bool e0 = (warp == 2 && lane == 0);
  const int cps = p.out_fp32 ? 32 : 64;  // columns per 128-byte slab row
  const int n_slabs = BN / cps;
  for (int s = 0; s < n_slabs; ++s, ++slab_ctr) {
    const int col0 = n_blk * BN + s * cps;
    const bool last = (s == n_slabs - 1) || (col0 + cps >= p.N);
    float f[64];
    {
      uint32_t v[32];
      tmem_ld_32x32(t_row + s * cps, v);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
      if (cps == 64) {
        tmem_ld_32x32(t_row + s * cps + 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) f[32 + j] = __uint_as_float(v[j]);
      }
    }
    if (last) {
      tc_fence_before();
      arrive_tmem_empty(tmem_empty_bar, remote_leader);  // the accumulator buffer can be overwritten by the next tile's MMAs
    }
    if (p.bias) {
      const __nv_bfloat16* b = reinterpret_cast<const __nv_bfloat16*>(p.bias) + col0;
#pragma unroll
      for (int j = 0; j < 64; ++j)
        if (j < cps && col0 + j < p.N) f[j] += __bfloat162float(b[j]);
    }
    if (p.act != ACT_NONE) {
#pragma unroll
      for (int j = 0; j < 64; ++j)
        if (j < cps) f[j] = apply_act(f[j], p.act);
    }
    if (mine) {
      // bf16-round my partial like the peers', then add theirs (they sit in my own inbox: local reads)
#pragma unroll
      for (int j = 0; j < 64; ++j) f[j] = __bfloat162float(__float2bfloat16(f[j]));
      if (row < p.M) {
        const size_t off = static_cast<size_t>(row) * p.N + col0;
        for (int src = 0; src < p.ar_world; ++src) {
          if (src == p.ar_rank) continue;
          const __nv_bfloat16* in = p.ar_inbox[p.ar_rank] + static_cast<size_t>(src) * p.ar_slot_elems + off;
          if (col0 + 64 <= p.N) {
#pragma unroll
            for (int j = 0; j < 64; j += 8) {
              const uint4 u = *reinterpret_cast<const uint4*>(in + j);
              const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                f[j + 2 * q] += __uint_as_float(w[q] << 16);
                f[j + 2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u);
              }
            }
          } else {
            for (int j = 0; j < 64 && col0 + j < p.N; ++j) f[j] += __bfloat162float(in[j]);
          }
        }
      }
    }
    uint8_t* buf = epi_smem + (slab_ctr & 1) * EPI_OFF_BYTES_SLAB;
    if (e0) tma_store_wait_read<1>();  // the store that last used this slab has finished reading it
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (p.out_fp32) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint4 u = make_uint4(__float_as_uint(f[4 * j]), __float_as_uint(f[4 * j + 1]), __float_as_uint(f[4 * j + 2]),
                                   __float_as_uint(f[4 * j + 3]));
        *reinterpret_cast<uint4*>(buf + sw128_offset(r, j)) = u;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        uint4 u;
        u.x = pack_bf16x2(f[8 * j + 0], f[8 * j + 1]);
        u.y = pack_bf16x2(f[8 * j + 2], f[8 * j + 3]);
        u.z = pack_bf16x2(f[8 * j + 4], f[8 * j + 5]);
        u.w = pack_bf16x2(f[8 * j + 6], f[8 * j + 7]);
        *reinterpret_cast<uint4*>(buf + sw128_offset(r, j)) = u;
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 2, 128;" ::: "memory");
    if (e0) {
      const int y = m_blk * BM;
      if (!ar) {
        if (p.accumulate) tma_reduce_add_2d(&maps.c, buf, col0, y);
        else tma_store_2d(&maps.c, buf, col0, y);
      } else if (!mine) {
        tma_store_2d(&maps.inbox[owner], buf, col0, y);
      } else if (p.ar_scatter) {
        tma_store_2d(&maps.c, buf, col0, y - p.ar_row_offset);  // C holds the owned rows only
      } else {
        tma_store_2d(&maps.c, buf, col0, y);
        for (int d = 0; d < p.ar_world; ++d)
          if (d != p.ar_rank) tma_store_2d(&maps.fin[d], buf, col0, y);
      }
      tma_store_commit();
    }
    if (last) {
      slab_ctr += 1;
      break;
    }
  }
  if (ar && e0) {
    // the tile's stores must have landed before the tile is counted on the receiving side
    tma_store_wait<0>();
    asm volatile("fence.proxy.async;" ::: "memory");
    __threadfence_system();
    if (!mine) {
      int* cnt = p.ar_cnt_part[owner] + p.ar_rank * AR_MAX_ROWS + m_blk;
      asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
    } else if (!p.ar_scatter) {
      for (int d = 0; d < p.ar_world; ++d) {
        if (d == p.ar_rank) continue;
        int* cnt = p.ar_cnt_final[d] + p.ar_rank * AR_MAX_ROWS + m_blk;
        asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int CG>
__global__ void __launch_bounds__(192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tma_a, const __grid_constant__ CUtensorMap tma_b,
                 const __grid_constant__ EpiMaps epi_maps, const GemmParams p) {
  using L = SmemLayout<BN, CG>;
  constexpr int BNH = BN / CG;  // rows of B this thread block stages
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
  // The grid is one-dimensional so that thread blocks start in index order: the pulling blocks of a fused all-gather
  // come first and are resident before any block that waits for their counters.
  const int n_pull = p.ag_world > 1 ? p.ag_pull_ctas : 0;  // CG == 2: an even number, so that a pair pulls or works as one
  if ((int)blockIdx.x < n_pull) {
    if (!ag_pull(p, blockIdx.x, n_pull, smem)) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
    return;
  }
  // A pair of thread blocks (CG == 2) walks the tiles together: `unit` rows of 128 * CG; block `cta_rank` of the pair
  // owns rows [cta_rank * 128, +128) of a tile and rows [cta_rank * BNH, +BNH) of the B tile.
  const int cta_rank = CG == 2 ? (int)cluster_ctarank() : 0;
  const bool leader = cta_rank == 0;
  const int num_m_units = (p.num_m_blocks + CG - 1) / CG;
  const int num_tiles = num_m_units * p.num_n_blocks;
  const int work_first = ((int)blockIdx.x - n_pull) / CG;
  const int work_step = ((int)gridDim.x - n_pull) / CG;
  // tile rows are walked in rotated order: fused all-reduce / reduce-scatter - the rows of the next rank first, the own
  // last; fused all-gather - the own rows (already local) first
  // (CG == 2: the host picks pairs only when every range starts on an even tile row, so a pair never straddles two)
  const int rot = (p.ar_world > 1 ? ar_range_start((p.ar_rank + 1) % p.ar_world, p.num_m_blocks, p.ar_world)
                                  : (p.ag_world > 1 ? ar_range_start(p.ag_rank, p.num_m_blocks, p.ag_world) : 0)) / CG;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 128 * CG);  // CG == 2: the epilogue threads of both blocks arrive on the leader's barrier
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tma_a);
    tma_prefetch_desc(&tma_b);
  }
  if (warp == 1) {
    if constexpr (CG == 2) {
      tmem_alloc_2cta(tmem_addr_slot, 2 * BN);  // the same warp of both blocks: the columns are allocated in both
      tmem_relinquish_2cta();
    } else {
      tmem_alloc(tmem_addr_slot, 2 * BN);
      tmem_relinquish();
    }
  }
  tc_fence_before();
  if constexpr (CG == 2) cluster_sync_all();  // the peer's barriers are initialised before anything signals them
  else __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_addr_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t ag_opened = 0;
      bool ok = true;
      // CG == 2: both blocks' loads report their bytes to the LEADER's barrier (its address in the cluster window is
      // this block's address with the pair bit cleared); only the leader announces the expected byte count
      constexpr uint32_t LEADER_MASK = CG == 2 ? 0xFEFFFFFFu : 0xFFFFFFFFu;
      for (int tile = work_first; tile < num_tiles && ok; tile += work_step) {
        int m_blk, n_blk;
        tile_coords_rot<(CG == 2 ? 8 : 16)>(tile, num_m_units, p.num_n_blocks, rot, m_blk, n_blk);
        m_blk = m_blk * CG + cta_rank;
        const int n_row0 = n_blk * BN + cta_rank * BNH;
        const CUtensorMap* map_a = &tma_a;
        int a_row0 = m_blk * BM;
        const CUtensorMap* map_b = p.group_rows > 0 ? group_b_map(epi_maps, a_row0 / p.group_rows) : &tma_b;
        if (n_pull > 0) {
          const int o = ar_owner(m_blk, p.num_m_blocks, p.ag_world);
          if (o == p.ag_rank) {
            // own rows: read from the shard in place (the full A receives them last, for the caller)
            map_a = &epi_maps.a_own;
            a_row0 -= ar_range_start(o, p.num_m_blocks, p.ag_world) * BM;
          } else if (!((ag_opened >> o) & 1u)) {
            // first tile of a peer's range: its rows must have been copied into the local A (bounded wait on the pull
            // counter); the copy was written by other blocks, the loads below go through the async proxy
            if (!spin_local_ge(p.ag_pulled + o, p.ag_pull_target)) {
              atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
              *abort_flag = 1;
              ok = false;
              break;
            }
            asm volatile("fence.proxy.async.global;" ::: "memory");
            ag_opened |= 1u << o;
          }
        }
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
          const uint32_t full_addr_s = smem_u32(&full_bar[s]) & LEADER_MASK;
          if (leader) mbar_expect_tx(&full_bar[s], L::STAGE_BYTES * CG);
          if constexpr (A_MN) {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d_to<CG>(sa + j * (64 * BK * 2), map_a, full_addr_s, a_row0 + j * 64, kb * BK);
          } else {
            tma_load_2d_to<CG>(sa, map_a, full_addr_s, kb * BK, a_row0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int j = 0; j < BNH / 64; ++j)
              tma_load_2d_to<CG>(sb + j * (64 * BK * 2), map_b, full_addr_s, n_row0 + j * 64, kb * BK);
          } else {
            tma_load_2d_to<CG>(sb, map_b, full_addr_s, kb * BK, n_row0);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // the whole warp walks this code in step; one elected lane issues each MMA and commit (see umma_f16_w)
    if (leader) {
      constexpr uint32_t idesc = make_idesc_bf16(BM * CG, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0;
      uint32_t local_tile = 0;
      bool ok = true;
      for (int tile = work_first; tile < num_tiles && ok; tile += work_step, ++local_tile) {
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
            if constexpr (CG == 2) umma_f16_2cta_w(d_tmem, adesc + a_adv, bdesc + b_adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            else umma_f16_w(d_tmem, adesc + a_adv, bdesc + b_adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit_cg_w<CG>(&empty_bar[s]);  // smem slot (of both blocks) is free once these MMAs retire
        }
        if (ok) umma_commit_cg_w<CG>(&tmem_full[acc]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ epilogue warps (2..5)
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    uint32_t local_tile = 0;
    uint32_t slab_ctr = 0;
    bool ok = true;
    for (int tile = work_first; tile < num_tiles && ok; tile += work_step, ++local_tile) {
      int m_blk, n_blk;
      tile_coords_rot<(CG == 2 ? 8 : 16)>(tile, num_m_units, p.num_n_blocks, rot, m_blk, n_blk);
      m_blk = m_blk * CG + cta_rank;
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
      const bool vec_ok = (p.ldc & 7) == 0;
      const bool ar = p.ar_world > 1;
      const int owner = ar ? ar_owner(m_blk, p.num_m_blocks, p.ar_world) : 0;
      const bool mine = ar && owner == p.ar_rank;
      if (p.tma_epi) {
        if (mine) {
          bool arrived = true;
          if (lane < p.ar_world && lane != p.ar_rank)
            arrived = spin_until_ge(p.ar_cnt_part[p.ar_rank] + lane * AR_MAX_ROWS + m_blk, p.ar_base + p.num_n_blocks);
          if (!__all_sync(0xffffffffu, arrived) && lane == 0) atomicExch(p.status, ST_TIMEOUT_PEER_FLAG);
        }
        epilogue_tile_tma<BN, L::EPI_SLAB_BYTES>(p, epi_maps, smem + L::EPI_OFFSET, t_row, m_blk, n_blk, quarter, lane, warp, slab_ctr,
                                                 &tmem_empty[acc], ar, owner, mine, !leader);
        continue;
      }
      if (mine) {
        // the peers computed my rows first; by now their partials normally sit in my inbox already
        bool arrived = true;
        if (lane < p.ar_world && lane != p.ar_rank)
          arrived = spin_until_ge(p.ar_cnt_part[p.ar_rank] + lane * AR_MAX_ROWS + m_blk, p.ar_base + p.num_n_blocks);
        if (!__all_sync(0xffffffffu, arrived)) {
          if (lane == 0) atomicExch(p.status, ST_TIMEOUT_PEER_FLAG);  // the sum below is then incomplete; the host sees the status
        }
      }
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
          if (ar) {
            const size_t off = static_cast<size_t>(row) * p.N + col0;
            if (!mine) {
              // partial tile -> my slot of the owner's inbox
              __nv_bfloat16* dst = p.ar_inbox[owner] + static_cast<size_t>(p.ar_rank) * p.ar_slot_elems + off;
              if (full) {
#pragma unroll
                for (int j = 0; j < 32; j += 8) {
                  uint4 o;
                  o.x = pack_bf16x2(f[j], f[j + 1]);
                  o.y = pack_bf16x2(f[j + 2], f[j + 3]);
                  o.z = pack_bf16x2(f[j + 4], f[j + 5]);
                  o.w = pack_bf16x2(f[j + 6], f[j + 7]);
                  *reinterpret_cast<uint4*>(dst + j) = o;
                }
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) dst[j] = __float2bfloat16(f[j]);
              }
            } else {
              // my own partial is rounded to bf16 like the peers' so that the sum does not depend on who owns the row
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = __bfloat162float(__float2bfloat16(f[j]));
              for (int src = 0; src < p.ar_world; ++src) {
                if (src == p.ar_rank) continue;
                const __nv_bfloat16* in = p.ar_inbox[p.ar_rank] + static_cast<size_t>(src) * p.ar_slot_elems + off;
                if (full) {
#pragma unroll
                  for (int j = 0; j < 32; j += 8) {
                    const uint4 u = *reinterpret_cast<const uint4*>(in + j);
                    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                      f[j + 2 * q] += __uint_as_float(w[q] << 16);
                      f[j + 2 * q + 1] += __uint_as_float(w[q] & 0xffff0000u);
                    }
                  }
                } else {
                  for (int j = 0; j < 32 && col0 + j < p.N; ++j) f[j] += __bfloat162float(in[j]);
                }
              }
              // final values: into my C and into every peer's `final` buffer
              uint4 o[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                o[j].x = pack_bf16x2(f[8 * j + 0], f[8 * j + 1]);
                o[j].y = pack_bf16x2(f[8 * j + 2], f[8 * j + 3]);
                o[j].z = pack_bf16x2(f[8 * j + 4], f[8 * j + 5]);
                o[j].w = pack_bf16x2(f[8 * j + 6], f[8 * j + 7]);
              }
              __nv_bfloat16* cdst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
              if (full && vec_ok) {
#pragma unroll
                for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(cdst + 8 * j) = o[j];
              } else {
                for (int j = 0; j < 32 && col0 + j < p.N; ++j) cdst[j] = __float2bfloat16(f[j]);
              }
              for (int d = 0; d < p.ar_world; ++d) {
                if (d == p.ar_rank) continue;
                __nv_bfloat16* fdst = p.ar_final[d] + off;
                if (full) {
#pragma unroll
                  for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(fdst + 8 * j) = o[j];
                } else {
                  for (int j = 0; j < 32 && col0 + j < p.N; ++j) fdst[j] = __float2bfloat16(f[j]);
                }
              }
            }
          } else if (p.out_fp32) {
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
            __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<size_t>(row) * p.ldc + col0;
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
      arrive_tmem_empty(&tmem_empty[acc], !leader);
      if (ar) {
        // all 128 epilogue threads have issued their stores for this tile: make them visible, then count the tile
        asm volatile("bar.sync 2, 128;" ::: "memory");
        if (warp == 2) {
          if (!mine && lane == 0) {
            __threadfence_system();
            int* cnt = p.ar_cnt_part[owner] + p.ar_rank * AR_MAX_ROWS + m_blk;
            asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
          } else if (mine && lane < p.ar_world && lane != p.ar_rank) {
            __threadfence_system();
            int* cnt = p.ar_cnt_final[lane] + p.ar_rank * AR_MAX_ROWS + m_blk;
            asm volatile("red.release.sys.global.add.s32 [%0], 1;" ::"l"(cnt) : "memory");
          }
        }
      }
    }
    if (p.tma_epi && warp == 2 && lane == 0) tma_store_wait<0>();  // shared memory must outlive the bulk stores
    if (p.ar_world > 1 && !p.ar_scatter && ok && work_first == 0) {
      // before the launch completes, the final tiles that the other owners push into my `final` buffer must have
      // landed: each epilogue thread of CTA 0 checks a share of the (tile row, owner) counters
      const int t = (warp - 2) * 32 + lane;
      bool all_in = true;
      for (int mb = t; mb < p.num_m_blocks; mb += 128) {
        const int o = ar_owner(mb, p.num_m_blocks, p.ar_world);
        if (o == p.ar_rank) continue;
        all_in = all_in && spin_until_ge(p.ar_cnt_final[p.ar_rank] + o * AR_MAX_ROWS + mb, p.ar_base + p.num_n_blocks);
      }
      if (!all_in) atomicExch(p.status, ST_TIMEOUT_PEER_FLAG);
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before();
  if constexpr (CG == 2) cluster_sync_all();  // both blocks are done with tensor memory and with each other's barriers
  else __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    if constexpr (CG == 2) tmem_dealloc_2cta(tmem_base, 2 * BN);
    else tmem_dealloc(tmem_base, 2 * BN);
  }
}

template <int BN, bool A_MN, bool B_MN, int CG = 1>
static int launch_gemm(const void* A, const void* B, const GemmParams& p, int lda, int ldb, int max_ctas,
                       cudaStream_t stream, const void* const* group_b = nullptr, int groups = 0) {
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
    r = make_tmap_2d_bf16(&tb, B, p.N, p.K, ldb, BK, BN / CG);
  if (r) return r;
  using L = SmemLayout<BN, CG>;
  auto kfn = gemm_bf16_kernel<BN, A_MN, B_MN, CG>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, L::DYN_BYTES);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  int tiles = ((p.num_m_blocks + CG - 1) / CG) * p.num_n_blocks;
  // thread blocks (CG == 1) or pairs (CG == 2); with a fused all-gather the pulling blocks keep their SMs, so that every
  // working block is resident from the start (tiles are dealt out round-robin: a block that started late would finish late)
  const int slots = (sm_count() - (p.ag_world > 1 ? p.ag_pull_ctas : 0)) / CG;
  int grid = tiles < slots ? tiles : slots;
  if (max_ctas > 0 && grid > max_ctas / CG) grid = max_ctas / CG > 0 ? max_ctas / CG : 1;
  grid *= CG;
  if (p.ag_world > 1) grid += p.ag_pull_ctas;  // the pulling blocks come first and leave when they are done
  GemmParams q = p;
  EpiMaps em = {};  // filled per launch and passed by value: no state shared between host threads
  const int eb = q.out_fp32 ? 4 : 2;
  const int cps = 128 / eb;
  q.tma_epi = ((reinterpret_cast<uintptr_t>(q.C) & 15) == 0 && ((size_t)q.ldc * eb) % 16 == 0) ? 1 : 0;
  if (q.ar_world > 1 && !q.tma_epi) return CSB_ERR_BAD_ARG;
  if (q.group_rows > 0) {
    // grouped form: one B per group, same shape and row pitch (B above is group 0's and only serves the prefetch)
    if (A_MN || q.ar_world > 1 || q.ag_world > 1 || groups < 1 || groups > MAX_GROUPS || group_b == nullptr ||
        q.group_rows % (BM * CG) != 0 || (long)groups * q.group_rows != q.M)
      return CSB_ERR_BAD_ARG;
    for (int g = 0; g < groups; ++g) {
      CUtensorMap* dst = const_cast<CUtensorMap*>(group_b_map(em, g));
      if (reinterpret_cast<uintptr_t>(group_b[g]) & 15) return CSB_ERR_BAD_ARG;
      if (B_MN)
        r = make_tmap_2d_bf16(dst, group_b[g], q.K, q.N, ldb, 64, BK);
      else
        r = make_tmap_2d_bf16(dst, group_b[g], q.N, q.K, ldb, BK, BN / CG);
      if (r) return r;
    }
  }
  if (q.ag_world > 1) {
    if (A_MN) return CSB_ERR_BAD_ARG;
    const int own0 = ar_range_start(q.ag_rank, q.num_m_blocks, q.ag_world) * BM;
    int own1 = ar_range_start(q.ag_rank + 1, q.num_m_blocks, q.ag_world) * BM;
    if (own1 > q.M) own1 = q.M;
    r = make_tmap_2d_bf16(&em.a_own, q.ag_src[q.ag_rank], own1 - own0, q.K, q.K, BK, BM);
    if (r) return r;
  }
  if (q.tma_epi) {
    r = make_tmap_2d_out(&em.c, q.C, q.M, q.N, q.ldc, q.out_fp32, cps, BM);
    if (r) return r;
    for (int d = 0; d < q.ar_world && q.ar_world > 1; ++d) {
      r = make_tmap_2d_out(&em.inbox[d], q.ar_inbox[d] + (size_t)q.ar_rank * q.ar_slot_elems, q.M, q.N, q.N, 0, cps, BM);
      if (r) return r;
      r = make_tmap_2d_out(&em.fin[d], q.ar_final[d], q.M, q.N, q.N, 0, cps, BM);
      if (r) return r;
    }
  }
  if constexpr (CG == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)grid);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = L::DYN_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2;
    at[0].val.clusterDim.y = 1;
    at[0].val.clusterDim.z = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kfn, ta, tb, em, q);
    if (e != cudaSuccess) {
      fprintf(stderr, "[cornstarch_b200] cluster launch of the GEMM failed: %s\n", cudaGetErrorString(e));
      return (int)e;
    }
    return launch_result();
  } else {
    kfn<<<grid, 192, L::DYN_BYTES, stream>>>(ta, tb, em, q);
    return launch_result();
  }
}

}  // namespace csb

namespace csb {
static int gemm_cg_choice() {
  static const int cg_env = []() { const char* e = getenv("CORNSTARCH_B200_GEMM_CG"); return e ? atoi(e) : 0; }();
  return (cg_env == 1 || cg_env == 2) ? cg_env : CSB_GEMM_DEFAULT_CG;
}
// Pairs of thread blocks serve a fused collective when every rank's range of tile rows starts on an even tile row:
// both blocks of a pair then work for the same owner.
static bool pairs_fit_ranges(int num_m_blocks, int world) { return num_m_blocks % (2 * world) == 0; }
static void no_collective(GemmParams& p) {
  p.group_rows = 0;
  p.ar_scatter = 0; p.ar_row_offset = 0;
  p.ag_world = 1; p.ag_rank = 0; p.ag_pull_ctas = 0;
  for (int i = 0; i < 8; ++i) p.ag_src[i] = nullptr;
  p.ag_dst = nullptr; p.ag_ready = nullptr; p.ag_ready_value = 0; p.ag_pulled = nullptr; p.ag_pull_target = 0;
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
  p.tma_epi = 0;
  p.ar_world = 1; p.ar_rank = 0; p.ar_base = 0; p.ar_slot_elems = 0;
  for (int i = 0; i < 8; ++i) { p.ar_inbox[i] = nullptr; p.ar_final[i] = nullptr; p.ar_cnt_part[i] = nullptr; p.ar_cnt_final[i] = nullptr; }
  no_collective(p);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CSB_DISPATCH(BNV)                                                                       \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BNV, false, false>(A, B, p, lda, ldb, max_ctas, s); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BNV, false, true>(A, B, p, lda, ldb, max_ctas, s);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BNV, true, false>(A, B, p, lda, ldb, max_ctas, s);   \
  return launch_gemm<BNV, true, true>(A, B, p, lda, ldb, max_ctas, s);
  // Pairs of thread blocks on one 256 x 256 tile (cta_group::2) when the problem has at least two tile rows and the
  // caller did not restrict the number of thread blocks (a restricted launch shares the GPU with another kernel).
  const int cg = gemm_cg_choice();
  if (bn == 256 && cg == 2 && p.num_m_blocks >= 2 && max_ctas <= 0) {
    if (!a_mn_major && !b_mn_major) return launch_gemm<256, false, false, 2>(A, B, p, lda, ldb, 0, s);
    if (!a_mn_major && b_mn_major) return launch_gemm<256, false, true, 2>(A, B, p, lda, ldb, 0, s);
    if (a_mn_major && !b_mn_major) return launch_gemm<256, true, false, 2>(A, B, p, lda, ldb, 0, s);
    return launch_gemm<256, true, true, 2>(A, B, p, lda, ldb, 0, s);
  }
  if (bn == 256) { CSB_DISPATCH(256) }
  CSB_DISPATCH(128)
#undef CSB_DISPATCH
}


// Grouped GEMM: `groups` problems of the same shape in ONE launch.  A is [groups * group_rows][K] (K-major) and C is
// [groups * group_rows][N]; rows [g * group_rows, (g + 1) * group_rows) use B_ptrs[g] (a HOST array of `groups` device
// pointers): [N][K] (b_mn_major = 0) or [K][N] (b_mn_major = 1), all with row pitch ldb.
//   C[g] (+)= A[g] * op(B[g])^T
// group_rows must be a multiple of 256 (the height of a tile of a pair of thread blocks); groups <= 16.  This is the
// expert MLP of a MoE layer whose experts all receive the same number of rows (capacity dispatch): the forward GEMMs
// (b_mn_major = 0) and the input-gradient GEMMs (b_mn_major = 1) of all local experts.
CSB_API int csb_gemm_grouped_bf16(const void* A, const void* const* B_ptrs, void* C, int groups, int group_rows, int N, int K,
                                  int lda, int ldb, int ldc, int b_mn_major, int out_fp32, int accumulate, int tile_n,
                                  int* status, void* stream) {
  using namespace csb;
  if (groups < 1 || groups > MAX_GROUPS || group_rows <= 0 || group_rows % 256 || N <= 0 || K <= 0 || (lda & 7) || (ldb & 7) ||
      B_ptrs == nullptr)
    return CSB_ERR_BAD_ARG;
  if (reinterpret_cast<uintptr_t>(A) & 15) return CSB_ERR_BAD_ARG;
  const int M = groups * group_rows;
  int bn = tile_n;
  if (bn != 128 && bn != 256) {
    long t256 = (long)((M + BM - 1) / BM) * ((N + 255) / 256);
    bn = (N >= 256 && t256 >= sm_count()) ? 256 : 128;
  }
  GemmParams p;
  p.C = C;
  p.bias = nullptr;
  p.M = M; p.N = N; p.K = K;
  p.ldc = ldc;
  p.out_fp32 = out_fp32;
  p.accumulate = accumulate;
  p.act = 0;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.num_k_blocks = (K + BK - 1) / BK;
  p.status = status;
  p.tma_epi = 0;
  p.ar_world = 1; p.ar_rank = 0; p.ar_base = 0; p.ar_slot_elems = 0;
  for (int i = 0; i < 8; ++i) { p.ar_inbox[i] = nullptr; p.ar_final[i] = nullptr; p.ar_cnt_part[i] = nullptr; p.ar_cnt_final[i] = nullptr; }
  no_collective(p);
  p.group_rows = group_rows;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const void* B0 = B_ptrs[0];
  if (bn == 256 && gemm_cg_choice() == 2) {
    if (b_mn_major) return launch_gemm<256, false, true, 2>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
    return launch_gemm<256, false, false, 2>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
  }
  if (bn == 256) {
    if (b_mn_major) return launch_gemm<256, false, true>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
    return launch_gemm<256, false, false>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
  }
  if (b_mn_major) return launch_gemm<128, false, true>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
  return launch_gemm<128, false, false>(A, B0, p, lda, ldb, 0, s, B_ptrs, groups);
}


// Fused GEMM + all-reduce across `world` ranks (2..8, one node) through peer-mapped memory:
//   C = sum over ranks of op(A_rank) * op(B_rank)^T      (bf16)
// On return of the launch, C holds the rows this rank owns (contiguous ranges of 128-row tile rows, range r for
// rank r, see csb_ar_owned_rows) and `final` (this rank's buffer in final_ptrs) holds every other row; the
// caller copies those rows from `final` into C (a plain device copy, stream-ordered after the launch).
//   inbox_ptrs[r] : inbox of rank r, `world` slots of slot_elems bf16          (>= M*N each)
//   final_ptrs[r] : final buffer of rank r, slot_elems bf16
//   cnt_part_ptrs[r], cnt_final_ptrs[r] : int32 [world][512] arrival counters of rank r (monotonic, zero at start)
// all four arrays hold `world` device pointers valid on THIS rank (own buffers + peer mappings).
// `base` = num_n_blocks(of this shape) * number of earlier calls on this set of buffers; a set of buffers serves one
// (M, N, tile_n) shape, and callers alternate between two sets so a rank never overwrites data a slower peer still reads.
static int gemm_allreduce_impl(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                               int a_mn_major, int b_mn_major, int world, int rank, void* const* inbox_ptrs,
                               void* const* final_ptrs, void* const* cnt_part_ptrs, void* const* cnt_final_ptrs,
                               long slot_elems, int base, int tile_n, int* status, void* stream, int scatter) {
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
  if (p.num_m_blocks > AR_MAX_ROWS || p.num_m_blocks < world || (long)M * N > slot_elems) return CSB_ERR_TOO_LARGE;
  p.status = status;
  p.tma_epi = 0;
  p.ar_world = world; p.ar_rank = rank; p.ar_base = base; p.ar_slot_elems = slot_elems;
  for (int i = 0; i < 8; ++i) {
    p.ar_inbox[i] = i < world ? reinterpret_cast<__nv_bfloat16*>(inbox_ptrs[i]) : nullptr;
    p.ar_final[i] = i < world ? reinterpret_cast<__nv_bfloat16*>(final_ptrs[i]) : nullptr;
    p.ar_cnt_part[i] = i < world ? reinterpret_cast<int*>(cnt_part_ptrs[i]) : nullptr;
    p.ar_cnt_final[i] = i < world ? reinterpret_cast<int*>(cnt_final_ptrs[i]) : nullptr;
  }
  no_collective(p);
  if (scatter) {
    p.ar_scatter = 1;
    p.ar_row_offset = ar_range_start(rank, p.num_m_blocks, world) * BM;
    // the C tensor map covers the owned rows only
    p.M = M;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
#define CSB_DISPATCH_AR(BNV)                                                                       \
  if (!a_mn_major && !b_mn_major) return launch_gemm<BNV, false, false>(A, B, p, lda, ldb, 0, s); \
  if (!a_mn_major && b_mn_major) return launch_gemm<BNV, false, true>(A, B, p, lda, ldb, 0, s);   \
  if (a_mn_major && !b_mn_major) return launch_gemm<BNV, true, false>(A, B, p, lda, ldb, 0, s);   \
  return launch_gemm<BNV, true, true>(A, B, p, lda, ldb, 0, s);
  if (bn == 256 && gemm_cg_choice() == 2 && pairs_fit_ranges(p.num_m_blocks, world)) {
    if (!a_mn_major && !b_mn_major) return launch_gemm<256, false, false, 2>(A, B, p, lda, ldb, 0, s);
    if (!a_mn_major && b_mn_major) return launch_gemm<256, false, true, 2>(A, B, p, lda, ldb, 0, s);
    if (a_mn_major && !b_mn_major) return launch_gemm<256, true, false, 2>(A, B, p, lda, ldb, 0, s);
    return launch_gemm<256, true, true, 2>(A, B, p, lda, ldb, 0, s);
  }
  if (bn == 256) { CSB_DISPATCH_AR(256) }
  CSB_DISPATCH_AR(128)
#undef CSB_DISPATCH_AR
}

CSB_API int csb_gemm_allreduce_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                    int a_mn_major, int b_mn_major, int world, int rank, void* const* inbox_ptrs,
                                    void* const* final_ptrs, void* const* cnt_part_ptrs, void* const* cnt_final_ptrs,
                                    long slot_elems, int base, int tile_n, int* status, void* stream) {
  return gemm_allreduce_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, world, rank, inbox_ptrs, final_ptrs,
                             cnt_part_ptrs, cnt_final_ptrs, slot_elems, base, tile_n, status, stream, 0);
}

// Fused GEMM + reduce-scatter: like csb_gemm_allreduce_bf16, but every rank keeps only the sum of the rows it owns
// (rows [row_begin, row_end) of csb_ar_layout) and nothing is sent back.  C is the OWNED part: [row_end - row_begin][N].
// final_ptrs / cnt_final_ptrs are not used (pass the same arrays).
CSB_API int csb_gemm_reducescatter_bf16(const void* A, const void* B, void* C, int M, int N, int K, int lda, int ldb, int ldc,
                                        int a_mn_major, int b_mn_major, int world, int rank, void* const* inbox_ptrs,
                                        void* const* final_ptrs, void* const* cnt_part_ptrs, void* const* cnt_final_ptrs,
                                        long slot_elems, int base, int tile_n, int* status, void* stream) {
  return gemm_allreduce_impl(A, B, C, M, N, K, lda, ldb, ldc, a_mn_major, b_mn_major, world, rank, inbox_ptrs, final_ptrs,
                             cnt_part_ptrs, cnt_final_ptrs, slot_elems, base, tile_n, status, stream, 1);
}

// Fused all-gather + GEMM: C[M,N] = A_full * op(B)^T where A_full [M][K] (K-major) is sharded by rows over `world`
// ranks (range r of csb_ar_layout on rank r).  shard_ptrs[r] = rank r's shard (peer-mapped, row pitch K); a_full = local
// [M][K] buffer whose PEER rows the kernel fills (the caller copies its own shard in; it may keep the buffer, e.g. for
// the weight gradient); ready = local
// int[world] counters (rank r stores ready_value there once its shard is staged); pulled = local int[world] counters,
// zero at start, advanced by pull_ctas per call: pass pull_target = pull_ctas * (number of calls so far, this one included).
CSB_API int csb_ag_gemm_bf16(void* const* shard_ptrs, void* a_full, const void* B, void* C, int M, int N, int K, int ldb,
                             int ldc, int b_mn_major, int world, int rank, const int* ready, int ready_value, int* pulled,
                             int pull_target, int pull_ctas, int tile_n, int* status, void* stream) {
  using namespace csb;
  if (M <= 0 || N <= 0 || K <= 0 || (K & 7) || (ldb & 7) || world < 2 || world > 8 || pull_ctas < 1 || pull_ctas > 64)
    return CSB_ERR_BAD_ARG;
  if ((reinterpret_cast<uintptr_t>(a_full) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return CSB_ERR_BAD_ARG;
  int bn = (tile_n == 128 || tile_n == 256) ? tile_n : ((N >= 256) ? 256 : 128);
  GemmParams p;
  p.C = C; p.bias = nullptr;
  p.M = M; p.N = N; p.K = K; p.ldc = ldc;
  p.out_fp32 = 0; p.accumulate = 0; p.act = 0;
  p.num_m_blocks = (M + BM - 1) / BM;
  p.num_n_blocks = (N + bn - 1) / bn;
  p.num_k_blocks = (K + BK - 1) / BK;
  if (p.num_m_blocks < world) return CSB_ERR_TOO_LARGE;
  p.status = status;
  p.tma_epi = 0;
  p.ar_world = 1; p.ar_rank = 0; p.ar_base = 0; p.ar_slot_elems = 0;
  for (int i = 0; i < 8; ++i) { p.ar_inbox[i] = nullptr; p.ar_final[i] = nullptr; p.ar_cnt_part[i] = nullptr; p.ar_cnt_final[i] = nullptr; }
  no_collective(p);
  p.ag_world = world; p.ag_rank = rank; p.ag_pull_ctas = pull_ctas;
  for (int i = 0; i < 8; ++i) p.ag_src[i] = reinterpret_cast<const uint4*>(shard_ptrs[i < world ? i : 0]);
  p.ag_dst = reinterpret_cast<uint4*>(a_full);
  p.ag_ready = ready; p.ag_ready_value = ready_value; p.ag_pulled = pulled; p.ag_pull_target = pull_target;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (bn == 256 && gemm_cg_choice() == 2 && pairs_fit_ranges(p.num_m_blocks, world) && (pull_ctas & 1) == 0) {
    if (b_mn_major) return launch_gemm<256, false, true, 2>(a_full, B, p, K, ldb, 0, s);
    return launch_gemm<256, false, false, 2>(a_full, B, p, K, ldb, 0, s);
  }
  if (bn == 256) {
    if (b_mn_major) return launch_gemm<256, false, true>(a_full, B, p, K, ldb, 0, s);
    return launch_gemm<256, false, false>(a_full, B, p, K, ldb, 0, s);
  }
  if (b_mn_major) return launch_gemm<128, false, true>(a_full, B, p, K, ldb, 0, s);
  return launch_gemm<128, false, false>(a_full, B, p, K, ldb, 0, s);
}

// Rows [row_begin, row_end) of an M-row output that rank `rank` of `world` owns in the fused all-reduce,
// and the tile width / tile-row count the launch will use for N columns.
CSB_API int csb_ar_layout(int M, int N, int world, int rank, int tile_n, int* row_begin, int* row_end, int* num_n_blocks) {
  using namespace csb;
  int bn = (tile_n == 128 || tile_n == 256) ? tile_n : ((N >= 256) ? 256 : 128);
  const int num_m = (M + BM - 1) / BM;
  *row_begin = ar_range_start(rank, num_m, world) * BM;
  int e = ar_range_start(rank + 1, num_m, world) * BM;
  *row_end = e < M ? e : M;
  *num_n_blocks = (N + bn - 1) / bn;
  return 0;
}

CSB_WAIT_LIMIT_SETTER(gemm)
