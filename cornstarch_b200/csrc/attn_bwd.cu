// Flash-attention backward for sm_100a (bitfield / causal / full masks, GQA, tile skipping).
//
// One CTA owns one 128-row K/V tile of one KV head and keeps dK and dV for it in TMEM for the
// whole kernel, looping over the query heads of the GQA group and over 64-row query tiles:
//
//   S^T  = K  Q^T              M=128(kv) N=64(q)  contraction D     -> TMEM S^T[2] (double buffer)
//   dP^T = V  dO^T             M=128     N=64     contraction D     -> TMEM dP^T
//   P^T  = exp2(S^T*c - LSE),  dS^T = P^T * (dP^T - delta) * scale   (P^T -> bf16 pairs in TMEM over S^T;
//                                                                     dS^T -> bf16 smem tile)
//   dV  += P^T  dO             M=128     N=D      contraction q=64
//   dK  += dS^T Q              M=128     N=D      contraction q=64
//   dQ^T = K^T  dS^T           M=128(d)  N=64(q)  contraction kv=128 -> TMEM dQ^T
//
// dK/dV need no atomics and are bit-reproducible: every query head that shares the KV head is
// handled by the same CTA.  dQ^T tiles are staged in shared memory as [q][d] rows and added into an fp32
// accumulator by TMA reduce-add (one 32x32 block per warp), then converted to bf16 by a final pass.
//
// Warp roles (576 threads by default): warp 0 = TMA producer (K/V once, Q/dO ring of 3 stages), warp 1 = MMA
// issuer, warps 2..17 = 512 compute threads (or 2..9 = 256).  Thread (r, group) owns KV row r (TMEM lane r) and 16
// (32) of the 64 query columns of S^T / dP^T, and head-dim row r of dQ^T.  The pipeline keeps S^T one
// iteration ahead: while the compute warps turn S^T(i), dP^T(i) into P^T, dS^T, the tensor core
// already holds S^T(i+1); dP^T(i+1) is issued as soon as dP^T(i) has been read, before the
// dV/dK/dQ^T MMAs of iteration i, so the next exponentials overlap those MMAs.  Per-tile query
// metadata (LSE, delta, positions, bitfields) is prefetched into registers one iteration early.
//
// Replaces cornstarch/kernel/bitfield_attention.py:526-929 (T8, T9: fp32 atomics for dQ, dK and dV)
// and cornstarch/kernel/attention.py:348-852.
#include "host.h"
#include "kv_segments.h"
#include "mask.cuh"
#include "ptx.cuh"

namespace csb {

constexpr int BW_BKV = 128;
constexpr int BW_BQ = 64;
constexpr int KV_CHUNK = 128 * 128;  // 128 rows x 128 B
constexpr int Q_CHUNK = 64 * 128;    // 64 rows x 128 B

struct AttnBwdParams {
  int B, Sq, Sk, Hq, Hk, D, dk16;
  int nQ64, nQ128, nK;
  float scale, scale_log2;
  int mask_mode;
  const int64_t* q_bits;
  const int64_t* k_bits;
  const int* q_pos;
  const int* k_pos;
  const int8_t* cls;  // [B][nQ128][nK]
  const float* lse;   // [B][Hq][Sq]
  const float* delta; // [B][Hq][Sq]
  float* dq_acc;      // [B][Sq][Hq][D] fp32, zeroed by the caller
  __nv_bfloat16* dK[CSB_MAX_SEG];  // per key segment: where its dK / dV tiles go (possibly a peer's inbox)
  __nv_bfloat16* dV[CSB_MAX_SEG];
  long dk_stride_b[CSB_MAX_SEG], dk_stride_s[CSB_MAX_SEG], dv_stride_b[CSB_MAX_SEG], dv_stride_s[CSB_MAX_SEG];
  int* status;
  int kj_slowest;  // block order: 1 = key block slowest (masks that leave key blocks unequal work), 0 = key block fastest
  // dense boolean mask (MASK_DENSE) and additive bias, as in the forward kernel
  const uint8_t* dmask;
  long dm_sb, dm_sq;
  const float* bias;
  long bias_sb, bias_sh, bias_sq;
  float inv_scale;
  SegInfo seg;
};

struct BwdSmem {
  static constexpr int QSTAGES = 3;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + 2 * KV_CHUNK;
  static constexpr int Q_OFF = V_OFF + 2 * KV_CHUNK;          // QSTAGES x (2 chunks x 8 KB)
  static constexpr int DO_OFF = Q_OFF + QSTAGES * 2 * Q_CHUNK;
  static constexpr int DST_OFF = DO_OFF + QSTAGES * 2 * Q_CHUNK;  // dS^T [128 kv][64 q] bf16
  static constexpr int DQ_OFF = DST_OFF + KV_CHUNK;           // dQ staging: 8 warps x [32 q][32 d] fp32 (row-major, 4 KB each)
  static constexpr int META_OFF = DQ_OFF + 8 * 4096;          // three buffers of: lse2[64] f32, delta*scale[64] f32, qpos[64] i32, qbits[64] i64
  static constexpr int META_STAGE = 64 * 4 * 3 + 64 * 8;
  static constexpr int LIST_OFF = META_OFF + 3 * META_STAGE;  // valid 64-row query tiles of this key block: int16 index, int8 class
  static constexpr int MAX_TILES = 1024;                      // sequences up to 65536 tokens
  static constexpr int BAR_OFF = LIST_OFF + MAX_TILES * 4;
  static constexpr int NBAR = 1 + QSTAGES + QSTAGES + 1 + 1 + 1 + 1 + 1 + 1;
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 32;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

// NCW compute warps (8 or 16): NCW / 4 warps share a TMEM lane quarter and split the 64 query columns between them.
template <int NCW>
struct BwdCfg {
  static constexpr int COMPUTE_THREADS = NCW * 32;
  static constexpr int THREADS = 64 + COMPUTE_THREADS;
  static constexpr int GROUPS = NCW / 4;       // column groups
  static constexpr int COLS = BW_BQ / GROUPS;  // query columns of S^T / dP^T / dQ^T per thread: 32 or 16
};

__device__ __forceinline__ bool bw_wait(uint64_t* bar, uint32_t phase, volatile int* abort_flag) {
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

// delta[b][h][q] = sum_d O[b][q][h][d] * dO[b][q][h][d]
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                  float* __restrict__ delta, int B, int Sq, int Hq, int D, long o_sb, long o_ss,
                                  long do_sb, long do_ss) {
  const long row = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;  // one warp per (b, q, h)
  const int lane = threadIdx.x & 31;
  const long total = (long)B * Sq * Hq;
  if (row >= total) return;
  const int h = row % Hq;
  const long bq = row / Hq;
  const int q = bq % Sq;
  const int b = bq / Sq;
  const __nv_bfloat16* o = O + b * o_sb + (long)q * o_ss + (long)h * D;
  const __nv_bfloat16* d = dO + b * do_sb + (long)q * do_ss + (long)h * D;
  float acc = 0.f;
  for (int i = lane * 2; i < D; i += 64) {
    float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(o + i));
    float2 c = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(d + i));
    acc += a.x * c.x + a.y * c.y;
  }
#pragma unroll
  for (int s = 16; s > 0; s >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, s);
  if (lane == 0) delta[((long)b * Hq + h) * Sq + q] = acc;
}

// dq (bf16, strided) = dq_acc (fp32, dense [B][Sq][Hq][D])
__global__ void attn_dq_convert_kernel(const float* __restrict__ acc, __nv_bfloat16* __restrict__ dq, long n_rows,
                                       int Sq, int HD, long dq_sb, long dq_ss) {
  const int vec = HD / 4;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n_rows * vec; i += (long)gridDim.x * blockDim.x) {
    const long row = i / vec;
    const int c = (i % vec) * 4;
    const int q = row % Sq;
    const long b = row / Sq;
    const float4 f = *reinterpret_cast<const float4*>(acc + row * HD + c);
    uint2 u;
    u.x = pack_bf16x2(f.x, f.y);
    u.y = pack_bf16x2(f.z, f.w);
    *reinterpret_cast<uint2*>(dq + b * dq_sb + (long)q * dq_ss + c) = u;
  }
}

template <int NCW>
__global__ void __launch_bounds__(BwdCfg<NCW>::THREADS, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ KvMaps kvm,
                const __grid_constant__ CUtensorMap tm_do, const __grid_constant__ CUtensorMap tm_dq,
                const AttnBwdParams p) {
  using L = BwdSmem;
  using CFG = BwdCfg<NCW>;
  constexpr int QS = L::QSTAGES;
  constexpr int COLS = CFG::COLS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;
  uint64_t* q_full = bars + 1;            // [QS]  Q + dO stage landed
  uint64_t* q_empty = q_full + QS;        // [QS]  stage consumed by the dV/dK MMAs
  uint64_t* sdp_full = q_empty + QS;      //       S^T and dP^T of an iteration ready in TMEM
  uint64_t* pds_full = sdp_full + 1;      //       P^T and dS^T tiles written to smem (256 arrivals)
  uint64_t* pds_empty = pds_full + 1;     //       ... and consumed by the MMAs
  uint64_t* dq_full = pds_empty + 1;      //       dQ^T ready in TMEM
  uint64_t* dq_free = dq_full + 1;        //       dQ^T drained (256 arrivals)
  uint64_t* dp_read = dq_free + 1;      //       S^T and dP^T of an iteration are in registers (256 arrivals): dP^T may be overwritten
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_valid_slot = reinterpret_cast<int*>(tmem_slot + 2);
  int* peer_ok_slot = reinterpret_cast<int*>(tmem_slot + 3);
  int16_t* tile_idx = reinterpret_cast<int16_t*>(smem + L::LIST_OFF);
  int8_t* tile_cls = reinterpret_cast<int8_t*>(smem + L::LIST_OFF + L::MAX_TILES * 2);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // One-dimensional grid, key block slowest: under causal masks the first key blocks meet the most query tiles, so
  // the heavy blocks of every head start first and the light ones fill the tail.
  // (With a full mask every block is equally heavy; key block fastest then keeps the Q / dO tiles of few heads in L2.)
  const int n_hb = p.Hk * p.B;
  const int hb = p.kj_slowest ? blockIdx.x % n_hb : blockIdx.x / p.nK;
  const int kj = p.kj_slowest ? blockIdx.x / n_hb : blockIdx.x % p.nK;
  const int hk = hb % p.Hk, b = hb / p.Hk;
  const int group = p.Hq / p.Hk;
  const int k0 = kj * BW_BKV;                              // index into k_bits / k_pos (padded gathered space)
  const int sg = seg_of_tile(p.seg, kj);                   // which K/V segment (rank) this key block belongs to
  const int row0 = (kj - p.seg.tile_start[sg]) * BW_BKV;   // first row of the block inside that segment

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int i = 0; i < QS; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
    }
    mbar_init(sdp_full, 1);
    mbar_init(pds_full, CFG::COMPUTE_THREADS);
    mbar_init(pds_empty, 1);
    mbar_init(dq_full, 1);
    mbar_init(dq_free, CFG::COMPUTE_THREADS);
    mbar_init(dp_read, CFG::COMPUTE_THREADS);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    // list of the 64-row query tiles that have at least one allowed pair with this key block (ordered compaction)
    int n = 0;
    for (int base = 0; base < p.nQ64 && n < L::MAX_TILES; base += 32) {
      const int i = base + lane;
      const int8_t c = (i < p.nQ64) ? p.cls[((long)b * p.nQ128 + (i >> 1)) * p.nK + kj] : int8_t(0);
      const uint32_t m = __ballot_sync(0xffffffffu, c != 0);
      const int pos = n + __popc(m & ((1u << lane) - 1u));
      if (c != 0 && pos < L::MAX_TILES) {
        tile_idx[pos] = static_cast<int16_t>(i);
        tile_cls[pos] = c;
      }
      n += __popc(m);
    }
    if (lane == 0) {
      *n_valid_slot = n < L::MAX_TILES ? n : L::MAX_TILES;
      // A key block of a peer: nothing of this CTA may touch that rank's memory (loads of K/V, stores of dK/dV
      // into its inbox) before the rank has staged its K/V, which also means it is done with its previous inbox.
      int ok = 1;
      if (p.seg.ready_flags != nullptr && sg != p.seg.my_seg) {
        ok = wait_peer_flag(p.seg.ready_flags + sg, p.seg.ready_value) ? 1 : 0;
        if (!ok) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
      }
      *peer_ok_slot = ok;
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int n_valid = *n_valid_slot;
  const bool peer_ready = *peer_ok_slot != 0;
  const int n_iter = peer_ready ? n_valid * group : 0;
  // TMEM columns: S^T[0] 0..63, S^T[1] 64..127, dP^T 128..191, dQ^T 192..255, dV 256..383, dK 384..511
  const uint32_t tmem_dPT = tmem_base + 128;
  const uint32_t tmem_dQT = tmem_base + 192;
  const uint32_t tmem_dV = tmem_base + 256;
  const uint32_t tmem_dK = tmem_base + 384;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_do);
      const bool peer_ok = peer_ready;
      if (peer_ok) {
        mbar_expect_tx(kv_full, 4 * KV_CHUNK);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(smem + L::K_OFF + c * KV_CHUNK, &kvm.k[sg], kv_full, c * 64, hk, row0, b);
          tma_load_4d(smem + L::V_OFF + c * KV_CHUNK, &kvm.v[sg], kv_full, c * 64, hk, row0, b);
        }
      }
      for (int it = 0; peer_ok && it < n_iter; ++it) {
        const int h = hk * group + it / n_valid;
        const int i = tile_idx[it % n_valid];
        const int st = it % QS;
        if (!bw_wait(&q_empty[st], ((it / QS) & 1) ^ 1, abort_flag)) {
          atomicCAS(p.status, 0, ST_TIMEOUT_EMPTY);
          *abort_flag = 1;
          break;
        }
        mbar_expect_tx(&q_full[st], 4 * Q_CHUNK);
        for (int c = 0; c < 2; ++c) {
          tma_load_4d(smem + L::Q_OFF + (st * 2 + c) * Q_CHUNK, &tm_q, &q_full[st], c * 64, h, i * BW_BQ, b);
          tma_load_4d(smem + L::DO_OFF + (st * 2 + c) * Q_CHUNK, &tm_do, &q_full[st], c * 64, h, i * BW_BQ, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks this code in step (every lane waits on the barriers; one elected lane issues each MMA and
    // commit): see umma_f16_w.  A 16-wide slice of a tile is the tile's descriptor plus the slice's byte offset / 16.
    {
      const uint32_t idesc_s = make_idesc_bf16(128, BW_BQ, 0, 0);
      const uint32_t idesc_dkv = make_idesc_bf16(128, p.dk16, 0, 1);
      const uint32_t idesc_dq = make_idesc_bf16(128, BW_BQ, 1, 1);
      const uint64_t k_km = make_desc_kmajor_sw128(smem_u32(smem + L::K_OFF));
      const uint64_t v_km = make_desc_kmajor_sw128(smem_u32(smem + L::V_OFF));
      const uint64_t k_mn = make_desc_mnmajor_sw128(smem_u32(smem + L::K_OFF), KV_CHUNK);
      const uint64_t dst_km = make_desc_kmajor_sw128(smem_u32(smem + L::DST_OFF));
      const uint64_t dst_mn = make_desc_mnmajor_sw128(smem_u32(smem + L::DST_OFF), KV_CHUNK);
      const int ksteps_d = p.dk16 / 16;
      bool ok = bw_wait(kv_full, 0, abort_flag);
      if (!ok) { atomicCAS(p.status, 0, ST_TIMEOUT_FULL); *abort_flag = 1; }
      auto kslice = [](int kk, int chunk_bytes) -> uint64_t {
        return static_cast<uint64_t>(((kk >> 2) * chunk_bytes + (kk & 3) * 32) >> 4);
      };

      // S^T(it) = K Q^T into ST[it & 1]; waits for the Q/dO stage of that iteration
      auto issue_st = [&](int it) -> bool {
        const int st = it % QS;
        if (!bw_wait(&q_full[st], (it / QS) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_FULL); *abort_flag = 1; return false; }
        tc_fence_after();
        const uint64_t q_km = make_desc_kmajor_sw128(smem_u32(smem + L::Q_OFF + st * 2 * Q_CHUNK));
        const uint32_t t_st = tmem_base + (it & 1) * 64;
        for (int kk = 0; kk < ksteps_d; ++kk)
          umma_f16_w(t_st, k_km + kslice(kk, KV_CHUNK), q_km + kslice(kk, Q_CHUNK), idesc_s, kk > 0);
        return true;
      };
      // dP^T(it) = V dO^T; its commit also covers S^T(it), issued earlier
      auto issue_dpt = [&](int it) {
        const int st = it % QS;
        const uint64_t do_km = make_desc_kmajor_sw128(smem_u32(smem + L::DO_OFF + st * 2 * Q_CHUNK));
        for (int kk = 0; kk < ksteps_d; ++kk)
          umma_f16_w(tmem_dPT, v_km + kslice(kk, KV_CHUNK), do_km + kslice(kk, Q_CHUNK), idesc_s, kk > 0);
        umma_commit_w(sdp_full);
      };

      if (ok && n_iter > 0) {
        ok = issue_st(0);
        if (ok) issue_dpt(0);
        if (ok && n_iter > 1) ok = issue_st(1);
      }
      for (int it = 0; ok && it < n_iter; ++it) {
        const int st = it % QS;
        // dP^T(it+1) is issued as soon as the compute warps hold dP^T(it) in registers, long before they are done with
        // the iteration: S^T(it+1) and dP^T(it+1) are then ready when they come back for the next one
        if (it + 1 < n_iter) {
          if (!bw_wait(dp_read, it & 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_MISC); *abort_flag = 1; break; }
          tc_fence_after();
          issue_dpt(it + 1);
        }
        if (!bw_wait(pds_full, it & 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_MISC); *abort_flag = 1; break; }
        tc_fence_after();
        const uint64_t q_mn = make_desc_mnmajor_sw128(smem_u32(smem + L::Q_OFF + st * 2 * Q_CHUNK), Q_CHUNK);
        const uint64_t do_mn = make_desc_mnmajor_sw128(smem_u32(smem + L::DO_OFF + st * 2 * Q_CHUNK), Q_CHUNK);
        // dV += P^T dO ; dK += dS^T Q   (contraction over the 64 query rows)
#pragma unroll
        for (int kk = 0; kk < BW_BQ / 16; ++kk)
          umma_f16_ts_w(tmem_dV, tmem_base + (it & 1) * 64 + (kk / (COLS / 16)) * COLS + (kk % (COLS / 16)) * 8,
                        do_mn + static_cast<uint64_t>((kk * 2048) >> 4), idesc_dkv, (it > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
        for (int kk = 0; kk < BW_BQ / 16; ++kk)
          umma_f16_w(tmem_dK, dst_km + static_cast<uint64_t>((kk * 32) >> 4), q_mn + static_cast<uint64_t>((kk * 2048) >> 4),
                     idesc_dkv, (it > 0 || kk > 0) ? 1u : 0u);
        umma_commit_w(&q_empty[st]);
        if (it > 0) {
          if (!bw_wait(dq_free, (it - 1) & 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_EMPTY); *abort_flag = 1; break; }
          tc_fence_after();
        }
        // dQ^T = K^T dS^T  (contraction over the 128 key rows)
#pragma unroll
        for (int kk = 0; kk < BW_BKV / 16; ++kk)
          umma_f16_w(tmem_dQT, k_mn + static_cast<uint64_t>((kk * 2048) >> 4), dst_mn + static_cast<uint64_t>((kk * 2048) >> 4),
                     idesc_dq, kk > 0 ? 1u : 0u);
        umma_commit_w(pds_empty);
        umma_commit_w(dq_full);
        if (it + 2 < n_iter) ok = issue_st(it + 2);  // ST[it & 1] was read before pds_full(it)
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ compute threads (NCW warps)
    const int cw = warp - 2;
    const int quarter = warp & 3;       // TMEM lane quarter this warp may touch
    const int half = cw >> 2;           // which group of COLS query columns (of 64) this warp handles
    const int r = quarter * 32 + lane;  // KV row in the tile == TMEM lane; also head-dim row of dQ^T
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int col0 = half * COLS;
    const int kidx = k0 + r;
    const int krow = row0 + r;  // row inside the segment
    const bool k_valid = krow < p.seg.rows[sg];
    const int64_t kb = (k_valid && p.k_bits) ? p.k_bits[(long)b * p.Sk + kidx] : 0;
    const int kpos = k_valid ? (p.k_pos ? p.k_pos[(long)b * p.Sk + kidx] : kidx) : -1;
    const float LOG2E = 1.4426950408889634f;
    // the 64 threads with half == 0 and r < 64 stage the metadata of query row (tile * 64 + r)
    const bool stager = (half == 0) && (r < 64);

    float pf_lse = 0.f, pf_delta = 0.f;
    int pf_qpos = -1;
    int64_t pf_qbits = 0;
    auto prefetch_meta = [&](int it) {
      if (!stager || it >= n_iter) return;
      const int h = hk * group + it / n_valid;
      const int q = tile_idx[it % n_valid] * BW_BQ + r;
      const bool qv = q < p.Sq;
      const long idx = ((long)b * p.Hq + h) * p.Sq + q;
      pf_lse = qv ? p.lse[idx] * LOG2E : INFINITY;
      pf_delta = qv ? p.delta[idx] * p.scale : 0.f;
      pf_qpos = qv ? (p.q_pos ? p.q_pos[(long)b * p.Sq + q] : q) : -1;
      pf_qbits = (qv && p.q_bits) ? p.q_bits[(long)b * p.Sq + q] : 0;
    };

    bool ok = true;
    auto drain_dq = [&](int pit) -> bool {
      if (!bw_wait(dq_full, pit & 1, abort_flag)) {
        if (lane == 0) atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        return false;
      }
      tc_fence_after();
      const int ph = hk * group + pit / n_valid;
      const int pi = tile_idx[pit % n_valid];
      uint32_t v[COLS];
      tmem_ld_cols<COLS>(tmem_dQT + col0 + lane_addr, v);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(dq_free);
      // this warp's [32 d][COLS q] block -> shared memory as [q][d] rows of 128 B -> one TMA reduce-add into dq_acc
      if (lane == 0) tma_store_wait_read<0>();  // the previous block has left the staging buffer
      __syncwarp();
      float* stage = reinterpret_cast<float*>(smem + L::DQ_OFF + cw * (COLS * 128));
#pragma unroll
      for (int c = 0; c < COLS; ++c) stage[c * 32 + lane] = __uint_as_float(v[c]);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0 && quarter * 32 < p.D) {
        tma_reduce_add_4d(&tm_dq, stage, quarter * 32, ph, pi * BW_BQ + col0, b);  // box: 32 d x COLS q
        tma_store_commit();
      }
      return true;
    };

    // Query metadata of iteration it lives in buffer it % 3.  The stagers write the metadata of iteration it + 1 right
    // after they hold S^T / dP^T of iteration it in registers and BEFORE they arrive on dp_read(it); the MMA warp issues
    // dP^T(it + 1) only after dp_read(it) is complete, so sdp_full(it + 1) also tells every thread that the metadata is
    // staged.  Three buffers: whoever stages it + 1 has seen sdp_full(it), i.e. every thread is past its loads of it - 1
    // and therefore done with the metadata of it - 2, the previous tenant of that buffer.
    auto stage_meta = [&](int it) {
      if (!stager || it >= n_iter) return;
      float* m = reinterpret_cast<float*>(smem + L::META_OFF + (it % 3) * L::META_STAGE);
      m[r] = pf_lse;
      m[64 + r] = pf_delta;
      reinterpret_cast<int*>(m + 128)[r] = pf_qpos;
      reinterpret_cast<int64_t*>(m + 192)[r] = pf_qbits;
    };
    prefetch_meta(0);
    stage_meta(0);
    prefetch_meta(1);
    // the metadata of iteration 0 is ordered by a barrier of its own (named barrier 1 over the compute threads)
    asm volatile("bar.sync 1, %0;" ::"n"(CFG::COMPUTE_THREADS) : "memory");
    for (int it = 0; it < n_iter && ok; ++it) {
      const int c = tile_cls[it % n_valid];
      float* m_lse = reinterpret_cast<float*>(smem + L::META_OFF + (it % 3) * L::META_STAGE);
      float* m_delta = m_lse + 64;
      int* m_qpos = reinterpret_cast<int*>(m_delta + 64);
      int64_t* m_qbits = reinterpret_cast<int64_t*>(m_qpos + 64);
      if (!bw_wait(sdp_full, it & 1, abort_flag)) {
        if (lane == 0) atomicCAS(p.status, 0, ST_TIMEOUT_TMEM_FULL);
        *abort_flag = 1;
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t sv[COLS], dv[COLS];
      tmem_ld_cols<COLS>(tmem_base + (it & 1) * 64 + col0 + lane_addr, sv);
      tmem_ld_cols<COLS>(tmem_dPT + col0 + lane_addr, dv);
      tmem_ld_wait();
      stage_meta(it + 1);
      prefetch_meta(it + 2);  // global loads for the tile after next fly while this one is processed
      tc_fence_before();
      mbar_arrive(dp_read);
      float pv[COLS], ds[COLS];
      const int q_base = tile_idx[it % n_valid] * BW_BQ + col0;  // first query row of this thread's columns
      if (p.bias != nullptr && k_valid) {
        const int hh = hk * group + it / n_valid;
        const float* bcol = p.bias + (long)b * p.bias_sb + (long)hh * p.bias_sh + kidx;
#pragma unroll
        for (int x = 0; x < COLS; ++x)
          if (q_base + x < p.Sq)
            sv[x] = __float_as_uint(fmaf(__ldg(bcol + (long)(q_base + x) * p.bias_sq), p.inv_scale, __uint_as_float(sv[x])));
      }
#pragma unroll
      for (int x4 = 0; x4 < COLS / 4; ++x4) {
        const float4 l4 = *reinterpret_cast<const float4*>(m_lse + col0 + x4 * 4);
        const float ls[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int y = 0; y < 4; ++y)
          pv[x4 * 4 + y] = fast_exp2(fmaf(__uint_as_float(sv[x4 * 4 + y]), p.scale_log2, -ls[y]));
      }
      if (c == 1) {
        if (p.mask_mode == MASK_DENSE) {
          const uint8_t* mcol = p.dmask + (long)b * p.dm_sb + kidx;
#pragma unroll
          for (int x = 0; x < COLS; ++x) {
            const bool allow = k_valid && m_qpos[col0 + x] >= 0 && __ldg(mcol + (long)(q_base + x) * p.dm_sq) != 0;
            pv[x] = allow ? pv[x] : 0.f;
          }
        } else {
#pragma unroll
          for (int x = 0; x < COLS; ++x) {
            const int col = col0 + x;
            const bool allow = k_valid && m_qpos[col] >= 0 && mask_allowed(p.mask_mode, m_qbits[col], kb, m_qpos[col], kpos);
            pv[x] = allow ? pv[x] : 0.f;
          }
        }
      }
#pragma unroll
      for (int x4 = 0; x4 < COLS / 4; ++x4) {
        const float4 d4 = *reinterpret_cast<const float4*>(m_delta + col0 + x4 * 4);
        const float dl[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
        for (int y = 0; y < 4; ++y)
          ds[x4 * 4 + y] = pv[x4 * 4 + y] * fmaf(__uint_as_float(dv[x4 * 4 + y]), p.scale, -dl[y]);
      }
      if (it > 0) {
        if (!bw_wait(pds_empty, (it - 1) & 1, abort_flag)) {
          if (lane == 0) atomicCAS(p.status, 0, ST_TIMEOUT_MISC);
          *abort_flag = 1;
          ok = false;
          break;
        }
      }
      // P^T -> packed bf16 pairs in tensor memory, over this thread's own S^T columns (the first half of them);
      // dS^T -> bf16 smem tile: row r, this warp's 16-byte pieces (8 query columns each)
      {
        uint32_t pk[COLS / 2];
#pragma unroll
        for (int x = 0; x < COLS / 2; ++x) pk[x] = pack_bf16x2(pv[2 * x], pv[2 * x + 1]);
        tmem_st_cols<COLS / 2>(tmem_base + (it & 1) * 64 + col0 + lane_addr, pk);
      }
#pragma unroll
      for (int pc = 0; pc < COLS / 8; ++pc) {
        uint4 w;
        w.x = pack_bf16x2(ds[pc * 8 + 0], ds[pc * 8 + 1]);
        w.y = pack_bf16x2(ds[pc * 8 + 2], ds[pc * 8 + 3]);
        w.z = pack_bf16x2(ds[pc * 8 + 4], ds[pc * 8 + 5]);
        w.w = pack_bf16x2(ds[pc * 8 + 6], ds[pc * 8 + 7]);
        *reinterpret_cast<uint4*>(smem + L::DST_OFF + sw128_offset(r, half * (COLS / 8) + pc)) = w;
      }
      tmem_st_wait();
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(pds_full);
      // drain dQ^T of the previous iteration while the MMAs of this one run
      if (it > 0) ok = drain_dq(it - 1);
    }
    if (ok && n_iter > 0) ok = drain_dq(n_iter - 1);
    if (lane == 0) tma_store_wait<0>();  // every reduce-add of this warp has completed
    __syncwarp();
    // ---- epilogue: dV and dK tiles (every MMA has retired once the last dQ^T was seen);
    //      the warps of a lane quarter split the head-dim columns
    if (ok && peer_ready) {
      tc_fence_after();
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        const uint32_t t = which == 0 ? tmem_dV : tmem_dK;
        __nv_bfloat16* base = which == 0
                                  ? p.dV[sg] + (long)b * p.dv_stride_b[sg] + (long)krow * p.dv_stride_s[sg] + (long)hk * p.D
                                  : p.dK[sg] + (long)b * p.dk_stride_b[sg] + (long)krow * p.dk_stride_s[sg] + (long)hk * p.D;
#pragma unroll
        for (int c2 = 0; c2 < 4 / CFG::GROUPS; ++c2) {
          const int cc = half * (4 / CFG::GROUPS) + c2;
          uint32_t v[32];
          if (n_iter > 0) {
            tmem_ld_32x32(t + cc * 32 + lane_addr, v);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x) v[x] = 0u;
          }
          if (k_valid) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const int col = cc * 32 + g * 8;
              if (col + 8 <= p.D) {
                uint4 u;
                u.x = pack_bf16x2(__uint_as_float(v[g * 8 + 0]), __uint_as_float(v[g * 8 + 1]));
                u.y = pack_bf16x2(__uint_as_float(v[g * 8 + 2]), __uint_as_float(v[g * 8 + 3]));
                u.z = pack_bf16x2(__uint_as_float(v[g * 8 + 4]), __uint_as_float(v[g * 8 + 5]));
                u.w = pack_bf16x2(__uint_as_float(v[g * 8 + 6]), __uint_as_float(v[g * 8 + 7]));
                *reinterpret_cast<uint4*>(base + col) = u;
              }
            }
          }
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

static int make_tmap_4d(CUtensorMap* tm, const void* base, int D, int H, int S, int B, long stride_s, long stride_b,
                        int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)stride_s * 2, (uint64_t)stride_b * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap_nd_bf16(tm, base, 4, dims, strides, box);
}

}  // namespace csb

using namespace csb;

// q / out / dout / dq are [B][Sq][Hq][D] bf16 views (head stride D; token / batch strides in elements); keys and values
// come as segments (kv_segments.h) and the dK / dV tiles of segment r are written to kv->dk[r] / kv->dv[r].
// lse: fp32 [B][Hq][Sq] from the forward; delta: fp32 [B][Hq][Sq] scratch; dq_acc: fp32 dense [B][Sq][Hq][D] scratch
// that the caller has zeroed.  Sk = padded gathered length; cls: tile classes for 128x128 tiles.
// Optional inputs of the dense-mask / bias form (same layout as in attn_fwd.cu).
struct CsbAttnExtras {
  const unsigned char* dmask;
  long dm_sb, dm_sq;
  const float* bias;
  long bias_sb, bias_sh, bias_sq;
};

static int attn_bwd_seg_impl(const void* q, const CsbKvSegments* kv, const void* out, const void* dout, const float* lse,
                             float* delta, float* dq_acc, void* dq, int B, int Sq, int Sk, int Hq, int Hk, int D, long q_ss,
                             long q_sb, long o_ss, long o_sb, long do_ss, long do_sb, long dq_ss, long dq_sb, float scale,
                             int mask_mode, const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                             const signed char* cls, int* status, void* stream, const CsbAttnExtras* ex) {
  if (D % 8 || D > 128 || D < 16 || Hq % Hk) return CSB_ERR_BAD_ARG;
  if (mask_mode == MASK_DENSE && (ex == nullptr || ex->dmask == nullptr)) return CSB_ERR_BAD_ARG;
  if (kv == nullptr || kv->n_seg < 1 || kv->n_seg > CSB_MAX_SEG) return CSB_ERR_BAD_ARG;
  if ((Sq + BW_BQ - 1) / BW_BQ > BwdSmem::MAX_TILES) return CSB_ERR_TOO_LARGE;
  if ((q_ss % 8) || (do_ss % 8) || (dq_ss % 4)) return CSB_ERR_BAD_ARG;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  {
    const long rows = (long)B * Sq * Hq;
    const int threads = 256;
    const long blocks = (rows * 32 + threads - 1) / threads;
    attn_delta_kernel<<<(unsigned)blocks, threads, 0, s>>>(reinterpret_cast<const __nv_bfloat16*>(out),
                                                           reinterpret_cast<const __nv_bfloat16*>(dout), delta, B, Sq, Hq,
                                                           D, o_sb, o_ss, do_sb, do_ss);
    if (int e = launch_result()) return e;
  }
  AttnBwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hk = Hk; p.D = D;
  p.dk16 = (D + 15) / 16 * 16;
  p.nQ64 = (Sq + BW_BQ - 1) / BW_BQ;
  p.nQ128 = (Sq + 127) / 128;
  p.nK = (Sk + BW_BKV - 1) / BW_BKV;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mask_mode = mask_mode;
  p.q_bits = reinterpret_cast<const int64_t*>(q_bits);
  p.k_bits = reinterpret_cast<const int64_t*>(k_bits);
  p.q_pos = q_pos; p.k_pos = k_pos;
  p.cls = reinterpret_cast<const int8_t*>(cls);
  p.lse = lse; p.delta = delta; p.dq_acc = dq_acc;
  p.status = status;
  p.dmask = ex ? ex->dmask : nullptr;
  p.dm_sb = ex ? ex->dm_sb : 0; p.dm_sq = ex ? ex->dm_sq : 0;
  p.bias = ex ? ex->bias : nullptr;
  p.bias_sb = ex ? ex->bias_sb : 0; p.bias_sh = ex ? ex->bias_sh : 0; p.bias_sq = ex ? ex->bias_sq : 0;
  p.inv_scale = scale != 0.f ? 1.f / scale : 0.f;
  p.kj_slowest = mask_mode != MASK_FULL;
  fill_seg_info(&p.seg, kv, BW_BKV);
  if (p.seg.tile_start[kv->n_seg] != p.nK) return CSB_ERR_BAD_ARG;
  CUtensorMap tq, tdo;
  KvMaps kvm;
  int r;
  if ((r = make_tmap_4d(&tq, q, D, Hq, Sq, B, q_ss, q_sb, BW_BQ))) return r;
  if ((r = make_tmap_4d(&tdo, dout, D, Hq, Sq, B, do_ss, do_sb, BW_BQ))) return r;
  for (int i = 0; i < CSB_MAX_SEG; ++i) {
    const int g = i < kv->n_seg ? i : 0;
    if ((kv->k_stride_s[g] % 8) || (kv->v_stride_s[g] % 8) || (kv->dk_stride_s[g] % 8) || (kv->dv_stride_s[g] % 8)) return CSB_ERR_BAD_ARG;
    if ((r = make_tmap_4d(&kvm.k[i], kv->k[g], D, Hk, kv->rows[g], B, kv->k_stride_s[g], kv->k_stride_b[g], BW_BKV))) return r;
    if ((r = make_tmap_4d(&kvm.v[i], kv->v[g], D, Hk, kv->rows[g], B, kv->v_stride_s[g], kv->v_stride_b[g], BW_BKV))) return r;
    p.dK[i] = reinterpret_cast<__nv_bfloat16*>(kv->dk[g]);
    p.dV[i] = reinterpret_cast<__nv_bfloat16*>(kv->dv[g]);
    p.dk_stride_s[i] = kv->dk_stride_s[g]; p.dk_stride_b[i] = kv->dk_stride_b[g];
    p.dv_stride_s[i] = kv->dv_stride_s[g]; p.dv_stride_b[i] = kv->dv_stride_b[g];
  }
  // 16 compute warps (four per scheduler: they hide the tensor-memory load and dependency latencies of each other;
  // measured 3 % faster than 8 at S = 8192 once the MMA warp issued as a converged warp), or 8 when the environment asks
  static const bool wide = []() {
    const char* e = getenv("CORNSTARCH_B200_ATTN_BWD_WARPS");
    return !(e && atoi(e) == 8);
  }();
  CUtensorMap tdq;
  {
    // dq_acc is dense fp32 [B][Sq][Hq][D]; a block is 32 head-dim elements (128 B) x 32 or 16 query rows
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hq, (uint64_t)Sq, (uint64_t)B};
    uint64_t strides[3] = {(uint64_t)D * 4, (uint64_t)Hq * D * 4, (uint64_t)Sq * Hq * D * 4};
    uint32_t box[4] = {32, 1, (uint32_t)(wide ? BwdCfg<16>::COLS : BwdCfg<8>::COLS), 1};
    if ((r = make_tmap_nd_f32(&tdq, dq_acc, 4, dims, strides, box))) return r;
  }
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::DYN_BYTES) != cudaSuccess ||
        cudaFuncSetAttribute(attn_bwd_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::DYN_BYTES) != cudaSuccess)
      return launch_result();
    attr = true;
  }
  const long n_blocks = (long)p.nK * Hk * B;
  if (n_blocks > 0x7fffffffL) return CSB_ERR_TOO_LARGE;
  dim3 grid((unsigned)n_blocks);
  if (wide)
    attn_bwd_kernel<16><<<grid, BwdCfg<16>::THREADS, BwdSmem::DYN_BYTES, s>>>(tq, kvm, tdo, tdq, p);
  else
    attn_bwd_kernel<8><<<grid, BwdCfg<8>::THREADS, BwdSmem::DYN_BYTES, s>>>(tq, kvm, tdo, tdq, p);
  int e = launch_result();
  if (e) return e;
  const long n_rows = (long)B * Sq;
  const int HD = Hq * D;
  long work = n_rows * (HD / 4);
  int blocks = (int)((work + 255) / 256 < (long)sm_count() * 16 ? (work + 255) / 256 : (long)sm_count() * 16);
  attn_dq_convert_kernel<<<blocks, 256, 0, s>>>(dq_acc, reinterpret_cast<__nv_bfloat16*>(dq), n_rows, Sq, HD, dq_sb, dq_ss);
  return launch_result();
}

CSB_API int csb_attn_bwd_seg(const void* q, const CsbKvSegments* kv, const void* out, const void* dout, const float* lse,
                             float* delta, float* dq_acc, void* dq, int B, int Sq, int Sk, int Hq, int Hk, int D, long q_ss,
                             long q_sb, long o_ss, long o_sb, long do_ss, long do_sb, long dq_ss, long dq_sb, float scale,
                             int mask_mode, const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                             const signed char* cls, int* status, void* stream) {
  return attn_bwd_seg_impl(q, kv, out, dout, lse, delta, dq_acc, dq, B, Sq, Sk, Hq, Hk, D, q_ss, q_sb, o_ss, o_sb, do_ss, do_sb,
                           dq_ss, dq_sb, scale, mask_mode, q_bits, k_bits, q_pos, k_pos, cls, status, stream, nullptr);
}

// One local K/V tensor with a dense boolean mask (mask_mode = MASK_DENSE) and / or an additive bias (no bias gradient).
CSB_API int csb_attn_bwd_dense(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                               int Sk, int Hq, int Hk, int D, long q_ss, long q_sb, long k_ss, long k_sb, long v_ss, long v_sb,
                               long o_ss, long o_sb, long do_ss, long do_sb, long dq_ss, long dq_sb, long dk_ss, long dk_sb,
                               long dv_ss, long dv_sb, float scale, int mask_mode, const signed char* cls,
                               const CsbAttnExtras* ex, int* status, void* stream) {
  CsbKvSegments kv = {};
  kv.n_seg = 1;
  kv.my_seg = 0;
  kv.rows[0] = Sk;
  kv.k[0] = k; kv.v[0] = v;
  kv.k_stride_s[0] = k_ss; kv.k_stride_b[0] = k_sb; kv.v_stride_s[0] = v_ss; kv.v_stride_b[0] = v_sb;
  kv.dk[0] = dk; kv.dv[0] = dv;
  kv.dk_stride_s[0] = dk_ss; kv.dk_stride_b[0] = dk_sb; kv.dv_stride_s[0] = dv_ss; kv.dv_stride_b[0] = dv_sb;
  kv.ready_flags = nullptr;
  return attn_bwd_seg_impl(q, &kv, out, dout, lse, delta, dq_acc, dq, B, Sq, Sk, Hq, Hk, D, q_ss, q_sb, o_ss, o_sb, do_ss, do_sb,
                           dq_ss, dq_sb, scale, mask_mode, nullptr, nullptr, nullptr, nullptr, cls, status, stream, ex);
}

// One local K/V tensor ([B][Sk][Hk][D] views) with dK / dV of the same shape.
CSB_API int csb_attn_bwd(const void* q, const void* k, const void* v, const void* out, const void* dout,
                         const float* lse, float* delta, float* dq_acc, void* dq, void* dk, void* dv, int B, int Sq,
                         int Sk, int Hq, int Hk, int D, long q_ss, long q_sb, long k_ss, long k_sb, long v_ss, long v_sb,
                         long o_ss, long o_sb, long do_ss, long do_sb, long dq_ss, long dq_sb, long dk_ss, long dk_sb,
                         long dv_ss, long dv_sb, float scale, int mask_mode, const long* q_bits, const long* k_bits,
                         const int* q_pos, const int* k_pos, const signed char* cls, int* status, void* stream) {
  CsbKvSegments kv = {};
  kv.n_seg = 1;
  kv.my_seg = 0;
  kv.rows[0] = Sk;
  kv.k[0] = k; kv.v[0] = v;
  kv.k_stride_s[0] = k_ss; kv.k_stride_b[0] = k_sb; kv.v_stride_s[0] = v_ss; kv.v_stride_b[0] = v_sb;
  kv.dk[0] = dk; kv.dv[0] = dv;
  kv.dk_stride_s[0] = dk_ss; kv.dk_stride_b[0] = dk_sb; kv.dv_stride_s[0] = dv_ss; kv.dv_stride_b[0] = dv_sb;
  kv.ready_flags = nullptr;
  return csb_attn_bwd_seg(q, &kv, out, dout, lse, delta, dq_acc, dq, B, Sq, Sk, Hq, Hk, D, q_ss, q_sb, o_ss, o_sb, do_ss,
                          do_sb, dq_ss, dq_sb, scale, mask_mode, q_bits, k_bits, q_pos, k_pos, cls, status, stream);
}

// --------------------------------------------------------------------------------------------- context-parallel glue
namespace csb {

// Tell every peer that this rank's event counter reached `value` (its K/V are staged, or its dK/dV tiles delivered):
// peer r's flag array has one int per source rank.  Ordered after all earlier work of the stream; the fence makes
// this rank's earlier stores (also those to peer memory) visible before the flag.
__global__ void cp_signal_kernel(int* const* flag_arrays, int world, int me, int value) {
  const int r = threadIdx.x;
  if (r >= world) return;
  __threadfence_system();
  int* f = flag_arrays[r] + me;
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(f), "r"(value) : "memory");
}

// Stream-ordered (bounded) wait until every rank's counter in the local flag array reached `value`.
__global__ void cp_wait_kernel(const int* flags, int world, int value, int* status) {
  if (threadIdx.x != 0) return;
  for (int r = 0; r < world; ++r)
    if (!wait_peer_flag(flags + r, value)) {
      atomicCAS(status, 0, ST_TIMEOUT_PEER_FLAG);
      return;
    }
}

struct CpReduceParams {
  const __nv_bfloat16* src[CSB_MAX_SEG];  // one inbox slot per source rank, all [n] elements
  int world;
  const int* flags;  // local flag array: flags[r] >= value once rank r delivered its tiles
  int value;
  int* status;
};

// out = sum over source ranks of their bf16 partial tiles (fp32 accumulation).
__global__ void __launch_bounds__(256) cp_reduce_kernel(CpReduceParams p, __nv_bfloat16* out, long n8) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) {
    int ok = 1;
    for (int r = 0; r < p.world && ok; ++r)
      if (!wait_peer_flag(p.flags + r, p.value)) ok = 0;
    if (!ok) atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
    ok_s = ok;
  }
  __syncthreads();
  if (!ok_s) return;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int r = 0; r < p.world; ++r) {
      const uint4 u = reinterpret_cast<const uint4*>(p.src[r])[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(h[k]);
        acc[2 * k] += f.x;
        acc[2 * k + 1] += f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16x2(acc[0], acc[1]);
    o.y = pack_bf16x2(acc[2], acc[3]);
    o.z = pack_bf16x2(acc[4], acc[5]);
    o.w = pack_bf16x2(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

}  // namespace csb

// flag_arrays: device array of `world` pointers, entry r = rank r's flag array (peer-mapped), each int[world].
CSB_API int csb_cp_signal(void* flag_arrays, int world, int me, int value, void* stream) {
  if (world < 1 || world > CSB_MAX_SEG) return CSB_ERR_BAD_ARG;
  cp_signal_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(reinterpret_cast<int* const*>(flag_arrays), world, me, value);
  return launch_result();
}

CSB_API int csb_cp_wait(const int* flags, int world, int value, int* status, void* stream) {
  if (world < 1 || world > CSB_MAX_SEG) return CSB_ERR_BAD_ARG;
  cp_wait_kernel<<<1, 32, 0, reinterpret_cast<cudaStream_t>(stream)>>>(flags, world, value, status);
  return launch_result();
}

// out[n] = sum_r src[r][n] once every rank's counter in `flags` reached `value` (n a multiple of 8).
CSB_API int csb_cp_reduce(const void* const* src, int world, const int* flags, int value, void* out, long n, int* status,
                          void* stream) {
  if (world < 1 || world > CSB_MAX_SEG || (n % 8)) return CSB_ERR_BAD_ARG;
  CpReduceParams p;
  for (int r = 0; r < CSB_MAX_SEG; ++r) p.src[r] = reinterpret_cast<const __nv_bfloat16*>(src[r < world ? r : 0]);
  p.world = world; p.flags = flags; p.value = value; p.status = status;
  const long n8 = n / 8;
  long blocks = (n8 + 255) / 256;
  if (blocks > (long)sm_count() * 8) blocks = (long)sm_count() * 8;
  if (blocks < 1) blocks = 1;
  cp_reduce_kernel<<<(unsigned)blocks, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p, reinterpret_cast<__nv_bfloat16*>(out), n8);
  return launch_result();
}

CSB_WAIT_LIMIT_SETTER(attn_bwd)
