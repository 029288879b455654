// Flash-attention forward for sm_100a with bitfield / causal / full masks, GQA and block skipping.
//
//   O = softmax(scale * Q K^T + mask) V,   LSE = log sum exp   (per query row)
//
// One CTA = one 128-row query tile of one head.  Both GEMMs run on tcgen05 with TMEM accumulators:
//   S = Q K^T    : A = Q tile (K-major smem), B = K tile (K-major smem)      -> TMEM S[2] (double buffer)
//   O[h] += P V  : A = P tile in TMEM (bf16 pairs written by the softmax threads over the columns of S), B = V tile
//                  (MN-major smem)                                            -> TMEM O[2]
// Warp roles: warp 0 = TMA producer (Q once, K/V ring of 2 stages), warp 1 = MMA issuer (the whole warp walks the code,
// one elected lane issues), warps 2..9 = softmax: two threads per query row (one TMEM lane), thread (r, h) owning key
// columns [64 h, 64 h + 64) of every tile.  Each thread is an independent online softmax over ITS columns (own running
// maximum and row sum), and the keys of column half h accumulate into their own output O[h]: no exchange between the two
// threads of a row inside the loop, and the P V of a half is issued as soon as that half's threads are done.  The epilogue
// merges the two partial results of a row.  The running maximum is only refreshed when it grows by more than 2^8 (lazy
// rescale), which keeps the TMEM read-modify-write of O off the common path.
//
// Mask handling: a [B][nQ][nK] int8 class map (0 = skip tile, 1 = evaluate the predicate per element,
// 2 = all allowed) is produced once per step by csb_mask_classify and shared by all layers, heads, the
// forward and the backward.  Token positions may be given explicitly (context parallelism assigns
// non-contiguous token sets to ranks), in which case causal order uses those global positions.
//
// Replaces the Triton kernels of the reference: cornstarch/kernel/bitfield_attention.py:215-523 (forward,
// split-KV partials :1279-1436, compressed mask :104-156) and cornstarch/kernel/attention.py:56-345.
#include "host.h"
#include "kv_segments.h"
#include "mask.cuh"
#include "ptx.cuh"

namespace csb {

constexpr int AT_BM = 128;
constexpr int AT_BN = 128;
constexpr int CHUNK_BYTES = 128 * 128;  // 128 rows x 64 bf16

struct AttnFwdParams {
  int B, Sq, Sk, Hq, Hk, D, dk16;
  int nQ, nK;
  float scale, scale_log2;
  int mask_mode;
  const int64_t* q_bits;
  const int64_t* k_bits;
  const int* q_pos;
  const int* k_pos;
  const int8_t* cls;
  __nv_bfloat16* O;
  long o_stride_b, o_stride_s;  // elements; head stride is D
  float* lse;                   // [B][Hq][Sq]
  int* status;
  int j_start;  // key tiles are visited in rotated order starting here (own segment first)
  // dense boolean mask (MASK_DENSE): bytes [B][Sq][Sk], key index contiguous, strides in bytes
  const uint8_t* dmask;
  long dm_sb, dm_sq;
  // additive bias (optional, any mode): fp32, key index contiguous; strides in elements, 0 for broadcast dimensions
  const float* bias;
  long bias_sb, bias_sh, bias_sq;
  float inv_scale;
  SegInfo seg;
};

// ---------------------------------------------------------------------------------------------
// Tile classification: cls[b][qi][kj] = 0 (no pair allowed) / 2 (every pair allowed) / 1 (mixed).
__global__ void __launch_bounds__(128)
mask_classify_kernel(int mode, const int64_t* __restrict__ q_bits, const int64_t* __restrict__ k_bits,
                     const int* __restrict__ q_pos, const int* __restrict__ k_pos, int Sq, int Sk, int bm, int bn,
                     int nQ, int nK, int8_t* __restrict__ cls, int* __restrict__ row_work) {
  extern __shared__ uint8_t sm[];
  int64_t* kb_s = reinterpret_cast<int64_t*>(sm);
  int* kp_s = reinterpret_cast<int*>(kb_s + bn);
  const int kj = blockIdx.x, qi = blockIdx.y, b = blockIdx.z;
  for (int i = threadIdx.x; i < bn; i += blockDim.x) {
    const int k = kj * bn + i;
    kb_s[i] = (k < Sk && k_bits) ? k_bits[(long)b * Sk + k] : 0;
    kp_s[i] = (k < Sk) ? (k_pos ? k_pos[(long)b * Sk + k] : k) : -1;
  }
  __syncthreads();
  int cnt = 0;
  for (int r = threadIdx.x; r < bm; r += blockDim.x) {
    const int q = qi * bm + r;
    if (q >= Sq) continue;
    const int64_t qb = q_bits ? q_bits[(long)b * Sq + q] : 0;
    const int qp = q_pos ? q_pos[(long)b * Sq + q] : q;
    for (int i = 0; i < bn; ++i) {
      const bool ok = kp_s[i] >= 0 && mask_allowed(mode, qb, kb_s[i], qp, kp_s[i]);
      cnt += ok ? 1 : 0;
    }
  }
  __shared__ int red[4];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int total = red[0] + red[1] + red[2] + red[3];
    const int valid_rows = min(bm, Sq - qi * bm);
    int8_t c = 1;
    if (total == 0) c = 0;
    else if (total == valid_rows * bn) c = 2;
    cls[((long)b * nQ + qi) * nK + kj] = c;
    // per query block: number of non-empty key blocks (the context-parallel partitioner's workload)
    if (row_work && c != 0) atomicAdd(&row_work[(long)b * nQ + qi], 1);
  }
}

// Tile classes of a dense boolean mask (bytes [B][Sq][Sk]): one thread block per 128 x 128 tile counts the allowed pairs.
__global__ void __launch_bounds__(128)
mask_classify_dense_kernel(const uint8_t* __restrict__ dmask, long sb, long sq, int Sq, int Sk, int bm, int bn, int nQ, int nK,
                           int8_t* __restrict__ cls, int* __restrict__ row_work) {
  const int kj = blockIdx.x, qi = blockIdx.y, b = blockIdx.z;
  const int k0 = kj * bn, k1 = min(Sk, k0 + bn);
  int cnt = 0;
  for (int r = threadIdx.x; r < bm; r += blockDim.x) {
    const int q = qi * bm + r;
    if (q >= Sq) continue;
    const uint8_t* row = dmask + (long)b * sb + (long)q * sq;
    for (int k = k0; k < k1; ++k) cnt += row[k] ? 1 : 0;
  }
  __shared__ int red[4];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = cnt;
  __syncthreads();
  if (threadIdx.x == 0) {
    const int total = red[0] + red[1] + red[2] + red[3];
    const int valid_rows = min(bm, Sq - qi * bm);
    int8_t c = 1;
    if (total == 0) c = 0;
    else if (total == valid_rows * bn) c = 2;  // only tiles that lie fully inside Sk can be "all allowed"
    cls[((long)b * nQ + qi) * nK + kj] = c;
    if (row_work && c != 0) atomicAdd(&row_work[(long)b * nQ + qi], 1);
  }
}

// ---------------------------------------------------------------------------------------------
template <int NCH>  // number of 64-wide head-dim chunks held in smem (1: D<=64, 2: D<=128)
struct AttnSmem {
  static constexpr int Q_BYTES = NCH * CHUNK_BYTES;
  static constexpr int KV_BYTES = NCH * CHUNK_BYTES;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + 2 * KV_BYTES;
  static constexpr int KB_OFF = V_OFF + 2 * KV_BYTES;         // int64 k bits  [2][128]
  static constexpr int KP_OFF = KB_OFF + 2 * 128 * 8;         // int   k pos   [2][128]
  static constexpr int XM_OFF = KP_OFF + 2 * 128 * 4;         // float row-max exchange [2 buffers][2 halves][128]
  static constexpr int CLS_OFF = XM_OFF + 6 * 128 * 4;        // + row-sum exchange [2 halves][128]; then the tile classes
  static constexpr int MAX_NK = 1024;                         // key blocks per row of the class map (131072 keys)
  static constexpr int BAR_OFF = CLS_OFF + MAX_NK;
  static constexpr int NBAR = 1 + 2 + 2 + 2 + 2 + 2 + 2 + 1 + 1 + 4 + 1;
  static constexpr int TOTAL = BAR_OFF + NBAR * 8 + 16;
  static constexpr int DYN_BYTES = TOTAL + 1024;
};

__device__ __forceinline__ bool at_wait(uint64_t* bar, uint32_t phase, volatile int* abort_flag) {
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

template <int NCH>
__global__ void __launch_bounds__(320, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ KvMaps kvm, const AttnFwdParams p) {
  using L = AttnSmem<NCH>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;
  uint64_t* k_empty = bars + 3;
  uint64_t* v_full = bars + 5;
  uint64_t* v_empty = bars + 7;
  uint64_t* s_full = bars + 9;
  uint64_t* p_full = bars + 11;   // [2] the threads of one column half have written their part of P
  uint64_t* pv_done = bars + 13;
  uint64_t* kb_full = bars + 14;  // key bits / positions of a partial tile staged by the softmax threads
  uint64_t* pair_bar = bars + 15; // [4] one per lane quarter: the two warps that share its query rows (epilogue)
  uint64_t* o_done = bars + 19;   // the last P V has retired: both O accumulators are final
  float* xm_s = reinterpret_cast<float*>(smem + L::XM_OFF);
  int8_t* cls_s = reinterpret_cast<int8_t*>(smem + L::CLS_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + L::NBAR);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int64_t* kb_s = reinterpret_cast<int64_t*>(smem + L::KB_OFF);
  int* kp_s = reinterpret_cast<int*>(smem + L::KP_OFF);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // The grid is one-dimensional so that thread blocks start in index order.  The first pull_ctas blocks bring the
  // remote K / V segments into local memory; they are resident before any block that waits for their counters.
  const int n_pull = p.seg.pull_ctas;
  if ((int)blockIdx.x < n_pull) {
    if (!pull_remote_segments(p.seg, blockIdx.x, n_pull, reinterpret_cast<int*>(smem)) && threadIdx.x == 0)
      atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG);
    return;
  }
  const int lin = blockIdx.x - n_pull;
  // Heaviest (last) query tiles first, over all heads and batch entries: under causal masks they have the most key
  // blocks, and the lightest tiles of every head fill the tail of the grid.
  const int hb = lin % (p.Hq * p.B);
  const int qi = p.nQ - 1 - lin / (p.Hq * p.B);
  const int h = hb % p.Hq, b = hb / p.Hq;
  const int hk = h / (p.Hq / p.Hk);
  const int q0 = qi * AT_BM;
  {
    // this query tile's row of the class map, read once (every role walks it)
    const int8_t* cls_g = p.cls + ((long)b * p.nQ + qi) * p.nK;
    for (int j = threadIdx.x; j < p.nK; j += blockDim.x) cls_s[j] = cls_g[j];
  }
  const int8_t* cls_row = cls_s;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
    }
    mbar_init(&p_full[0], 128);
    mbar_init(&p_full[1], 128);
    mbar_init(pv_done, 1);
    mbar_init(o_done, 1);
    mbar_init(kb_full, 256);
    for (int i = 0; i < 4; ++i) mbar_init(&pair_bar[i], 64);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_S = tmem_base;        // 2 x 128 columns
  const uint32_t tmem_O = tmem_base + 256;  // 2 x (up to 128) columns: O[h] accumulates the keys of column half h of every tile

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tm_q);
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int c = 0; c < NCH; ++c) tma_load_4d(smem + L::Q_OFF + c * CHUNK_BYTES, &tm_q, q_full, c * 64, h, q0, b);
      uint32_t it = 0;
      uint32_t opened = p.seg.my_seg >= 0 ? (1u << p.seg.my_seg) : 0u;
      if (p.seg.ready_flags == nullptr) opened = 0xffu;
      for (int t = 0; t < p.nK; ++t) {
        int j = t + p.j_start;
        if (j >= p.nK) j -= p.nK;
        if (cls_row[j] == 0) continue;
        const int sg = seg_of_tile(p.seg, j);
        const int row0 = (j - p.seg.tile_start[sg]) * AT_BN;
        if (!((opened >> sg) & 1u)) {
          // first tile from this peer: its K/V must have been staged (bounded wait on the counter it stores here)
          const bool arrived = n_pull > 0 ? wait_local_count(p.seg.pulled + sg, p.seg.pull_target)
                                          : wait_peer_flag(p.seg.ready_flags + sg, p.seg.ready_value);
          if (!arrived) { atomicCAS(p.status, 0, ST_TIMEOUT_PEER_FLAG); *abort_flag = 1; break; }
          // the copy was written with ordinary stores by other blocks; the loads below go through the async proxy
          asm volatile("fence.proxy.async.global;" ::: "memory");
          opened |= 1u << sg;
        }
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!at_wait(&k_empty[st], ph ^ 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_EMPTY); *abort_flag = 1; break; }
        mbar_expect_tx(&k_full[st], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_4d(smem + L::K_OFF + st * L::KV_BYTES + c * CHUNK_BYTES, &kvm.k[sg], &k_full[st], c * 64, hk, row0, b);
        if (!at_wait(&v_empty[st], ph ^ 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_EMPTY); *abort_flag = 1; break; }
        mbar_expect_tx(&v_full[st], L::KV_BYTES);
#pragma unroll
        for (int c = 0; c < NCH; ++c)
          tma_load_4d(smem + L::V_OFF + st * L::KV_BYTES + c * CHUNK_BYTES, &kvm.v[sg], &v_full[st], c * 64, hk, row0, b);
        ++it;
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    // The whole warp walks this code in step (every lane waits on the barriers; one elected lane issues each MMA and
    // commit): see umma_f16_w.
    {
      const uint32_t idesc_s = make_idesc_bf16(AT_BM, AT_BN, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(AT_BM, p.dk16, 0, 1);
      const uint64_t q_desc = make_desc_kmajor_sw128(smem_u32(smem + L::Q_OFF));
      const int ksteps_s = p.dk16 / 16;
      bool ok = at_wait(q_full, 0, abort_flag);
      if (!ok) { atomicCAS(p.status, 0, ST_TIMEOUT_FULL); *abort_flag = 1; }
      // number of non-empty key blocks
      int n = 0;
      for (int j = 0; j < p.nK; ++j) n += (cls_row[j] != 0);

      // tcgen05.mma operations of one CTA execute in issue order.  S(it+1) is issued after P(it-1) V(it-1), the last
      // reader of the TMEM buffer it overwrites (P(it-1) lives in the columns of S(it-1)); the softmax threads are done
      // with that buffer because their p_full(it-1) arrival preceded that MMA.
      auto issue_s = [&](uint32_t it) -> bool {
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!at_wait(&k_full[st], ph, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_FULL); *abort_flag = 1; return false; }
        tc_fence_after();
        // descriptors of the k-th 16-wide slice: the tile's descriptor plus the slice's byte offset / 16
        const uint64_t k_desc = make_desc_kmajor_sw128(smem_u32(smem + L::K_OFF + st * L::KV_BYTES));
        for (int kk = 0; kk < ksteps_s; ++kk) {
          const uint64_t off = static_cast<uint64_t>(((kk >> 2) * CHUNK_BYTES + (kk & 3) * 32) >> 4);
          umma_f16_w(tmem_S + st * 128, q_desc + off, k_desc + off, idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit_w(&k_empty[st]);
        umma_commit_w(&s_full[st]);
        return true;
      };
      if (ok && n > 0) ok = issue_s(0);
      for (uint32_t it = 0; ok && it < (uint32_t)n; ++it) {
        if (it + 1 < (uint32_t)n) {
          ok = issue_s(it + 1);
          if (!ok) break;
        }
        const int st = it & 1;
        const uint32_t ph = (it >> 1) & 1;
        if (!at_wait(&v_full[st], ph, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_FULL); *abort_flag = 1; break; }
        const uint64_t v_desc = make_desc_mnmajor_sw128(smem_u32(smem + L::V_OFF + st * L::KV_BYTES), CHUNK_BYTES);
        // O[h] += P_h V_h for the two column halves of the tile, each as soon as its threads have written P_h (packed
        // bf16 pairs in the first 32 columns of that half of the S buffer: 16 keys of a row = 8 columns per step)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
          if (!at_wait(&p_full[hh], it & 1, abort_flag)) { atomicCAS(p.status, 0, ST_TIMEOUT_MISC); *abort_flag = 1; ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < AT_BN / 32; ++kk)
            umma_f16_ts_w(tmem_O + hh * 128, tmem_S + st * 128 + hh * 64 + kk * 8,
                          v_desc + static_cast<uint64_t>(((hh * 4 + kk) * 2048) >> 4), idesc_o, (it > 0 || kk > 0) ? 1u : 0u);
        }
        if (!ok) break;
        umma_commit_w(&v_empty[st]);
        umma_commit_w(pv_done);
        if (it + 1 == (uint32_t)n) umma_commit_w(o_done);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    // Two threads per query row: warps 2..5 take key columns 0..63 of a tile, warps 6..9 columns 64..127 (a warp
    // may only touch the TMEM lane quarter warp%4).  The pair exchanges its row maximum through shared memory.
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;  // row inside the tile == TMEM lane
    const int q = q0 + r;
    const bool row_valid = q < p.Sq;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    int64_t qb = 0;
    int qpos = q;
    if (row_valid) {
      if (p.q_bits) qb = p.q_bits[(long)b * p.Sq + q];
      if (p.q_pos) qpos = p.q_pos[(long)b * p.Sq + q];
    }
    float m_used = -INFINITY, l_sum = 0.f;
    uint32_t it = 0, n_partial = 0;
    bool ok = true;
    auto fail = [&](int code) {
      if (lane == 0) atomicCAS(p.status, 0, code);
      *abort_flag = 1;
      ok = false;
    };
    for (int t = 0; t < p.nK && ok; ++t) {
      int j = t + p.j_start;
      if (j >= p.nK) j -= p.nK;
      const int c = cls_row[j];
      if (c == 0) continue;
      const int buf = it & 1;
      if (!at_wait(&s_full[buf], (it >> 1) & 1, abort_flag)) { fail(ST_TIMEOUT_TMEM_FULL); break; }
      tc_fence_after();
      float s[64];
      {
        uint32_t v0[32], v1[32];
        tmem_ld_32x32(tmem_S + buf * 128 + half * 64 + lane_addr, v0);
        tmem_ld_32x32(tmem_S + buf * 128 + half * 64 + 32 + lane_addr, v1);
        // Key metadata of a partial tile is staged only now: S(it) being ready means P(it-2) V(it-2) was issued, i.e.
        // every thread has finished the tile that used this staging buffer before.
        if (c == 1) {
          if (half == 0) {
            const int k = j * AT_BN + r;
            const bool kv = k < p.Sk;
            kb_s[buf * 128 + r] = (kv && p.k_bits) ? p.k_bits[(long)b * p.Sk + k] : 0;
            kp_s[buf * 128 + r] = kv ? (p.k_pos ? p.k_pos[(long)b * p.Sk + k] : k) : -1;
          }
          mbar_arrive(kb_full);
          if (!at_wait(kb_full, n_partial & 1, abort_flag)) {
            tmem_ld_wait();
            fail(ST_TIMEOUT_MISC);
            break;
          }
          ++n_partial;
        }
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          s[i] = __uint_as_float(v0[i]);
          s[32 + i] = __uint_as_float(v1[i]);
        }
      }
      if (p.bias != nullptr && row_valid) {
        // additive bias in score units: folded in as bias / scale so that the scaled exponent below stays one FMA
        const int kc0 = j * AT_BN + half * 64;
        const float* brow = p.bias + (long)b * p.bias_sb + (long)h * p.bias_sh + (long)q * p.bias_sq + kc0;
#pragma unroll
        for (int i = 0; i < 64; ++i)
          if (kc0 + i < p.Sk) s[i] = fmaf(__ldg(brow + i), p.inv_scale, s[i]);
      }
      if (c == 1) {
        const int64_t* kb = kb_s + buf * 128 + half * 64;
        const int* kp = kp_s + buf * 128 + half * 64;
        if (p.mask_mode == MASK_DENSE) {
          const int kc0 = j * AT_BN + half * 64;
          const uint8_t* mrow = p.dmask + (long)b * p.dm_sb + (long)(row_valid ? q : 0) * p.dm_sq + kc0;
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const bool allow = row_valid && kp[i] >= 0 && __ldg(mrow + i) != 0;
            s[i] = allow ? s[i] : -INFINITY;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int kpos = kp[i];
            const bool allow = row_valid && kpos >= 0 && mask_allowed(p.mask_mode, qb, kb[i], qpos, kpos);
            s[i] = allow ? s[i] : -INFINITY;
          }
        }
      }
      float mx0 = s[0], mx1 = s[1], mx2 = s[2], mx3 = s[3];
#pragma unroll
      for (int i = 4; i < 64; i += 4) {
        mx0 = fmaxf(mx0, s[i]);
        mx1 = fmaxf(mx1, s[i + 1]);
        mx2 = fmaxf(mx2, s[i + 2]);
        mx3 = fmaxf(mx3, s[i + 3]);
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));  // of this thread's half of the row only
      const float m_new = fmaxf(m_used, mx);
      const bool need = (m_new - m_used) * p.scale_log2 > 8.f;  // also true when m_used is -inf and m_new is finite
      if (it > 0 && __any_sync(0xffffffffu, need)) {
        // rare (lazy rescale): O[half] is only touched once the previous P V has retired
        if (!at_wait(pv_done, (it - 1) & 1, abort_flag)) { fail(ST_TIMEOUT_MISC); break; }
        tc_fence_after();
        float alpha = 1.f;
        if (need) alpha = (m_used == -INFINITY) ? 0.f : fast_exp2((m_used - m_new) * p.scale_log2);
#pragma unroll 1
        for (int cc = 0; cc < 2 * NCH; ++cc) {
          uint32_t v[32];
          tmem_ld_32x32(tmem_O + half * 128 + cc * 32 + lane_addr, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          tmem_st_32x32(tmem_O + half * 128 + cc * 32 + lane_addr, v);
        }
        tmem_st_wait();
        l_sum *= alpha;
      }
      if (need) m_used = m_new;
      const float m_eff = (m_used == -INFINITY) ? 0.f : m_used * p.scale_log2;
      // probabilities -> packed bf16 pairs -> tensor memory, over the first 32 of this thread's own 64 columns of the
      // tile's S buffer (its scores are in registers by now)
      uint32_t pk[32];
      float ls0 = 0.f, ls1 = 0.f, ls2 = 0.f, ls3 = 0.f;
#pragma unroll
      for (int i = 0; i < 64; i += 4) {
        const float e0 = fast_exp2(fmaf(s[i], p.scale_log2, -m_eff));
        const float e1 = fast_exp2(fmaf(s[i + 1], p.scale_log2, -m_eff));
        const float e2 = fast_exp2(fmaf(s[i + 2], p.scale_log2, -m_eff));
        const float e3 = fast_exp2(fmaf(s[i + 3], p.scale_log2, -m_eff));
        ls0 += e0;
        ls1 += e1;
        ls2 += e2;
        ls3 += e3;
        pk[i / 2] = pack_bf16x2(e0, e1);
        pk[i / 2 + 1] = pack_bf16x2(e2, e3);
      }
      tmem_st_32x32(tmem_S + buf * 128 + half * 64 + lane_addr, pk);
      tmem_st_wait();
      l_sum += (ls0 + ls1) + (ls2 + ls3);
      // Arrive for tile `it` only once P V(it-1) has retired.  Without this, nothing bounds how far the softmax threads
      // run ahead of the MMA warp (S(it+1) is issued before it waits for p_full(it)): while it waits for a slow V tile,
      // p_full could complete two phases, which its parity wait cannot tell from none; a fast thread could also arrive
      // twice within one phase.  The exponentials above are already done, so the wait is normally free.
      if (it > 0 && !at_wait(pv_done, (it - 1) & 1, abort_flag)) { fail(ST_TIMEOUT_MISC); break; }
      tc_fence_before();
      mbar_arrive(&p_full[half]);
      ++it;
    }
    // ---- epilogue
    if (ok && it > 0) {
      // (pv_done cannot be used here: two phases may still be pending, which a parity wait cannot tell from none)
      if (!at_wait(o_done, 0, abort_flag)) fail(ST_TIMEOUT_MISC);
    }
    if (ok) {
      // merge the two halves' partial softmax results (running maximum, row sum, accumulator) of this row
      xm_s[half * 128 + r] = m_used;
      xm_s[(2 + half) * 128 + r] = l_sum;
      mbar_arrive(&pair_bar[quarter]);
      if (!at_wait(&pair_bar[quarter], 0, abort_flag)) fail(ST_TIMEOUT_MISC);
    }
    if (ok) {
      tc_fence_after();
      const float m0 = xm_s[r], m1 = xm_s[128 + r];
      const float l0 = xm_s[256 + r], l1 = xm_s[384 + r];
      const float m = fmaxf(m0, m1);
      const float a0 = (m0 == -INFINITY) ? 0.f : fast_exp2((m0 - m) * p.scale_log2);
      const float a1 = (m1 == -INFINITY) ? 0.f : fast_exp2((m1 - m) * p.scale_log2);
      const float l = l0 * a0 + l1 * a1;
      const float inv = l > 0.f ? 1.f / l : 0.f;
      const float w0 = a0 * inv, w1 = a1 * inv;
      __nv_bfloat16* o_row = p.O + (long)b * p.o_stride_b + (long)q * p.o_stride_s + (long)h * p.D;
      // thread (r, half) writes output columns [half * NCH * 32, +NCH * 32) of row r
#pragma unroll
      for (int cc = 0; cc < NCH; ++cc) {
        const int col0 = (half * NCH + cc) * 32;
        float o[32];
        if (it > 0) {
          uint32_t v0[32], v1[32];
          tmem_ld_32x32(tmem_O + col0 + lane_addr, v0);
          tmem_ld_32x32(tmem_O + 128 + col0 + lane_addr, v1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __uint_as_float(v0[i]) * w0 + __uint_as_float(v1[i]) * w1;
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (row_valid) {
#pragma unroll
          for (int g = 0; g < 4; ++g) {
            const int col = col0 + g * 8;
            if (col + 8 <= p.D) {
              uint4 u;
              u.x = pack_bf16x2(o[g * 8 + 0], o[g * 8 + 1]);
              u.y = pack_bf16x2(o[g * 8 + 2], o[g * 8 + 3]);
              u.z = pack_bf16x2(o[g * 8 + 4], o[g * 8 + 5]);
              u.w = pack_bf16x2(o[g * 8 + 6], o[g * 8 + 7]);
              *reinterpret_cast<uint4*>(o_row + col) = u;
            }
          }
        }
      }
      if (row_valid && half == 0)
        p.lse[((long)b * p.Hq + h) * p.Sq + q] = l > 0.f ? m * p.scale + logf(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

// 4-D view {D, H, S, B} of a [B][S][H][D]-like bf16 tensor with arbitrary token / batch strides.
static int make_qkv_tmap(CUtensorMap* tm, const void* base, int D, int H, int S, int B, long stride_s, long stride_b) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)D * 2, (uint64_t)stride_s * 2, (uint64_t)stride_b * 2};
  uint32_t box[4] = {64, 1, 128, 1};
  return make_tmap_nd_bf16(tm, base, 4, dims, strides, box);
}

}  // namespace csb

using namespace csb;

// cls: int8 [B][nQ][nK] with nQ = ceil(Sq/bm), nK = ceil(Sk/bn).  row_work (optional, int32 [B][nQ],
// zeroed by the caller) receives the number of non-empty key blocks of each query block.
CSB_API int csb_mask_classify(int mode, const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                              int B, int Sq, int Sk, int bm, int bn, signed char* cls, int* row_work, void* stream) {
  if (bm <= 0 || bn <= 0 || bn > 1024) return CSB_ERR_BAD_ARG;
  const int nQ = (Sq + bm - 1) / bm, nK = (Sk + bn - 1) / bn;
  dim3 grid(nK, nQ, B);
  mask_classify_kernel<<<grid, 128, bn * 12, reinterpret_cast<cudaStream_t>(stream)>>>(
      mode, reinterpret_cast<const int64_t*>(q_bits), reinterpret_cast<const int64_t*>(k_bits), q_pos, k_pos, Sq, Sk,
      bm, bn, nQ, nK, reinterpret_cast<int8_t*>(cls), row_work);
  return launch_result();
}

// q: [B][Sq][Hq][D]; keys / values as segments (see kv_segments.h), each a [B][rows][Hk][D] bf16 view (head stride D,
// token / batch strides in elements); Sk = sum of the segments' rows rounded up to 128 each (the padded gathered
// length that k_bits / k_pos / cls are indexed by); out: [B][Sq][Hq][D] view; lse: fp32 [B][Hq][Sq]; cls from
// csb_mask_classify with bm = bn = 128.
// Optional inputs of the dense-mask / bias form (flash attention with a boolean mask or an additive bias).
struct CsbAttnExtras {
  const unsigned char* dmask;  // bytes [B][Sq][Sk] (nonzero = attend), key index contiguous; used when mask_mode = MASK_DENSE
  long dm_sb, dm_sq;           // byte strides of batch and query index
  const float* bias;           // fp32, key index contiguous; null = none
  long bias_sb, bias_sh, bias_sq;  // element strides (0 = broadcast)
};

static int attn_fwd_seg_impl(const void* q, const CsbKvSegments* kv, void* out, float* lse, int B, int Sq, int Sk, int Hq,
                             int Hk, int D, long q_stride_s, long q_stride_b, long o_stride_s, long o_stride_b, float scale,
                             int mask_mode, const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                             const signed char* cls, int* status, void* stream, const CsbAttnExtras* ex) {
  if (D % 8 || D > 128 || D < 16 || Hq % Hk) return CSB_ERR_BAD_ARG;
  if (mask_mode == MASK_DENSE && (ex == nullptr || ex->dmask == nullptr)) return CSB_ERR_BAD_ARG;
  if (kv == nullptr || kv->n_seg < 1 || kv->n_seg > CSB_MAX_SEG) return CSB_ERR_BAD_ARG;
  if ((Sk + AT_BN - 1) / AT_BN > AttnSmem<2>::MAX_NK) return CSB_ERR_TOO_LARGE;
  if ((q_stride_s % 8) || (o_stride_s % 8)) return CSB_ERR_BAD_ARG;
  AttnFwdParams p;
  p.B = B; p.Sq = Sq; p.Sk = Sk; p.Hq = Hq; p.Hk = Hk; p.D = D;
  p.dk16 = (D + 15) / 16 * 16;
  p.nQ = (Sq + AT_BM - 1) / AT_BM;
  p.nK = (Sk + AT_BN - 1) / AT_BN;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.mask_mode = mask_mode;
  p.q_bits = reinterpret_cast<const int64_t*>(q_bits);
  p.k_bits = reinterpret_cast<const int64_t*>(k_bits);
  p.q_pos = q_pos; p.k_pos = k_pos;
  p.cls = reinterpret_cast<const int8_t*>(cls);
  p.O = reinterpret_cast<__nv_bfloat16*>(out);
  p.o_stride_b = o_stride_b; p.o_stride_s = o_stride_s;
  p.lse = lse;
  p.status = status;
  p.dmask = ex ? ex->dmask : nullptr;
  p.dm_sb = ex ? ex->dm_sb : 0; p.dm_sq = ex ? ex->dm_sq : 0;
  p.bias = ex ? ex->bias : nullptr;
  p.bias_sb = ex ? ex->bias_sb : 0; p.bias_sh = ex ? ex->bias_sh : 0; p.bias_sq = ex ? ex->bias_sq : 0;
  p.inv_scale = scale != 0.f ? 1.f / scale : 0.f;
  fill_seg_info(&p.seg, kv, AT_BN);
  if (p.seg.tile_start[kv->n_seg] != p.nK) return CSB_ERR_BAD_ARG;  // Sk must be the padded gathered length
  p.j_start = (kv->my_seg >= 0 && kv->my_seg < kv->n_seg) ? p.seg.tile_start[kv->my_seg] : 0;
  if (p.j_start >= p.nK) p.j_start = 0;
  CUtensorMap tq;
  KvMaps kvm;
  int r;
  if ((r = make_qkv_tmap(&tq, q, D, Hq, Sq, B, q_stride_s, q_stride_b))) return r;
  for (int i = 0; i < CSB_MAX_SEG; ++i) {
    const int g = i < kv->n_seg ? i : 0;  // unused slots repeat segment 0 (never dereferenced)
    if ((kv->k_stride_s[g] % 8) || (kv->v_stride_s[g] % 8)) return CSB_ERR_BAD_ARG;
    // with pulling blocks the tiles of a remote segment are read from its local copy
    const bool local_copy = p.seg.pull_ctas > 0 && g != kv->my_seg;
    if (local_copy && (kv->pull_k[g] == nullptr || kv->pull_v[g] == nullptr || (kv->pull_elems[g] % 8))) return CSB_ERR_BAD_ARG;
    const void* kb = local_copy ? kv->pull_k[g] : kv->k[g];
    const void* vb = local_copy ? kv->pull_v[g] : kv->v[g];
    if ((r = make_qkv_tmap(&kvm.k[i], kb, D, Hk, kv->rows[g], B, kv->k_stride_s[g], kv->k_stride_b[g]))) return r;
    if ((r = make_qkv_tmap(&kvm.v[i], vb, D, Hk, kv->rows[g], B, kv->v_stride_s[g], kv->v_stride_b[g]))) return r;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const long n_blocks = (long)p.nQ * Hq * B + p.seg.pull_ctas;
  if (n_blocks > 0x7fffffffL) return CSB_ERR_TOO_LARGE;
  dim3 grid((unsigned)n_blocks);
  if (D <= 64) {
    auto kfn = attn_fwd_kernel<1>;
    static bool set1 = false;
    if (!set1) { if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<1>::DYN_BYTES) != cudaSuccess) return launch_result(); set1 = true; }
    kfn<<<grid, 320, AttnSmem<1>::DYN_BYTES, s>>>(tq, kvm, p);
  } else {
    auto kfn = attn_fwd_kernel<2>;
    static bool set2 = false;
    if (!set2) { if (cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<2>::DYN_BYTES) != cudaSuccess) return launch_result(); set2 = true; }
    kfn<<<grid, 320, AttnSmem<2>::DYN_BYTES, s>>>(tq, kvm, p);
  }
  return launch_result();
}

CSB_API int csb_attn_fwd_seg(const void* q, const CsbKvSegments* kv, void* out, float* lse, int B, int Sq, int Sk, int Hq,
                             int Hk, int D, long q_stride_s, long q_stride_b, long o_stride_s, long o_stride_b, float scale,
                             int mask_mode, const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                             const signed char* cls, int* status, void* stream) {
  return attn_fwd_seg_impl(q, kv, out, lse, B, Sq, Sk, Hq, Hk, D, q_stride_s, q_stride_b, o_stride_s, o_stride_b, scale,
                           mask_mode, q_bits, k_bits, q_pos, k_pos, cls, status, stream, nullptr);
}

// Tile classes (128 x 128) of a dense boolean mask: bytes [B][Sq][Sk] with byte strides sb / sq.
CSB_API int csb_mask_classify_dense(const unsigned char* dmask, long sb, long sq, int B, int Sq, int Sk, signed char* cls,
                                    int* row_work, void* stream) {
  const int nQ = (Sq + 127) / 128, nK = (Sk + 127) / 128;
  dim3 grid(nK, nQ, B);
  mask_classify_dense_kernel<<<grid, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(dmask, sb, sq, Sq, Sk, 128, 128, nQ, nK,
                                                                                      reinterpret_cast<int8_t*>(cls), row_work);
  return launch_result();
}

// One local K/V tensor with a dense boolean mask (mask_mode = MASK_DENSE) and / or an additive bias.
CSB_API int csb_attn_fwd_dense(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                               int Hq, int Hk, int D, long q_stride_s, long q_stride_b, long k_stride_s, long k_stride_b,
                               long v_stride_s, long v_stride_b, long o_stride_s, long o_stride_b, float scale, int mask_mode,
                               const signed char* cls, const CsbAttnExtras* ex, int* status, void* stream) {
  CsbKvSegments kv = {};
  kv.n_seg = 1;
  kv.my_seg = 0;
  kv.rows[0] = Sk;
  kv.k[0] = k; kv.v[0] = v;
  kv.k_stride_s[0] = k_stride_s; kv.k_stride_b[0] = k_stride_b;
  kv.v_stride_s[0] = v_stride_s; kv.v_stride_b[0] = v_stride_b;
  kv.ready_flags = nullptr;
  return attn_fwd_seg_impl(q, &kv, out, lse, B, Sq, Sk, Hq, Hk, D, q_stride_s, q_stride_b, o_stride_s, o_stride_b, scale,
                           mask_mode, nullptr, nullptr, nullptr, nullptr, cls, status, stream, ex);
}

// One local K/V tensor: q: [B][Sq][Hq][D], k/v: [B][Sk][Hk][D] bf16 views.
CSB_API int csb_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int Sq, int Sk,
                         int Hq, int Hk, int D, long q_stride_s, long q_stride_b, long k_stride_s, long k_stride_b,
                         long v_stride_s, long v_stride_b, long o_stride_s, long o_stride_b, float scale, int mask_mode,
                         const long* q_bits, const long* k_bits, const int* q_pos, const int* k_pos,
                         const signed char* cls, int* status, void* stream) {
  CsbKvSegments kv = {};
  kv.n_seg = 1;
  kv.my_seg = 0;
  kv.rows[0] = Sk;
  kv.k[0] = k; kv.v[0] = v;
  kv.k_stride_s[0] = k_stride_s; kv.k_stride_b[0] = k_stride_b;
  kv.v_stride_s[0] = v_stride_s; kv.v_stride_b[0] = v_stride_b;
  kv.ready_flags = nullptr;
  // the kernel indexes k_bits / k_pos / cls by the unpadded Sk when there is a single segment
  return csb_attn_fwd_seg(q, &kv, out, lse, B, Sq, Sk, Hq, Hk, D, q_stride_s, q_stride_b, o_stride_s, o_stride_b, scale,
                          mask_mode, q_bits, k_bits, q_pos, k_pos, cls, status, stream);
}

CSB_WAIT_LIMIT_SETTER(attn_fwd)
