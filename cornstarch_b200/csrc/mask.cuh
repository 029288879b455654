// Attention-mask predicate shared by the mask-classification kernel and the attention kernels.
//
// Bitfield attention mask: one int64 per token.  Bit 0 = "is text"; bits 1..61 = modality ids; value
// 0 = padding.  Only the low 62 bits take part (bit 62 is set on text tokens by convention and is
// ignored).  Rule of the reference kernel (cornstarch/kernel/bitfield_attention.py:86-101):
//     text query      : k <= q  and  (q.bits & k.bits) != 0
//     modality query  : q.bits == k.bits            (bidirectional inside the same modality bits)
//     padding (0) attends to nothing and is attended by nothing.
// PREFIX_CAUSAL adds, for a modality query, every earlier non-padding key (k < q): an image is
// bidirectional inside itself and causal to everything before it.
#pragma once
#include <stdint.h>

namespace csb {

// MASK_DENSE: a boolean [B][Sq][Sk] byte matrix decides (read by the kernels for tiles of class 1); the predicate below
// is not used for it.
enum MaskMode : int { MASK_FULL = 0, MASK_CAUSAL = 1, MASK_BITFIELD = 2, MASK_BITFIELD_PREFIX_CAUSAL = 3, MASK_DENSE = 4 };

constexpr int64_t BITFIELD_LOW62 = (int64_t(1) << 62) - 1;

__host__ __device__ __forceinline__ bool mask_allowed(int mode, int64_t qb, int64_t kb, int qpos, int kpos) {
  if (mode == MASK_FULL) return true;
  if (mode == MASK_CAUSAL) return kpos <= qpos;
  qb &= BITFIELD_LOW62;
  kb &= BITFIELD_LOW62;
  if (qb == 0 || kb == 0) return false;
  if (qb & 1) return (kpos <= qpos) && ((qb & kb) != 0);
  if (qb == kb) return true;
  return (mode == MASK_BITFIELD_PREFIX_CAUSAL) && (kpos < qpos);
}

}  // namespace csb
