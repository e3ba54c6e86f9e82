// Lane side of the encoder, shared by the encode kernels and the fused update
// kernel: append one tile's exponent pairs of a lane to its bit stream.
#pragma once

#include "common.cuh"

namespace lct {

// Unroll factor of the lane-phase loop (16 pairs per tile).
#ifndef LCT_ENCODE_UNROLL
#define LCT_ENCODE_UNROLL 16
#endif
#define LCT_ENCODE_PRAGMA(x) _Pragma(#x)
#define LCT_ENCODE_UNROLL_(n) LCT_ENCODE_PRAGMA(unroll n)
#define LCT_ENCODE_UNROLL_PRAGMA LCT_ENCODE_UNROLL_(LCT_ENCODE_UNROLL)

// Lane phase of one tile.  Returns false once the lane has overflowed.
template <bool kCheckValid>
__device__ __forceinline__ bool encode_tile_rows(const uint2* table, const uint8_t* tile_bytes,
                                                 uint32_t* payload_column, int64_t word_stride,
                                                 int lane32, int lane_mask,
                                                 int step0, int valid, int budget_bits, int& pos,
                                                 uint32_t& lo, int& extra_start) {
  LCT_ENCODE_UNROLL_PRAGMA
  for (int p = 0; p < kTilePairs; ++p) {
    // Tiles start on multiples of 32 rows, so the low mask bits of pair p are 2p & lane_mask.
    const uint8_t* e = tile_bytes + 2 * (p * 32 + (lane32 ^ ((2 * p) & lane_mask)));
    uint2 c0 = table[e[0]];
    uint2 c1 = table[e[1]];
    if (kCheckValid) {  // padding carries no bits
      if (step0 + 2 * p >= valid) c0 = make_uint2(0u, 0u);
      if (step0 + 2 * p + 1 >= valid) c1 = make_uint2(0u, 0u);
    }
    const uint32_t code = c0.x | (c1.x << c0.y);
    const int length = (int)(c0.y + c1.y);
    const int shift = pos & 31;
    const int next = pos + length;
    if (next > budget_bits) {
      // First pair that does not fit: freeze the current word and stop.
      extra_start = step0 + 2 * p;
      if (pos < budget_bits) payload_column[(pos >> 5) * word_stride] = lo;
      return false;
    }
    lo |= code << shift;
    if (shift + length >= 32) {
      payload_column[(pos >> 5) * word_stride] = lo;
      lo = __funnelshift_l(code, 0u, shift);  // the bits that did not fit; 0 when shift == 0
    }
    pos = next;
  }
  return true;
}

}  // namespace lct
