// Lane side of the encoder, shared by the encode kernels and the fused update
// kernel: append one tile's exponent pairs of a lane to its bit stream.
#pragma once

#include "common.cuh"
#include "decode_core.cuh"

namespace lct {

// Shared encode table: one uint2 per raw exponent byte, x = code bits (LSB first),
// y = code length.
__device__ __forceinline__ uint2 load_shared_code(uint32_t table, uint32_t exponent_byte) {
  uint2 c;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(c.x), "=r"(c.y) : "r"(table + exponent_byte * 8u));
  return c;
}

// Where a lane's finished 32-bit words go.  append() adds a pair's code to the word under
// construction and, when the pair that moved the position from `pos` to `next` left that word,
// stores it - as predicated instructions, no branch.
//
// ... its column of the block's shared payload image,
struct SharedWordSink {
  uint32_t column;  // shared address of word 0 of this lane
  __device__ __forceinline__ uint32_t address(int pos) const {
    return column + ((uint32_t)pos & ~31u) * (uint32_t)(kLanes * 4 / 32);
  }
  __device__ __forceinline__ void store(int pos, uint32_t word) const {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(address(pos)), "r"(word) : "memory");
  }
  // lo |= code << (pos & 31); when the pair left the word `pos` is in, store that word and start
  // the next one with the bits of `code` that did not fit (none when pos is word aligned).
  __device__ __forceinline__ void append(int pos, int next, uint32_t code, uint32_t& lo) const {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 t, d, w;\n\t"
        "shf.l.wrap.b32 t, 0, %1, %2;\n\t"
        "or.b32 %0, %0, t;\n\t"
        "xor.b32 d, %2, %3;\n\t"
        "setp.ge.u32 p, d, 32;\n\t"
        "and.b32 w, %2, -32;\n\t"
        "mad.lo.u32 w, w, 32, %4;\n\t"
        "@p st.shared.u32 [w], %0;\n\t"
        "@p shf.l.wrap.b32 %0, %1, 0, %2;\n\t"
        "}"
        : "+r"(lo)
        : "r"(code), "r"(pos), "r"(next), "r"(column)
        : "memory");
  }
};
// ... or straight to the payload in global memory (row stride = number of streams).
struct GlobalWordSink {
  uint32_t* column;
  int64_t stride;
  __device__ __forceinline__ uint32_t* address(int pos) const {
    return column + (int64_t)(pos >> 5) * stride;
  }
  __device__ __forceinline__ void store(int pos, uint32_t word) const { *address(pos) = word; }
  __device__ __forceinline__ void append(int pos, int next, uint32_t code, uint32_t& lo) const {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b32 t, d;\n\t"
        "shf.l.wrap.b32 t, 0, %1, %2;\n\t"
        "or.b32 %0, %0, t;\n\t"
        "xor.b32 d, %2, %3;\n\t"
        "setp.ge.u32 p, d, 32;\n\t"
        "@p st.global.u32 [%4], %0;\n\t"
        "@p shf.l.wrap.b32 %0, %1, 0, %2;\n\t"
        "}"
        : "+r"(lo)
        : "r"(code), "r"(pos), "r"(next), "l"(address(pos))
        : "memory");
  }
};

// One pair of one lane (kPair: its index in the tile).  Returns false when the pair does not fit
// the lane's budget any more.  The instruction sequence is spelled out: two byte loads of the
// lane's exponents, their table rows (address = byte * 8 + table on the multiplier pipe), code
// and position, then the append; a finished word is stored by predicated instructions.
template <bool kCheckValid, int kPair, typename WordSink, typename Slices>
__device__ __forceinline__ bool encode_pair(uint32_t table, const uint32_t (&slot)[4],
                                            const WordSink& sink, int step0, int valid,
                                            int budget_bits, int& pos, uint32_t& lo,
                                            int& extra_start, Slices& slices) {
  uint32_t code0, length0, code1, length1;
  asm volatile(
      "{\n\t.reg .b32 a0, a1;\n\t"
      "ld.shared.u8 a0, [%4+%5];\n\t"
      "ld.shared.u8 a1, [%4+%6];\n\t"
      "mad.lo.u32 a0, a0, 8, %7;\n\t"
      "mad.lo.u32 a1, a1, 8, %7;\n\t"
      "ld.shared.v2.u32 {%0, %1}, [a0];\n\t"
      "ld.shared.v2.u32 {%2, %3}, [a1];\n\t"
      "}"
      : "=r"(code0), "=r"(length0), "=r"(code1), "=r"(length1)
      : "r"(slot[kPair & 3]), "n"(kPair * 64), "n"(kPair * 64 + 1), "r"(table));
  // Issued behind the lookups and ahead of their first use: this is what runs while they are
  // in flight (a warp issues in order).
  slices.template slice<kPair % kHalfPairs>();
  if (kCheckValid) {  // padding carries no bits
    if (step0 + 2 * kPair >= valid) { code0 = 0u; length0 = 0u; }
    if (step0 + 2 * kPair + 1 >= valid) { code1 = 0u; length1 = 0u; }
  }
  const uint32_t code = code0 | (code1 << length0);
  const int next = pos + (int)length0 + (int)length1;
  if (next > budget_bits) {
    // First pair that does not fit: freeze the current word and stop.
    extra_start = step0 + 2 * kPair;
    if (pos < budget_bits) sink.store(pos, lo);
    return false;
  }
  sink.append(pos, next, code, lo);
  pos = next;
  return true;
}

// Pairs kPair .. kEnd - 1 of a tile of one lane, unrolled; after each pair one slice of the
// caller's row-side work is issued (see NoSlices in decode_core.cuh).  A lane that has
// overflowed (`open` false) only runs the slices.
template <bool kCheckValid, int kPair, int kEnd, typename WordSink, typename Slices>
struct EncodePairs {
  static __device__ __forceinline__ void run(uint32_t table, const uint32_t (&slot)[4],
                                             const WordSink& sink, int step0, int valid,
                                             int budget_bits, int& pos, uint32_t& lo,
                                             int& extra_start, bool& open, Slices& slices) {
    if (open)
      open = encode_pair<kCheckValid, kPair>(table, slot, sink, step0, valid, budget_bits, pos, lo,
                                             extra_start, slices);
    else
      slices.template slice<kPair % kHalfPairs>();
    EncodePairs<kCheckValid, kPair + 1, kEnd, WordSink, Slices>::run(
        table, slot, sink, step0, valid, budget_bits, pos, lo, extra_start, open, slices);
  }
};
template <bool kCheckValid, int kEnd, typename WordSink, typename Slices>
struct EncodePairs<kCheckValid, kEnd, kEnd, WordSink, Slices> {
  static __device__ __forceinline__ void run(uint32_t, const uint32_t (&)[4], const WordSink&, int,
                                             int, int, int&, uint32_t&, int&, bool&, Slices&) {}
};

// Lane phase of part of a tile (row pairs kHalf * kPairs .. + kPairs - 1, half a tile by default,
// of the tile that starts at row `step0`;
// tile layout: see tile_slot_xor).  `open` turns false once the lane has overflowed.  `table`:
// shared address of the encode table; `tile_lane`: shared address of this lane's slot in row
// pair 0 of the warp's tile.
template <bool kCheckValid, int kLaneMask, int kHalf, typename WordSink, typename Slices,
          int kPairs = kHalfPairs>
__device__ __forceinline__ void encode_half_rows(uint32_t table, uint32_t tile_lane,
                                                 const WordSink& sink, int lane_mask, int step0,
                                                 int valid, int budget_bits, int& pos,
                                                 uint32_t& lo, int& extra_start, bool& open,
                                                 Slices& slices) {
  const uint32_t slot[4] = {tile_lane ^ tile_slot_xor<kLaneMask>(0, lane_mask),
                            tile_lane ^ tile_slot_xor<kLaneMask>(1, lane_mask),
                            tile_lane ^ tile_slot_xor<kLaneMask>(2, lane_mask),
                            tile_lane ^ tile_slot_xor<kLaneMask>(3, lane_mask)};
  EncodePairs<kCheckValid, kHalf * kPairs, (kHalf + 1) * kPairs, WordSink, Slices>::run(
      table, slot, sink, step0, valid, budget_bits, pos, lo, extra_start, open, slices);
}

// Lane phase of one whole tile, nothing interleaved.  Returns false once the lane has overflowed.
template <bool kCheckValid, int kLaneMask, typename WordSink>
__device__ __forceinline__ bool encode_tile_rows(uint32_t table, uint32_t tile_lane,
                                                 const WordSink& sink, int lane_mask, int step0,
                                                 int valid, int budget_bits, int& pos,
                                                 uint32_t& lo, int& extra_start) {
  NoSlices none;
  bool open = true;
#pragma unroll 1
  for (int part = 0; part < kTilePairs / kLoopPairs; ++part)  // one copy of the code: see decode_tile_rows
    encode_half_rows<kCheckValid, kLaneMask, 0, WordSink, NoSlices, kLoopPairs>(
        table, tile_lane + (uint32_t)(part * kLoopPairs * 64), sink, lane_mask,
        step0 + part * 2 * kLoopPairs, valid, budget_bits, pos, lo, extra_start, open, none);
  return open;
}

}  // namespace lct
