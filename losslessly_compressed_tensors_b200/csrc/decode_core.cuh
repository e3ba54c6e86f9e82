// Device building blocks shared by the decoder, the fused pointwise kernels and
// the fused update kernel: operand views, the per-CTA prologue (staging of the
// payload and of the center's two-symbol table, overflow map), the lane-side
// stream cursor and tile decoder, the row-side BF16 join/split, the arithmetic
// of the fused operations, and the host-side argument checks.
#pragma once

#include "common.cuh"
#include "lct_b200.h"

namespace lct {

struct OperandView {
  const uint32_t* encoded;
  const uint8_t* side;
  const int32_t* center;
  const uint32_t* pair_table;
  const uint8_t* lanes;
  const uint8_t* starts;
  const uint8_t* tail;
  const int32_t* descriptor;
  const int32_t* count;
  const int32_t* blocks;
  int64_t base;
  int mode;
};

struct Shape {
  int64_t size;
  int64_t logical_numel;
  int64_t streams;
  int64_t n_blocks;
  int block_symbols;
  int steps;
  int fixed_words;
  int rare_length;
  int lane_mask;  // 254: lane ^ (row & 254) ("swizzle"); 0: "linear"
};

// Shared memory of a decoding CTA with n operands (n = 2 only for the fused operation on two
// compressed tensors):
//
//   table 0 .. n-1   the 4096-entry two-symbol table of each operand's center, 16 KB each.  They
//                    come first so that their shared addresses do not depend on the geometry:
//                    a lookup is then one load at (window & 0x3FFC) + a constant.
//   (the fused update keeps its 2 KB encode table here, for the same reason)
//   then per operand:
//   image            the block's payload: fixed_words rows of 256 words,
//                    then two zero rows                                          (fixed_words + 2) KB
//   DecodeHead       warp tiles, byte table, overflow map, scan scratch         kHeadBytes
//
// A lane opens its stream with the image row in FRONT of its first word (see ShiftCursor), so
// the kilobyte before the image must be readable: it is the end of the tables or of the
// previous operand's head.  A well-formed stream is never read past the image's second zero
// row; a lane's fetch address is pulled back to that row once per half tile and can run at
// most 8 rows further inside one, which is the head (garbage in, garbage out, but never an
// out-of-range access).
struct __align__(16) DecodeHead {
  uint16_t tile[kWarps][kTilePairs * 32];
  uint8_t index_to_byte[256];
  uint16_t overflow_start[kLanes];
  int32_t overflow_offset[kLanes];
  int scan[36];
};
constexpr size_t kHeadBytes = 10240;
constexpr size_t kTableBytes = (size_t)kPairEntries * 4;
static_assert(sizeof(DecodeHead) <= kHeadBytes, "head must fit its slot");
static_assert(kHeadBytes % 1024 == 0 && kHeadBytes >= 9 * 1024,
              "a lane may fetch up to 9 rows past the image");

struct OperandShared {
  DecodeHead* head;
  uint32_t* image;
  uint32_t* table;
};

static inline __host__ __device__ size_t payload_image_bytes(int fixed_words) {
  return (size_t)(fixed_words + 2) * kLanes * 4;
}
// Shared memory per operand (its table included).
static inline __host__ __device__ size_t operand_shared_bytes(int fixed_words) {
  return kTableBytes + kHeadBytes + payload_image_bytes(fixed_words);
}
// Operand `index` of `count` in the CTA's dynamic shared memory.  `extra_bytes` (a multiple of
// 16) are left free between the tables and the first operand's head for the caller's own
// fixed-address data.
__device__ __forceinline__ OperandShared carve_operand(unsigned char* base, int index, int count,
                                                       int fixed_words, size_t extra_bytes = 0) {
  const size_t rest = kHeadBytes + payload_image_bytes(fixed_words);
  unsigned char* own = base + (size_t)count * kTableBytes + extra_bytes + (size_t)index * rest;
  OperandShared s;
  s.table = reinterpret_cast<uint32_t*>(base + (size_t)index * kTableBytes);
  s.image = reinterpret_cast<uint32_t*>(own);
  s.head = reinterpret_cast<DecodeHead*>(own + payload_image_bytes(fixed_words));
  return s;
}

__device__ __forceinline__ void cp_async_16(void* shared_dst, const void* global_src) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(shared_dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(global_src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* shared_dst, const void* global_src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                   (uint32_t)__cvta_generic_to_shared(shared_dst)),
               "l"(global_src));
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;\n" ::: "memory");
}

// ---- shared memory by 32-bit address (lane phases) -------------------------
// The lane phases address shared memory with 32-bit window addresses and constant
// byte offsets, so that a lookup is one load with an immediate and no 64-bit
// pointer arithmetic.
__device__ __forceinline__ uint32_t shared_address(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
template <int kByteOffset = 0>
__device__ __forceinline__ uint32_t load_shared_u32(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(address), "n"(kByteOffset));
  return v;
}
__device__ __forceinline__ uint32_t load_shared_u8(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u8 %0, [%1];" : "=r"(v) : "r"(address));
  return v;
}
template <int kByteOffset = 0>
__device__ __forceinline__ uint32_t load_shared_u16(uint32_t address) {
  uint32_t v;
  asm volatile("ld.shared.u16 %0, [%1+%2];" : "=r"(v) : "r"(address), "n"(kByteOffset));
  return v;
}
template <int kByteOffset = 0>
__device__ __forceinline__ void store_shared_u16(uint32_t address, uint32_t value) {
  asm volatile("st.shared.u16 [%0+%1], %2;" ::"r"(address), "n"(kByteOffset),
               "h"((unsigned short)value)
               : "memory");
}
__device__ __forceinline__ void store_shared_u16_at(uint32_t address, uint32_t value) {
  asm volatile("st.shared.u16 [%0], %1;" ::"r"(address), "h"((unsigned short)value) : "memory");
}

__device__ __forceinline__ uint32_t funnel_right(uint32_t low, uint32_t high, uint32_t amount) {
  return __funnelshift_r(low, high, amount);  // the amount is taken modulo 32
}
// a + sum over the four bytes of e (unsigned) * w (signed): with w = -1 in one byte this
// subtracts that byte of e from a.
__device__ __forceinline__ int dot_bytes(uint32_t e, int w, int a) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(e), "r"(w), "r"(a));
  return d;
}

// Shared address of the table entry for the window at bits 2..13 of `bits4` (the two low bits
// are ignored).  The tables sit at fixed offsets of the CTA's shared memory, so `table` is a
// constant that folds into the load's immediate.
__device__ __forceinline__ uint32_t entry_address(uint32_t bits4, uint32_t table) {
  return (bits4 & 0x3FFCu) + table;
}

// Read position of one lane: the next 94 stream bits in three registers, already shifted so
// that the bit under the position is bit 2 of `lo` (bits 0..1 are the two bits before it).
// A lookup is then  entry = table[lo & 0x3FFC]  and consuming n bits is three funnel shifts
// whose amount is the low five bits of a register, i.e. the table entry itself, so the
// dependent chain from one lookup to the next is  mask -> shared load -> shift.
// `valid` counts the loaded bits of the 96 (at least 64 at every check): when fewer than 64
// are left, the next word of the lane's column is inserted above them.  Refills are off the
// lookup chain.  Up to 31 bits may be consumed between two checks.
struct ShiftCursor {
  uint32_t lo, mid, hi;
  int valid;
  uint32_t next;  // shared address of the next unread word of this lane
  uint32_t last;  // shared address of this lane's word in the image's second zero row

  __device__ __forceinline__ void open(const uint32_t* image, int lane, int fixed_words) {
    const uint32_t before = shared_address(image + lane) - (uint32_t)(kLanes * 4);
    const uint32_t v0 = load_shared_u32<0>(before);  // shifted out: any readable word will do
    const uint32_t v1 = load_shared_u32<kLanes * 4>(before);
    const uint32_t v2 = load_shared_u32<2 * kLanes * 4>(before);
    lo = funnel_right(v0, v1, 30u);
    mid = funnel_right(v1, v2, 30u);
    hi = v2 >> 30;
    valid = 66;
    next = before + 3u * kLanes * 4u;
    last = before + (uint32_t)(fixed_words + 2) * kLanes * 4u;
  }
  __device__ __forceinline__ uint32_t window() const { return lo; }
  // `amount`: only its low five bits count.
  __device__ __forceinline__ void shift_out(uint32_t amount) {
    lo = funnel_right(lo, mid, amount);
    mid = funnel_right(mid, hi, amount);
    hi = funnel_right(hi, 0u, amount);
  }
  // When fewer than 64 bits are loaded, insert the lane's next word above them.
  __device__ __forceinline__ void refill() {
    if (valid < 64) {
      const uint32_t word = load_shared_u32<0>(next);
      next += (uint32_t)(kLanes * 4);
      mid |= __funnelshift_l(0u, word, (uint32_t)valid);  // word << (valid - 32)
      hi = __funnelshift_l(word, 0u, (uint32_t)valid);    // the bits of word that did not fit
      valid += 32;
    }
  }
  // Once per half tile: a lane never fetches more than 9 words past this (8 pairs of at most 32
  // bits), which still lies inside the CTA's shared memory (the image is followed by the head).
  __device__ __forceinline__ void half_start() { next = min(next, last); }
  // Consume a full-pair entry (refill separately).
  __device__ __forceinline__ void take_pair(uint32_t entry) {
    shift_out(entry);
    valid = dot_bytes(entry, (int)0xFF000000u, valid);
  }
  // Consume `bits` (<= 31) and refill.
  __device__ __forceinline__ void take(uint32_t bits) {
    shift_out(bits);
    valid -= (int)bits;
    refill();
  }
};

using LaneReader = ShiftCursor;


// What the lane phase of one thread needs besides its cursor.
struct LaneTables {
  uint32_t table;       // shared address of the two-symbol table
  uint32_t byte_table;  // shared address of index_to_byte[256]
  uint32_t tile_lane;   // shared address of this lane's slot in row pair 0 of the warp's tile
};

// Tile layout.  tile[p][x], x = 0..31, holds e(row 2p) | e(row 2p+1) << 8 of the lane
// x ^ (2p & lane_mask & 6), i.e. of column c = x ^ (2p & lane_mask & 0x18): inside an aligned
// group of 8 the tile is in column order, while the groups keep the lanes' order.  A lane
// therefore only applies the two low mask bits (four address values, constant when the loop is
// unrolled), and the row side, which needs the group bits for its side bytes anyway, reads or
// writes group j ^ (2p & lane_mask & 0x18) / 8 for its columns 8j..8j+7.
template <int kLaneMask>
__device__ __forceinline__ uint32_t tile_slot_xor(int p, int lane_mask) {
  const int mask = kLaneMask >= 0 ? kLaneMask : lane_mask;
  return (uint32_t)(((2 * p) & mask & 6) << 1);
}

constexpr unsigned kFullWarp = 0xFFFFFFFFu;

// The rest of a pair whose table entry is not a full pair.  The entry still carries its
// first symbol and that symbol's length, and take_pair(entry) has already shifted that length
// out of the cursor (and subtracted the entry's flag byte from the bit counter, which is put
// right here); `before` is the window the entry was looked up with.  Accounts for the first
// symbol, looks the second one up on its own and consumes it.
// Returns (e0 | e1 << 8) << 8, the form a full-pair entry has.
template <typename Reader>
__device__ __forceinline__ uint32_t finish_slow_pair(Reader& r, uint32_t entry, uint32_t before,
                                                     const LaneTables& t, int rare_length) {
  // All three lookups are issued before any of them is used: the literal of the first symbol,
  // the entry of the second (the cursor's low word is valid whatever the bit counter says) and
  // the literal it would have.
  const uint32_t bits1 = r.window();
  const uint32_t literal0 = load_shared_u8(t.byte_table + ((before >> (rare_length + 2)) & 255u));
  const uint32_t second = load_shared_u32(entry_address(bits1, t.table));
  const uint32_t literal1 = load_shared_u8(t.byte_table + ((bits1 >> (rare_length + 2)) & 255u));
  r.valid += (int)(entry >> 24) - (int)(entry & 31u);
  r.refill();
  const uint32_t e0 = (entry & kEscape) ? literal0 : entry_first_symbol(entry);
  const uint32_t e1 = (second & kEscape) ? literal1 : entry_first_symbol(second);
  r.take(entry_first_length(second));
  return (e0 << 8) | (e1 << 16);
}

constexpr int kHalfPairs = kTilePairs / 2;  // a half tile: 8 row pairs = 16 rows

// Work of the caller that is issued between the pairs of a lane phase (slice<k>() after pair k
// of a half tile, k = 0..7; rest() for whatever the lane phase did not get to).  The lane
// phase is one dependent chain per lane (mask -> table load -> shift); independent row-side
// work placed between its links fills the chain's latency, and spreads the row side's memory
// traffic over the whole iteration.
struct NoSlices {
  template <int k> __device__ __forceinline__ void slice() {}
  __device__ __forceinline__ void rest() {}
};

// One fully coded pair of every lane of the warp (kPair: its index in the tile, a compile-time
// constant so that the tile address is a register plus an immediate).
template <int kPair, typename Reader, typename Slices>
__device__ __forceinline__ void decode_pair_uniform(Reader& r, const LaneTables& t,
                                                    const uint32_t (&slot)[4], int rare_length,
                                                    Slices& slices) {
  const uint32_t before = r.window();
  uint32_t entry = load_shared_u32(entry_address(before, t.table));
  // Issued behind the lookup and ahead of its first use: this is what runs while the lookup is
  // in flight (a warp issues in order).
  slices.template slice<kPair % kHalfPairs>();
  r.take_pair(entry);
  // The rare entry that is not a full pair: a plain divergent branch.  (Asking the warp first
  // with a vote, so that the common case is a uniform branch, was measured 5 % slower: the vote
  // and its predicate sit on every pair's path.)
  if ((int32_t)entry < 0) entry = finish_slow_pair(r, entry, before, t, rare_length);
  if (kPair & 1) r.refill();  // two full pairs take at most 24 bits: one check serves both
  store_shared_u16<kPair * 64>(slot[kPair & 3], entry >> 8);
}

// Pairs kPair .. kEnd - 1 of a tile, unrolled.
template <int kPair, int kEnd, typename Reader, typename Slices>
struct UniformPairs {
  static __device__ __forceinline__ void run(Reader& r, const LaneTables& t,
                                             const uint32_t (&slot)[4], int rare_length,
                                             Slices& slices) {
    decode_pair_uniform<kPair>(r, t, slot, rare_length, slices);
    UniformPairs<kPair + 1, kEnd, Reader, Slices>::run(r, t, slot, rare_length, slices);
  }
};
template <int kEnd, typename Reader, typename Slices>
struct UniformPairs<kEnd, kEnd, Reader, Slices> {
  static __device__ __forceinline__ void run(Reader&, const LaneTables&, const uint32_t (&)[4], int,
                                             Slices&) {}
};

// Lane phase for part of a tile: row pairs kHalf * kPairs .. + kPairs - 1 (half a tile by
// default) of the tile that starts at row `step0` of the block.  `coded` = number of leading steps of this lane that are in the bit stream (its
// overflow start or its valid length, whichever is first); steps from `tail_from` on come from
// the raw tail.  `slices`: see NoSlices; all of its work has been issued on return.
template <int kLaneMask, int kHalf, typename Reader, typename Slices, int kPairs = kHalfPairs>
__device__ __forceinline__ void decode_half_rows(Reader& r, const LaneTables& t, int step0,
                                                 int coded, int tail_from,
                                                 const uint8_t* tail_bytes, int rare_length,
                                                 int lane_mask, Slices& slices) {
  static_assert(kPairs % 2 == 0 && kPairs <= kHalfPairs, "whole refill periods, at most half a tile");
  const int first = step0 + kHalf * 2 * kPairs;
  r.half_start();
  if (__all_sync(kFullWarp, first + 2 * kPairs <= coded)) {
    // Every lane of the warp has all 16 rows in its stream: no per-lane conditions except the
    // rare entry that is not a full pair.  The four tile addresses a lane uses (see
    // tile_slot_xor):
    const uint32_t slot[4] = {t.tile_lane ^ tile_slot_xor<kLaneMask>(0, lane_mask),
                              t.tile_lane ^ tile_slot_xor<kLaneMask>(1, lane_mask),
                              t.tile_lane ^ tile_slot_xor<kLaneMask>(2, lane_mask),
                              t.tile_lane ^ tile_slot_xor<kLaneMask>(3, lane_mask)};
    UniformPairs<kHalf * kPairs, (kHalf + 1) * kPairs, Reader, Slices>::run(r, t, slot, rare_length,
                                                                            slices);
    return;
  }
#pragma unroll 1
  for (int p = kHalf * kPairs; p < (kHalf + 1) * kPairs; ++p) {
    const int step = step0 + 2 * p;
    uint32_t pair = 0;
    if (step + 2 <= coded) {
      const uint32_t before = r.window();
      pair = load_shared_u32(entry_address(before, t.table));
      r.take_pair(pair);
      if ((int32_t)pair < 0) {
        pair = finish_slow_pair(r, pair, before, t, rare_length);
      } else {
        r.refill();
      }
      pair >>= 8;
    } else if (step >= tail_from) {
      const uint32_t t0 = tail_bytes[step - tail_from], t1 = tail_bytes[step + 1 - tail_from];
      pair = ((t0 + 127u) & 255u) | (((t1 + 127u) & 255u) << 8);
    } else if (step + 1 == coded) {
      // The lane's last coded step is the first row of this pair.
      const uint32_t before = r.window();
      const uint32_t entry = load_shared_u32(entry_address(before, t.table));
      pair = entry_first_symbol(entry);
      if (entry & kEscape)
        pair = load_shared_u8(t.byte_table + ((before >> (rare_length + 2)) & 255u));
      r.take(entry_first_length(entry));
    }
    store_shared_u16_at((t.tile_lane ^ tile_slot_xor<kLaneMask>(p, lane_mask)) + (uint32_t)(p * 64),
                        pair);
  }
  slices.rest();
}

// Lane phase for one whole tile, nothing interleaved.  The tile's row pairs run through ONE copy
// of the code for kLoopPairs pairs (each part's tile rows are kLoopPairs * 64 bytes further on),
// which keeps kernels that also hold an encoder within the instruction cache.
constexpr int kLoopPairs = 8;  // measured on the fused update: 8 -> 62.1 us, 4 -> 63.0, 2 -> 64.5, 16 (unrolled) -> 69.8
template <int kLaneMask, typename Reader>
__device__ __forceinline__ void decode_tile_rows(Reader& r, const LaneTables& t, int step0,
                                                 int coded, int tail_from,
                                                 const uint8_t* tail_bytes, int rare_length,
                                                 int lane_mask) {
  NoSlices none;
  LaneTables part_tables = t;
#pragma unroll 1
  for (int part = 0; part < kTilePairs / kLoopPairs; ++part) {
    decode_half_rows<kLaneMask, 0, Reader, NoSlices, kLoopPairs>(
        r, part_tables, step0 + part * 2 * kLoopPairs, coded, tail_from, tail_bytes, rare_length,
        lane_mask, none);
    part_tables.tile_lane += (uint32_t)(kLoopPairs * 64);
  }
}

struct NoExtraWork {
  __device__ __forceinline__ void operator()() const {}
};

// CTA prologue: stage the payload and the symbol table of the tensor's center,
// expand this block's overflow map.  Ends with a block barrier.
// `before_barrier` runs once per thread after this block's loads have been issued and before
// the closing barrier (work of the caller that the same barrier should publish).
template <typename Extra = NoExtraWork>
__device__ __forceinline__ void prepare_block(const OperandShared& sh, const OperandView& a,
                                              const Shape& g, int64_t block,
                                              Extra before_barrier = Extra()) {
  const int tid = threadIdx.x;
  DecodeHead& head = *sh.head;
  // Word w of the block's 256 streams is one contiguous, 1 KB aligned row.
  const uint32_t* rows = a.encoded + block * kLanes;
  for (int i = tid; i < g.fixed_words * (kLanes / 4); i += kThreads) {
    const int w = i >> 6, c = (i & 63) * 4;
    cp_async_16(&sh.image[w * kLanes + c], rows + (int64_t)w * g.streams + c);
  }
  sh.image[g.fixed_words * kLanes + tid] = 0u;
  sh.image[(g.fixed_words + 1) * kLanes + tid] = 0u;

  // The codebook's table for this tensor's center, ready to use (symbols are exponent bytes).
  const int center = *a.center;
  const uint32_t* source = a.pair_table + (size_t)((center + 128) & 255) * kPairEntries;
  for (int i = tid; i < kPairEntries / 4; i += kThreads) cp_async_16(&sh.table[4 * i], source + 4 * i);
  head.index_to_byte[tid] = (uint8_t)index_to_exponent_byte((uint32_t)tid, center);
  head.overflow_start[tid] = (uint16_t)g.steps;
  head.overflow_offset[tid] = 0;
  __syncthreads();
  if (a.mode != 0) {
    bool usable = true;
    int64_t region = 0;
    int total = 0;
    if (a.mode == 2) {
      usable = a.descriptor[2] == 0;
      region = a.descriptor[0];
      total = *a.count;
    }
    const int count = usable ? a.blocks[block] : 0;
    if (count > 0) {  // uniform across the CTA
      const int64_t first = a.blocks[g.n_blocks + block];
      const int byte_base = a.blocks[2 * g.n_blocks + block];
      const int64_t lane_at = (a.mode == 2 ? region : 0) + first;
      const int64_t start_at = (a.mode == 2 ? region + total : 0) + first;
      int lane = 0, start = g.steps;
      if (tid < count) {
        lane = a.lanes[lane_at + tid];
        start = a.starts[start_at + tid];
      }
      int unused;
      const int prefix = block_exclusive_scan(tid < count ? g.steps - start : 0, head.scan, &unused);
      if (tid < count) {
        head.overflow_start[lane] = (uint16_t)start;
        head.overflow_offset[lane] = byte_base + prefix;
      }
    }
  }
  before_barrier();
  cp_async_wait_all();
  __syncthreads();
}

__device__ __forceinline__ const uint8_t* tail_origin(const OperandView& a) {
  if (a.mode == 2) return a.tail + a.descriptor[0] + 2 * (int64_t)(*a.count);
  return a.tail + a.base;
}

// Per-lane state of a decoding thread, set up after prepare_block.
struct LaneState {
  LaneReader reader;
  LaneTables tables;
  const uint8_t* tail_bytes;
  int tail_from;
  int coded;
};

__device__ __forceinline__ LaneState open_lane(const OperandShared& sh, const OperandView& a,
                                               const Shape& g, int valid) {
  const int tid = threadIdx.x;
  LaneState s;
  s.tail_from = sh.head->overflow_start[tid];
  s.coded = min(valid, s.tail_from);
  s.tail_bytes = a.mode ? tail_origin(a) + sh.head->overflow_offset[tid] : nullptr;
  s.reader.open(sh.image, tid, g.fixed_words);
  s.tables.table = shared_address(sh.table);
  s.tables.byte_table = shared_address(sh.head->index_to_byte);
  s.tables.tile_lane = shared_address(&sh.head->tile[tid >> 5][tid & 31]);
  return s;
}

// Where one row-phase unit (row pair p of the tile, 8-column subgroup j4 of the
// warp's 32 columns) lives in the tensor and in the tile.
struct UnitPlace {
  int64_t logical;   // element offset of the top row's first column
  int64_t storage;   // byte offset of the top row's first lane in the side bytes
  uint32_t q;        // pair permutation between lane order and column order
  int tile_index;    // uint16 index of the unit's 8 tile entries (column order)
};

__device__ __forceinline__ UnitPlace place_unit(int warp, int p, int j4, int64_t row0, int step0,
                                                int64_t block_base, int lane_mask) {
  // All 32 rows of a tile share mask bits 5..7; bits 1..4 of pair p are 2p (all & lane_mask).
  const int64_t tile_row = row0 + step0;
  const int in_tile = (2 * p) & lane_mask;
  const int group = warp ^ ((int)(tile_row & lane_mask) >> 5);
  const int swapped = (8 * j4) ^ (in_tile & 0x18);
  UnitPlace u;
  u.logical = (tile_row + 2 * p) * kLanes + 32 * group + 8 * j4;
  u.storage = block_base + (int64_t)(step0 + 2 * p) * kLanes + 32 * warp + swapped;
  u.q = (uint32_t)(in_tile >> 1) & 3u;
  u.tile_index = p * 32 + swapped;
  return u;
}

// PRMT selectors that spread the side bytes of lane pair (i ^ q) of an 8-lane group over the
// two BF16 halves of output word i: bytes [s_a, s_a, s_b, s_b].
struct SideSelectors {
  uint32_t word[4];
};
__device__ __forceinline__ SideSelectors side_selectors(uint32_t q) {
  SideSelectors s;
#pragma unroll
  for (uint32_t i = 0; i < 4; ++i) s.word[i] = 0x1100u + 2u * (i ^ q) * 0x1111u;
  return s;
}

// Rebuild the 8 BF16 values (4 words, column order) of one row from the unit's tile words
// (column pairs, both rows) and that row's side bytes (lane order).  Per output word:
// exponents of the row into bits 7..14 of both halves (one shift), side bytes spread by one
// byte permute, merged by one bit select.
__device__ __forceinline__ void join_row(const uint4& tile_words, uint2 side_lane_order,
                                         const SideSelectors& sel, bool second_row,
                                         uint32_t out[4]) {
  const uint32_t tw[4] = {tile_words.x, tile_words.y, tile_words.z, tile_words.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const uint32_t exponents = second_row ? (tw[i] >> 1) : (tw[i] << 7);
    const uint32_t sides = prmt(side_lane_order.x, side_lane_order.y, sel.word[i]);
    out[i] = (exponents & 0x7F807F80u) | (sides & 0x807F807Fu);
  }
}

struct OpSpec {
  const float* alpha;
  const float* beta;
  int op;
  int alpha_is_one;
  int beta_is_one;
};

__device__ __forceinline__ float bf16_low(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_high(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

__device__ __forceinline__ uint32_t pack_rn(float low, float high) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(low, high);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// torch.lerp(start, end, weight) in float32, as PyTorch's CUDA kernel evaluates it.
__device__ __forceinline__ float lerp_f32(float start, float end, float weight) {
  const float d = __fsub_rn(end, start);
  return fabsf(weight) < 0.5f ? __fmaf_rn(weight, d, start)
                              : __fmaf_rn(-d, __fsub_rn(1.0f, weight), end);
}
// Two lanes of lerp(start, end, weight), rounded to BF16.
__device__ __forceinline__ uint32_t lerp_pair(uint32_t start, uint32_t end, float weight) {
  return pack_rn(lerp_f32(bf16_low(start), bf16_low(end), weight),
                 lerp_f32(bf16_high(start), bf16_high(end), weight));
}

// Two lanes of `left (op) right`, rounded once to BF16.
__device__ __forceinline__ uint32_t apply_op(uint32_t left, uint32_t right, int op, bool alpha_one,
                                             bool beta_one, float alpha, float beta) {
  if (op == LCT_OP_ADD) {
    const __nv_bfloat162 r = __hadd2(*reinterpret_cast<const __nv_bfloat162*>(&left),
                                     *reinterpret_cast<const __nv_bfloat162*>(&right));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  if (op == LCT_OP_MULTIPLY) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&left),
                                     *reinterpret_cast<const __nv_bfloat162*>(&right));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  if (op == LCT_OP_LERP) return lerp_pair(left, right, alpha);
  const float l0 = bf16_low(left), l1 = bf16_high(left);
  const float r0 = bf16_low(right), r1 = bf16_high(right);
  if (op == LCT_OP_EMA_SQUARE) {
    const uint32_t scaled = pack_rn(__fmul_rn(l0, alpha), __fmul_rn(l1, alpha));
    return pack_rn(__fmaf_rn(beta, __fmul_rn(r0, r0), bf16_low(scaled)),
                   __fmaf_rn(beta, __fmul_rn(r1, r1), bf16_high(scaled)));
  }
  if (alpha_one) {
    if (beta_one) return pack_rn(__fadd_rn(l0, r0), __fadd_rn(l1, r1));
    return pack_rn(__fmaf_rn(r0, beta, l0), __fmaf_rn(r1, beta, l1));
  }
  if (beta_one) return pack_rn(__fmaf_rn(l0, alpha, r0), __fmaf_rn(l1, alpha, r1));
  return pack_rn(__fmaf_rn(l0, alpha, __fmul_rn(r0, beta)), __fmaf_rn(l1, alpha, __fmul_rn(r1, beta)));
}

// Load 8 dense BF16 values of one row (zero beyond the tensor's end).
__device__ __forceinline__ void load_dense8(const uint16_t* other, int64_t at, int64_t numel,
                                            bool vector_ok, uint32_t w[4]) {
  if (vector_ok && at + 8 <= numel) {
    const uint4 v = __ldcs(reinterpret_cast<const uint4*>(other + at));
    w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    return;
  }
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t a = at + 2 * k < numel ? other[at + 2 * k] : 0u;
    const uint32_t b = at + 2 * k + 1 < numel ? other[at + 2 * k + 1] : 0u;
    w[k] = a | (b << 16);
  }
}

// Emit one row of results: dense BF16, or side bytes (storage order) plus
// exponent bytes (logical order) for the encoder.
__device__ __forceinline__ void store_row(uint32_t r[4], bool compressed, void* output,
                                          uint8_t* auxiliary, int64_t at, int64_t numel,
                                          int64_t storage_at, uint32_t q) {
  if (!compressed) {
    uint16_t* out = static_cast<uint16_t*>(output);
    if (at + 8 <= numel) {
      __stcs(reinterpret_cast<uint4*>(out + at), make_uint4(r[0], r[1], r[2], r[3]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (at + i < numel) out[at + i] = (uint16_t)(r[i >> 1] >> (16 * (i & 1)));
    }
    return;
  }
  if (at + 8 > numel) {  // padding counts as +0.0
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (at + i >= numel) r[i >> 1] &= (i & 1) ? 0x0000FFFFu : 0xFFFF0000u;
  }
  const uint32_t l03 = prmt(r[0], r[1], 0x6420), h03 = prmt(r[0], r[1], 0x7531);
  const uint32_t l47 = prmt(r[2], r[3], 0x6420), h47 = prmt(r[2], r[3], 0x7531);
  const uint32_t e03 = exponent_bytes(l03, h03), e47 = exponent_bytes(l47, h47);
  const uint32_t c03 = side_bytes(l03, h03), c47 = side_bytes(l47, h47);
  const uint2 side_lane_order =
      make_uint2(prmt(c03, c47, pair_selector_low(q)), prmt(c03, c47, pair_selector_high(q)));
  *reinterpret_cast<uint2*>(static_cast<uint8_t*>(output) + storage_at) = side_lane_order;
  if (at + 8 <= numel) {
    *reinterpret_cast<uint2*>(auxiliary + at) = make_uint2(e03, e47);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (at + i < numel) auxiliary[at + i] = (uint8_t)((i < 4 ? e03 : e47) >> (8 * (i & 3)));
  }
}

// ---------------------------------------------------------------------------
// Host-side launch helpers
// ---------------------------------------------------------------------------

static inline int check_shape(int64_t size, int64_t logical_numel, int block_symbols, int steps,
                       int fixed_words, int rare_length, Shape* g) {
  if (steps != 128 && steps != 256) return LCT_E_BAD_GEOMETRY;
  if (block_symbols != steps * kLanes) return LCT_E_BAD_GEOMETRY;
  if (fixed_words < 2 || fixed_words > 64) return LCT_E_BAD_GEOMETRY;
  if (rare_length < 0 || rare_length > 8) return LCT_E_BAD_ARGUMENT;
  if (size <= 0 || size % block_symbols != 0) return LCT_E_BAD_ARGUMENT;
  if (logical_numel <= 0 || logical_numel > size) return LCT_E_BAD_ARGUMENT;
  const int64_t blocks = size / block_symbols;
  if (blocks > 0x7FFFFFFFLL) return LCT_E_TOO_LARGE;
  g->size = size;
  g->logical_numel = logical_numel;
  g->n_blocks = blocks;
  g->streams = blocks * kLanes;
  g->block_symbols = block_symbols;
  g->steps = steps;
  g->fixed_words = fixed_words;
  g->rare_length = rare_length;
  g->lane_mask = lane_mask_now();
  return 0;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static inline int view_of(const lct_operand* in, OperandView* v) {
  if (in == nullptr || in->encoded == nullptr || in->side == nullptr || in->center == nullptr ||
      in->pair_table == nullptr)
    return LCT_E_NULL_POINTER;
  if (!aligned16(in->side) || !aligned16(in->pair_table) || !aligned16(in->encoded))
    return LCT_E_ALIGNMENT;
  const lct_overflow& o = in->overflow;
  if (o.mode < 0 || o.mode > 2) return LCT_E_BAD_ARGUMENT;
  if (o.mode != 0 && (o.blocks == nullptr || o.tail == nullptr || o.lanes == nullptr ||
                      o.starts == nullptr))
    return LCT_E_NULL_POINTER;
  if (o.mode == 2 && (o.descriptor == nullptr || o.count == nullptr)) return LCT_E_NULL_POINTER;
  v->encoded = reinterpret_cast<const uint32_t*>(in->encoded);
  v->side = in->side;
  v->center = in->center;
  v->pair_table = in->pair_table;
  v->lanes = o.lanes;
  v->starts = o.starts;
  v->tail = o.tail;
  v->descriptor = o.descriptor;
  v->count = o.count;
  v->blocks = o.blocks;
  v->base = o.base;
  v->mode = o.mode;
  return 0;
}

// Operation code and its scalars: which of alpha / beta the kernels will read.
static inline int check_op(int op, const float* alpha, const float* beta, int* alpha_is_one,
                           int* beta_is_one) {
  if (op < LCT_OP_ADD || op > LCT_OP_EMA_SQUARE) return LCT_E_BAD_ARGUMENT;
  if (op == LCT_OP_SCALAR_MUL_ADD) {
    if (!*alpha_is_one && alpha == nullptr) return LCT_E_NULL_POINTER;
    if (!*beta_is_one && beta == nullptr) return LCT_E_NULL_POINTER;
  } else if (op == LCT_OP_LERP) {
    if (alpha == nullptr) return LCT_E_NULL_POINTER;
    *alpha_is_one = 0;
    *beta_is_one = beta == nullptr;  // beta: weight of the Nesterov direction, when one is emitted
  } else if (op == LCT_OP_EMA_SQUARE) {
    if (alpha == nullptr || beta == nullptr) return LCT_E_NULL_POINTER;
    *alpha_is_one = *beta_is_one = 0;
  } else {
    *alpha_is_one = *beta_is_one = 1;
  }
  return 0;
}

template <typename Kernel>
static inline int opt_in_shared(Kernel kernel, size_t bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace lct
