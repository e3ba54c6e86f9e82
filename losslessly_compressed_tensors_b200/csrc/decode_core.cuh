// Device building blocks shared by the decoder, the fused pointwise kernels and
// the fused update kernel: operand views, the per-CTA prologue (staging of the
// payload and of the center's two-symbol table, overflow map), the lane-side bit reader and
// tile decoder, the row-side BF16 join/split, the arithmetic of the fused
// operations, and the host-side argument checks.
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

// Shared memory of a CTA: the payload image(s) first (fixed_words + 2 rows of
// 256 words each, the last two zero), then one DecodeShared per operand.  A
// lane's refill pointer is clamped to the image once per tile; inside a tile a
// corrupt stream can run at most 16 rows past it, which still lands in the
// tables below (garbage in, garbage out, but never an out-of-range access).
struct __align__(16) DecodeShared {
  uint32_t table[kPairEntries];
  uint16_t tile[kWarps][kTilePairs * 32];
  uint8_t index_to_byte[256];
  uint16_t overflow_start[kLanes];
  int32_t overflow_offset[kLanes];
  int scan[36];
};

static inline size_t payload_image_bytes(int fixed_words) {
  return (size_t)(fixed_words + 2) * kLanes * 4;
}
static inline size_t operand_shared_bytes(int fixed_words) {
  return sizeof(DecodeShared) + payload_image_bytes(fixed_words);
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

// Read position of one lane: a 96-bit register window over the shared payload
// image (the word under the position and the two after it) plus the bit
// offset inside the first word.  Lookups take their bits from registers; the
// only shared-memory access is the refill of the third word, which is not on
// the lookup's dependency chain.
struct BitReader {
  const uint32_t* next_row;  // image word that enters the window at the next refill
  const uint32_t* last_row;  // the image's second zero row
  uint32_t cur, n1, n2;
  int shift;                 // 0..31 between pairs

  // `column`: this lane's column of an image of fixed_words + 2 rows.
  __device__ __forceinline__ void open(const uint32_t* column, int fixed_words) {
    cur = column[0];
    n1 = column[kLanes];
    n2 = column[2 * kLanes];
    next_row = column + 3 * kLanes;
    last_row = column + (fixed_words + 1) * kLanes;
    shift = 0;
  }
  // A well-formed stream never refills past the image's second zero row; a
  // corrupt one is pulled back here, once per tile (at most 16 refills each).
  __device__ __forceinline__ void tile_start() {
    if (next_row > last_row) next_row = last_row;
  }
  // 32 stream bits starting `extra` bits after the position (shift + extra < 64).
  __device__ __forceinline__ uint32_t peek(int extra) const {
    const int s = shift + extra;
    const bool far = s >= 32;
    return __funnelshift_r(far ? n1 : cur, far ? n2 : n1, s);  // amount is taken modulo 32
  }
  __device__ __forceinline__ uint32_t peek0() const { return __funnelshift_r(cur, n1, shift); }
  __device__ __forceinline__ void advance(int bits) {  // bits <= 32
    shift += bits;
    if (shift >= 32) {
      shift -= 32;
      cur = n1;
      n1 = n2;
      n2 = *next_row;
      next_row += kLanes;
    }
  }
};

// Unroll factor of the lane-phase loop (16 pairs per tile).  Measured on B200
// (64 Mi elements): 16 -> 81.9 us, 8 -> 80.8, 4 -> 80.0, 2 -> 80.9; the fully
// unrolled loop pays in instruction-cache misses for what it saves in address
// arithmetic.
#ifndef LCT_DECODE_UNROLL
#define LCT_DECODE_UNROLL 4
#endif
#define LCT_PRAGMA(x) _Pragma(#x)
#define LCT_UNROLL(n) LCT_PRAGMA(unroll n)

// One symbol from a table entry and the stream bits it was looked up with.
__device__ __forceinline__ uint32_t symbol_of(uint32_t entry, uint32_t bits, const DecodeShared& sh,
                                              int rare_length, int* length) {
  if (entry & kEscape) {
    *length = rare_length + 8;
    return sh.index_to_byte[(bits >> rare_length) & 255u];
  }
  *length = (int)((entry >> 16) & 15u);
  return entry & 255u;
}

// Pair whose table entry is not "two direct symbols": take the first symbol
// from the entry already in hand, look the second one up on its own.
// Returns the pair in table-entry form (bytes: first, second, -, bits consumed).
template <typename Reader>
__device__ __forceinline__ uint32_t slow_pair(const Reader& r, uint32_t entry, uint32_t bits,
                                              const DecodeShared& sh, int rare_length) {
  // Every entry carries the length of its first symbol, escapes included, so the second
  // lookup does not wait for an escape test; literals are patched in afterwards.
  const uint32_t l0 = (entry >> 16) & 31u;
  const uint32_t bits1 = r.peek((int)l0);
  const uint32_t second = sh.table[table_slot(bits1)];
  uint32_t e0 = entry & 255u, e1 = second & 255u;
  if ((entry | second) & kEscape) {
    if (entry & kEscape) e0 = sh.index_to_byte[(bits >> rare_length) & 255u];
    if (second & kEscape) e1 = sh.index_to_byte[(bits1 >> rare_length) & 255u];
  }
  return e0 | (e1 << 8) | ((l0 + ((second >> 16) & 31u)) << 24);
}

// Lane phase for one tile.  `coded` = number of leading steps of this lane that
// are in the bit stream (its overflow start or its valid length, whichever is
// first); steps from `tail_from` on come from the raw tail.
template <typename Reader>
__device__ __forceinline__ void decode_tile_rows(Reader& r, const DecodeShared& sh,
                                                 uint16_t* tile, int lane32, int step0, int coded,
                                                 int tail_from, const uint8_t* tail_bytes,
                                                 int rare_length, int lane_mask) {
  r.tile_start();
  // Tiles start on multiples of 32 rows, so the low mask bits of pair p are 2p & lane_mask.
  if (__all_sync(0xFFFFFFFFu, step0 + kTileRows <= coded)) {
    LCT_UNROLL(LCT_DECODE_UNROLL)
    for (int p = 0; p < kTilePairs; ++p) {
      const uint32_t bits = r.peek0();
      uint32_t entry = sh.table[table_slot(bits)];
      if ((int32_t)entry < 0) entry = slow_pair(r, entry, bits, sh, rare_length);
      tile[p * 32 + (lane32 ^ ((2 * p) & lane_mask))] = (uint16_t)entry;
      r.advance((int)(entry >> 24));
    }
    return;
  }
  for (int p = 0; p < kTilePairs; ++p) {
    const int step = step0 + 2 * p;
    uint32_t pair = 0;
    if (step + 2 <= coded) {
      const uint32_t bits = r.peek0();
      pair = sh.table[table_slot(bits)];
      if ((int32_t)pair < 0) pair = slow_pair(r, pair, bits, sh, rare_length);
      r.advance((int)(pair >> 24));
    } else if (step >= tail_from) {
      const uint32_t t0 = tail_bytes[step - tail_from], t1 = tail_bytes[step + 1 - tail_from];
      pair = ((t0 + 127u) & 255u) | (((t1 + 127u) & 255u) << 8);
    } else if (step + 1 == coded) {
      int l0;
      const uint32_t bits = r.peek0();
      pair = symbol_of(sh.table[table_slot(bits)], bits, sh, rare_length, &l0);
      r.advance(l0);
    }
    tile[p * 32 + (lane32 ^ ((2 * p) & lane_mask))] = (uint16_t)pair;
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
__device__ __forceinline__ void prepare_block(DecodeShared& sh, uint32_t* payload,
                                              const OperandView& a, const Shape& g, int64_t block,
                                              Extra before_barrier = Extra()) {
  const int tid = threadIdx.x;
  // Word w of the block's 256 streams is one contiguous, 1 KB aligned row.
  const uint32_t* rows = a.encoded + block * kLanes;
  for (int i = tid; i < g.fixed_words * (kLanes / 4); i += kThreads) {
    const int w = i >> 6, c = (i & 63) * 4;
    cp_async_16(&payload[w * kLanes + c], rows + (int64_t)w * g.streams + c);
  }
  payload[g.fixed_words * kLanes + tid] = 0u;
  payload[(g.fixed_words + 1) * kLanes + tid] = 0u;

  // The codebook's table for this tensor's center, ready to use (symbols are exponent bytes).
  const int center = *a.center;
  const uint32_t* source = a.pair_table + (size_t)((center + 128) & 255) * kPairEntries;
  for (int i = tid; i < kPairEntries / 4; i += kThreads) cp_async_16(&sh.table[4 * i], source + 4 * i);
  sh.index_to_byte[tid] = (uint8_t)index_to_exponent_byte((uint32_t)tid, center);
  sh.overflow_start[tid] = (uint16_t)g.steps;
  sh.overflow_offset[tid] = 0;
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
      const int prefix = block_exclusive_scan(tid < count ? g.steps - start : 0, sh.scan, &unused);
      if (tid < count) {
        sh.overflow_start[lane] = (uint16_t)start;
        sh.overflow_offset[lane] = byte_base + prefix;
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

// Where one row-phase unit (row pair p of the tile, 8-column subgroup j4 of the
// warp's 32 columns) lives in the tensor.
struct UnitPlace {
  int64_t logical;   // element offset of the top row's first column
  int64_t storage;   // byte offset of the top row's first lane in the side bytes
  uint32_t q;        // pair permutation between lane order and column order
};

__device__ __forceinline__ UnitPlace place_unit(int warp, int p, int j4, int64_t row0, int step0,
                                                int64_t block_base, int lane_mask) {
  // All 32 rows of a tile share mask bits 5..7; bits 1..4 of pair p are 2p (all & lane_mask).
  const int64_t tile_row = row0 + step0;
  const int in_tile = (2 * p) & lane_mask;
  const int group = warp ^ ((int)(tile_row & lane_mask) >> 5);
  UnitPlace u;
  u.logical = (tile_row + 2 * p) * kLanes + 32 * group + 8 * j4;
  u.storage = block_base + (int64_t)(step0 + 2 * p) * kLanes + 32 * warp + ((8 * j4) ^ (in_tile & 0x18));
  u.q = (uint32_t)(in_tile >> 1) & 3u;
  return u;
}

// Rebuild the 8 BF16 values (4 words, column order) of one row from the unit's
// tile words and that row's side bytes (lane order).
__device__ __forceinline__ void join_row(const uint4& tile_words, uint2 side_lane_order, uint32_t q,
                                         bool second_row, uint32_t out[4]) {
  const uint32_t pick = second_row ? 0x7531u : 0x6420u;
  const uint32_t e03 = prmt(tile_words.x, tile_words.y, pick);
  const uint32_t e47 = prmt(tile_words.z, tile_words.w, pick);
  const uint32_t s03 = prmt(side_lane_order.x, side_lane_order.y, pair_selector_low(q));
  const uint32_t s47 = prmt(side_lane_order.x, side_lane_order.y, pair_selector_high(q));
  const uint32_t l03 = bf16_low_bytes(e03, s03), h03 = bf16_high_bytes(e03, s03);
  const uint32_t l47 = bf16_low_bytes(e47, s47), h47 = bf16_high_bytes(e47, s47);
  out[0] = prmt(l03, h03, 0x5140);
  out[1] = prmt(l03, h03, 0x7362);
  out[2] = prmt(l47, h47, 0x5140);
  out[3] = prmt(l47, h47, 0x7362);
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
  const float l0 = bf16_low(left), l1 = bf16_high(left);
  const float r0 = bf16_low(right), r1 = bf16_high(right);
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

template <typename Kernel>
static inline int opt_in_shared(Kernel kernel, size_t bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace lct
