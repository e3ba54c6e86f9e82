// Table-driven decoder and the fused decode -> pointwise operation kernels.
//
// One CTA (256 threads) per codec block.  Per 32-row tile:
//   lane phase  - thread = lane: walks its bit stream two symbols per lookup
//                 (12-bit two-symbol table in shared memory, remapped to this
//                 tensor's center at CTA start) and drops the exponent bytes
//                 into the column-ordered shared tile;
//   row phase   - thread = 8 columns of a row pair: 128-bit read of the tile,
//                 64-bit reads of the side bytes, byte permutes to rebuild the
//                 BF16 words, optional arithmetic, 128-bit streaming stores.
// Overflow lanes switch from the bit stream to their raw tail bytes at their
// recorded start step, inside the same launch.
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
};

struct __align__(16) DecodeShared {
  uint32_t table[kPairEntries];
  uint16_t tile[kTilePairs * kLanes];
  uint8_t index_to_byte[256];
  uint16_t overflow_start[kLanes];
  int32_t overflow_offset[kLanes];
  int scan[33];
};

// Per-lane read position in the fixed payload: a 64-bit window plus one
// prefetched word, so the dependent lookup chain never waits on HBM.
struct LaneReader {
  const uint32_t* next_ptr;  // word index word + 2 of this stream
  int64_t stride;            // words between consecutive words of one stream
  uint32_t lo, hi, next;
  int shift, word, fixed_words;

  __device__ __forceinline__ void open(const uint32_t* encoded, int64_t streams, int64_t stream,
                                       int fw) {
    const uint32_t* p = encoded + stream;
    stride = streams;
    fixed_words = fw;
    lo = __ldcs(p);
    hi = __ldcs(p + streams);
    next = fw > 2 ? __ldcs(p + 2 * streams) : 0u;
    next_ptr = p + 3 * streams;
    shift = 0;
    word = 0;
  }
  __device__ __forceinline__ void advance(int bits) {
    shift += bits;
    if (shift >= 32) {
      shift -= 32;
      lo = hi;
      hi = next;
      ++word;
      next = (word + 2 < fixed_words) ? __ldcs(next_ptr) : 0u;
      next_ptr += stride;
    }
  }
};

// Decode one symbol at bit offset 0 of `bits` (>= 16 valid bits).
__device__ __forceinline__ void one_symbol(uint32_t bits, const DecodeShared& sh, int rare_length,
                                           uint32_t* exponent_byte, int* length) {
  const uint32_t entry = sh.table[bits & (kPairEntries - 1)];
  if (entry & kEscape) {
    *exponent_byte = sh.index_to_byte[(bits >> rare_length) & 255u];
    *length = rare_length + 8;
  } else {
    *exponent_byte = entry & 255u;
    *length = (int)((entry >> 24) & 15u);
  }
}

// Pair whose table entry is not "two direct symbols": decode them one by one.
__device__ __noinline__ uint32_t slow_pair(uint32_t lo, uint32_t hi, int shift,
                                           const DecodeShared& sh, int rare_length, int* consumed) {
  const uint64_t window = (((uint64_t)hi << 32) | lo) >> shift;
  uint32_t e0, e1;
  int l0, l1;
  one_symbol((uint32_t)window, sh, rare_length, &e0, &l0);
  one_symbol((uint32_t)(window >> l0), sh, rare_length, &e1, &l1);
  *consumed = l0 + l1;
  return e0 | (e1 << 8);
}

// Lane phase for one tile.  `coded` = number of leading steps of this lane that
// are in the bit stream (its overflow start or its valid length, whichever is
// first); steps from `tail_from` on come from the raw tail.
__device__ __forceinline__ void decode_tile_rows(LaneReader& r, DecodeShared& sh, uint16_t* tile,
                                                 int lane, int64_t row0, int step0, int coded,
                                                 int tail_from, const uint8_t* tail_bytes,
                                                 int rare_length) {
  if (step0 + kTileRows <= coded) {
#pragma unroll 4
    for (int p = 0; p < kTilePairs; ++p) {
      const int mask = (int)((row0 + step0 + 2 * p) & 254);
      const uint32_t bits = __funnelshift_r(r.lo, r.hi, r.shift);
      uint32_t entry = sh.table[bits & (kPairEntries - 1)];
      int consumed;
      if ((int32_t)entry < 0) {
        entry = slow_pair(r.lo, r.hi, r.shift, sh, rare_length, &consumed);
      } else {
        consumed = (int)prmt(entry, 0, 0x4442);
      }
      tile[p * kLanes + (lane ^ mask)] = (uint16_t)entry;
      r.advance(consumed);
    }
    return;
  }
  for (int p = 0; p < kTilePairs; ++p) {
    const int step = step0 + 2 * p;
    const int mask = (int)((row0 + step) & 254);
    uint32_t pair = 0;
    if (step + 2 <= coded) {
      int consumed;
      pair = slow_pair(r.lo, r.hi, r.shift, sh, rare_length, &consumed);
      r.advance(consumed);
    } else if (step >= tail_from) {
      const uint32_t t0 = tail_bytes[step - tail_from], t1 = tail_bytes[step + 1 - tail_from];
      pair = ((t0 + 127u) & 255u) | (((t1 + 127u) & 255u) << 8);
    } else if (step + 1 == coded) {
      const uint64_t window = (((uint64_t)r.hi << 32) | r.lo) >> r.shift;
      uint32_t e0;
      int l0;
      one_symbol((uint32_t)window, sh, rare_length, &e0, &l0);
      r.advance(l0);
      pair = e0;
    }
    tile[p * kLanes + (lane ^ mask)] = (uint16_t)pair;
  }
}

// CTA prologue: center-specific symbol table and this block's overflow map.
__device__ __forceinline__ void prepare_block(DecodeShared& sh, const OperandView& a,
                                              const Shape& g, int64_t block) {
  const int tid = threadIdx.x;
  const int center = *a.center;
  sh.index_to_byte[tid] = (uint8_t)index_to_exponent_byte((uint32_t)tid, center);
  sh.overflow_start[tid] = (uint16_t)g.steps;
  sh.overflow_offset[tid] = 0;
  __syncthreads();
  const uint4* source = reinterpret_cast<const uint4*>(a.pair_table);
  uint4* target = reinterpret_cast<uint4*>(sh.table);
  for (int i = tid; i < kPairEntries / 4; i += kThreads) {
    uint4 e = __ldg(source + i);
    uint32_t* w = &e.x;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint32_t b0 = sh.index_to_byte[w[k] & 255u];
      const uint32_t b1 = sh.index_to_byte[(w[k] >> 8) & 255u];
      w[k] = (w[k] & 0xFFFF0000u) | b0 | (b1 << 8);
    }
    target[i] = e;
  }
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
  __syncthreads();
}

__device__ __forceinline__ const uint8_t* tail_origin(const OperandView& a) {
  if (a.mode == 2) return a.tail + a.descriptor[0] + 2 * (int64_t)(*a.count);
  return a.tail + a.base;
}

// Rebuild the 8 BF16 values (4 words, column order) of one row from the tile
// words and that row's side bytes.  `second_row` picks the high exponent byte.
__device__ __forceinline__ void join_row(const uint4& tile_words, uint2 side_lane_order, uint32_t q,
                                         bool second_row, uint32_t out[4]) {
  const uint32_t p0 = prmt(side_lane_order.x, side_lane_order.y, pair_selector_low(q));
  const uint32_t p1 = prmt(side_lane_order.x, side_lane_order.y, pair_selector_high(q));
  if (!second_row) {
    out[0] = join_bf16x2(prmt(tile_words.x, p0, 0x2504));
    out[1] = join_bf16x2(prmt(tile_words.y, p0, 0x2706));
    out[2] = join_bf16x2(prmt(tile_words.z, p1, 0x2504));
    out[3] = join_bf16x2(prmt(tile_words.w, p1, 0x2706));
  } else {
    out[0] = join_bf16x2(prmt(tile_words.x, p0, 0x3514));
    out[1] = join_bf16x2(prmt(tile_words.y, p0, 0x3716));
    out[2] = join_bf16x2(prmt(tile_words.z, p1, 0x3514));
    out[3] = join_bf16x2(prmt(tile_words.w, p1, 0x3716));
  }
}

// ---------------------------------------------------------------------------
// Plain decode
// ---------------------------------------------------------------------------

__global__ void __launch_bounds__(kThreads)
decode_kernel(OperandView a, Shape g, uint16_t* __restrict__ out) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  DecodeShared& sh = *reinterpret_cast<DecodeShared*>(smem_raw);
  const int64_t block = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t row0 = block * g.steps;
  prepare_block(sh, a, g, block);

  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel);
  const int tail_from = sh.overflow_start[tid];
  const int coded = min(valid, tail_from);
  const uint8_t* tail_bytes = a.mode ? tail_origin(a) + sh.overflow_offset[tid] : nullptr;
  LaneReader reader;
  reader.open(a.encoded, g.streams, block * kLanes + tid, g.fixed_words);
  const bool full_block = (block + 1) * (int64_t)g.block_symbols <= g.logical_numel;
  const uint8_t* side_block = a.side + block * (int64_t)g.block_symbols;

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    // Side bytes of the two row-phase units of this thread, fetched early.
    uint2 side_regs[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = (tid >> 5) + 8 * u;
      const int j = tid & 31;
      const int step = step0 + 2 * p;
      const int mask = (int)((row0 + step) & 254);
      const int lane_group = (8 * j) ^ (mask & 0xF8);
      const uint8_t* s = side_block + (int64_t)step * kLanes + lane_group;
      side_regs[u][0] = __ldcs(reinterpret_cast<const uint2*>(s));
      side_regs[u][1] = __ldcs(reinterpret_cast<const uint2*>(s + kLanes));
    }
    decode_tile_rows(reader, sh, sh.tile, tid, row0, step0, coded, tail_from, tail_bytes,
                     g.rare_length);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = (tid >> 5) + 8 * u;
      const int j = tid & 31;
      const int64_t row = row0 + step0 + 2 * p;
      const uint32_t q = (uint32_t)(row >> 1) & 3u;
      const uint4 words = *reinterpret_cast<const uint4*>(&sh.tile[p * kLanes + 8 * j]);
      uint32_t top[4], bottom[4];
      join_row(words, side_regs[u][0], q, false, top);
      join_row(words, side_regs[u][1], q, true, bottom);
      const int64_t at = row * kLanes + 8 * j;
      if (full_block || at + kLanes + 8 <= g.logical_numel) {
        __stcs(reinterpret_cast<uint4*>(out + at), make_uint4(top[0], top[1], top[2], top[3]));
        __stcs(reinterpret_cast<uint4*>(out + at + kLanes),
               make_uint4(bottom[0], bottom[1], bottom[2], bottom[3]));
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint32_t t = top[i >> 1] >> (16 * (i & 1));
          const uint32_t b = bottom[i >> 1] >> (16 * (i & 1));
          if (at + i < g.logical_numel) out[at + i] = (uint16_t)t;
          if (at + kLanes + i < g.logical_numel) out[at + kLanes + i] = (uint16_t)b;
        }
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Fused pointwise operations
// ---------------------------------------------------------------------------

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
  const uint32_t e01 = prmt(exponents_of(r[0]), exponents_of(r[1]), 0x6420);
  const uint32_t e23 = prmt(exponents_of(r[2]), exponents_of(r[3]), 0x6420);
  const uint32_t c01 = prmt(sides_of(r[0]), sides_of(r[1]), 0x6420);
  const uint32_t c23 = prmt(sides_of(r[2]), sides_of(r[3]), 0x6420);
  const uint2 side_lane_order =
      make_uint2(prmt(c01, c23, pair_selector_low(q)), prmt(c01, c23, pair_selector_high(q)));
  *reinterpret_cast<uint2*>(static_cast<uint8_t*>(output) + storage_at) = side_lane_order;
  if (at + 8 <= numel) {
    *reinterpret_cast<uint2*>(auxiliary + at) = make_uint2(e01, e23);
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (at + i < numel) auxiliary[at + i] = (uint8_t)((i < 4 ? e01 : e23) >> (8 * (i & 3)));
  }
}

template <bool kDual>
__global__ void __launch_bounds__(kThreads)
pointwise_kernel(OperandView a, OperandView b, Shape g, const uint16_t* __restrict__ other,
                 bool other_vector_ok, void* output, uint8_t* auxiliary, OpSpec spec,
                 bool compressed) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  DecodeShared& sh = *reinterpret_cast<DecodeShared*>(smem_raw);
  DecodeShared& sh_b = *reinterpret_cast<DecodeShared*>(smem_raw + (kDual ? sizeof(DecodeShared) : 0));
  const int64_t block = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t row0 = block * g.steps;
  prepare_block(sh, a, g, block);
  if (kDual) prepare_block(sh_b, b, g, block);

  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel);
  const int a_tail_from = sh.overflow_start[tid];
  const int a_coded = min(valid, a_tail_from);
  const uint8_t* a_tail = a.mode ? tail_origin(a) + sh.overflow_offset[tid] : nullptr;
  LaneReader reader_a, reader_b;
  reader_a.open(a.encoded, g.streams, block * kLanes + tid, g.fixed_words);
  int b_tail_from = g.steps, b_coded = 0;
  const uint8_t* b_tail = nullptr;
  if (kDual) {
    b_tail_from = sh_b.overflow_start[tid];
    b_coded = min(valid, b_tail_from);
    b_tail = b.mode ? tail_origin(b) + sh_b.overflow_offset[tid] : nullptr;
    reader_b.open(b.encoded, g.streams, block * kLanes + tid, g.fixed_words);
  }
  const int64_t block_base = block * (int64_t)g.block_symbols;

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    decode_tile_rows(reader_a, sh, sh.tile, tid, row0, step0, a_coded, a_tail_from, a_tail,
                     g.rare_length);
    if (kDual)
      decode_tile_rows(reader_b, sh_b, sh_b.tile, tid, row0, step0, b_coded, b_tail_from, b_tail,
                       g.rare_length);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = (tid >> 5) + 8 * u;
      const int j = tid & 31;
      const int step = step0 + 2 * p;
      const int64_t row = row0 + step;
      const int mask = (int)(row & 254);
      const uint32_t q = (uint32_t)(mask >> 1) & 3u;
      const int lane_group = (8 * j) ^ (mask & 0xF8);
      const int64_t storage_at = block_base + (int64_t)step * kLanes + lane_group;
      const int64_t at = row * kLanes + 8 * j;
      const uint4 words = *reinterpret_cast<const uint4*>(&sh.tile[p * kLanes + 8 * j]);
      uint4 words_b = make_uint4(0, 0, 0, 0);
      if (kDual) words_b = *reinterpret_cast<const uint4*>(&sh_b.tile[p * kLanes + 8 * j]);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t s_at = storage_at + half * kLanes;
        const int64_t l_at = at + half * kLanes;
        uint32_t left[4], right[4], result[4];
        join_row(words, __ldcs(reinterpret_cast<const uint2*>(a.side + s_at)), q, half == 1, left);
        if (kDual) {
          join_row(words_b, __ldcs(reinterpret_cast<const uint2*>(b.side + s_at)), q, half == 1,
                   right);
        } else {
          load_dense8(other, l_at, g.logical_numel, other_vector_ok, right);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
          result[k] = apply_op(left[k], right[k], spec.op, spec.alpha_is_one != 0,
                               spec.beta_is_one != 0, alpha, beta);
        store_row(result, compressed, output, auxiliary, l_at, g.logical_numel, s_at, q);
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Host-side launch helpers
// ---------------------------------------------------------------------------

static int check_shape(int64_t size, int64_t logical_numel, int block_symbols, int steps,
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
  return 0;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int view_of(const lct_operand* in, OperandView* v) {
  if (in == nullptr || in->encoded == nullptr || in->side == nullptr || in->center == nullptr ||
      in->pair_table == nullptr)
    return LCT_E_NULL_POINTER;
  if (!aligned16(in->side) || !aligned16(in->pair_table)) return LCT_E_ALIGNMENT;
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
static int opt_in_shared(Kernel kernel, size_t bytes) {
  return (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

}  // namespace lct

extern "C" {

int lct_decode(const lct_operand* a, int16_t* out, int64_t size, int64_t logical_numel,
               int block_symbols, int steps, int fixed_words, int rare_length, void* stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = lct::view_of(a, &va)) != 0) return rc;
  if (out == nullptr) return LCT_E_NULL_POINTER;
  if (!lct::aligned16(out)) return LCT_E_ALIGNMENT;
  const size_t shared = sizeof(lct::DecodeShared);
  if ((rc = lct::opt_in_shared(lct::decode_kernel, shared)) != 0) return rc;
  lct::decode_kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared,
                       static_cast<cudaStream_t>(stream)>>>(va, g, reinterpret_cast<uint16_t*>(out));
  return (int)cudaGetLastError();
}

int lct_pointwise(const lct_operand* a, const void* other, void* output, uint8_t* auxiliary,
                  const float* alpha, const float* beta, int op, int alpha_is_one,
                  int beta_is_one, int compressed_output, int64_t size, int64_t logical_numel,
                  int block_symbols, int steps, int fixed_words, int rare_length, void* stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = lct::view_of(a, &va)) != 0) return rc;
  if (other == nullptr || output == nullptr) return LCT_E_NULL_POINTER;
  if (compressed_output && auxiliary == nullptr) return LCT_E_NULL_POINTER;
  if (op < LCT_OP_ADD || op > LCT_OP_SCALAR_MUL_ADD) return LCT_E_BAD_ARGUMENT;
  if (op == LCT_OP_SCALAR_MUL_ADD) {
    if (!alpha_is_one && alpha == nullptr) return LCT_E_NULL_POINTER;
    if (!beta_is_one && beta == nullptr) return LCT_E_NULL_POINTER;
  } else {
    alpha_is_one = beta_is_one = 1;
  }
  if (!lct::aligned16(output) || (compressed_output && !lct::aligned16(auxiliary)))
    return LCT_E_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(other) & 1u) != 0) return LCT_E_ALIGNMENT;
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const size_t shared = sizeof(lct::DecodeShared);
  if ((rc = lct::opt_in_shared(lct::pointwise_kernel<false>, shared)) != 0) return rc;
  lct::pointwise_kernel<false><<<(unsigned)g.n_blocks, lct::kThreads, shared,
                                 static_cast<cudaStream_t>(stream)>>>(
      va, va, g, static_cast<const uint16_t*>(other), lct::aligned16(other), output, auxiliary,
      spec, compressed_output != 0);
  return (int)cudaGetLastError();
}

int lct_dual_scale_add(const lct_operand* a, const lct_operand* b, void* output,
                       uint8_t* auxiliary, const float* alpha, int compressed_output,
                       int64_t size, int64_t logical_numel, int block_symbols, int steps,
                       int fixed_words, int rare_length, void* stream) {
  lct::Shape g;
  lct::OperandView va, vb;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = lct::view_of(a, &va)) != 0) return rc;
  if ((rc = lct::view_of(b, &vb)) != 0) return rc;
  if (output == nullptr || alpha == nullptr) return LCT_E_NULL_POINTER;
  if (compressed_output && auxiliary == nullptr) return LCT_E_NULL_POINTER;
  if (!lct::aligned16(output) || (compressed_output && !lct::aligned16(auxiliary)))
    return LCT_E_ALIGNMENT;
  // fma(a, alpha, b): the scaled operation with beta == 1.
  const lct::OpSpec spec{alpha, nullptr, LCT_OP_SCALAR_MUL_ADD, 0, 1};
  const size_t shared = 2 * sizeof(lct::DecodeShared);
  if ((rc = lct::opt_in_shared(lct::pointwise_kernel<true>, shared)) != 0) return rc;
  lct::pointwise_kernel<true><<<(unsigned)g.n_blocks, lct::kThreads, shared,
                                static_cast<cudaStream_t>(stream)>>>(
      va, vb, g, nullptr, false, output, auxiliary, spec, compressed_output != 0);
  return (int)cudaGetLastError();
}

}  // extern "C"
