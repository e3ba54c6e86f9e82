/*
 * CPU oracle for the BF16 lossless codec hot path.  TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C, single-threaded restatement of what the reference's Triton
 * kernels compute, written lane by lane from their source.  It exists so the
 * CUDA kernels can be checked bit for bit; nothing in the shipped package may
 * import, link or call it.  Parity of this file with the reference itself is
 * pinned by the fixtures in tests/golden/, which were produced by running the
 * reference's own code (tests/golden/make_golden.py).
 *
 * Each function names the reference source it follows (paths are relative to
 * the reference project's root).
 *
 * Build: gcc -O2 -fopenmp -fPIC -shared -ffp-contract=off -o liblct_oracle.so lct_oracle.c -lm
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define LANES 256

/* Blocks are independent, so the block loops below run in parallel when built
 * with OpenMP; results do not depend on the thread count. */
int orc_set_threads(int n) {
#ifdef _OPENMP
  if (n > 0) omp_set_num_threads(n);
  return omp_get_max_threads();
#else
  (void)n;
  return 1;
#endif
}
#define FIRST_MASK 1023

/* ------------------------------------------------------------------------ */
/* Geometry helpers: LCT/kernels/generic/layout.py:15-18                     */
/* ------------------------------------------------------------------------ */

/* layout.py:15-33: the default "swizzle" mapping XORs the lane with the even
 * row mask (row & 254); "linear" (config.lane_mapping) leaves the lane as it is. */
static int g_lane_mask = 254;

void orc_set_lane_mapping(int linear) { g_lane_mask = linear ? 0 : 254; }

/* Logical (flattened tensor) offset of storage position (block, step, lane). */
static int64_t logical_offset(int64_t block, int steps, int step, int lane) {
  int64_t row = block * steps + step;
  return row * LANES + (lane ^ (int)(row & g_lane_mask));
}

/* ------------------------------------------------------------------------ */
/* Center estimate and shifted tables: LCT/kernels/common/tables.py:9-118    */
/* ------------------------------------------------------------------------ */

/* tables.py:9-49.  src is int16 BF16 bits, or uint8 exponent bytes when
 * precomputed.  n is the logical element count. */
int orc_estimate_center(const void *src, int64_t n, int precomputed) {
  int64_t samples = n < 4096 ? n : 4096;
  int64_t total = 0, kept = 0;
  for (int64_t idx = 0; idx < samples; ++idx) {
    uint32_t hashed = (uint32_t)idx * 0x9E3779B9u;
    int64_t start = idx * n / samples;
    int64_t end = (idx + 1) * n / samples;
    uint64_t jitter = ((uint64_t)hashed * (uint64_t)(end - start)) >> 32;
    int64_t pos = start + (int64_t)jitter;
    int exp;
    if (precomputed)
      exp = (int)((const uint8_t *)src)[pos] - 127;
    else
      exp = (((int)((const int16_t *)src)[pos] >> 7) & 0xFF) - 127;
    if (exp >= -120) { total += exp; ++kept; }
  }
  int64_t safe = kept > 0 ? kept : 1;
  int64_t center = total >= 0 ? (total + safe / 2) / safe : -((-total + safe / 2) / safe);
  if (kept == 0) center = 0;
  if (center < -128) center = -128;
  if (center > 127) center = 127;
  return (int)center;
}

/* tables.py:52-67 (encode, indexed by raw exponent byte) and :102-118 (decode). */
void orc_shift_tables(const int32_t *base_enc, const int32_t *base_dec, int center,
                      int32_t *enc_out, int32_t *dec_out) {
  int zero_delta = (-127 - center) & 255;
  for (int raw = 0; raw < 256; ++raw) {
    int exp = raw - 127;
    int delta = (exp - center) & 255;
    int index = exp == -127 ? 0 : delta + (delta < zero_delta);
    enc_out[raw] = base_enc[index];
  }
  for (int i = 0; i <= FIRST_MASK; ++i) {
    int32_t packed = base_dec[i];
    int length = packed & 255;
    int symbol = (packed >> 8) & 255;
    int delta = symbol == 0 ? 0 : symbol - (symbol <= zero_delta);
    if (delta >= 128) delta -= 256;
    int exponent = symbol == 0 ? -127 : delta + center;
    dec_out[i] = length == 0 ? 0 : (int32_t)(length | (exponent * 256));
  }
}

/* ------------------------------------------------------------------------ */
/* Encoder: LCT/kernels/generic/encode.py:10-169                             */
/* ------------------------------------------------------------------------ */

/*
 * One call encodes the whole tensor.  `encoded` (int32[streams*fw + 4]),
 * `side` (uint8[size]) must be zero-filled by the caller; `defined`
 * (uint8[streams*fw + 4], may be NULL) receives 1 for every payload word the
 * reference kernel stores (the rest is uninitialised memory there).
 * `side_defined` (uint8[size], may be NULL) likewise for side bytes.
 * summaries: int32[4*blocks]; only [0, 2*blocks) is written here.
 */
void orc_encode(const void *src, int precomputed, int64_t logical_numel, int64_t size,
                int block_symbols, int steps, int fw, const int32_t *shifted_enc,
                uint8_t *side, uint8_t *side_defined, int32_t *encoded, uint8_t *defined,
                uint8_t *extra_starts, int32_t *summaries) {
  int64_t blocks = (size + block_symbols - 1) / block_symbols;
  int64_t streams = blocks * LANES;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    int count = 0, total = 0;
    for (int lane = 0; lane < LANES; ++lane) {
      int64_t stream = b * LANES + lane;
      int word = 0, shift = 0, overflow = 0, extra_start = steps;
      uint32_t word_value = 0;
      for (int step = 0; step < steps; step += 2) {
        uint32_t packed[2];
        int valid0 = 0;
        for (int k = 0; k < 2; ++k) {
          int64_t storage = b * (int64_t)block_symbols + (int64_t)(step + k) * LANES + lane;
          int64_t logical = logical_offset(b, steps, step + k, lane);
          int in_range = logical < logical_numel;
          int value = 0;
          if (in_range)
            value = precomputed ? (int)((const uint8_t *)src)[logical]
                                : (int)((const int16_t *)src)[logical];
          int byte;
          if (precomputed) {
            byte = value & 255;
          } else {
            byte = (value >> 7) & 0xFF;
            if (in_range && storage < size) {
              side[storage] = (uint8_t)((value & 0x7F) | ((value >> 8) & 0x80));
              if (side_defined) side_defined[storage] = 1;
            }
          }
          packed[k] = in_range ? (uint32_t)shifted_enc[byte] : 0u;
          if (k == 0) valid0 = storage < size;
        }
        int length0 = (int)(packed[0] >> 20), length1 = (int)(packed[1] >> 20);
        int length = length0 + length1;
        uint32_t code = (packed[0] & 0xFFFFFu) | ((packed[1] & 0xFFFFFu) << length0);
        uint32_t new_word = word_value | (code << shift);
        int crosses = shift + length >= 32;
        int pair_overflow = ((int64_t)word * 32 + shift + length > (int64_t)fw * 32) && valid0;
        int first_overflow = !overflow && pair_overflow;
        if (first_overflow) extra_start = step;
        if (crosses && word < fw) {
          int64_t at = (int64_t)word * streams + stream;
          encoded[at] = (int32_t)(first_overflow ? word_value : new_word);
          if (defined) defined[at] = 1;
        }
        if (crosses) {
          /* A 32-bit pair landing on an empty word leaves nothing to carry. */
          word_value = shift == 0 ? 0u : code >> (32 - shift);
          ++word;
          shift = shift + length - 32;
        } else {
          word_value = new_word;
          shift += length;
        }
        overflow |= pair_overflow;
      }
      if (word < fw && shift != 0) {
        int64_t at = (int64_t)word * streams + stream;
        encoded[at] = (int32_t)word_value;
        if (defined) defined[at] = 1;
      }
      extra_starts[stream] = overflow ? (uint8_t)extra_start : 255;
      if (overflow) { ++count; total += steps - extra_start; }
    }
    summaries[b] = count;
    summaries[blocks + b] = total;
  }
}

/* Exclusive scans of the block summaries: LCT/kernels/generic/metadata.py:20-31. */
void orc_prefix(int32_t *summaries, int64_t blocks, int32_t *counts) {
  int32_t c = 0, t = 0;
  for (int64_t b = 0; b < blocks; ++b) {
    summaries[2 * blocks + b] = c;
    summaries[3 * blocks + b] = t;
    c += summaries[b];
    t += summaries[blocks + b];
  }
  counts[0] = c; counts[1] = t; counts[2] = 0; counts[3] = 0;
}

/*
 * Overflow compaction with metadata: LCT/kernels/generic/compaction.py:99-190
 * (BUILD_META path).  lanes/starts/tail are written at lane_off/start_off/
 * tail_off, which are 0/0/0 for private storage and base/base+count/
 * base+2*count inside a shared arena.
 */
void orc_compact(const void *src, int precomputed, int64_t logical_numel, int64_t size,
                 int block_symbols, int steps, const uint8_t *extra_starts,
                 const int32_t *summaries, uint8_t *lanes, int64_t lane_off,
                 uint8_t *starts, int64_t start_off, uint8_t *tail, int64_t tail_off,
                 int32_t *blocks_out) {
  int64_t blocks = (size + block_symbols - 1) / block_symbols;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    int32_t count = summaries[b];
    int32_t first = summaries[2 * blocks + b];
    int32_t byte_base = summaries[3 * blocks + b];
    if (count > 0) {
      int rank = 0, local = 0;
      for (int lane = 0; lane < LANES; ++lane) {
        int start = extra_starts[b * LANES + lane];
        if (start == 255) continue;
        lanes[lane_off + first + rank] = (uint8_t)lane;
        starts[start_off + first + rank] = (uint8_t)start;
        for (int row = start; row < steps; ++row) {
          int64_t logical = logical_offset(b, steps, row, lane);
          int value = 0;
          if (logical < logical_numel)
            value = precomputed ? (int)((const uint8_t *)src)[logical]
                                : (int)((const int16_t *)src)[logical];
          int exp = precomputed ? value - 127 : ((value >> 7) & 255) - 127;
          tail[tail_off + byte_base + local + (row - start)] = (uint8_t)(int8_t)exp;
        }
        local += steps - start;
        ++rank;
      }
    }
    blocks_out[b] = count;
    blocks_out[blocks + b] = first;
    blocks_out[2 * blocks + b] = byte_base;
  }
}

/* ------------------------------------------------------------------------ */
/* Decoder: LCT/kernels/primitives.py:7-36, generic/decode.py:12-257         */
/* ------------------------------------------------------------------------ */

static int pack_bf16(int value, int sm) {
  return (((value + 127) & 255) << 7) | (sm & 0x7F) | ((sm & 0x80) << 8);
}

static void decode_symbol(uint64_t current, const int32_t *dec, int center, int rare_length,
                          int *value, int *length) {
  int32_t first = dec[current & FIRST_MASK];
  int first_length = first & 255;
  int symbol = (int)((current >> rare_length) & 255);
  int zero_delta = (-127 - center) & 255;
  int delta = symbol == 0 ? 0 : symbol - (symbol <= zero_delta);
  if (delta >= 128) delta -= 256;
  int escaped = symbol == 0 ? -127 : delta + center;
  if (first_length == 0) { *value = escaped; *length = rare_length + 8; }
  else { *value = first >> 8; *length = first_length; }
}

/* Per-lane reader shared by decode and the fused operations. */
typedef struct {
  const int32_t *encoded;
  const int32_t *dec;
  int64_t streams, stream;
  int fw, center, rare_length;
  int word, shift;
  uint64_t window;
} lane_reader;

static void reader_open(lane_reader *r, const int32_t *encoded, const int32_t *dec,
                        int64_t streams, int64_t stream, int fw, int center, int rare_length) {
  r->encoded = encoded; r->dec = dec; r->streams = streams; r->stream = stream;
  r->fw = fw; r->center = center; r->rare_length = rare_length;
  r->word = 0; r->shift = 0;
  uint64_t w0 = (uint32_t)encoded[stream];
  uint64_t w1 = (uint32_t)encoded[streams + stream];
  r->window = w0 | (w1 << 32);
}

/* Decode the pair of symbols at the read position; consume only the bits of
 * symbols whose storage position is valid (decode.py:137-169). */
static void reader_pair(lane_reader *r, int valid0, int valid1, int *value0, int *value1) {
  int next = r->word + 2 < r->fw - 1 ? r->word + 2 : r->fw - 1;
  uint64_t prefetch = (uint32_t)r->encoded[(int64_t)next * r->streams + r->stream];
  int length0, length1;
  decode_symbol(r->window >> r->shift, r->dec, r->center, r->rare_length, value0, &length0);
  int shift1 = r->shift + (valid0 ? length0 : 0);
  decode_symbol(r->window >> shift1, r->dec, r->center, r->rare_length, value1, &length1);
  int next_shift = shift1 + (valid1 ? length1 : 0);
  if (next_shift >= 32) {
    r->window = (r->window >> 32) | (prefetch << 32);
    ++r->word;
    r->shift = next_shift - 32;
  } else {
    r->shift = next_shift;
  }
}

/* Per-lane overflow view of one block: decode.py:195-240. */
typedef struct { int start[LANES]; int64_t offset[LANES]; } block_overflow;

static void map_block(block_overflow *m, int steps, const int32_t *blocks_meta, int64_t blocks,
                      int64_t b, const uint8_t *lanes, int64_t lane_off,
                      const uint8_t *starts, int64_t start_off) {
  for (int l = 0; l < LANES; ++l) { m->start[l] = steps; m->offset[l] = 0; }
  if (!blocks_meta) return;
  int count = blocks_meta[b];
  int64_t first = blocks_meta[blocks + b];
  int64_t running = blocks_meta[2 * blocks + b];
  for (int e = 0; e < count; ++e) {
    int lane = lanes[lane_off + first + e];
    int start = starts[start_off + first + e];
    m->start[lane] = start;
    m->offset[lane] = running;
    running += steps - start;
  }
}

/*
 * Full decode.  blocks_meta == NULL selects the plain decoder; otherwise the
 * overflow overlay with lanes/starts/tail at the given offsets.
 */
void orc_decode(const int32_t *encoded, const uint8_t *side, const int32_t *shifted_dec,
                int center, int rare_length, int64_t logical_numel, int64_t size,
                int block_symbols, int steps, int fw, const int32_t *blocks_meta,
                const uint8_t *lanes, int64_t lane_off, const uint8_t *starts,
                int64_t start_off, const uint8_t *tail, int64_t tail_off, int16_t *out) {
  int64_t blocks = (size + block_symbols - 1) / block_symbols;
  int64_t streams = blocks * LANES;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    block_overflow map;
    map_block(&map, steps, blocks_meta, blocks, b, lanes, lane_off, starts, start_off);
    for (int lane = 0; lane < LANES; ++lane) {
      lane_reader r;
      reader_open(&r, encoded, shifted_dec, streams, b * LANES + lane, fw, center, rare_length);
      for (int step = 0; step < steps; step += 2) {
        int64_t s0 = b * (int64_t)block_symbols + (int64_t)step * LANES + lane;
        int64_t s1 = s0 + LANES;
        int v[2];
        reader_pair(&r, s0 < size, s1 < size, &v[0], &v[1]);
        for (int k = 0; k < 2; ++k) {
          int64_t storage = k ? s1 : s0;
          int64_t logical = logical_offset(b, steps, step + k, lane);
          int value = v[k];
          if (step + k >= map.start[lane])
            value = (int)tail[tail_off + map.offset[lane] + (step + k - map.start[lane])];
          int sm = storage < size ? side[storage] : 0;
          if (logical < logical_numel) out[logical] = (int16_t)pack_bf16(value, sm);
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Fused pointwise operations: LCT/kernels/generic/pointwise.py:31-363,      */
/* pointwise_scalar_dual.py:118-346                                          */
/* ------------------------------------------------------------------------ */

static float bf16_to_float(uint16_t bits) {
  uint32_t u = (uint32_t)bits << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* Round-to-nearest-even float -> bf16, NaN canonicalised as the GPU's
 * cvt.rn.bf16.f32 does (0x7FFF). */
static uint16_t float_to_bf16(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7FFFFFFFu) > 0x7F800000u) return 0x7FFF;
  u += 0x7FFFu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

/* Correctly rounded double -> bf16 (single rounding, subnormals included). */
static uint16_t double_to_bf16(double d) {
  if (d != d) return 0x7FFF;
  uint16_t sign = signbit(d) ? 0x8000 : 0;
  double a = fabs(d);
  if (a == 0.0) return sign;
  if (isinf(a)) return sign | 0x7F80;
  int e;
  frexp(a, &e);                 /* a = m * 2^e, m in [0.5, 1) */
  int exp = e - 1;              /* a in [2^exp, 2^(exp+1)) */
  if (exp < -126) exp = -126;   /* subnormal spacing */
  double scaled = ldexp(a, 7 - exp);       /* units of the bf16 ulp; exact */
  double q = nearbyint(scaled);            /* default rounding mode: nearest even */
  if (exp > 127) return sign | 0x7F80;
  uint32_t mant = (uint32_t)q;             /* in [0, 256] */
  uint32_t bits;
  if (mant < 128) bits = mant;                         /* subnormal or zero */
  else bits = ((uint32_t)(exp + 127) << 7) + (mant - 128); /* carry propagates into exponent */
  if (bits >= 0x7F80) bits = 0x7F80;
  return sign | (uint16_t)bits;
}

enum { OP_ADD = 0, OP_MULTIPLY = 1, OP_SCALED = 2, OP_LERP = 3, OP_EMA_SQUARE = 4 };

/* torch.lerp(start, end, weight) on float32 as PyTorch's CUDA kernel evaluates it (the formula
 * of ATen/native/Lerp.h with the multiply-adds contracted; pinned against torch on a GPU by
 * tests/test_gpu_momentum.py): what LCT/components/sparse_utils.py:88-90,193 computes. */
static float lerp_f32(float start, float end, float weight) {
  float d = end - start;
  return fabsf(weight) < 0.5f ? fmaf(weight, d, start) : fmaf(-d, 1.0f - weight, end);
}

/* pointwise.py:340-363 followed by the BF16 rounding of :50. */
static uint16_t apply_op(int op, uint16_t left, uint16_t right, float alpha, float beta,
                         int alpha_is_one, int beta_is_one) {
  float a = bf16_to_float(left), b = bf16_to_float(right);
  /* BF16 add/multiply round the exact result once; double holds it exactly
   * (products) or to far more than twice the target precision (sums). */
  if (op == OP_ADD) return double_to_bf16((double)a + (double)b);
  if (op == OP_MULTIPLY) return double_to_bf16((double)a * (double)b);
  if (op == OP_LERP) return float_to_bf16(lerp_f32(a, b, alpha));
  if (op == OP_EMA_SQUARE) { /* sparse_utils.py:194: mul_(beta2) rounds, then addcmul_ */
    float scaled = bf16_to_float(float_to_bf16(a * alpha));
    return float_to_bf16(fmaf(beta, b * b, scaled));
  }
  float r;
  if (alpha_is_one) r = beta_is_one ? a + b : fmaf(b, beta, a);
  else r = fmaf(a, alpha, beta_is_one ? b : b * beta);
  return float_to_bf16(r);
}

/*
 * compA (op) dense B.  dense_out != NULL: BF16 bits at logical offsets.
 * Otherwise side_out (storage order, every storage position written) and
 * exp_out (logical order, valid positions only), padding treated as +0.0.
 */
void orc_pointwise(const int32_t *encoded, const uint8_t *side, const int32_t *shifted_dec,
                   int center, int rare_length, int64_t logical_numel, int64_t size,
                   int block_symbols, int steps, int fw, const int32_t *blocks_meta,
                   const uint8_t *lanes, int64_t lane_off, const uint8_t *starts,
                   int64_t start_off, const uint8_t *tail, int64_t tail_off,
                   const uint16_t *other, int op, float alpha, float beta, int alpha_is_one,
                   int beta_is_one, uint16_t *dense_out, uint8_t *side_out, uint8_t *exp_out) {
  int64_t blocks = (size + block_symbols - 1) / block_symbols;
  int64_t streams = blocks * LANES;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    block_overflow map;
    map_block(&map, steps, blocks_meta, blocks, b, lanes, lane_off, starts, start_off);
    for (int lane = 0; lane < LANES; ++lane) {
      lane_reader r;
      reader_open(&r, encoded, shifted_dec, streams, b * LANES + lane, fw, center, rare_length);
      for (int step = 0; step < steps; step += 2) {
        int64_t s0 = b * (int64_t)block_symbols + (int64_t)step * LANES + lane;
        int v[2];
        reader_pair(&r, s0 < size, s0 + LANES < size, &v[0], &v[1]);
        for (int k = 0; k < 2; ++k) {
          int64_t storage = s0 + (int64_t)k * LANES;
          int64_t logical = logical_offset(b, steps, step + k, lane);
          int value = v[k];
          if (step + k >= map.start[lane])
            value = (int)tail[tail_off + map.offset[lane] + (step + k - map.start[lane])];
          int sm = storage < size ? side[storage] : 0;
          int in_range = logical < logical_numel;
          uint16_t left = (uint16_t)pack_bf16(value, sm);
          uint16_t right = in_range ? other[logical] : 0;
          uint16_t res = apply_op(op, left, right, alpha, beta, alpha_is_one, beta_is_one);
          if (dense_out) {
            if (in_range) dense_out[logical] = res;
          } else {
            if (!in_range) res = 0;
            if (storage < size) side_out[storage] = (uint8_t)((res & 0x7F) | ((res >> 8) & 0x80));
            if (in_range) exp_out[logical] = (uint8_t)((res >> 7) & 0xFF);
          }
        }
      }
    }
  }
}

/* out = bf16(lerp(start, end, weight)) elementwise on BF16 bit patterns: the Nesterov direction
 * grad.lerp_(momentum, mu) of sparse_utils.py:90. */
void orc_lerp_dense(const uint16_t *start, const uint16_t *end, float weight, int64_t n,
                    uint16_t *out) {
#pragma omp parallel for schedule(static)
  for (int64_t i = 0; i < n; ++i)
    out[i] = float_to_bf16(lerp_f32(bf16_to_float(start[i]), bf16_to_float(end[i]), weight));
}

/* alpha * compA + compB: pointwise_scalar_dual.py:118-346. */
void orc_dual(const int32_t *a_encoded, const uint8_t *a_side, const int32_t *a_dec, int a_center,
              const int32_t *a_meta, const uint8_t *a_lanes, int64_t a_lane_off,
              const uint8_t *a_starts, int64_t a_start_off, const uint8_t *a_tail, int64_t a_tail_off,
              const int32_t *b_encoded, const uint8_t *b_side, const int32_t *b_dec, int b_center,
              const int32_t *b_meta, const uint8_t *b_lanes, int64_t b_lane_off,
              const uint8_t *b_starts, int64_t b_start_off, const uint8_t *b_tail, int64_t b_tail_off,
              int rare_length, int64_t logical_numel, int64_t size, int block_symbols, int steps,
              int fw, float alpha, uint16_t *dense_out, uint8_t *side_out, uint8_t *exp_out) {
  int64_t blocks = (size + block_symbols - 1) / block_symbols;
  int64_t streams = blocks * LANES;
#pragma omp parallel for schedule(static)
  for (int64_t b = 0; b < blocks; ++b) {
    block_overflow ma, mb;
    map_block(&ma, steps, a_meta, blocks, b, a_lanes, a_lane_off, a_starts, a_start_off);
    map_block(&mb, steps, b_meta, blocks, b, b_lanes, b_lane_off, b_starts, b_start_off);
    for (int lane = 0; lane < LANES; ++lane) {
      lane_reader ra, rb;
      reader_open(&ra, a_encoded, a_dec, streams, b * LANES + lane, fw, a_center, rare_length);
      reader_open(&rb, b_encoded, b_dec, streams, b * LANES + lane, fw, b_center, rare_length);
      for (int step = 0; step < steps; step += 2) {
        int64_t s0 = b * (int64_t)block_symbols + (int64_t)step * LANES + lane;
        int va[2], vb[2];
        /* Symbols taken from the tail consume no payload bits (dual.py:211-214). */
        reader_pair(&ra, s0 < size && step < ma.start[lane],
                    s0 + LANES < size && step + 1 < ma.start[lane], &va[0], &va[1]);
        reader_pair(&rb, s0 < size && step < mb.start[lane],
                    s0 + LANES < size && step + 1 < mb.start[lane], &vb[0], &vb[1]);
        for (int k = 0; k < 2; ++k) {
          int64_t storage = s0 + (int64_t)k * LANES;
          int64_t logical = logical_offset(b, steps, step + k, lane);
          int xa = va[k], xb = vb[k];
          if (step + k >= ma.start[lane])
            xa = (int)a_tail[a_tail_off + ma.offset[lane] + (step + k - ma.start[lane])];
          if (step + k >= mb.start[lane])
            xb = (int)b_tail[b_tail_off + mb.offset[lane] + (step + k - mb.start[lane])];
          int in_range = logical < logical_numel;
          int sa = storage < size ? a_side[storage] : 0;
          int sb = storage < size ? b_side[storage] : 0;
          float fa = bf16_to_float((uint16_t)pack_bf16(xa, sa));
          float fb = bf16_to_float((uint16_t)pack_bf16(xb, sb));
          uint16_t res = float_to_bf16(fmaf(fa, alpha, fb));
          if (dense_out) {
            if (in_range) dense_out[logical] = res;
          } else {
            if (!in_range) res = 0;
            if (storage < size) side_out[storage] = (uint8_t)((res & 0x7F) | ((res >> 8) & 0x80));
            if (in_range) exp_out[logical] = (uint8_t)((res >> 7) & 0xFF);
          }
        }
      }
    }
  }
}

/* ------------------------------------------------------------------------ */
/* Arena allocator: LCT/kernels/tensor_buffer.py:18-179                      */
/* meta = int32[2*R + 3]: free_starts[R] | free_sizes[R] | count | lock | gen */
/* ------------------------------------------------------------------------ */

void orc_buf_reset(int32_t *meta, int regions, int32_t capacity) {
  for (int i = 0; i < 2 * regions; ++i) meta[i] = 0;
  meta[regions] = capacity;
  meta[2 * regions] = 1;
  meta[2 * regions + 1] = 0;
  meta[2 * regions + 2] += 1;
}

/* tensor_buffer.py:37-91; request = bytes + items * item_bytes, aligned up. */
void orc_buf_alloc(int32_t *meta, int regions, int32_t bytes, int32_t items, int item_bytes,
                   int alignment, int32_t *descriptor) {
  int32_t *starts = meta, *sizes = meta + regions, *count = meta + 2 * regions;
  int32_t request = bytes + items * item_bytes;
  int32_t size = (request + alignment - 1) / alignment * alignment;
  int slot = regions;
  for (int i = 0; i < *count; ++i)
    if (sizes[i] >= size) { slot = i; break; }
  int ok = request > 0 && slot < *count;
  int32_t start = ok ? starts[slot] : 0;
  if (ok && sizes[slot] == size) {
    for (int i = slot; i + 1 < *count; ++i) { starts[i] = starts[i + 1]; sizes[i] = sizes[i + 1]; }
    *count -= 1;
  } else if (ok) {
    starts[slot] = start + size;
    sizes[slot] -= size;
  }
  descriptor[0] = ok ? start : -1;
  descriptor[1] = ok ? size : 0;
  descriptor[2] = request <= 0 ? 2 : (ok ? 0 : 1);
  descriptor[3] = meta[2 * regions + 2];
}

/* tensor_buffer.py:94-179; returns the status word (0 ok, 3 list full, 4 invalid/stale). */
int orc_buf_free(int32_t *meta, int regions, int32_t *descriptor) {
  int32_t *starts = meta, *sizes = meta + regions, *count = meta + 2 * regions;
  int32_t offset = descriptor[0], size = descriptor[1];
  int valid = descriptor[2] == 0 && descriptor[3] == meta[2 * regions + 2] && offset >= 0 && size > 0;
  if (!valid) return 4;
  int n = *count, insert = 0;
  for (int i = 0; i < n; ++i) insert += starts[i] < offset;
  int merge_prev = insert > 0 && starts[insert - 1] + sizes[insert - 1] == offset;
  int merge_next = insert < n && offset + size == starts[insert];
  if (merge_prev && merge_next) {
    sizes[insert - 1] += size + sizes[insert];
    for (int i = insert; i + 1 < n; ++i) { starts[i] = starts[i + 1]; sizes[i] = sizes[i + 1]; }
    *count = n - 1;
  } else if (merge_prev) {
    sizes[insert - 1] += size;
  } else if (merge_next) {
    starts[insert] = offset;
    sizes[insert] += size;
  } else {
    if (n >= regions) return 3;
    for (int i = n; i > insert; --i) { starts[i] = starts[i - 1]; sizes[i] = sizes[i - 1]; }
    starts[insert] = offset;
    sizes[insert] = size;
    *count = n + 1;
  }
  descriptor[2] = 5;
  return 0;
}
