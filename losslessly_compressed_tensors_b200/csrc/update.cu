// Fused update of compressed state: decode -> pointwise operation -> re-encode in
// ONE launch per tensor, with no dense or split intermediate in HBM.
//
// The re-encoded tensor gets a fresh exponent center, sampled from the RESULT at
// (up to) 4096 hashed positions - the same positions and the same rounding the
// reference uses when it re-estimates the center from its split intermediate
// (LCT/codec/pointwise.py:263-278 -> LCT/codec/encode.py:59-65).  So a tiny
// pre-pass computes just those result values (each sample decodes its lane's
// stream up to the sampled step), the ordinary center kernel turns the samples
// into center + tables, and the main kernel then has everything it needs:
//
//   per codec block (one CTA), per 32-row tile, per warp:
//     lane side  decode this lane's pairs            -> exponent tile (shared)
//     row side   join with side bytes, load B, op    -> new side bytes to HBM,
//                new exponent bytes back into the tile
//     lane side  encode this lane's pairs from the tile into the output payload image
//
// Lanes whose output overflows their bit budget also store their raw result
// exponents from the overflow step on into `spill` (logical order), which is
// what the tail compaction reads afterwards; nothing else touches `spill`.
#include "decode_core.cuh"
#include "encode_core.cuh"

namespace lct {

constexpr int kSampleCount = 4096;

// Shared memory of the sample kernel: just the center-specific table.
struct __align__(16) SampleShared {
  uint32_t table[kPairEntries];
  uint8_t index_to_byte[256];
};

// One symbol at the head of a 64-bit window read straight from global memory.
struct GlobalReader {
  const uint32_t* next_ptr;
  int64_t stride;
  uint32_t lo, hi;
  int shift, word, fixed_words;

  __device__ __forceinline__ void open(const uint32_t* encoded, int64_t streams, int64_t stream,
                                       int fw) {
    const uint32_t* p = encoded + stream;
    stride = streams;
    fixed_words = fw;
    lo = p[0];
    hi = p[streams];
    next_ptr = p + 2 * streams;
    shift = 0;
    word = 0;
  }
  __device__ __forceinline__ uint32_t peek() const { return __funnelshift_r(lo, hi, shift); }
  __device__ __forceinline__ void advance(int bits) {  // bits <= 16
    shift += bits;
    if (shift >= 32) {
      shift -= 32;
      lo = hi;
      ++word;
      hi = (word + 1 < fixed_words) ? *next_ptr : 0u;
      next_ptr += stride;
    }
  }
};

// Exponent byte of A at storage position (block, step, lane).
__device__ __forceinline__ uint32_t exponent_at(const OperandView& a, const Shape& g,
                                                const SampleShared& sh, int64_t block, int step,
                                                int lane) {
  if (a.mode != 0 && (a.mode != 2 || a.descriptor[2] == 0)) {
    const int count = a.blocks[block];
    if (count > 0) {
      const int64_t region = a.mode == 2 ? a.descriptor[0] : 0;
      const int64_t total = a.mode == 2 ? *a.count : 0;
      const int64_t first = a.blocks[g.n_blocks + block];
      int64_t offset = a.blocks[2 * g.n_blocks + block];
      for (int e = 0; e < count; ++e) {
        const int entry_lane = a.lanes[region + first + e];
        const int entry_start = a.starts[region + total + first + e];
        if (entry_lane == lane) {
          if (step >= entry_start)
            return ((uint32_t)tail_origin(a)[offset + step - entry_start] + 127u) & 255u;
          break;
        }
        offset += g.steps - entry_start;
      }
    }
  }
  GlobalReader r;
  r.open(a.encoded, g.streams, block * kLanes + lane, g.fixed_words);
  uint32_t exponent = 0;
  for (int s = 0; s <= step; ++s) {
    const uint32_t bits = r.peek();
    const uint32_t entry = sh.table[table_slot(bits)];
    int length;
    if (entry & kEscape) {
      exponent = sh.index_to_byte[(bits >> g.rare_length) & 255u];
      length = g.rare_length + 8;
    } else {
      exponent = entry & 255u;
      length = (int)((entry >> 24) & 15u);
    }
    r.advance(length);
  }
  return exponent;
}

// Result exponent bytes at the center-sample positions of the result tensor.
__global__ void __launch_bounds__(kThreads)
update_sample_kernel(OperandView a, Shape g, const uint16_t* __restrict__ other, OpSpec spec,
                     uint8_t* __restrict__ samples) {
  __shared__ SampleShared sh;
  const int tid = threadIdx.x;
  const int center = *a.center;
  sh.index_to_byte[tid] = (uint8_t)index_to_exponent_byte((uint32_t)tid, center);
  __syncthreads();
  for (int i = tid; i < kPairEntries; i += kThreads) {
    const uint32_t e = a.pair_table[i];
    sh.table[i] = (e & 0xFFFF0000u) | sh.index_to_byte[e & 255u] |
                  ((uint32_t)sh.index_to_byte[(e >> 8) & 255u] << 8);
  }
  __syncthreads();
  const int64_t n = g.logical_numel;
  const int64_t count = n < kSampleCount ? n : kSampleCount;
  const int64_t idx = (int64_t)blockIdx.x * kThreads + tid;
  if (idx >= count) return;
  // Same jittered position as the center estimate (one per equal slice of the tensor).
  const uint32_t hashed = (uint32_t)idx * 0x9E3779B9u;
  const int64_t start = idx * n / count, end = (idx + 1) * n / count;
  const int64_t pos = start + (int64_t)(((uint64_t)hashed * (uint64_t)(end - start)) >> 32);
  const int64_t row = pos >> 8;
  const int lane = (int)(pos & 255) ^ (int)(row & 254);
  const int64_t block = row / g.steps;
  const int step = (int)(row - block * g.steps);
  const uint32_t exponent = exponent_at(a, g, sh, block, step, lane);
  const uint32_t side = a.side[block * (int64_t)g.block_symbols + (int64_t)step * kLanes + lane];
  const uint32_t left = (exponent << 7) | (side & 0x7Fu) | ((side & 0x80u) << 8);
  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  const uint32_t result = apply_op(left, other[pos], spec.op, spec.alpha_is_one != 0,
                                   spec.beta_is_one != 0, alpha, beta);
  samples[idx] = (uint8_t)((result >> 7) & 0xFFu);
}


// Split one row of results (4 words, column order; padding already zeroed):
// exponent bytes stay in column order, side bytes go to lane order.
__device__ __forceinline__ void split_row(const uint32_t r[4], uint32_t q, uint32_t* e03,
                                          uint32_t* e47, uint2* side_lane_order) {
  const uint32_t l03 = prmt(r[0], r[1], 0x6420), h03 = prmt(r[0], r[1], 0x7531);
  const uint32_t l47 = prmt(r[2], r[3], 0x6420), h47 = prmt(r[2], r[3], 0x7531);
  *e03 = exponent_bytes(l03, h03);
  *e47 = exponent_bytes(l47, h47);
  const uint32_t c03 = side_bytes(l03, h03), c47 = side_bytes(l47, h47);
  *side_lane_order =
      make_uint2(prmt(c03, c47, pair_selector_low(q)), prmt(c03, c47, pair_selector_high(q)));
}

// Shared memory: [input payload image | DecodeShared | encode table | output payload image].
__global__ void __launch_bounds__(kThreads, 2)
update_fused_kernel(OperandView a, Shape g, const uint16_t* __restrict__ other, bool other_vector_ok,
                    OpSpec spec, const int32_t* __restrict__ shifted_encode,
                    uint8_t* __restrict__ side_out, uint32_t* __restrict__ encoded_out,
                    uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries,
                    uint8_t* __restrict__ spill) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const size_t image = (size_t)(g.fixed_words + 2) * kLanes * 4;
  uint32_t* payload = reinterpret_cast<uint32_t*>(smem_raw);
  DecodeShared& sh = *reinterpret_cast<DecodeShared*>(smem_raw + image);
  uint2* encode_table = reinterpret_cast<uint2*>(smem_raw + image + sizeof(DecodeShared));
  uint32_t* out_image = reinterpret_cast<uint32_t*>(encode_table + 256);

  const int64_t block = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  const bool full_block = block_base + g.block_symbols <= g.logical_numel;
  {
    const uint32_t packed = (uint32_t)shifted_encode[tid];
    encode_table[tid] = make_uint2(packed & 0xFFFFFu, packed >> 20);
  }
  for (int w = 0; w < g.fixed_words; ++w) out_image[w * kLanes + tid] = 0u;
  if (block == 0 && tid < 4) encoded_out[g.streams * g.fixed_words + tid] = 0u;
  prepare_block(sh, payload, a, g, block);  // ends with a block barrier

  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel);
  const int tail_from = sh.overflow_start[tid];
  const int coded = min(valid, tail_from);
  const uint8_t* tail_bytes = a.mode ? tail_origin(a) + sh.overflow_offset[tid] : nullptr;
  BitReader reader;
  reader.open(payload + tid);
  const uint32_t* last_row = payload + tid + (g.fixed_words + 2) * kLanes;
  uint16_t* tile = sh.tile[warp];
  const uint8_t* tile_bytes = reinterpret_cast<const uint8_t*>(tile);
  uint32_t* out_column = out_image + tid;
  const int budget_bits = g.fixed_words * 32;
  uint32_t lo = 0;
  int pos = 0, extra_start = -1;
  bool open = true;

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    decode_tile_rows(reader, sh, tile, lane32, step0, coded, tail_from, tail_bytes, g.rare_length,
                     last_row);
    __syncwarp();
    // ---- row side: A (op) B, new side bytes out, new exponents back into the tile ----
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = (lane32 >> 2) + 8 * u, j4 = lane32 & 3;
      const UnitPlace place = place_unit(warp, p, j4, row0, step0, block_base);
      uint4* slot = reinterpret_cast<uint4*>(&tile[p * 32 + 8 * j4]);
      const uint4 words = *slot;
      uint32_t e_top03, e_top47, e_bot03, e_bot47;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t s_at = place.storage + half * kLanes;
        const int64_t l_at = place.logical + half * kLanes;
        uint32_t left[4], right[4], result[4];
        join_row(words, __ldcs(reinterpret_cast<const uint2*>(a.side + s_at)), place.q, half == 1,
                 left);
        load_dense8(other, l_at, g.logical_numel, other_vector_ok, right);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          result[k] = apply_op(left[k], right[k], spec.op, spec.alpha_is_one != 0,
                               spec.beta_is_one != 0, alpha, beta);
        if (!full_block && l_at + 8 > g.logical_numel) {  // padding counts as +0.0
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (l_at + i >= g.logical_numel) result[i >> 1] &= (i & 1) ? 0x0000FFFFu : 0xFFFF0000u;
        }
        uint2 side_lane_order;
        split_row(result, place.q, half ? &e_bot03 : &e_top03, half ? &e_bot47 : &e_top47,
                  &side_lane_order);
        __stcs(reinterpret_cast<uint2*>(side_out + s_at), side_lane_order);
      }
      *slot = make_uint4(prmt(e_top03, e_bot03, 0x5140), prmt(e_top03, e_bot03, 0x7362),
                         prmt(e_top47, e_bot47, 0x5140), prmt(e_top47, e_bot47, 0x7362));
    }
    __syncwarp();
    // ---- lane side: encode the result exponents ----
    if (open) {
      if (full_block)
        open = encode_tile_rows<false>(encode_table, tile_bytes, out_column, lane32, step0, valid,
                                       budget_bits, pos, lo, extra_start);
      else
        open = encode_tile_rows<true>(encode_table, tile_bytes, out_column, lane32, step0, valid,
                                      budget_bits, pos, lo, extra_start);
    }
    if (!open) {
      // Raw exponents of the overflowed lane, from its overflow step on, for the tail pass.
      const int from = extra_start > step0 ? (extra_start - step0) >> 1 : 0;
      const int64_t tile_row = row0 + step0;
      const int group = warp ^ ((int)(tile_row >> 5) & 7);
      for (int p = from; p < kTilePairs; ++p) {
        const int column = lane32 ^ (2 * p);
        const int64_t logical = (tile_row + 2 * p) * kLanes + 32 * group + column;
        const uint8_t* e = tile_bytes + 2 * (p * 32 + column);
        if (logical < g.logical_numel) spill[logical] = e[0];
        if (logical + kLanes < g.logical_numel) spill[logical + kLanes] = e[1];
      }
    }
    __syncwarp();
  }
  if (open && (pos & 31) != 0) out_column[(pos >> 5) * kLanes] = lo;
  extra_starts[block * kLanes + tid] = extra_start < 0 ? (uint8_t)255 : (uint8_t)extra_start;

  int bad = extra_start >= 0 ? 1 : 0;
  int bytes = extra_start >= 0 ? g.steps - extra_start : 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    bad += __shfl_down_sync(0xFFFFFFFFu, bad, d);
    bytes += __shfl_down_sync(0xFFFFFFFFu, bytes, d);
  }
  if (lane32 == 0) { sh.scan[warp] = bad; sh.scan[8 + warp] = bytes; }
  __syncthreads();  // also publishes every lane's output words
  if (tid == 0) {
    int total_bad = 0, total_bytes = 0;
    for (int w = 0; w < kWarps; ++w) { total_bad += sh.scan[w]; total_bytes += sh.scan[8 + w]; }
    summaries[block] = total_bad;
    summaries[g.n_blocks + block] = total_bytes;
  }
  uint32_t* out = encoded_out + block * kLanes;
  for (int i = tid; i < g.fixed_words * (kLanes / 4); i += kThreads) {
    const int w = i >> 6, c = (i & 63) * 4;
    const uint4 v = *reinterpret_cast<const uint4*>(&out_image[w * kLanes + c]);
    __stcs(reinterpret_cast<uint4*>(out + (int64_t)w * g.streams + c), v);
  }
}

}  // namespace lct

extern "C" {

static int check_update_args(const lct_operand* a, const void* other, const float* alpha,
                             const float* beta, int op, int* alpha_is_one, int* beta_is_one,
                             lct::OperandView* view) {
  int rc = lct::view_of(a, view);
  if (rc) return rc;
  if (other == nullptr) return LCT_E_NULL_POINTER;
  if ((reinterpret_cast<uintptr_t>(other) & 1u) != 0) return LCT_E_ALIGNMENT;
  if (op < LCT_OP_ADD || op > LCT_OP_SCALAR_MUL_ADD) return LCT_E_BAD_ARGUMENT;
  if (op == LCT_OP_SCALAR_MUL_ADD) {
    if (!*alpha_is_one && alpha == nullptr) return LCT_E_NULL_POINTER;
    if (!*beta_is_one && beta == nullptr) return LCT_E_NULL_POINTER;
  } else {
    *alpha_is_one = *beta_is_one = 1;
  }
  return 0;
}

int lct_update_sample(const lct_operand* a, const void* other, const float* alpha,
                      const float* beta, int op, int alpha_is_one, int beta_is_one,
                      uint8_t* samples, int64_t size, int64_t logical_numel, int block_symbols,
                      int steps, int fixed_words, int rare_length, void* stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = check_update_args(a, other, alpha, beta, op, &alpha_is_one, &beta_is_one, &va))) return rc;
  if (samples == nullptr) return LCT_E_NULL_POINTER;
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const int64_t count = logical_numel < lct::kSampleCount ? logical_numel : lct::kSampleCount;
  const unsigned grid = (unsigned)((count + lct::kThreads - 1) / lct::kThreads);
  lct::update_sample_kernel<<<grid, lct::kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      va, g, static_cast<const uint16_t*>(other), spec, samples);
  return (int)cudaGetLastError();
}

int lct_update_fused(const lct_operand* a, const void* other, const float* alpha,
                     const float* beta, int op, int alpha_is_one, int beta_is_one,
                     const int32_t* shifted_encode, uint8_t* side_out, int32_t* encoded_out,
                     uint8_t* extra_starts, int32_t* summaries, uint8_t* spill, int64_t size,
                     int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                     int rare_length, void* stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = check_update_args(a, other, alpha, beta, op, &alpha_is_one, &beta_is_one, &va))) return rc;
  if (shifted_encode == nullptr || side_out == nullptr || encoded_out == nullptr ||
      extra_starts == nullptr || summaries == nullptr || spill == nullptr)
    return LCT_E_NULL_POINTER;
  if (!lct::aligned16(side_out) || !lct::aligned16(encoded_out)) return LCT_E_ALIGNMENT;
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const size_t shared = lct::operand_shared_bytes(fixed_words) + 256 * sizeof(uint2) +
                        (size_t)fixed_words * lct::kLanes * 4;
  if ((rc = lct::opt_in_shared(lct::update_fused_kernel, shared)) != 0) return rc;
  lct::update_fused_kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared,
                             static_cast<cudaStream_t>(stream)>>>(
      va, g, static_cast<const uint16_t*>(other), lct::aligned16(other), spec, shifted_encode,
      side_out, reinterpret_cast<uint32_t*>(encoded_out), extra_starts, summaries, spill);
  return (int)cudaGetLastError();
}

}  // extern "C"
