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
//     lane side  encode this lane's pairs from the tile; finished words go straight
//                to the output payload in HBM
//
// lct_update strings the five launches of an update (sample, center, this kernel,
// scan, tail compaction) together behind one call, each scheduled while its
// predecessor runs (programmatic stream serialisation, see batch.cuh).
//
// Lanes whose output overflows their bit budget also store their raw result
// exponents from the overflow step on into `spill` (logical order), which is
// what the tail compaction reads afterwards; nothing else touches `spill`.
#include "batch.cuh"
#include "center.cuh"
#include "decode_core.cuh"
#include "encode_core.cuh"

namespace lct {

// The sample kernel walks bit streams with the two-symbol table of the tensor's
// center read straight from global memory (16 KB, L1-resident after the first
// touches).  Shared memory holds one payload column per thread: fixed_words + 3
// rows of 256 words (the window refill may read one row past the two zero rows
// when a stream uses its whole budget; the refill pointer is clamped to that
// last row on every pair).

// Read position of one sampled lane: a 96-bit register window over its shared column (the
// word under the position and the two after it) plus the bit offset inside the first word.
struct BitReader {
  const uint32_t* next_row;  // column word that enters the window at the next refill
  const uint32_t* last_row;  // the column's last zero row
  uint32_t cur, n1, n2;
  int shift;                 // 0..31 between pairs

  // `column`: fixed_words + 2 rows with stride kLanes, the last two zero.
  __device__ __forceinline__ void open(const uint32_t* column, int fixed_words) {
    cur = column[0];
    n1 = column[kLanes];
    n2 = column[2 * kLanes];
    next_row = column + 3 * kLanes;
    last_row = column + (fixed_words + 1) * kLanes;
    shift = 0;
  }
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

// One symbol (exponent byte) from an entry and the bits it was looked up with.
__device__ __forceinline__ uint32_t byte_of(uint32_t entry, uint32_t bits, int rare_length,
                                            int center, int* length) {
  *length = (int)entry_first_length(entry);
  if (entry & kEscape) return index_to_exponent_byte((bits >> rare_length) & 255u, center);
  return entry_first_symbol(entry);
}

// Raw-tail exponent byte of A at (block, step, lane), or -1 when that step is in the bit stream.
__device__ __forceinline__ int tail_exponent_at(const OperandView& a, const Shape& g, int64_t block,
                                                int step, int lane) {
  if (a.mode == 0 || (a.mode == 2 && a.descriptor[2] != 0)) return -1;
  const int count = a.blocks[block];
  if (count <= 0) return -1;
  const int64_t region = a.mode == 2 ? a.descriptor[0] : 0;
  const int64_t total = a.mode == 2 ? *a.count : 0;
  const int64_t first = a.blocks[g.n_blocks + block];
  int64_t offset = a.blocks[2 * g.n_blocks + block];
  for (int e = 0; e < count; ++e) {
    const int entry_lane = a.lanes[region + first + e];
    const int entry_start = a.starts[region + total + first + e];
    if (entry_lane == lane) {
      if (step < entry_start) return -1;
      return (int)(((uint32_t)tail_origin(a)[offset + step - entry_start] + 127u) & 255u);
    }
    offset += g.steps - entry_start;
  }
  return -1;
}

// Exponent byte of the symbol at `step` of the stream staged in `column`.
__device__ __forceinline__ uint32_t walk_to(const uint32_t* __restrict__ table, const Shape& g,
                                            const uint32_t* column, int step, int center) {
  BitReader r;
  r.open(column, g.fixed_words + 1);  // the column has one more (zero) row than a decoder image
  uint32_t first = 0, second = 0;
  for (int p = 0; p <= (step >> 1); ++p) {
    r.tile_start();
    const uint32_t bits = r.peek0();
    const uint32_t entry = __ldg(table + table_slot(bits));
    int consumed;
    if ((int32_t)entry < 0) {
      int l0, l1;
      first = byte_of(entry, bits, g.rare_length, center, &l0);
      const uint32_t bits1 = r.peek(l0);
      second = byte_of(__ldg(table + table_slot(bits1)), bits1, g.rare_length, center, &l1);
      consumed = l0 + l1;
    } else {
      first = entry_first_symbol(entry);
      second = entry_second_symbol(entry);
      consumed = (int)(entry & 31u);
    }
    r.advance(consumed);
  }
  return (step & 1) ? second : first;
}

// Result exponent bytes at the center-sample positions of the result tensor.
// The kernel is a chain of memory latencies in front of a serial bit-stream
// walk, so everything independent starts first: the lane's payload words go to
// its shared column asynchronously while the overflow map is consulted.
// `chunk`: which 256 of the (up to) 4096 samples this CTA computes.
__device__ __forceinline__ void update_sample_chunk(const OperandView& a, const Shape& g,
                                                    const uint16_t* __restrict__ other,
                                                    const OpSpec& spec,
                                                    const uint16_t* __restrict__ known,
                                                    uint8_t* __restrict__ samples,
                                                    uint16_t* __restrict__ values, int chunk) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x;
  const int64_t n = g.logical_numel;
  const int64_t count = n < kSampleCount ? n : kSampleCount;
  const int64_t idx = (int64_t)chunk * kThreads + tid;
  if (idx >= count) return;
  // Same jittered position as the center estimate (one per equal slice of the tensor).
  const int64_t pos = sample_position(idx, n);
  const uint32_t right = other[pos];
  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  uint32_t left;
  if (known != nullptr) {
    // A's values at the sample positions were kept when A was made: no stream to walk.
    left = known[idx];
  } else {
    uint32_t* column = reinterpret_cast<uint32_t*>(smem_raw) + tid;
    const int64_t row = pos >> 8;
    const int lane = (int)(pos & 255) ^ (int)(row & g.lane_mask);
    const int64_t block = row / g.steps;
    const int step = (int)(row - block * g.steps);
    const uint32_t* words = a.encoded + block * kLanes + lane;
    for (int w = 0; w < g.fixed_words; ++w)
      cp_async_4(column + w * kLanes, words + (int64_t)w * g.streams);
    column[g.fixed_words * kLanes] = 0u;
    column[(g.fixed_words + 1) * kLanes] = 0u;
    column[(g.fixed_words + 2) * kLanes] = 0u;
    const uint32_t side = a.side[block * (int64_t)g.block_symbols + (int64_t)step * kLanes + lane];
    const int center = *a.center;
    const uint32_t* table = a.pair_table + (size_t)((center + 128) & 255) * kPairEntries;
    const int tail = tail_exponent_at(a, g, block, step, lane);
    cp_async_wait_all();
    const uint32_t exponent = tail >= 0 ? (uint32_t)tail : walk_to(table, g, column, step, center);
    left = (exponent << 7) | (side & 0x7Fu) | ((side & 0x80u) << 8);
  }
  const uint32_t result = apply_op(left, right, spec.op, spec.alpha_is_one != 0,
                                   spec.beta_is_one != 0, alpha, beta);
  samples[idx] = (uint8_t)((result >> 7) & 0xFFu);
  if (values != nullptr) values[idx] = (uint16_t)result;
}

__global__ void __launch_bounds__(kThreads)
update_sample_kernel(OperandView a, Shape g, const uint16_t* __restrict__ other, OpSpec spec,
                     const uint16_t* __restrict__ known, uint8_t* __restrict__ samples,
                     uint16_t* __restrict__ values) {
  cudaTriggerProgrammaticLaunchCompletion();  // the center kernel behind this one waits on its own
  update_sample_chunk(a, g, other, spec, known, samples, values, (int)blockIdx.x);
}

// The sample pre-pass and the center kernel in one, for an operand that carries the BF16
// values at its sample positions (every result of a fused update does): one CTA, four samples
// per thread computed from `known` and B, the results kept for the next update, then the
// center and the shifted tables.  Launched as an ordinary kernel, so everything queued before
// the update is complete when it starts.
__global__ void __launch_bounds__(kTableThreads)
update_center_known_kernel(const uint16_t* __restrict__ other, int64_t n, OpSpec spec,
                           const uint16_t* __restrict__ known, uint16_t* __restrict__ values,
                           const int32_t* __restrict__ base_encode,
                           const int32_t* __restrict__ base_decode, int32_t* center_out,
                           int32_t* shifted_encode, int32_t* shifted_decode) {
  cudaTriggerProgrammaticLaunchCompletion();  // the fused kernel may start its prologue
  const int64_t count = n < kSampleCount ? n : kSampleCount;
  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  int raw[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t idx = threadIdx.x + k * kTableThreads;
    raw[k] = -1;
    if (idx < count) {
      const uint32_t right = other[sample_position(idx, n)];
      const uint32_t result = apply_op(known[idx], right, spec.op, spec.alpha_is_one != 0,
                                       spec.beta_is_one != 0, alpha, beta) & 0xFFFFu;
      raw[k] = (int)((result >> 7) & 0xFFu);
      if (values != nullptr) values[idx] = (uint16_t)result;
    }
  }
  center_from_samples(raw, base_encode, base_decode, center_out, shifted_encode, shifted_decode);
}

// Geometry of one job of a batched update (all jobs share `common`).
__device__ __forceinline__ Shape shape_of_update(const lct_update_job& job, const Shape& common) {
  Shape g = common;
  g.size = job.size;
  g.logical_numel = job.logical_numel;
  g.n_blocks = job.size / common.block_symbols;
  g.streams = g.n_blocks * kLanes;
  return g;
}

__device__ __forceinline__ OperandView view_of_update(const lct_operand& in) {
  OperandView v;
  v.encoded = reinterpret_cast<const uint32_t*>(in.encoded);
  v.side = in.side;
  v.center = in.center;
  v.pair_table = in.pair_table;
  v.lanes = in.overflow.lanes;
  v.starts = in.overflow.starts;
  v.tail = in.overflow.tail;
  v.descriptor = in.overflow.descriptor;
  v.count = in.overflow.count;
  v.blocks = in.overflow.blocks;
  v.base = in.overflow.base;
  v.mode = in.overflow.mode;
  return v;
}

// Sample pre-pass of every job of a batch: grid (16, n_jobs); job j's samples go to
// samples + 4096 * j.
__global__ void __launch_bounds__(kThreads)
update_sample_batch_kernel(const lct_update_job* __restrict__ jobs, Shape common, OpSpec spec,
                           uint8_t* __restrict__ samples) {
  cudaTriggerProgrammaticLaunchCompletion();
  const lct_update_job& job = jobs[blockIdx.y];
  update_sample_chunk(view_of_update(job.a), shape_of_update(job, common),
                      static_cast<const uint16_t*>(job.other), spec, job.known_values,
                      samples + (int64_t)kSampleCount * blockIdx.y, job.result_values,
                      (int)blockIdx.x);
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

// Shared memory: [decode table | encode table | the input operand (head | payload image)].  Finished output
// words go straight to global memory (a warp's lanes write neighbouring words of the same
// payload rows; L2 merges the sectors), which keeps four CTAs resident per SM.
// One codec block.  extra_starts and summaries are the tensor's own arrays.
// kEmit (LCT_EMIT_*): also write a dense BF16 tensor - the result itself or the Nesterov
// direction lerp(B, result, beta) - to dense_out, which may alias `other` (hence neither is
// `__restrict__` here: a thread reads its eight values of B before it overwrites them).
template <int kLaneMask, int kEmit>
__device__ __forceinline__ void update_fused_block(
    const OperandView& a, const Shape& g_in, const uint16_t* other,
    bool other_vector_ok, const OpSpec& spec, const int32_t* __restrict__ shifted_encode,
    uint8_t* __restrict__ side_out, uint32_t* __restrict__ encoded_out,
    uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries,
    uint8_t* __restrict__ spill, uint16_t* dense_out, int64_t block) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Shape g = g_in;
  if (kLaneMask >= 0) g.lane_mask = kLaneMask;  // compile-time lane mapping, see decode_block
  const OperandShared sh = carve_operand(smem_raw, 0, 1, g.fixed_words, 256 * sizeof(uint2));
  uint2* encode_table = reinterpret_cast<uint2*>(smem_raw + kTableBytes);

  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  const bool full_block = block_base + g.block_symbols <= g.logical_numel;
  if (block == 0 && tid < 4) encoded_out[g.streams * g.fixed_words + tid] = 0u;
  // The input operand does not depend on the result's center: its payload is staged and its
  // tables are built before this grid waits for the kernel that writes the shifted encode
  // table (which may still be running when the grid was launched by lct_update).
  prepare_block(sh, a, g, block, [&] {
    cudaGridDependencySynchronize();
    const uint32_t packed = (uint32_t)shifted_encode[tid];
    encode_table[tid] = make_uint2(packed & 0xFFFFFu, packed >> 20);
  });  // ends with a block barrier

  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  // A job table comes from the caller's device memory: an unaligned by-product pointer takes
  // the scalar stores, a missing one is skipped.
  const bool dense_vector_ok = (reinterpret_cast<uintptr_t>(dense_out) & 15u) == 0;
  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel, g.lane_mask);
  LaneState lane = open_lane(sh, a, g, valid);
  uint16_t* tile = sh.head->tile[warp];
  const uint8_t* tile_bytes = reinterpret_cast<const uint8_t*>(tile);
  const uint32_t encode_table_address = shared_address(encode_table);
  uint32_t* out_column = encoded_out + block * kLanes + tid;
  const GlobalWordSink sink{out_column, g.streams};
  const SideSelectors selectors = side_selectors((uint32_t)(((2 * (lane32 >> 2)) & g.lane_mask) >> 1) & 3u);
  const int budget_bits = g.fixed_words * 32;
  uint32_t lo = 0;
  int pos = 0, extra_start = -1;
  bool open = true;

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    decode_tile_rows<kLaneMask>(lane.reader, lane.tables, step0, lane.coded, lane.tail_from,
                                lane.tail_bytes, g.rare_length, g.lane_mask);
    __syncwarp();
    // ---- row side: A (op) B, new side bytes out, new exponents back into the tile ----
    // Side bytes of all four rows first (registers allow no more at four CTAs per SM); B's
    // rows are requested two at a time, each pair ahead of the arithmetic that uses it.
    UnitPlace place_of[2];
    uint2 side_in[2][2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      place_of[u] = place_unit(warp, (lane32 >> 2) + 8 * u, lane32 & 3, row0, step0, block_base,
                               g.lane_mask);
#pragma unroll
      for (int half = 0; half < 2; ++half)
        side_in[u][half] =
            __ldcs(reinterpret_cast<const uint2*>(a.side + place_of[u].storage + half * kLanes));
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const UnitPlace place = place_of[u];
      uint32_t right_in[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half)
        load_dense8(other, place.logical + half * kLanes, g.logical_numel, other_vector_ok,
                    right_in[half]);
      uint4* slot = reinterpret_cast<uint4*>(&tile[place.tile_index]);
      const uint4 words = *slot;
      uint32_t e_top03, e_top47, e_bot03, e_bot47;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t s_at = place.storage + half * kLanes;
        const int64_t l_at = place.logical + half * kLanes;
        uint32_t left[4], result[4];
        const uint32_t* right = right_in[half];
        join_row(words, side_in[u][half], selectors, half == 1, left);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          result[k] = apply_op(left[k], right[k], spec.op, spec.alpha_is_one != 0,
                               spec.beta_is_one != 0, alpha, beta);
        if (!full_block && l_at + 8 > g.logical_numel) {  // padding counts as +0.0
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (l_at + i >= g.logical_numel) result[i >> 1] &= (i & 1) ? 0x0000FFFFu : 0xFFFF0000u;
        }
        if (kEmit != LCT_EMIT_NONE && dense_out != nullptr) {
          uint32_t dense[4];
#pragma unroll
          for (int k = 0; k < 4; ++k)
            dense[k] = kEmit == LCT_EMIT_NESTEROV ? lerp_pair(right[k], result[k], beta) : result[k];
          if (dense_vector_ok && l_at + 8 <= g.logical_numel) {
            __stcs(reinterpret_cast<uint4*>(dense_out + l_at),
                   make_uint4(dense[0], dense[1], dense[2], dense[3]));
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              if (l_at + i < g.logical_numel)
                dense_out[l_at + i] = (uint16_t)(dense[i >> 1] >> (16 * (i & 1)));
          }
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
        open = encode_tile_rows<false, kLaneMask>(encode_table_address, lane.tables.tile_lane, sink,
                                                  g.lane_mask, step0, valid, budget_bits, pos, lo,
                                                  extra_start);
      else
        open = encode_tile_rows<true, kLaneMask>(encode_table_address, lane.tables.tile_lane, sink,
                                                 g.lane_mask, step0, valid, budget_bits, pos, lo,
                                                 extra_start);
    }
    if (!open) {
      // Raw exponents of the overflowed lane, from its overflow step on, for the tail pass.
      const int from = extra_start > step0 ? (extra_start - step0) >> 1 : 0;
      const int64_t tile_row = row0 + step0;
      const int group = warp ^ ((int)(tile_row & g.lane_mask) >> 5);
      for (int p = from; p < kTilePairs; ++p) {
        const int column = lane32 ^ ((2 * p) & g.lane_mask);
        const int64_t logical = (tile_row + 2 * p) * kLanes + 32 * group + column;
        const uint8_t* e = tile_bytes + 2 * (p * 32 + (lane32 ^ ((2 * p) & g.lane_mask & 6)));
        if (logical < g.logical_numel) spill[logical] = e[0];
        if (logical + kLanes < g.logical_numel) spill[logical + kLanes] = e[1];
      }
    }
    __syncwarp();
  }
  if (open) {
    if ((pos & 31) != 0) out_column[(int64_t)(pos >> 5) * g.streams] = lo;
    // Unused words of the lane are zero, as in the stand-alone encoder.
    for (int w = (pos + 31) >> 5; w < g.fixed_words; ++w) out_column[(int64_t)w * g.streams] = 0u;
  }
  extra_starts[block * kLanes + tid] = extra_start < 0 ? (uint8_t)255 : (uint8_t)extra_start;

  int bad = extra_start >= 0 ? 1 : 0;
  int bytes = extra_start >= 0 ? g.steps - extra_start : 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    bad += __shfl_down_sync(0xFFFFFFFFu, bad, d);
    bytes += __shfl_down_sync(0xFFFFFFFFu, bytes, d);
  }
  if (lane32 == 0) { sh.head->scan[warp] = bad; sh.head->scan[8 + warp] = bytes; }
  __syncthreads();
  if (tid == 0) {
    int total_bad = 0, total_bytes = 0;
    for (int w = 0; w < kWarps; ++w) { total_bad += sh.head->scan[w]; total_bytes += sh.head->scan[8 + w]; }
    summaries[block] = total_bad;
    summaries[g.n_blocks + block] = total_bytes;
  }
}

template <int kLaneMask, int kEmit>
__global__ void __launch_bounds__(kThreads, 4)
update_fused_kernel(OperandView a, Shape g, const uint16_t* other, bool other_vector_ok,
                    OpSpec spec, const int32_t* __restrict__ shifted_encode,
                    uint8_t* __restrict__ side_out, uint32_t* __restrict__ encoded_out,
                    uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries,
                    uint8_t* __restrict__ spill, uint16_t* dense_out) {
  update_fused_block<kLaneMask, kEmit>(a, g, other, other_vector_ok, spec, shifted_encode,
                                       side_out, encoded_out, extra_starts, summaries, spill,
                                       dense_out, blockIdx.x);
}

// Every block of every job of a batch: CTA b serves the job whose block range contains b.
template <int kLaneMask, int kEmit>
__global__ void __launch_bounds__(kThreads, 4)
update_fused_batch_kernel(const lct_update_job* __restrict__ jobs, int n_jobs, Shape common,
                          OpSpec spec, const int32_t* __restrict__ shifted_encode,
                          uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries) {
  const int64_t block = blockIdx.x;
  int lo = 0, hi = n_jobs - 1;
  while (lo < hi) {  // last job with first_block <= block
    const int mid = (lo + hi + 1) >> 1;
    if (jobs[mid].first_block <= block) lo = mid; else hi = mid - 1;
  }
  const lct_update_job& job = jobs[lo];
  const bool vector_ok = (reinterpret_cast<uintptr_t>(job.other) & 15u) == 0;
  update_fused_block<kLaneMask, kEmit>(
      view_of_update(job.a), shape_of_update(job, common), static_cast<const uint16_t*>(job.other),
      vector_ok, spec, shifted_encode + 256 * (int64_t)lo, job.side_out,
      reinterpret_cast<uint32_t*>(job.encoded_out), extra_starts + job.first_block * kLanes,
      summaries + 4 * job.first_block, job.spill, static_cast<uint16_t*>(job.dense_out),
      block - job.first_block);
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
  return lct::check_op(op, alpha, beta, alpha_is_one, beta_is_one);
}

static int launch_sample(const lct_operand* a, const void* other, const float* alpha,
                         const float* beta, int op, int alpha_is_one, int beta_is_one,
                         uint8_t* samples, const uint16_t* known_values, uint16_t* result_values,
                         int64_t size, int64_t logical_numel, int block_symbols,
                         int steps, int fixed_words, int rare_length, cudaStream_t stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = check_update_args(a, other, alpha, beta, op, &alpha_is_one, &beta_is_one, &va))) return rc;
  if (samples == nullptr) return LCT_E_NULL_POINTER;
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const int64_t count = logical_numel < lct::kSampleCount ? logical_numel : lct::kSampleCount;
  const unsigned grid = (unsigned)((count + lct::kThreads - 1) / lct::kThreads);
  const size_t shared = lct::payload_image_bytes(fixed_words + 1);
  if ((rc = lct::opt_in_shared(lct::update_sample_kernel, shared)) != 0) return rc;
  if ((reinterpret_cast<uintptr_t>(known_values) | reinterpret_cast<uintptr_t>(result_values)) & 1u)
    return LCT_E_ALIGNMENT;
  lct::update_sample_kernel<<<grid, lct::kThreads, shared, stream>>>(
      va, g, static_cast<const uint16_t*>(other), spec, known_values, samples, result_values);
  return (int)cudaGetLastError();
}

static int launch_fused(const lct_operand* a, const void* other, const float* alpha,
                        const float* beta, int op, int alpha_is_one, int beta_is_one,
                        const int32_t* shifted_encode, uint8_t* side_out, int32_t* encoded_out,
                        uint8_t* extra_starts, int32_t* summaries, uint8_t* spill, int64_t size,
                        int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                        int rare_length, bool overlapped, void* dense_out, int emit,
                        cudaStream_t stream) {
  lct::Shape g;
  lct::OperandView va;
  int rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
  if (rc) return rc;
  if ((rc = check_update_args(a, other, alpha, beta, op, &alpha_is_one, &beta_is_one, &va))) return rc;
  if (shifted_encode == nullptr || side_out == nullptr || encoded_out == nullptr ||
      extra_starts == nullptr || summaries == nullptr || spill == nullptr)
    return LCT_E_NULL_POINTER;
  if (!lct::aligned16(side_out) || !lct::aligned16(encoded_out)) return LCT_E_ALIGNMENT;
  if (emit < LCT_EMIT_NONE || emit > LCT_EMIT_NESTEROV) return LCT_E_BAD_ARGUMENT;
  if (emit != LCT_EMIT_NONE) {
    if (dense_out == nullptr) return LCT_E_NULL_POINTER;
    if (!lct::aligned16(dense_out)) return LCT_E_ALIGNMENT;
    if (emit == LCT_EMIT_NESTEROV && (op != LCT_OP_LERP || beta == nullptr)) return LCT_E_BAD_ARGUMENT;
  }
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const size_t shared = lct::operand_shared_bytes(fixed_words) + 256 * sizeof(uint2);
  const bool swizzled = g.lane_mask == 254;
  auto kernel = emit == LCT_EMIT_NESTEROV
                    ? (swizzled ? lct::update_fused_kernel<254, LCT_EMIT_NESTEROV>
                                : lct::update_fused_kernel<-1, LCT_EMIT_NESTEROV>)
                : emit == LCT_EMIT_RESULT
                    ? (swizzled ? lct::update_fused_kernel<254, LCT_EMIT_RESULT>
                                : lct::update_fused_kernel<-1, LCT_EMIT_RESULT>)
                    : (swizzled ? lct::update_fused_kernel<254, LCT_EMIT_NONE>
                                : lct::update_fused_kernel<-1, LCT_EMIT_NONE>);
  if ((rc = lct::opt_in_shared(kernel, shared)) != 0) return rc;
  const uint16_t* dense = static_cast<const uint16_t*>(other);
  uint32_t* words = reinterpret_cast<uint32_t*>(encoded_out);
  uint16_t* emitted = static_cast<uint16_t*>(dense_out);
  if (overlapped)
    return lct::launch_overlapped(kernel, (unsigned)g.n_blocks, lct::kThreads, shared, stream, va,
                                  g, dense, lct::aligned16(other), spec, shifted_encode, side_out,
                                  words, extra_starts, summaries, spill, emitted);
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared, stream>>>(
      va, g, dense, lct::aligned16(other), spec, shifted_encode, side_out, words, extra_starts,
      summaries, spill, emitted);
  return (int)cudaGetLastError();
}

int lct_update_sample(const lct_operand* a, const void* other, const float* alpha,
                      const float* beta, int op, int alpha_is_one, int beta_is_one,
                      uint8_t* samples, const uint16_t* known_values, uint16_t* result_values,
                      int64_t size, int64_t logical_numel, int block_symbols,
                      int steps, int fixed_words, int rare_length, void* stream) {
  return launch_sample(a, other, alpha, beta, op, alpha_is_one, beta_is_one, samples, known_values,
                       result_values, size, logical_numel, block_symbols, steps, fixed_words,
                       rare_length, static_cast<cudaStream_t>(stream));
}

int lct_update_fused(const lct_operand* a, const void* other, const float* alpha,
                     const float* beta, int op, int alpha_is_one, int beta_is_one,
                     const int32_t* shifted_encode, uint8_t* side_out, int32_t* encoded_out,
                     uint8_t* extra_starts, int32_t* summaries, uint8_t* spill, int64_t size,
                     int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                     int rare_length, void* stream) {
  return launch_fused(a, other, alpha, beta, op, alpha_is_one, beta_is_one, shifted_encode,
                      side_out, encoded_out, extra_starts, summaries, spill, size, logical_numel,
                      block_symbols, steps, fixed_words, rare_length, false, nullptr, LCT_EMIT_NONE,
                      static_cast<cudaStream_t>(stream));
}

int lct_update_emit(const lct_operand* a, const void* other, const float* alpha,
                    const float* beta, int op, int alpha_is_one, int beta_is_one,
                    const int32_t* encode_table, const int32_t* decode_table, uint8_t* samples,
                    const uint16_t* known_values, uint16_t* result_values, int32_t* center,
                    int32_t* shifted_encode, int32_t* shifted_decode, uint8_t* side_out,
                    int32_t* encoded_out, uint8_t* extra_starts, int32_t* summaries,
                    uint8_t* spill, int32_t* counts, int32_t* descriptor, int32_t* blocks_out,
                    void* arena_storage, int max_free_regions, int64_t size,
                    int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                    int rare_length, void* dense_out, int emit, int32_t* release_descriptor,
                    int32_t* release_status, void* stream) {
  if (encode_table == nullptr || decode_table == nullptr || center == nullptr ||
      counts == nullptr || descriptor == nullptr || arena_storage == nullptr)
    return LCT_E_NULL_POINTER;
  if (max_free_regions <= 0 || (max_free_regions & (max_free_regions - 1))) return LCT_E_BAD_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc;
  if (known_values != nullptr) {
    // 1+2. sample pre-pass and center in one ordinary launch (so everything queued before this
    //      call is complete and visible before any kernel of the update starts).
    lct::Shape g;
    lct::OperandView va;
    rc = lct::check_shape(size, logical_numel, block_symbols, steps, fixed_words, rare_length, &g);
    if (rc) return rc;
    if ((rc = check_update_args(a, other, alpha, beta, op, &alpha_is_one, &beta_is_one, &va))) return rc;
    if ((reinterpret_cast<uintptr_t>(known_values) | reinterpret_cast<uintptr_t>(result_values)) & 1u)
      return LCT_E_ALIGNMENT;
    if (shifted_encode == nullptr || shifted_decode == nullptr) return LCT_E_NULL_POINTER;
    const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
    lct::update_center_known_kernel<<<1, lct::kTableThreads, 0, st>>>(
        static_cast<const uint16_t*>(other), logical_numel, spec, known_values, result_values,
        encode_table, decode_table, center, shifted_encode, shifted_decode);
    if ((rc = (int)cudaGetLastError()) != 0) return rc;
  } else {
    // 1. the sample pre-pass: an ordinary launch, as above.
    rc = launch_sample(a, other, alpha, beta, op, alpha_is_one, beta_is_one, samples,
                       known_values, result_values, size, logical_numel, block_symbols, steps,
                       fixed_words, rare_length, st);
    if (rc) return rc;
    // 2. the center from the samples.
    const int64_t count = logical_numel < lct::kSampleCount ? logical_numel : lct::kSampleCount;
    rc = lct::launch_center(samples, count, true, encode_table, decode_table, center,
                            shifted_encode, shifted_decode, true, st);
    if (rc) return rc;
  }
  // 3-5. each may be scheduled while its predecessor runs and waits for it on the device.
  rc = launch_fused(a, other, alpha, beta, op, alpha_is_one, beta_is_one, shifted_encode, side_out,
                    encoded_out, extra_starts, summaries, spill, size, logical_numel, block_symbols,
                    steps, fixed_words, rare_length, true, dense_out, emit, st);
  if (rc) return rc;
  rc = lct::launch_scan_allocate(summaries, counts, descriptor, arena_storage, size / block_symbols,
                                 max_free_regions, true, st, release_descriptor, release_status);
  if (rc) return rc;
  const size_t metadata = ((size_t)8 * max_free_regions + 12 + 15) / 16 * 16;
  uint8_t* payload = static_cast<uint8_t*>(arena_storage) + metadata;
  return lct::launch_compact(spill, payload, payload, payload, descriptor, counts, blocks_out,
                             extra_starts, summaries, size, logical_numel, block_symbols, steps, 1,
                             true, st);
}

int lct_update(const lct_operand* a, const void* other, const float* alpha, const float* beta,
               int op, int alpha_is_one, int beta_is_one, const int32_t* encode_table,
               const int32_t* decode_table, uint8_t* samples, const uint16_t* known_values,
               uint16_t* result_values, int32_t* center,
               int32_t* shifted_encode, int32_t* shifted_decode, uint8_t* side_out,
               int32_t* encoded_out, uint8_t* extra_starts, int32_t* summaries, uint8_t* spill,
               int32_t* counts, int32_t* descriptor, int32_t* blocks_out, void* arena_storage,
               int max_free_regions, int64_t size, int64_t logical_numel, int block_symbols,
               int steps, int fixed_words, int rare_length, void* stream) {
  return lct_update_emit(a, other, alpha, beta, op, alpha_is_one, beta_is_one, encode_table,
                         decode_table, samples, known_values, result_values, center,
                         shifted_encode, shifted_decode, side_out, encoded_out, extra_starts,
                         summaries, spill, counts, descriptor, blocks_out, arena_storage,
                         max_free_regions, size, logical_numel, block_symbols, steps, fixed_words,
                         rare_length, nullptr, LCT_EMIT_NONE, nullptr, nullptr, stream);
}

int lct_update_batch_emit(const lct_update_job* jobs, int n_jobs, int64_t total_blocks,
                          const float* alpha, const float* beta, int op, int alpha_is_one,
                          int beta_is_one, const int32_t* encode_table,
                          const int32_t* decode_table, void* arena_storage, int max_free_regions,
                          uint8_t* samples, int32_t* shifted_encode, uint8_t* extra_starts,
                          int32_t* summaries, int block_symbols, int steps, int fixed_words,
                          int rare_length, int emit, void* stream) {
  if (jobs == nullptr || encode_table == nullptr || decode_table == nullptr ||
      arena_storage == nullptr || samples == nullptr || shifted_encode == nullptr ||
      extra_starts == nullptr || summaries == nullptr)
    return LCT_E_NULL_POINTER;
  if (n_jobs <= 0 || n_jobs > 65535 || total_blocks <= 0 || total_blocks > 0x7FFFFFFFLL)
    return LCT_E_BAD_ARGUMENT;
  if (max_free_regions <= 0 || (max_free_regions & (max_free_regions - 1))) return LCT_E_BAD_ARGUMENT;
  lct::Shape g;
  int rc = lct::check_op(op, alpha, beta, &alpha_is_one, &beta_is_one);
  if (rc) return rc;
  rc = lct::check_shape(block_symbols, block_symbols, block_symbols, steps, fixed_words,
                        rare_length, &g);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  // 1. samples of all jobs: an ordinary launch, so everything queued before this call is
  //    complete and visible before any of the five kernels starts.
  const size_t sample_shared = lct::payload_image_bytes(fixed_words + 1);
  if ((rc = lct::opt_in_shared(lct::update_sample_batch_kernel, sample_shared)) != 0) return rc;
  lct::update_sample_batch_kernel<<<dim3(lct::kSampleCount / lct::kThreads, (unsigned)n_jobs),
                                    lct::kThreads, sample_shared, st>>>(jobs, g, spec, samples);
  if ((rc = (int)cudaGetLastError()) != 0) return rc;
  // 2-5. each may be scheduled while its predecessor runs and waits for it on the device.
  if ((rc = lct::launch_center_batch(jobs, n_jobs, encode_table, decode_table, samples,
                                     shifted_encode, st)))
    return rc;
  const size_t shared = lct::operand_shared_bytes(fixed_words) + 256 * sizeof(uint2);
  if (emit < LCT_EMIT_NONE || emit > LCT_EMIT_NESTEROV) return LCT_E_BAD_ARGUMENT;
  if (emit == LCT_EMIT_NESTEROV && (op != LCT_OP_LERP || beta == nullptr)) return LCT_E_BAD_ARGUMENT;
  const bool swizzled = g.lane_mask == 254;
  auto kernel = emit == LCT_EMIT_NESTEROV
                    ? (swizzled ? lct::update_fused_batch_kernel<254, LCT_EMIT_NESTEROV>
                                : lct::update_fused_batch_kernel<-1, LCT_EMIT_NESTEROV>)
                : emit == LCT_EMIT_RESULT
                    ? (swizzled ? lct::update_fused_batch_kernel<254, LCT_EMIT_RESULT>
                                : lct::update_fused_batch_kernel<-1, LCT_EMIT_RESULT>)
                    : (swizzled ? lct::update_fused_batch_kernel<254, LCT_EMIT_NONE>
                                : lct::update_fused_batch_kernel<-1, LCT_EMIT_NONE>);
  if ((rc = lct::opt_in_shared(kernel, shared)) != 0) return rc;
  if ((rc = lct::launch_overlapped(kernel, (unsigned)total_blocks, lct::kThreads, shared, st, jobs,
                                   n_jobs, g, spec, shifted_encode, extra_starts, summaries)))
    return rc;
  if ((rc = lct::launch_scan_batch(jobs, n_jobs, summaries, arena_storage, max_free_regions,
                                   block_symbols, st)))
    return rc;
  const size_t metadata = ((size_t)8 * max_free_regions + 12 + 15) / 16 * 16;
  return lct::launch_compact_batch(jobs, n_jobs, total_blocks,
                                   static_cast<uint8_t*>(arena_storage) + metadata, extra_starts,
                                   summaries, block_symbols, steps, fixed_words, st);
}

int lct_update_batch(const lct_update_job* jobs, int n_jobs, int64_t total_blocks,
                     const float* alpha, const float* beta, int op, int alpha_is_one,
                     int beta_is_one, const int32_t* encode_table, const int32_t* decode_table,
                     void* arena_storage, int max_free_regions, uint8_t* samples,
                     int32_t* shifted_encode, uint8_t* extra_starts, int32_t* summaries,
                     int block_symbols, int steps, int fixed_words, int rare_length,
                     void* stream) {
  return lct_update_batch_emit(jobs, n_jobs, total_blocks, alpha, beta, op, alpha_is_one,
                               beta_is_one, encode_table, decode_table, arena_storage,
                               max_free_regions, samples, shifted_encode, extra_starts, summaries,
                               block_symbols, steps, fixed_words, rare_length, LCT_EMIT_NONE, stream);
}

}  // extern "C"
