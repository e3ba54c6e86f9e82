// Table-driven decoder and the fused decode -> pointwise operation kernels.
//
// One CTA (256 threads) per codec block.
//
// Prologue: the block's payload tile (fixed_words rows of 256 words) and the
// 16 KB two-symbol table of this tensor's center are copied into shared memory
// with cp.async while the block's overflow map is expanded.
//
// Then, software pipelined over half tiles of 16 rows:
//   lane side - thread = lane: the next 94 bits of its stream in three registers,
//               pre-shifted so that 12 of them index the two-symbol table (two
//               exponent bytes + bits consumed per lookup); consuming is three
//               funnel shifts by the table entry itself, refills from the shared
//               image are off the lookup chain (decode_core.cuh: ShiftCursor).
//               The only divergent path is the rare entry that is not a full
//               pair, decoded one symbol at a time;
//   row side  - thread = 8 columns of a row pair of the PREVIOUS half tile:
//               128-bit read of the tile, 64-bit side-byte loads (requested a
//               half tile earlier), four bytes at a time rebuilt into BF16,
//               optional arithmetic, 128-bit streaming stores.  In the plain
//               decoder its instructions are issued between the lane side's
//               lookups, and two neighbouring warps share their rows out so
//               that every store instruction writes full 128-byte lines.
// Overflow lanes switch from the bit stream to their raw tail bytes at their
// recorded start step, inside the same launch.
#include "decode_core.cuh"

namespace lct {

// ---------------------------------------------------------------------------
// Plain decode
// ---------------------------------------------------------------------------

// kLaneMask: the lane mapping as a compile-time constant (254, the default mapping: the masked
// tile and row addresses fold into constants, 80 instead of 82 us per 64 Mi elements), or -1 to
// take it from the shape at run time (the linear mapping).
// Row side of one half tile (16 rows) for one thread: 8 columns of one row pair.  Cut into
// slices that the lane phase of the NEXT half tile issues between its pairs.
struct DecodeRowSlices {
  const uint16_t* tile;
  uint16_t* out;
  SideSelectors selectors;
  int64_t logical_numel;
  bool full_block;
  // the half tile being finished:
  UnitPlace place;
  uint2 side[2];
  uint4 words;
  uint32_t top[4], bottom[4];

  __device__ __forceinline__ void store(const uint32_t (&row)[4], int64_t at) {
    if (full_block || at + 8 <= logical_numel) {
      __stcs(reinterpret_cast<uint4*>(out + at), make_uint4(row[0], row[1], row[2], row[3]));
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (at + i < logical_numel) out[at + i] = (uint16_t)(row[i >> 1] >> (16 * (i & 1)));
    }
  }
  template <int k>
  __device__ __forceinline__ void slice() {
    if (k == 0) words = *reinterpret_cast<const uint4*>(&tile[place.tile_index]);
    if (k == 1) join_row(words, side[0], selectors, false, top);
    if (k == 2) store(top, place.logical);
    if (k == 3) join_row(words, side[1], selectors, true, bottom);
    if (k == 4) store(bottom, place.logical + kLanes);
  }
  __device__ __forceinline__ void rest() {
    slice<0>(); slice<1>(); slice<2>(); slice<3>(); slice<4>();
  }
};

// One codec block.  The work is software pipelined over half tiles of 16 rows: while a warp's
// lanes decode half tile h into one half of the warp's tile buffer, the row side of half tile
// h - 1 (join with the side bytes, 128-bit stores) is issued between the lookups from the other
// half of the buffer, and the side bytes of half tile h were requested one iteration earlier.
// kLaneMask: the lane mapping as a compile-time constant (254, the default mapping), or -1 to
// take it from the shape at run time (the linear mapping).
template <int kLaneMask>
__device__ __forceinline__ void decode_block(const OperandView& a, const Shape& g_in,
                                             uint16_t* __restrict__ out, int64_t block) {
  Shape g = g_in;
  if (kLaneMask >= 0) g.lane_mask = kLaneMask;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  const OperandShared sh = carve_operand(smem_raw, 0, 1, g.fixed_words);
  prepare_block(sh, a, g, block);

  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel, g.lane_mask);
  LaneState lane = open_lane(sh, a, g, valid);
  const bool full_block = block_base + g.block_symbols <= g.logical_numel;
  // Rows of this block that hold elements: half tiles of pure padding (the tail of a ragged or
  // tiny tensor) have nothing to decode and nothing to store.
  const int rows_used =
      full_block ? g.steps : (int)((g.logical_numel - block_base + kLanes - 1) / kLanes);
  const int halves = (rows_used + kTileRows / 2 - 1) / (kTileRows / 2);

  // Row side: kRowWarps neighbouring warps work as one group.  Their lanes cover one aligned
  // segment of 32 * kRowWarps columns in every row (the lane mapping's bits 5..7 move whole
  // aligned groups), and the group's threads share that segment out so that 4 * kRowWarps
  // neighbouring threads cover one row: 128-bit stores of full 128-byte lines from two warps on.
  constexpr int kRowWarps = 2, kRowShift = 1;  // measured: 1 -> 76.8 us, 2 -> 75.9, 4 -> 78.0 (64 Mi elements)
  const int group = warp >> kRowShift;
  const int in_group = ((warp & (kRowWarps - 1)) << 5) + lane32;
  const int column8 = in_group & (4 * kRowWarps - 1);  // which 8 columns of the segment
  const int pair8 = in_group >> (2 + kRowShift);        // which row pair of a half tile, 0..7
  auto group_barrier = [&] {
    if (kRowWarps == 1) __syncwarp();
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "n"(32 * kRowWarps) : "memory");
  };

  DecodeRowSlices rows;
  rows.out = out;
  // Every row-side unit of a thread has the same pair permutation (its pair index mod 4).
  rows.selectors = side_selectors((uint32_t)(((2 * pair8) & g.lane_mask) >> 1) & 3u);
  rows.logical_numel = g.logical_numel;
  rows.full_block = full_block;

  // Side bytes of half tile h for this thread's unit (row pair 8 * (h & 1) + pair8 of tile h / 2).
  UnitPlace next_place;
  const uint16_t* next_tile;
  uint2 next_side[2];
  auto request = [&](int h) {
    const int step0 = kTileRows * (h >> 1);
    // The warp of the group whose lanes hold these columns in this tile.
    const int moved = (int)((row0 + step0) & g.lane_mask) >> 5;
    const int owner = (group << kRowShift) + ((column8 >> 2) ^ (moved & (kRowWarps - 1)));
    next_place = place_unit(owner, kHalfPairs * (h & 1) + pair8, column8 & 3, row0, step0,
                            block_base, g.lane_mask);
    next_tile = sh.head->tile[owner];
    const uint8_t* s = a.side + next_place.storage;
    next_side[0] = __ldcs(reinterpret_cast<const uint2*>(s));
    next_side[1] = __ldcs(reinterpret_cast<const uint2*>(s + kLanes));
  };
  auto hand_over = [&] {
    rows.place = next_place;
    rows.tile = next_tile;
    rows.side[0] = next_side[0];
    rows.side[1] = next_side[1];
  };
  NoSlices nothing;
  request(0);
  // Half tile 0: nothing to finish yet.
  decode_half_rows<kLaneMask, 0>(lane.reader, lane.tables, 0, lane.coded, lane.tail_from,
                                 lane.tail_bytes, g.rare_length, g.lane_mask, nothing);
  hand_over();
  group_barrier();
  // One copy of the code serves both halves of the tile buffer (the second half's rows are
  // 512 bytes further on): the loop stays within the instruction cache.
  LaneTables tables = lane.tables;
#pragma unroll 1
  for (int h = 1; h < halves; ++h) {
    request(h);
    tables.tile_lane = lane.tables.tile_lane + (uint32_t)((h & 1) * kHalfPairs * 64);
    decode_half_rows<kLaneMask, 0>(lane.reader, tables, (kTileRows / 2) * h, lane.coded,
                                   lane.tail_from, lane.tail_bytes, g.rare_length, g.lane_mask, rows);
    hand_over();
    group_barrier();
  }
  rows.rest();  // the last half tile
}

// Resident CTAs per SM the decoder is compiled for (shared memory allows no more; three cost 8 %).
constexpr int kDecodeMinCtas = 4;
template <int kLaneMask>
__global__ void __launch_bounds__(kThreads, kDecodeMinCtas)
decode_kernel(OperandView a, Shape g, uint16_t* __restrict__ out) {
  decode_block<kLaneMask>(a, g, out, blockIdx.x);
}

// Many tensors of one geometry in one launch: CTA b serves the job whose block
// range contains b.  Jobs are sorted by first_block.
__device__ __forceinline__ OperandView view_of_job(const lct_operand& in) {
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

template <typename Job>
__device__ __forceinline__ int find_job(const Job* jobs, int n_jobs, int64_t block) {
  int lo = 0, hi = n_jobs - 1;
  while (lo < hi) {  // last job with first_block <= block
    const int mid = (lo + hi + 1) >> 1;
    if (jobs[mid].first_block <= block) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// Operand in a peer GPU's memory: bring one block's side bytes over in full 16-byte requests
// (four in flight per thread) so that the decoder reads a local copy.  `chunks` (2048 or 4096)
// is a multiple of 4 * kThreads.  Not inlined: its registers are dead before the decoder starts.
static __device__ __noinline__ void stage_side_bytes(const uint8_t* __restrict__ from_bytes,
                                                     uint8_t* __restrict__ to_bytes, int chunks) {
  const uint4* from = reinterpret_cast<const uint4*>(from_bytes);
  uint4* to = reinterpret_cast<uint4*>(to_bytes);
  for (int i = threadIdx.x; i < chunks; i += 4 * kThreads) {
    uint4 v[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) v[k] = __ldcs(from + i + k * kThreads);
#pragma unroll
    for (int k = 0; k < 4; ++k) to[i + k * kThreads] = v[k];
  }
  __syncthreads();  // the copy is read by other threads of this CTA only
}

template <int kLaneMask>
__global__ void __launch_bounds__(kThreads, kDecodeMinCtas)
decode_batch_kernel(const lct_decode_job* __restrict__ jobs, int n_jobs, Shape common) {
  const int64_t block = blockIdx.x;
  const lct_decode_job& job = jobs[find_job(jobs, n_jobs, block)];
  Shape g = common;
  g.size = job.size;
  g.logical_numel = job.logical_numel;
  g.n_blocks = job.size / common.block_symbols;
  g.streams = g.n_blocks * kLanes;
  OperandView view = view_of_job(job.operand);
  const int64_t local_block = block - job.first_block;
  if (job.side_stage != nullptr) {
    const int64_t base = local_block * (int64_t)g.block_symbols;
    stage_side_bytes(view.side + base, job.side_stage + base, g.block_symbols / 16);
    view.side = job.side_stage;
  }
  decode_block<kLaneMask>(view, g, reinterpret_cast<uint16_t*>(job.out), local_block);
}

// ---------------------------------------------------------------------------
// Fused pointwise operations
// ---------------------------------------------------------------------------

template <bool kDual, int kLaneMask>
__global__ void __launch_bounds__(kThreads)
pointwise_kernel(OperandView a, OperandView b, Shape g_in, const uint16_t* __restrict__ other,
                 bool other_vector_ok, void* output, uint8_t* auxiliary, OpSpec spec,
                 bool compressed) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  Shape g = g_in;
  if (kLaneMask >= 0) g.lane_mask = kLaneMask;  // see decode_block
  const OperandShared sh = carve_operand(smem_raw, 0, kDual ? 2 : 1, g.fixed_words);
  const OperandShared sh_b = carve_operand(smem_raw, kDual ? 1 : 0, kDual ? 2 : 1, g.fixed_words);
  const int64_t block = blockIdx.x;
  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  prepare_block(sh, a, g, block);
  if (kDual) prepare_block(sh_b, b, g, block);

  const float alpha = spec.alpha_is_one ? 1.0f : *spec.alpha;
  const float beta = spec.beta_is_one ? 1.0f : *spec.beta;
  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel, g.lane_mask);
  LaneState lane_a = open_lane(sh, a, g, valid);
  LaneState lane_b = lane_a;
  if (kDual) lane_b = open_lane(sh_b, b, g, valid);
  const uint16_t* tile = sh.head->tile[warp];
  const uint16_t* tile_b = sh_b.head->tile[warp];
  const SideSelectors selectors = side_selectors((uint32_t)(((2 * (lane32 >> 2)) & g.lane_mask) >> 1) & 3u);

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    decode_tile_rows<kLaneMask>(lane_a.reader, lane_a.tables, step0, lane_a.coded, lane_a.tail_from,
                                lane_a.tail_bytes, g.rare_length, g.lane_mask);
    if (kDual)
      decode_tile_rows<kLaneMask>(lane_b.reader, lane_b.tables, step0, lane_b.coded,
                                  lane_b.tail_from, lane_b.tail_bytes, g.rare_length, g.lane_mask);
    __syncwarp();
    // All global loads of the tile's four rows first, so their latencies overlap.
    UnitPlace place_of[2];
    uint2 side_a[2][2], side_b[2][2];
    uint32_t dense_in[2][2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      place_of[u] = place_unit(warp, (lane32 >> 2) + 8 * u, lane32 & 3, row0, step0, block_base,
                               g.lane_mask);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t s_at = place_of[u].storage + half * kLanes;
        side_a[u][half] = __ldcs(reinterpret_cast<const uint2*>(a.side + s_at));
        if (kDual)
          side_b[u][half] = __ldcs(reinterpret_cast<const uint2*>(b.side + s_at));
        else
          load_dense8(other, place_of[u].logical + half * kLanes, g.logical_numel, other_vector_ok,
                      dense_in[u][half]);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const UnitPlace place = place_of[u];
      const uint4 words = *reinterpret_cast<const uint4*>(&tile[place.tile_index]);
      uint4 words_b = make_uint4(0, 0, 0, 0);
      if (kDual) words_b = *reinterpret_cast<const uint4*>(&tile_b[place.tile_index]);
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int64_t s_at = place.storage + half * kLanes;
        const int64_t l_at = place.logical + half * kLanes;
        uint32_t left[4], right[4], result[4];
        join_row(words, side_a[u][half], selectors, half == 1, left);
        if (kDual) {
          join_row(words_b, side_b[u][half], selectors, half == 1, right);
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) right[k] = dense_in[u][half][k];
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
          result[k] = apply_op(left[k], right[k], spec.op, spec.alpha_is_one != 0,
                               spec.beta_is_one != 0, alpha, beta);
        store_row(result, compressed, output, auxiliary, l_at, g.logical_numel, s_at, place.q);
      }
    }
    __syncwarp();
  }
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
  const size_t shared = lct::operand_shared_bytes(fixed_words);
  auto kernel = g.lane_mask == 254 ? lct::decode_kernel<254> : lct::decode_kernel<-1>;
  if ((rc = lct::opt_in_shared(kernel, shared)) != 0) return rc;
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared, static_cast<cudaStream_t>(stream)>>>(
      va, g, reinterpret_cast<uint16_t*>(out));
  return (int)cudaGetLastError();
}

int lct_decode_batch(const lct_decode_job* jobs, int n_jobs, int64_t total_blocks,
                     int block_symbols, int steps, int fixed_words, int rare_length, void* stream) {
  if (jobs == nullptr) return LCT_E_NULL_POINTER;
  if (n_jobs <= 0 || total_blocks <= 0 || total_blocks > 0x7FFFFFFFLL) return LCT_E_BAD_ARGUMENT;
  lct::Shape g;
  int rc = lct::check_shape(block_symbols, block_symbols, block_symbols, steps, fixed_words,
                            rare_length, &g);
  if (rc) return rc;
  const size_t shared = lct::operand_shared_bytes(fixed_words);
  auto kernel = g.lane_mask == 254 ? lct::decode_batch_kernel<254> : lct::decode_batch_kernel<-1>;
  if ((rc = lct::opt_in_shared(kernel, shared)) != 0) return rc;
  kernel<<<(unsigned)total_blocks, lct::kThreads, shared, static_cast<cudaStream_t>(stream)>>>(
      jobs, n_jobs, g);
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
  if ((rc = lct::check_op(op, alpha, beta, &alpha_is_one, &beta_is_one)) != 0) return rc;
  if (!lct::aligned16(output) || (compressed_output && !lct::aligned16(auxiliary)))
    return LCT_E_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(other) & 1u) != 0) return LCT_E_ALIGNMENT;
  const lct::OpSpec spec{alpha, beta, op, alpha_is_one, beta_is_one};
  const size_t shared = lct::operand_shared_bytes(fixed_words);
  auto kernel = g.lane_mask == 254 ? lct::pointwise_kernel<false, 254> : lct::pointwise_kernel<false, -1>;
  if ((rc = lct::opt_in_shared(kernel, shared)) != 0) return rc;
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared, static_cast<cudaStream_t>(stream)>>>(
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
  const size_t one = lct::operand_shared_bytes(fixed_words);
  auto kernel = g.lane_mask == 254 ? lct::pointwise_kernel<true, 254> : lct::pointwise_kernel<true, -1>;
  if ((rc = lct::opt_in_shared(kernel, 2 * one)) != 0) return rc;
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, 2 * one, static_cast<cudaStream_t>(stream)>>>(
      va, vb, g, nullptr, false, output, auxiliary, spec, compressed_output != 0);
  return (int)cudaGetLastError();
}

}  // extern "C"
