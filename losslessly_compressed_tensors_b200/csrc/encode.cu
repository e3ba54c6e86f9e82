// Field split + fixed-budget Huffman encoder, and the overflow tail compaction.
//
// One CTA (256 threads) per codec block; between the prologue and the epilogue
// every warp runs on its own (see common.cuh: a warp's 32 lanes own one
// 64-byte segment of every row).  Per half tile of 16 rows, per warp:
//   row side  - thread = 8 columns of a row pair: 128-bit loads of the BF16
//               source (requested one half tile ahead), four values at a time
//               split into exponent bytes -> the warp's shared tile and side
//               bytes -> lane order, stored 64 bits at a time;
//   lane side - thread = lane: two byte loads of its exponent pair from the
//               tile, both (code, length) rows of the shared encode table,
//               code appended at the lane's bit position; a finished 32-bit
//               word goes into a shared image of the block's payload by
//               predicated instructions (encode_core.cuh).
// At the end the payload image (zero where nothing was written, so the output
// is deterministic) is copied out with coalesced 128-bit stores, and the
// block's overflow summary is reduced.
#include <type_traits>

#include "batch.cuh"
#include "common.cuh"
#include "encode_core.cuh"
#include "lct_b200.h"

namespace lct {

// Resident CTAs per SM the encoder is compiled for (register cap = 65536 / 256 / this; five or
// six were measured slower, 63.5 and 65.7 us against 61.5 for 64 Mi elements).
constexpr int kEncodeMinCtas = 4;

struct EncodeShape {
  int64_t size;
  int64_t logical_numel;
  int64_t streams;
  int64_t n_blocks;
  int block_symbols;
  int steps;
  int fixed_words;
  int lane_mask;  // 254: lane ^ (row & 254) ("swizzle"); 0: "linear"
};

// Fixed part of the dynamic shared memory; the payload image follows it.
struct __align__(16) EncodeSharedHead {
  uint2 table[256];                        // x = code bits (LSB first), y = code length
  uint16_t tile[kWarps][kTilePairs * 32];
  int scan[36];
};

// Source values of one row-phase unit: 8 columns of two consecutive rows.
struct UnitSource {
  uint4 top, bottom;  // BF16 bits; for precomputed exponent bytes only .x/.y are used
};

__device__ __forceinline__ uint32_t load_pair_guarded(const uint16_t* src, int64_t at, int64_t numel) {
  const uint32_t a = at < numel ? src[at] : 0u;
  const uint32_t b = at + 1 < numel ? src[at + 1] : 0u;
  return a | (b << 16);
}

template <bool kPrecomputed>
__device__ __forceinline__ UnitSource load_unit(const void* src, int64_t at, int64_t numel,
                                                bool vector_ok, bool full_block) {
  UnitSource u;
  u.top = make_uint4(0, 0, 0, 0);
  u.bottom = make_uint4(0, 0, 0, 0);
  if (kPrecomputed) {
    const uint8_t* bytes = static_cast<const uint8_t*>(src);
    if (vector_ok && (full_block || at + kLanes + 8 <= numel)) {
      const uint2 t = __ldcs(reinterpret_cast<const uint2*>(bytes + at));
      const uint2 b = __ldcs(reinterpret_cast<const uint2*>(bytes + at + kLanes));
      u.top.x = t.x; u.top.y = t.y; u.bottom.x = b.x; u.bottom.y = b.y;
    } else {
      uint32_t* top = &u.top.x;
      uint32_t* bottom = &u.bottom.x;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (at + i < numel) top[i >> 2] |= (uint32_t)bytes[at + i] << (8 * (i & 3));
        if (at + kLanes + i < numel) bottom[i >> 2] |= (uint32_t)bytes[at + kLanes + i] << (8 * (i & 3));
      }
    }
  } else {
    const uint16_t* bits = static_cast<const uint16_t*>(src);
    if (vector_ok && (full_block || at + kLanes + 8 <= numel)) {
      u.top = __ldcs(reinterpret_cast<const uint4*>(bits + at));
      u.bottom = __ldcs(reinterpret_cast<const uint4*>(bits + at + kLanes));
    } else {
      uint32_t* top = &u.top.x;
      uint32_t* bottom = &u.bottom.x;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        top[k] = load_pair_guarded(bits, at + 2 * k, numel);
        bottom[k] = load_pair_guarded(bits, at + kLanes + 2 * k, numel);
      }
    }
  }
  return u;
}

// Row side of one half tile (16 rows) for one thread: 8 columns of one row pair - field split,
// side bytes to global memory in lane order, exponent bytes into the warp's tile.  Cut into
// slices (the form a lane phase can issue between its lookups); the last slice requests the
// source of the half tile after this one.
template <bool kPrecomputed>
struct EncodeRowSlices {
  const void* src;
  uint8_t* side;
  uint16_t* tile;
  int64_t logical_numel, row0, block_base;
  int halves, warp, lane32, lane_mask;
  bool vector_ok, full_block;
  int h = 0;           // the half tile whose source is in `source`
  UnitSource source;
  uint32_t l03, h03, l47, h47, bl03, bh03, bl47, bh47;
  uint32_t e_top03, e_top47, e_bot03, e_bot47;

  __device__ __forceinline__ int pair() const { return kHalfPairs * (h & 1) + (lane32 >> 2); }
  // Request the source rows of half tile `which` (nothing when it does not exist).
  __device__ __forceinline__ void request(int which) {
    h = which;
    if (which >= halves) return;
    const int64_t row = row0 + kTileRows * (which >> 1) + 2 * pair();
    const int64_t logical =
        row * kLanes + 32 * (warp ^ ((int)(row & lane_mask) >> 5)) + 8 * (lane32 & 3);
    source = load_unit<kPrecomputed>(src, logical, logical_numel, vector_ok, full_block);
  }
  template <int k>
  __device__ __forceinline__ void slice() {
    const int p = pair();
    const int in_tile = (2 * p) & lane_mask;
    const int swapped = (8 * (lane32 & 3)) ^ (in_tile & 0x18);
    if (kPrecomputed) {
      if (k == 0) {
        e_top03 = source.top.x; e_top47 = source.top.y;
        e_bot03 = source.bottom.x; e_bot47 = source.bottom.y;
      }
    } else {
      const uint32_t q = (uint32_t)(in_tile >> 1) & 3u;
      uint8_t* s = side + block_base + (int64_t)(kTileRows * (h >> 1) + 2 * p) * kLanes + 32 * warp + swapped;
      if (k == 0) {
        const uint4 t = source.top;
        l03 = prmt(t.x, t.y, 0x6420); h03 = prmt(t.x, t.y, 0x7531);
        l47 = prmt(t.z, t.w, 0x6420); h47 = prmt(t.z, t.w, 0x7531);
      }
      if (k == 1) {
        const uint4 b = source.bottom;
        bl03 = prmt(b.x, b.y, 0x6420); bh03 = prmt(b.x, b.y, 0x7531);
        bl47 = prmt(b.z, b.w, 0x6420); bh47 = prmt(b.z, b.w, 0x7531);
      }
      if (k == 2) {
        e_top03 = exponent_bytes(l03, h03); e_top47 = exponent_bytes(l47, h47);
        // Side bytes: column order -> lane order, one 8-byte store per row.
        const uint32_t s03 = side_bytes(l03, h03), s47 = side_bytes(l47, h47);
        __stcs(reinterpret_cast<uint2*>(s),
               make_uint2(prmt(s03, s47, pair_selector_low(q)), prmt(s03, s47, pair_selector_high(q))));
      }
      if (k == 3) {
        e_bot03 = exponent_bytes(bl03, bh03); e_bot47 = exponent_bytes(bl47, bh47);
        const uint32_t s03 = side_bytes(bl03, bh03), s47 = side_bytes(bl47, bh47);
        __stcs(reinterpret_cast<uint2*>(s + kLanes),
               make_uint2(prmt(s03, s47, pair_selector_low(q)), prmt(s03, s47, pair_selector_high(q))));
      }
    }
    if (k == 4) {
      // tile word for columns (2k, 2k+1): [e_top(2k), e_bot(2k), e_top(2k+1), e_bot(2k+1)];
      // the unit's group of 8 sits where its lanes are (see tile_slot_xor).
      *reinterpret_cast<uint4*>(&tile[p * 32 + swapped]) =
          make_uint4(prmt(e_top03, e_bot03, 0x5140), prmt(e_top03, e_bot03, 0x7362),
                     prmt(e_top47, e_bot47, 0x5140), prmt(e_top47, e_bot47, 0x7362));
    }
    if (k == 5) request(h + 1);
  }
  __device__ __forceinline__ void rest() {
    slice<0>(); slice<1>(); slice<2>(); slice<3>(); slice<4>(); slice<5>();
  }
};

// One codec block.  extra_starts and summaries are the tensor's own arrays
// (summaries holds g.n_blocks entries per row).
// kLaneMask: the lane mapping as a compile-time constant (254, the default mapping), or -1 to
// take it from the shape at run time.
template <bool kPrecomputed, int kLaneMask>
__device__ __forceinline__ void encode_block(const void* __restrict__ src, bool src_vector_ok,
                                             uint8_t* __restrict__ side,
                                             uint32_t* __restrict__ encoded,
                                             const int32_t* __restrict__ shifted_encode,
                                             uint8_t* __restrict__ extra_starts,
                                             int32_t* __restrict__ summaries, const EncodeShape& g_in,
                                             int64_t block) {
  EncodeShape g = g_in;
  if (kLaneMask >= 0) g.lane_mask = kLaneMask;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  EncodeSharedHead& sh = *reinterpret_cast<EncodeSharedHead*>(smem_raw);
  uint32_t* payload = reinterpret_cast<uint32_t*>(smem_raw + sizeof(EncodeSharedHead));

  const int tid = threadIdx.x, warp = tid >> 5, lane32 = tid & 31;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  const bool full_block = block_base + g.block_symbols <= g.logical_numel;

  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel, g.lane_mask);
  const int budget_bits = g.fixed_words * 32;
  uint16_t* tile = sh.tile[warp];
  const uint32_t tile_lane = shared_address(&tile[lane32]);
  const uint32_t table_address = shared_address(sh.table);
  uint32_t* payload_column = payload + tid;
  const SharedWordSink sink{shared_address(payload_column)};
  uint32_t lo = 0;
  int pos = 0;
  int extra_start = -1;  // first overflowing step, -1 = none
  bool open = true;

  // Rows of this block that hold elements.  Half tiles of pure padding (the tail of a ragged or
  // tiny tensor) carry no bits; their side bytes are cleared in one sweep after the loop.
  const int rows_used =
      full_block ? g.steps : (int)((g.logical_numel - block_base + kLanes - 1) / kLanes);
  const int halves = (rows_used + kTileRows / 2 - 1) / (kTileRows / 2);

  EncodeRowSlices<kPrecomputed> rows;
  rows.src = src;
  rows.side = side;
  rows.tile = tile;
  rows.logical_numel = g.logical_numel;
  rows.vector_ok = src_vector_ok;
  rows.full_block = full_block;
  rows.halves = halves;
  rows.warp = warp;
  rows.lane32 = lane32;
  rows.row0 = row0;
  rows.block_base = block_base;
  rows.lane_mask = g.lane_mask;
  rows.request(0);
  // Everything above is independent of the tensor's center.  The shifted table may come from
  // a kernel that is still running when this grid was launched with programmatic stream
  // serialisation (lct_compress): wait for it only now, with the first source rows in flight.
  cudaGridDependencySynchronize();
  {
    const uint32_t packed = (uint32_t)shifted_encode[tid];
    // Clearing the payload image hides the latency of the table load.
    for (int w = 0; w < g.fixed_words; ++w) payload[w * kLanes + tid] = 0u;
    if (block == 0 && tid < 4) encoded[g.streams * g.fixed_words + tid] = 0u;  // trailing pad words
    sh.table[tid] = make_uint2(packed & 0xFFFFFu, packed >> 20);
  }
  __syncthreads();

  // Half tiles of 16 rows alternate between the two sides: the row side splits half tile h + 1
  // into the free half of the warp's tile buffer (and ends by requesting the source of half
  // tile h + 2, which then has a whole lane phase to arrive), the lanes encode half tile h.
  // Issuing the row side's work between the lanes' lookups instead (one instruction stream)
  // was measured slower: 66-68 us against 61.5 for 64 Mi elements.
  rows.rest();   // half tile 0; leaves the source of half tile 1 requested
  __syncwarp();
  NoSlices nothing;
  auto lanes = [&](auto half_tag, int h) {
    constexpr int kHalf = decltype(half_tag)::value;
    if (full_block)
      encode_half_rows<false, kLaneMask, kHalf>(table_address, tile_lane, sink, g.lane_mask,
                                                kTileRows * (h >> 1), valid, budget_bits, pos, lo,
                                                extra_start, open, nothing);
    else
      encode_half_rows<true, kLaneMask, kHalf>(table_address, tile_lane, sink, g.lane_mask,
                                               kTileRows * (h >> 1), valid, budget_bits, pos, lo,
                                               extra_start, open, nothing);
  };
  for (int h = 0; h < halves; h += 2) {
    lanes(std::integral_constant<int, 0>(), h);
    __syncwarp();
    if (h + 1 < halves) {
      rows.rest();
      __syncwarp();
      lanes(std::integral_constant<int, 1>(), h + 1);
      __syncwarp();
      if (h + 2 < halves) {
        rows.rest();
        __syncwarp();
      }
    }
  }
  if (!kPrecomputed && !full_block) {
    const int first_untouched = halves * (kTileRows / 2);
    uint4* rest = reinterpret_cast<uint4*>(side + block_base + (int64_t)first_untouched * kLanes);
    for (int i = tid; i < (g.steps - first_untouched) * (kLanes / 16); i += kThreads)
      __stcs(rest + i, make_uint4(0u, 0u, 0u, 0u));
  }
  if (open && (pos & 31) != 0) payload_column[(pos >> 5) * kLanes] = lo;
  extra_starts[block * kLanes + tid] = extra_start < 0 ? (uint8_t)255 : (uint8_t)extra_start;

  // Block summary: overflowing lanes and their tail bytes.
  int bad = extra_start >= 0 ? 1 : 0;
  int bytes = extra_start >= 0 ? g.steps - extra_start : 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    bad += __shfl_down_sync(0xFFFFFFFFu, bad, d);
    bytes += __shfl_down_sync(0xFFFFFFFFu, bytes, d);
  }
  if (lane32 == 0) { sh.scan[warp] = bad; sh.scan[8 + warp] = bytes; }
  __syncthreads();  // also publishes every lane's payload words
  if (tid == 0) {
    int total_bad = 0, total_bytes = 0;
    for (int w = 0; w < kWarps; ++w) { total_bad += sh.scan[w]; total_bytes += sh.scan[8 + w]; }
    summaries[block] = total_bad;
    summaries[g.n_blocks + block] = total_bytes;
  }
  // Payload image -> global: word w of the block's 256 streams is one 1 KB row.
  uint32_t* out = encoded + block * kLanes;
  for (int i = tid; i < g.fixed_words * (kLanes / 4); i += kThreads) {
    const int w = i >> 6, c = (i & 63) * 4;
    const uint4 v = *reinterpret_cast<const uint4*>(&payload[w * kLanes + c]);
    __stcs(reinterpret_cast<uint4*>(out + (int64_t)w * g.streams + c), v);
  }
}

template <bool kPrecomputed, int kLaneMask>
__global__ void __launch_bounds__(kThreads, kEncodeMinCtas)
encode_kernel(const void* __restrict__ src, bool src_vector_ok, uint8_t* __restrict__ side,
              uint32_t* __restrict__ encoded, const int32_t* __restrict__ shifted_encode,
              uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries, EncodeShape g) {
  encode_block<kPrecomputed, kLaneMask>(src, src_vector_ok, side, encoded, shifted_encode,
                                        extra_starts, summaries, g, blockIdx.x);
}

// Shape of one job of a batch (all jobs share the geometry in `common`).
template <typename Job>
__device__ __forceinline__ EncodeShape shape_of_job(const Job& job, const EncodeShape& common) {
  EncodeShape g = common;
  g.size = job.size;
  g.logical_numel = job.logical_numel;
  g.n_blocks = job.size / common.block_symbols;
  g.streams = g.n_blocks * kLanes;
  return g;
}

template <typename Job>
__device__ __forceinline__ int find_encode_job(const Job* jobs, int n_jobs, int64_t block) {
  int lo = 0, hi = n_jobs - 1;
  while (lo < hi) {  // last job with first_block <= block
    const int mid = (lo + hi + 1) >> 1;
    if (jobs[mid].first_block <= block) lo = mid; else hi = mid - 1;
  }
  return lo;
}

template <int kLaneMask>
__global__ void __launch_bounds__(kThreads, kEncodeMinCtas)
encode_batch_kernel(const lct_encode_job* __restrict__ jobs, int n_jobs,
                    const int32_t* __restrict__ shifted_encode, uint8_t* __restrict__ extra_starts,
                    int32_t* __restrict__ summaries, EncodeShape common) {
  const int64_t block = blockIdx.x;
  const int j = find_encode_job(jobs, n_jobs, block);
  const lct_encode_job& job = jobs[j];
  const EncodeShape g = shape_of_job(job, common);
  const bool vector_ok = (reinterpret_cast<uintptr_t>(job.src) & 15u) == 0;
  encode_block<false, kLaneMask>(job.src, vector_ok, job.side,
                                 reinterpret_cast<uint32_t*>(job.encoded),
                                 shifted_encode + 256 * (int64_t)j,
                                 extra_starts + job.first_block * kLanes,
                                 summaries + 4 * job.first_block, g, block - job.first_block);
}

// Compact overflow metadata and raw exponent tails of one block.  Lanes are
// listed in increasing order; a lane's tail holds exponent - 127 for every
// row from its overflow start to the end of the block (padding rows read as
// exponent byte 0).
template <bool kPrecomputed>
__device__ __forceinline__ void compact_block(const void* __restrict__ src, uint8_t* lanes,
                                              uint8_t* starts, uint8_t* tail,
                                              const int32_t* descriptor, const int32_t* counts,
                                              int32_t* blocks_out,
                                              const uint8_t* __restrict__ extra_starts,
                                              const int32_t* __restrict__ summaries,
                                              const EncodeShape& g, int64_t block) {
  __shared__ int scan[33];
  const int tid = threadIdx.x;
  const int count = summaries[block];
  const int first = summaries[2 * g.n_blocks + block];
  const int byte_base = summaries[3 * g.n_blocks + block];
  if (tid == 0) {
    blocks_out[block] = count;
    blocks_out[g.n_blocks + block] = first;
    blocks_out[2 * g.n_blocks + block] = byte_base;
  }
  if (count == 0) return;
  int64_t lane_off = 0, start_off = 0, tail_off = 0;
  if (descriptor != nullptr) {
    if (descriptor[2] != 0) return;  // no arena region: nothing may be written
    const int64_t total = counts[0];
    lane_off = descriptor[0];
    start_off = lane_off + total;
    tail_off = lane_off + 2 * total;
  }
  const int start = extra_starts[block * kLanes + tid];
  const bool bad = start != 255;
  int unused;
  const int rank = block_exclusive_scan(bad ? 1 : 0, scan, &unused);
  const int local = block_exclusive_scan(bad ? g.steps - start : 0, scan, &unused);
  if (bad) {
    lanes[lane_off + first + rank] = (uint8_t)tid;
    starts[start_off + first + rank] = (uint8_t)start;
  }
  // Each warp copies the tails of its own 32 lanes, one lane at a time, with
  // the 32 threads striding over that lane's rows.
  const int lane_in_warp = tid & 31;
  const int warp_first_lane = tid & ~31;
  unsigned pending = __ballot_sync(0xFFFFFFFFu, bad);
  const int64_t row0 = block * g.steps;
  while (pending) {
    const int owner = __ffs(pending) - 1;
    pending &= pending - 1;
    const int lane = warp_first_lane + owner;
    const int lane_start = __shfl_sync(0xFFFFFFFFu, start, owner);
    const int lane_local = __shfl_sync(0xFFFFFFFFu, local, owner);
    uint8_t* dst = tail + tail_off + byte_base + lane_local;
    for (int row = lane_start + lane_in_warp; row < g.steps; row += 32) {
      const int64_t n = row0 + row;
      const int64_t logical = n * kLanes + (lane ^ (int)(n & g.lane_mask));
      int byte = 0;
      if (logical < g.logical_numel) {
        byte = kPrecomputed ? (int)static_cast<const uint8_t*>(src)[logical]
                            : ((int)static_cast<const uint16_t*>(src)[logical] >> 7) & 255;
      }
      dst[row - lane_start] = (uint8_t)(byte - 127);
    }
  }
}

template <bool kPrecomputed>
__global__ void __launch_bounds__(kThreads)
compact_tails_kernel(const void* __restrict__ src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                     const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                     const uint8_t* __restrict__ extra_starts, const int32_t* __restrict__ summaries,
                     EncodeShape g) {
  cudaGridDependencySynchronize();  // prefixes and the reservation come from the scan in front
  compact_block<kPrecomputed>(src, lanes, starts, tail, descriptor, counts, blocks_out,
                              extra_starts, summaries, g, blockIdx.x);
}

// Where the tail pass finds a job's exponents: the BF16 source of an encode job, the raw
// result exponents a fused update left for its overflowing lanes.
__device__ __forceinline__ const void* tail_source(const lct_encode_job& job) { return job.src; }
__device__ __forceinline__ const void* tail_source(const lct_update_job& job) { return job.spill; }

template <typename Job, bool kPrecomputed>
__global__ void __launch_bounds__(kThreads)
compact_batch_kernel(const Job* __restrict__ jobs, int n_jobs, uint8_t* arena_payload,
                     const uint8_t* __restrict__ extra_starts, const int32_t* __restrict__ summaries,
                     EncodeShape common) {
  cudaGridDependencySynchronize();  // prefixes and reservations come from the scan in front
  const int64_t block = blockIdx.x;
  const Job& job = jobs[find_encode_job(jobs, n_jobs, block)];
  const EncodeShape g = shape_of_job(job, common);
  compact_block<kPrecomputed>(tail_source(job), arena_payload, arena_payload, arena_payload,
                              job.descriptor, job.counts, job.blocks_out,
                              extra_starts + job.first_block * kLanes,
                              summaries + 4 * job.first_block, g, block - job.first_block);
}

static int check_encode_shape(int64_t size, int64_t logical_numel, int block_symbols, int steps,
                              int fixed_words, EncodeShape* g) {
  if (steps != 128 && steps != 256) return LCT_E_BAD_GEOMETRY;
  if (block_symbols != steps * kLanes) return LCT_E_BAD_GEOMETRY;
  if (fixed_words < 2 || fixed_words > 64) return LCT_E_BAD_GEOMETRY;
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
  g->lane_mask = lct::lane_mask_now();
  return 0;
}

}  // namespace lct

extern "C" {

// Argument checks and launch shared by lct_encode and lct_compress.
static int launch_encode(const void* src, uint8_t* side, int32_t* encoded,
                         const int32_t* shifted_encode, uint8_t* extra_starts, int32_t* summaries,
                         int64_t size, int64_t logical_numel, int block_symbols, int steps,
                         int fixed_words, int precomputed, bool overlapped, cudaStream_t st) {
  lct::EncodeShape g;
  int rc = lct::check_encode_shape(size, logical_numel, block_symbols, steps, fixed_words, &g);
  if (rc) return rc;
  if (src == nullptr || encoded == nullptr || shifted_encode == nullptr ||
      extra_starts == nullptr || summaries == nullptr)
    return LCT_E_NULL_POINTER;
  if (!precomputed && side == nullptr) return LCT_E_NULL_POINTER;
  const uintptr_t s = reinterpret_cast<uintptr_t>(src);
  if (!precomputed && (s & 1u)) return LCT_E_ALIGNMENT;
  if ((reinterpret_cast<uintptr_t>(encoded) & 15u) ||
      (!precomputed && (reinterpret_cast<uintptr_t>(side) & 15u)))
    return LCT_E_ALIGNMENT;
  const bool vector_ok = (s & (precomputed ? 7u : 15u)) == 0;
  const size_t shared = sizeof(lct::EncodeSharedHead) + (size_t)fixed_words * lct::kLanes * 4;
  uint32_t* words = reinterpret_cast<uint32_t*>(encoded);
  const bool swizzled = g.lane_mask == 254;
  auto kernel = precomputed ? (swizzled ? lct::encode_kernel<true, 254> : lct::encode_kernel<true, -1>)
                            : (swizzled ? lct::encode_kernel<false, 254> : lct::encode_kernel<false, -1>);
  rc = (int)cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
  if (rc) return rc;
  if (overlapped)
    return lct::launch_overlapped(kernel, (unsigned)g.n_blocks, lct::kThreads, shared, st, src,
                                  vector_ok, side, words, shifted_encode, extra_starts, summaries, g);
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, shared, st>>>(src, vector_ok, side, words,
                                                              shifted_encode, extra_starts,
                                                              summaries, g);
  return (int)cudaGetLastError();
}

}  // extern "C"

namespace lct {

int launch_compact_batch(const lct_update_job* jobs, int n_jobs, int64_t total_blocks,
                         uint8_t* arena_payload, const uint8_t* extra_starts,
                         const int32_t* summaries, int block_symbols, int steps, int fixed_words,
                         cudaStream_t stream) {
  EncodeShape g;
  const int rc = check_encode_shape(block_symbols, block_symbols, block_symbols, steps, fixed_words, &g);
  if (rc) return rc;
  return launch_overlapped(compact_batch_kernel<lct_update_job, true>, (unsigned)total_blocks,
                           kThreads, 0, stream, jobs, n_jobs, arena_payload, extra_starts,
                           summaries, g);
}

int launch_compact(const void* src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                          const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                          const uint8_t* extra_starts, const int32_t* summaries, int64_t size,
                          int64_t logical_numel, int block_symbols, int steps, int precomputed,
                          bool overlapped, cudaStream_t st) {
  lct::EncodeShape g;
  int rc = lct::check_encode_shape(size, logical_numel, block_symbols, steps, 2, &g);
  if (rc) return rc;
  if (src == nullptr || counts == nullptr || blocks_out == nullptr || extra_starts == nullptr ||
      summaries == nullptr)
    return LCT_E_NULL_POINTER;
  // lanes/starts/tail may be NULL only when the tensor has no overflow at all
  // (zero-size private tensors); the kernel then never dereferences them.
  auto kernel = precomputed ? lct::compact_tails_kernel<true> : lct::compact_tails_kernel<false>;
  if (overlapped)
    return lct::launch_overlapped(kernel, (unsigned)g.n_blocks, lct::kThreads, 0, st, src, lanes,
                                  starts, tail, descriptor, counts, blocks_out, extra_starts,
                                  summaries, g);
  kernel<<<(unsigned)g.n_blocks, lct::kThreads, 0, st>>>(src, lanes, starts, tail, descriptor,
                                                         counts, blocks_out, extra_starts,
                                                         summaries, g);
  return (int)cudaGetLastError();
}

}  // namespace lct

extern "C" {

int lct_encode(const void* src, uint8_t* side, int32_t* encoded, const int32_t* shifted_encode,
               uint8_t* extra_starts, int32_t* summaries, int64_t size, int64_t logical_numel,
               int block_symbols, int steps, int fixed_words, int precomputed, void* stream) {
  return launch_encode(src, side, encoded, shifted_encode, extra_starts, summaries, size,
                       logical_numel, block_symbols, steps, fixed_words, precomputed, false,
                       static_cast<cudaStream_t>(stream));
}

int lct_compact_tails(const void* src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                      const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                      const uint8_t* extra_starts, const int32_t* summaries, int64_t size,
                      int64_t logical_numel, int block_symbols, int steps, int precomputed,
                      void* stream) {
  return lct::launch_compact(src, lanes, starts, tail, descriptor, counts, blocks_out, extra_starts,
                        summaries, size, logical_numel, block_symbols, steps, precomputed, false,
                        static_cast<cudaStream_t>(stream));
}

int lct_compress(const void* src, int precomputed, uint8_t* side, int32_t* encoded,
                 const int32_t* encode_table, const int32_t* decode_table, int32_t* center,
                 int32_t* shifted_encode, int32_t* shifted_decode, uint8_t* extra_starts,
                 int32_t* summaries, int32_t* counts, int32_t* descriptor, int32_t* blocks_out,
                 void* arena_storage, int max_free_regions, int64_t size, int64_t logical_numel,
                 int block_symbols, int steps, int fixed_words, void* stream) {
  if (encode_table == nullptr || decode_table == nullptr || center == nullptr ||
      shifted_encode == nullptr || counts == nullptr || descriptor == nullptr ||
      arena_storage == nullptr || src == nullptr)
    return LCT_E_NULL_POINTER;
  if (max_free_regions <= 0 || (max_free_regions & (max_free_regions - 1))) return LCT_E_BAD_ARGUMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 1. center + tables: an ordinary launch, so everything queued before this call is complete
  //    and visible before any of the four kernels starts.
  int rc = lct::launch_center(src, logical_numel, precomputed != 0, encode_table, decode_table,
                              center, shifted_encode, shifted_decode, false, st);
  if (rc) return rc;
  // 2-4. each of these may be scheduled while its predecessor still runs and waits on the
  //    device for it where its first dependent read is.
  rc = launch_encode(src, side, encoded, shifted_encode, extra_starts, summaries, size,
                     logical_numel, block_symbols, steps, fixed_words, precomputed, true, st);
  if (rc) return rc;
  rc = lct::launch_scan_allocate(summaries, counts, descriptor, arena_storage, size / block_symbols,
                                 max_free_regions, true, st);
  if (rc) return rc;
  // The arena payload starts after the allocator words, padded to 16 bytes.
  const size_t metadata = ((size_t)8 * max_free_regions + 12 + 15) / 16 * 16;
  uint8_t* payload = static_cast<uint8_t*>(arena_storage) + metadata;
  return lct::launch_compact(src, payload, payload, payload, descriptor, counts, blocks_out,
                        extra_starts, summaries, size, logical_numel, block_symbols, steps,
                        precomputed, true, st);
}

}  // extern "C"

extern "C" {

int lct_compress_batch(const lct_encode_job* jobs, int n_jobs, int64_t total_blocks,
                       const int32_t* encode_table, const int32_t* decode_table,
                       void* arena_storage, int max_free_regions, uint8_t* extra_starts,
                       int32_t* summaries, int32_t* shifted_encode, int block_symbols, int steps,
                       int fixed_words, void* stream) {
  if (jobs == nullptr || encode_table == nullptr || decode_table == nullptr ||
      arena_storage == nullptr || extra_starts == nullptr || summaries == nullptr ||
      shifted_encode == nullptr)
    return LCT_E_NULL_POINTER;
  if (n_jobs <= 0 || total_blocks <= 0 || total_blocks > 0x7FFFFFFFLL) return LCT_E_BAD_ARGUMENT;
  if (max_free_regions <= 0 || (max_free_regions & (max_free_regions - 1))) return LCT_E_BAD_ARGUMENT;
  lct::EncodeShape g;
  int rc = lct::check_encode_shape(block_symbols, block_symbols, block_symbols, steps, fixed_words, &g);
  if (rc) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if ((rc = lct::launch_center_batch(jobs, n_jobs, encode_table, decode_table, shifted_encode, st)))
    return rc;
  const size_t shared = sizeof(lct::EncodeSharedHead) + (size_t)fixed_words * lct::kLanes * 4;
  auto encode_all = g.lane_mask == 254 ? lct::encode_batch_kernel<254> : lct::encode_batch_kernel<-1>;
  rc = (int)cudaFuncSetAttribute(encode_all, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
  if (rc) return rc;
  // Centers first (ordinary launch); the three kernels behind it may each be scheduled while
  // their predecessor still runs and wait for it on the device.
  if ((rc = lct::launch_overlapped(encode_all, (unsigned)total_blocks, lct::kThreads,
                                   shared, st, jobs, n_jobs, shifted_encode, extra_starts,
                                   summaries, g)))
    return rc;
  if ((rc = lct::launch_scan_batch(jobs, n_jobs, summaries, arena_storage, max_free_regions,
                                   block_symbols, st)))
    return rc;
  // The arena payload starts after the allocator words, padded to 16 bytes.
  const size_t metadata = ((size_t)8 * max_free_regions + 12 + 15) / 16 * 16;
  return lct::launch_overlapped(lct::compact_batch_kernel<lct_encode_job, false>,
                                (unsigned)total_blocks, lct::kThreads, 0, st, jobs, n_jobs,
                                static_cast<uint8_t*>(arena_storage) + metadata, extra_starts,
                                summaries, g);
}

}  // extern "C"

// ---------------------------------------------------------------------------
// Encode without any caller-side scratch: lct_encode_noalloc
// ---------------------------------------------------------------------------
//
// lct_encode needs two work buffers from its caller (one "first overflow step"
// byte per stream and four ints per block) that exist only to be handed to the
// summary scan.  Some callers cannot provide them: a serving loop that must
// not allocate once it has started, a host that gave all device memory to
// another allocator at start-up, or a C program that links this library and
// has no allocator at all.  For them the work buffers below live in the
// library image itself.  The first call on a GPU looks the array's address up
// and should come before any stream capture.

namespace lct {

// Largest tensor the built-in scratch serves: 1024 codec blocks (64 Mi
// elements in the 65536-element layouts, 32 Mi in the 32768-element ones).
constexpr int kNoAllocMaxBlocks = 1024;
constexpr size_t kNoAllocSummaryBytes = (size_t)kNoAllocMaxBlocks * 4 * sizeof(int32_t);
constexpr size_t kNoAllocBytes = kNoAllocSummaryBytes + (size_t)kNoAllocMaxBlocks * kLanes;

// 272 KiB per GPU that loads the library, held until the process exits.
// [0, 16 KiB): block summaries, int32[4 * blocks]; then one byte per stream.
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

constexpr int kMaxDevices = 64;
static unsigned char* g_noalloc_address[kMaxDevices];  // device address of the array, per GPU

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an
// address a kernel may use; the device address has to be asked for, once per
// GPU, while that GPU is current.  Returns 0 or a cudaError_t.
static int noalloc_scratch_address(unsigned char** out) {
  int device = -1;
  cudaError_t rc = cudaGetDevice(&device);
  if (rc != cudaSuccess) return (int)rc;
  if (device < 0 || device >= kMaxDevices) return LCT_E_BAD_ARGUMENT;
  unsigned char* known = __atomic_load_n(&g_noalloc_address[device], __ATOMIC_ACQUIRE);
  if (known == nullptr) {
    void* address = nullptr;
    rc = cudaGetSymbolAddress(&address, g_noalloc_scratch);
    if (rc != cudaSuccess) return (int)rc;
    if (address == nullptr) return (int)cudaErrorInvalidSymbol;
    known = static_cast<unsigned char*>(address);
    // Two threads racing here store the same value.
    __atomic_store_n(&g_noalloc_address[device], known, __ATOMIC_RELEASE);
  }
  *out = known;
  return 0;
}

}  // namespace lct

extern "C" {

int lct_scan_allocate(int32_t* summaries, int32_t* counts, int32_t* descriptor,
                      void* arena_storage, int64_t blocks, int max_free_regions, void* stream);

int lct_encode_noalloc(const void* src, uint8_t* side, int32_t* encoded,
                       const int32_t* shifted_encode, int32_t* counts, int64_t size,
                       int64_t logical_numel, int block_symbols, int steps, int fixed_words,
                       int precomputed, void* stream) {
  if (counts == nullptr) return LCT_E_NULL_POINTER;
  if (block_symbols <= 0 || size <= 0) return LCT_E_BAD_ARGUMENT;
  const int64_t blocks = (size + block_symbols - 1) / block_symbols;
  if (blocks > lct::kNoAllocMaxBlocks) return LCT_E_SCRATCH_LIMIT;
  unsigned char* scratch = nullptr;
  int rc = lct::noalloc_scratch_address(&scratch);
  if (rc) return rc;
  int32_t* summaries = reinterpret_cast<int32_t*>(scratch);
  uint8_t* extra_starts = scratch + lct::kNoAllocSummaryBytes;
  // Both kernels overwrite every scratch byte they later read (all streams of
  // the tensor, all four summary rows), so nothing left by an earlier call is
  // ever consumed and nothing has to be cleared first.
  rc = lct_encode(src, side, encoded, shifted_encode, extra_starts, summaries, size, logical_numel,
                  block_symbols, steps, fixed_words, precomputed, stream);
  if (rc) return rc;
  return lct_scan_allocate(summaries, counts, nullptr, nullptr, blocks, 256, stream);
}

}  // extern "C"
