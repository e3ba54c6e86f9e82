// Field split + fixed-budget Huffman encoder, and the overflow tail compaction.
//
// One CTA (256 threads) per codec block.  Per 32-row tile:
//   row phase  - thread = 8 columns of a row pair: 128-bit loads of the BF16
//                source, exponent bytes into the column-ordered shared tile,
//                side bytes permuted to lane order and stored 64 bits at a time;
//   lane phase - thread = lane: reads its exponent pair from the tile, looks
//                both codes up in the shared encode table, appends them to a
//                64-bit accumulator and drops finished 32-bit words into a
//                shared image of the block's payload.
// At the end the payload image (zero where nothing was written, so the output
// is deterministic) is copied out with coalesced stores, and the block's
// overflow summary is reduced.
#include "common.cuh"
#include "lct_b200.h"

namespace lct {

struct EncodeShape {
  int64_t size;
  int64_t logical_numel;
  int64_t streams;
  int64_t n_blocks;
  int block_symbols;
  int steps;
  int fixed_words;
};

// Dynamic shared memory: encode table | tile | scan scratch | payload image.
struct __align__(16) EncodeSharedHead {
  uint32_t table[256];
  uint16_t tile[kTilePairs * kLanes];
  int scan[33];
  int pad[3];
};

__device__ __forceinline__ uint32_t load_pair_guarded(const uint16_t* src, int64_t at, int64_t numel) {
  const uint32_t a = at < numel ? src[at] : 0u;
  const uint32_t b = at + 1 < numel ? src[at + 1] : 0u;
  return a | (b << 16);
}

template <bool kPrecomputed>
__global__ void __launch_bounds__(kThreads)
encode_kernel(const void* __restrict__ src, bool src_vector_ok, uint8_t* __restrict__ side,
              uint32_t* __restrict__ encoded, const int32_t* __restrict__ shifted_encode,
              uint8_t* __restrict__ extra_starts, int32_t* __restrict__ summaries, EncodeShape g) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  EncodeSharedHead& sh = *reinterpret_cast<EncodeSharedHead*>(smem_raw);
  uint32_t* payload = reinterpret_cast<uint32_t*>(smem_raw + sizeof(EncodeSharedHead));

  const int64_t block = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t row0 = block * g.steps;
  const int64_t block_base = block * (int64_t)g.block_symbols;
  const bool full_block = block_base + g.block_symbols <= g.logical_numel;

  sh.table[tid] = (uint32_t)shifted_encode[tid];
  for (int w = 0; w < g.fixed_words; ++w) payload[w * kLanes + tid] = 0u;
  if (block == 0 && tid < 4) encoded[g.streams * g.fixed_words + tid] = 0u;  // trailing pad words

  const int valid = valid_steps_of(block, tid, g.steps, g.block_symbols, g.logical_numel);
  const int budget_bits = g.fixed_words * 32;
  uint64_t acc = 0;
  int shift = 0, word = 0;
  int extra_start = -1;  // first overflowing step, -1 = none

  for (int step0 = 0; step0 < g.steps; step0 += kTileRows) {
    __syncthreads();  // table/payload ready; previous tile fully consumed
    // ---- row phase ----
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int p = (tid >> 5) + 8 * u;
      const int j = tid & 31;
      const int step = step0 + 2 * p;
      const int64_t row = row0 + step;
      const int64_t at = row * kLanes + 8 * j;
      uint32_t tile_words[4];
      if (kPrecomputed) {
        const uint8_t* bytes = static_cast<const uint8_t*>(src);
        uint32_t top[2], bottom[2];
        if (src_vector_ok && at + kLanes + 8 <= g.logical_numel) {
          const uint2 t = __ldcs(reinterpret_cast<const uint2*>(bytes + at));
          const uint2 b = __ldcs(reinterpret_cast<const uint2*>(bytes + at + kLanes));
          top[0] = t.x; top[1] = t.y; bottom[0] = b.x; bottom[1] = b.y;
        } else {
          top[0] = top[1] = bottom[0] = bottom[1] = 0u;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            if (at + i < g.logical_numel) top[i >> 2] |= (uint32_t)bytes[at + i] << (8 * (i & 3));
            if (at + kLanes + i < g.logical_numel)
              bottom[i >> 2] |= (uint32_t)bytes[at + kLanes + i] << (8 * (i & 3));
          }
        }
        tile_words[0] = prmt(top[0], bottom[0], 0x5140);
        tile_words[1] = prmt(top[0], bottom[0], 0x7362);
        tile_words[2] = prmt(top[1], bottom[1], 0x5140);
        tile_words[3] = prmt(top[1], bottom[1], 0x7362);
      } else {
        const uint16_t* bits = static_cast<const uint16_t*>(src);
        uint32_t top[4], bottom[4];
        if (src_vector_ok && (full_block || at + kLanes + 8 <= g.logical_numel)) {
          const uint4 t = __ldcs(reinterpret_cast<const uint4*>(bits + at));
          const uint4 b = __ldcs(reinterpret_cast<const uint4*>(bits + at + kLanes));
          top[0] = t.x; top[1] = t.y; top[2] = t.z; top[3] = t.w;
          bottom[0] = b.x; bottom[1] = b.y; bottom[2] = b.z; bottom[3] = b.w;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            top[k] = load_pair_guarded(bits, at + 2 * k, g.logical_numel);
            bottom[k] = load_pair_guarded(bits, at + kLanes + 2 * k, g.logical_numel);
          }
        }
#pragma unroll
        for (int k = 0; k < 4; ++k)
          tile_words[k] = prmt(exponents_of(top[k]), exponents_of(bottom[k]), 0x6240);
        // Side bytes: column order -> lane order, one 8-byte store per row.
        const int mask = (int)(row & 254);
        const uint32_t q = (uint32_t)(mask >> 1) & 3u;
        const int lane_group = (8 * j) ^ (mask & 0xF8);
        uint8_t* s = side + block_base + (int64_t)step * kLanes + lane_group;
        const uint32_t t01 = prmt(sides_of(top[0]), sides_of(top[1]), 0x6420);
        const uint32_t t23 = prmt(sides_of(top[2]), sides_of(top[3]), 0x6420);
        const uint32_t b01 = prmt(sides_of(bottom[0]), sides_of(bottom[1]), 0x6420);
        const uint32_t b23 = prmt(sides_of(bottom[2]), sides_of(bottom[3]), 0x6420);
        __stcs(reinterpret_cast<uint2*>(s),
               make_uint2(prmt(t01, t23, pair_selector_low(q)), prmt(t01, t23, pair_selector_high(q))));
        __stcs(reinterpret_cast<uint2*>(s + kLanes),
               make_uint2(prmt(b01, b23, pair_selector_low(q)), prmt(b01, b23, pair_selector_high(q))));
      }
      *reinterpret_cast<uint4*>(&sh.tile[p * kLanes + 8 * j]) =
          make_uint4(tile_words[0], tile_words[1], tile_words[2], tile_words[3]);
    }
    __syncthreads();
    // ---- lane phase ----
    if (extra_start < 0) {
#pragma unroll 4
      for (int p = 0; p < kTilePairs; ++p) {
        const int step = step0 + 2 * p;
        const int mask = (int)((row0 + step) & 254);
        const uint32_t pair = sh.tile[p * kLanes + (tid ^ mask)];
        uint32_t c0 = sh.table[pair & 255u];
        uint32_t c1 = sh.table[pair >> 8];
        if (step >= valid) c0 = 0u;          // padding carries no bits
        if (step + 1 >= valid) c1 = 0u;
        const int length0 = (int)(c0 >> 20);
        const int length = (int)((c0 + c1) >> 20);  // codes are < 2^16: no carry into bit 20
        const uint32_t code = (c0 & 0xFFFFFu) | ((c1 & 0xFFFFFu) << length0);
        if (word * 32 + shift + length > budget_bits) {
          // First pair that does not fit: freeze the current word and stop.
          extra_start = step;
          if (word < g.fixed_words) payload[word * kLanes + tid] = (uint32_t)acc;
          word = g.fixed_words;
          break;
        }
        acc |= (uint64_t)code << shift;
        shift += length;
        if (shift >= 32) {
          payload[word * kLanes + tid] = (uint32_t)acc;
          acc >>= 32;
          shift -= 32;
          ++word;
        }
      }
    }
  }
  if (extra_start < 0 && word < g.fixed_words && shift != 0)
    payload[word * kLanes + tid] = (uint32_t)acc;
  extra_starts[block * kLanes + tid] = extra_start < 0 ? (uint8_t)255 : (uint8_t)extra_start;

  // Block summary: overflowing lanes and their tail bytes.
  int bad = extra_start >= 0 ? 1 : 0;
  int bytes = extra_start >= 0 ? g.steps - extra_start : 0;
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    bad += __shfl_down_sync(0xFFFFFFFFu, bad, d);
    bytes += __shfl_down_sync(0xFFFFFFFFu, bytes, d);
  }
  __syncthreads();
  if ((tid & 31) == 0) { sh.scan[tid >> 5] = bad; sh.scan[8 + (tid >> 5)] = bytes; }
  __syncthreads();  // also publishes every lane's payload words
  if (tid == 0) {
    int total_bad = 0, total_bytes = 0;
    for (int w = 0; w < kThreads / 32; ++w) { total_bad += sh.scan[w]; total_bytes += sh.scan[8 + w]; }
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

// Compact overflow metadata and raw exponent tails of one block.  Lanes are
// listed in increasing order; a lane's tail holds exponent - 127 for every
// row from its overflow start to the end of the block (padding rows read as
// exponent byte 0).
template <bool kPrecomputed>
__global__ void __launch_bounds__(kThreads)
compact_tails_kernel(const void* __restrict__ src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                     const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                     const uint8_t* __restrict__ extra_starts, const int32_t* __restrict__ summaries,
                     EncodeShape g) {
  __shared__ int scan[33];
  const int64_t block = blockIdx.x;
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
      const int64_t logical = n * kLanes + (lane ^ (int)(n & 254));
      int byte = 0;
      if (logical < g.logical_numel) {
        byte = kPrecomputed ? (int)static_cast<const uint8_t*>(src)[logical]
                            : ((int)static_cast<const uint16_t*>(src)[logical] >> 7) & 255;
      }
      dst[row - lane_start] = (uint8_t)(byte - 127);
    }
  }
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
  return 0;
}

}  // namespace lct

extern "C" {

int lct_encode(const void* src, uint8_t* side, int32_t* encoded, const int32_t* shifted_encode,
               uint8_t* extra_starts, int32_t* summaries, int64_t size, int64_t logical_numel,
               int block_symbols, int steps, int fixed_words, int precomputed, void* stream) {
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* words = reinterpret_cast<uint32_t*>(encoded);
  if (precomputed) {
    rc = (int)cudaFuncSetAttribute(lct::encode_kernel<true>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (rc) return rc;
    lct::encode_kernel<true><<<(unsigned)g.n_blocks, lct::kThreads, shared, st>>>(
        src, vector_ok, side, words, shifted_encode, extra_starts, summaries, g);
  } else {
    rc = (int)cudaFuncSetAttribute(lct::encode_kernel<false>,
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
    if (rc) return rc;
    lct::encode_kernel<false><<<(unsigned)g.n_blocks, lct::kThreads, shared, st>>>(
        src, vector_ok, side, words, shifted_encode, extra_starts, summaries, g);
  }
  return (int)cudaGetLastError();
}

int lct_compact_tails(const void* src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                      const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                      const uint8_t* extra_starts, const int32_t* summaries, int64_t size,
                      int64_t logical_numel, int block_symbols, int steps, int precomputed,
                      void* stream) {
  lct::EncodeShape g;
  int rc = lct::check_encode_shape(size, logical_numel, block_symbols, steps, 2, &g);
  if (rc) return rc;
  if (src == nullptr || counts == nullptr || blocks_out == nullptr || extra_starts == nullptr ||
      summaries == nullptr)
    return LCT_E_NULL_POINTER;
  // lanes/starts/tail may be NULL only when the tensor has no overflow at all
  // (zero-size private tensors); the kernel then never dereferences them.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (precomputed)
    lct::compact_tails_kernel<true><<<(unsigned)g.n_blocks, lct::kThreads, 0, st>>>(
        src, lanes, starts, tail, descriptor, counts, blocks_out, extra_starts, summaries, g);
  else
    lct::compact_tails_kernel<false><<<(unsigned)g.n_blocks, lct::kThreads, 0, st>>>(
        src, lanes, starts, tail, descriptor, counts, blocks_out, extra_starts, summaries, g);
  return (int)cudaGetLastError();
}

}  // extern "C"
