// Shared device helpers of the sm_100a codec kernels.
//
// Data layout recap.  A block is `steps` rows of 256 lanes.  Lane l at global
// row n holds logical element n*256 + (l ^ (n & lane_mask)), lane_mask = 254 (the
// default "swizzle" mapping; 0 = the reference's "linear" mapping, for which every
// XOR below vanishes and the same code runs unchanged); rows 2k and 2k+1 share
// one XOR mask, and the mask is even, so lanes 2p/2p+1 stay adjacent.  The
// mask's bits 5..7 move a warp's 32 lanes to another aligned group of 32
// columns and its bits 1..4 permute them inside that group, so in every row
// one warp's lanes cover exactly one 64-byte segment of the BF16 row.  That
// makes the pipeline warp-private: a warp (32 lanes of a block) passes its
// data through its own shared-memory tile, 32 rows at a time:
//
//     tile[pair p][x] = e(row 2p) | e(row 2p+1) << 8  of lane  x ^ (2p & lane_mask & 6)
//
// i.e. column order inside every aligned group of 8, lane order between the
// groups (decode_core.cuh: tile_slot_xor).  One side of each kernel works
// lane-wise (a thread owns a lane and walks its bit stream); the other side
// works row-wise (a thread owns 8 adjacent columns of a row pair: 128-bit
// global accesses).  __syncwarp(), or a barrier of two warps where they share
// rows, separates the two.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lct {

constexpr int kLanes = 256;
constexpr int kThreads = 256;           // one thread per lane
constexpr int kWarps = kThreads / 32;
constexpr int kTilePairs = 16;          // row pairs per warp tile (32 rows)
constexpr int kTileRows = 2 * kTilePairs;
constexpr int kPairBits = 12;           // stream bits indexing the two-symbol table
constexpr int kPairEntries = 1 << kPairBits;
constexpr int kCenterValues = 256;     // centers -128..127: one two-symbol table each
constexpr int kFirstMask = 1023;        // the codebook's first-level table covers 10 bits
constexpr int kSampleCount = 4096;     // positions the exponent center is estimated from

// Two-symbol table entry (one per 12-bit stream window):
//
//   bits 0..4    bits to consume: both code lengths of a full pair (two directly coded
//                symbols that fit the window together), else the first symbol's length
//                (an escape: prefix + 8-bit literal).  A funnel shift takes its amount from
//                the low five bits of a register, so the entry itself is the shift operand.
//   bits 5..7    first code length - 1 of a full pair (for a reader that wants one symbol)
//   byte 1       first symbol as an exponent byte (undefined for an escape)
//   byte 2       second symbol of a full pair
//   bits 24..28  copy of bits 0..4 for a full pair, else 0: one byte dot product subtracts it
//                from a bit counter
//   bit 30       kEscape: the first symbol is an escape
//   bit 31       kSlow: not a full pair (the sign bit, so one signed compare finds it)
constexpr uint32_t kSlow = 0x80000000u;
constexpr uint32_t kEscape = 0x40000000u;

__host__ __device__ __forceinline__ uint32_t make_pair_entry(uint32_t len0, uint32_t byte0,
                                                             uint32_t len1, uint32_t byte1) {
  const uint32_t total = len0 + len1;
  return total | ((len0 - 1u) << 5) | (byte0 << 8) | (byte1 << 16) | (total << 24);
}
__host__ __device__ __forceinline__ uint32_t make_single_entry(uint32_t len0, uint32_t byte0,
                                                               bool escape) {
  return kSlow | (escape ? kEscape : 0u) | len0 | (byte0 << 8);
}
// Length of the entry's first symbol.
__device__ __forceinline__ uint32_t entry_first_length(uint32_t entry) {
  return (int32_t)entry < 0 ? (entry & 31u) : ((entry >> 5) & 7u) + 1u;
}
__device__ __forceinline__ uint32_t entry_first_symbol(uint32_t entry) { return (entry >> 8) & 255u; }
__device__ __forceinline__ uint32_t entry_second_symbol(uint32_t entry) { return (entry >> 16) & 255u; }

// Slot of the two-symbol table that holds the entry for a 12-bit stream window (the window is
// the low kPairBits bits of `stream_bits`; higher bits are ignored): the window itself.
// Folding the window's top bits onto the shared-memory bank bits was measured too: it removes
// a tenth of the bank conflicts and costs two instructions on every lookup's dependent chain,
// for no change in the decoder's time.
__device__ __forceinline__ uint32_t table_slot(uint32_t stream_bits) {
  return stream_bits & (kPairEntries - 1);
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t selector) {
  return __byte_perm(a, b, selector);
}

// Selectors that reorder the four byte pairs of an 8-byte group by XOR-ing the
// pair index with q (q = (row & 6) >> 1).  The same permutation maps lane
// order to column order and back.
__device__ __forceinline__ uint32_t pair_selector_low(uint32_t q) { return 0x3210u ^ (q * 0x2222u); }
__device__ __forceinline__ uint32_t pair_selector_high(uint32_t q) { return 0x7654u ^ (q * 0x2222u); }

// Four exponent bytes + four side bytes (same columns) -> the low bytes and the
// high bytes of the four BF16 values: low = mantissa | exponent bit 0 << 7,
// high = sign | exponent >> 1.
__device__ __forceinline__ uint32_t bf16_low_bytes(uint32_t e4, uint32_t s4) {
  return (s4 & 0x7F7F7F7Fu) | ((e4 << 7) & 0x80808080u);
}
__device__ __forceinline__ uint32_t bf16_high_bytes(uint32_t e4, uint32_t s4) {
  return (s4 & 0x80808080u) | ((e4 >> 1) & 0x7F7F7F7Fu);
}
// ... and back: low/high bytes of four BF16 values -> exponent bytes, side bytes.
__device__ __forceinline__ uint32_t exponent_bytes(uint32_t low4, uint32_t high4) {
  return ((low4 >> 7) & 0x01010101u) | ((high4 << 1) & 0xFEFEFEFEu);
}
__device__ __forceinline__ uint32_t side_bytes(uint32_t low4, uint32_t high4) {
  return (low4 & 0x7F7F7F7Fu) | (high4 & 0x80808080u);
}

// Table index (0 = exact zero, else centred exponent delta) -> raw exponent byte.
__device__ __forceinline__ uint32_t index_to_exponent_byte(uint32_t index, int center) {
  const uint32_t zero_delta = (uint32_t)(-127 - center) & 255u;
  if (index == 0) return 0;
  return (index - (index <= zero_delta ? 1u : 0u) + (uint32_t)(center + 127)) & 255u;
}

// Position of center sample `idx` in a tensor of n elements: one jittered
// position per equal slice, floor(idx*n/count) + floor(hash * slice / 2^32)
// with count = min(n, 4096).  For n < 4096 every slice is one element, and
// for n >= 4096 the divisor is 2^12, so no division is needed.
__device__ __forceinline__ int64_t sample_position(int64_t idx, int64_t n) {
  if (n < kSampleCount) return idx;
  const int64_t start = (idx * n) >> 12, end = ((idx + 1) * n) >> 12;
  const uint32_t hashed = (uint32_t)idx * 0x9E3779B9u;
  return start + (int64_t)(((uint64_t)hashed * (uint64_t)(end - start)) >> 32);
}

// Lane mapping in force (host side, process-wide like the reference's import-time
// config.lane_mapping): 254 or 0.  Set through lct_set_lane_mapping (capi.cu).
int lane_mask_now();

// Number of leading steps of `lane` in block `block` that hold real elements.
__device__ __forceinline__ int valid_steps_of(int64_t block, int lane, int steps, int block_symbols,
                                              int64_t logical_numel, int lane_mask) {
  const int64_t in_block = logical_numel - block * (int64_t)block_symbols;
  if (in_block >= block_symbols) return steps;
  if (in_block <= 0) return 0;
  const int full_rows = (int)(in_block >> 8);
  const int rem = (int)(in_block & 255);
  const int mask = (int)((block * steps + full_rows) & lane_mask);
  return full_rows + ((rem > 0 && ((lane ^ mask) < rem)) ? 1 : 0);
}

// Block-wide exclusive prefix sum of one int per thread (blockDim.x <= 1024).
// `scratch` needs 33 ints.  Returns the exclusive prefix; *total gets the sum.
__device__ __forceinline__ int block_exclusive_scan(int value, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int inclusive = value;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    int up = __shfl_up_sync(0xFFFFFFFFu, inclusive, d);
    if (lane >= d) inclusive += up;
  }
  if (lane == 31) scratch[warp] = inclusive;
  __syncthreads();
  if (warp == 0) {
    const int warps = (blockDim.x + 31) >> 5;
    int w = lane < warps ? scratch[lane] : 0;
    int winc = w;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
      int up = __shfl_up_sync(0xFFFFFFFFu, winc, d);
      if (lane >= d) winc += up;
    }
    scratch[lane] = winc - w;
    if (lane == 31) scratch[32] = winc;
  }
  __syncthreads();
  const int result = scratch[warp] + inclusive - value;
  *total = scratch[32];
  __syncthreads();
  return result;
}

// ---- shared overflow arena ------------------------------------------------
// int32 free_starts[R] | free_sizes[R] | free_count | lock | generation
struct Arena {
  volatile int32_t* starts;
  volatile int32_t* sizes;
  volatile int32_t* count;
  int32_t* lock;
  volatile int32_t* generation;
};

__device__ __forceinline__ Arena arena_of(void* storage, int regions) {
  int32_t* m = reinterpret_cast<int32_t*>(storage);
  return Arena{m, m + regions, m + 2 * regions, m + 2 * regions + 1, m + 2 * regions + 2};
}

constexpr int kLockSpins = 200000;  // bounded wait: ~0.1 s worst case, then status 7
constexpr int kStatusLockTimeout = 7;

// Thread 0 of the CTA takes the arena lock; all threads learn the outcome.
__device__ __forceinline__ bool arena_lock(const Arena& a, int* shared_flag) {
  if (threadIdx.x == 0) {
    int spins = 0;
    bool got = false;
    while (spins++ < kLockSpins) {
      if (atomicCAS(a.lock, 0, 1) == 0) { got = true; break; }
      __nanosleep(256);
    }
    __threadfence();
    *shared_flag = got ? 1 : 0;
  }
  __syncthreads();
  const bool ok = *shared_flag != 0;
  __syncthreads();
  return ok;
}

__device__ __forceinline__ void arena_unlock(const Arena& a) {
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    atomicExch(a.lock, 0);
  }
}

// First-fit reservation by a whole CTA (same results as the reference's
// single-program allocator: lowest-index region that fits; exact fit removes
// the region, otherwise it shrinks from the front).  `scratch` needs 2 ints.
// The reservation itself, by a CTA that holds the arena lock.
__device__ inline void arena_allocate_locked(const Arena& a, int regions, int32_t request,
                                             int32_t* descriptor, int* scratch) {
  const int32_t size = (request + 15) / 16 * 16;
  const int count = *a.count;
  if (threadIdx.x == 0) scratch[1] = regions;
  __syncthreads();
  for (int i = threadIdx.x; i < count; i += blockDim.x)
    if (a.sizes[i] >= size) atomicMin(&scratch[1], i);
  __syncthreads();
  const int slot = scratch[1];
  const bool success = request > 0 && slot < count;
  int32_t start = 0, region = 0;
  if (success) { start = a.starts[slot]; region = a.sizes[slot]; }
  __syncthreads();
  if (success && region == size) {
    // Remove the region: shift the list left, chunk by chunk, reads before writes.
    for (int base = slot; base + 1 < count; base += blockDim.x) {
      const int i = base + threadIdx.x;
      int32_t ns = 0, nz = 0;
      const bool move = i + 1 < count;
      if (move) { ns = a.starts[i + 1]; nz = a.sizes[i + 1]; }
      __syncthreads();
      if (move) { a.starts[i] = ns; a.sizes[i] = nz; }
      __syncthreads();
    }
    if (threadIdx.x == 0) *a.count = count - 1;
  } else if (success && threadIdx.x == 0) {
    a.starts[slot] = start + size;
    a.sizes[slot] = region - size;
  }
  if (threadIdx.x == 0) {
    descriptor[0] = success ? start : -1;
    descriptor[1] = success ? size : 0;
    descriptor[2] = request <= 0 ? 2 : (success ? 0 : 1);
    descriptor[3] = *a.generation;
  }
  __syncthreads();
}

// Descriptor of a reservation that gave up waiting for the lock.
__device__ inline void arena_allocate_timed_out(const Arena& a, int32_t* descriptor) {
  if (threadIdx.x == 0) {
    descriptor[0] = -1; descriptor[1] = 0; descriptor[2] = kStatusLockTimeout;
    descriptor[3] = *a.generation;
  }
}

__device__ inline void arena_allocate(const Arena& a, int regions, int32_t request,
                                      int32_t* descriptor, int* scratch) {
  if (!arena_lock(a, scratch)) {
    arena_allocate_timed_out(a, descriptor);
    return;
  }
  arena_allocate_locked(a, regions, request, descriptor, scratch);
  arena_unlock(a);
}

}  // namespace lct
