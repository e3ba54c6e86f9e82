// Center estimate and per-tensor shifted tables: the part shared by the codebook kernels
// (tables.cu) and the fused update's merged sample + center kernel (update.cu).
#pragma once

#include "common.cuh"

namespace lct {

constexpr int kTableThreads = 1024;

static_assert(kTableThreads == kFirstMask + 1, "one first-level decode entry per thread");
static_assert(kSampleCount == 4 * kTableThreads, "four center samples per thread");

__device__ __forceinline__ int32_t shifted_encode_entry(const int32_t* base_encode, int raw,
                                                        int center) {
  const int zero_delta = (-127 - center) & 255;
  const int exponent = raw - 127;
  const int delta = (exponent - center) & 255;
  const int index = exponent == -127 ? 0 : delta + (delta < zero_delta ? 1 : 0);
  return base_encode[index];
}

__device__ __forceinline__ int32_t shifted_decode_entry(int32_t packed, int center) {
  const int zero_delta = (-127 - center) & 255;
  const int length = packed & 255;
  const int symbol = (packed >> 8) & 255;
  int delta = symbol == 0 ? 0 : symbol - (symbol <= zero_delta ? 1 : 0);
  if (delta >= 128) delta -= 256;
  const int exponent = symbol == 0 ? -127 : delta + center;
  return length == 0 ? 0 : (int32_t)((uint32_t)length | ((uint32_t)exponent << 8));
}

// One CTA of 1024 threads, four samples per thread in raw[] (exponent bytes, -1 = no sample): the
// mean exponent of the samples with exponent >= -120, rounded half away from zero, is the
// center; then the shifted tables for it.  The base-table rows are requested before the
// reductions so that their latency is hidden.
__device__ __forceinline__ void center_from_samples(const int (&raw)[4],
                                                    const int32_t* __restrict__ base_encode,
                                                    const int32_t* __restrict__ base_decode,
                                                    int32_t* center_out, int32_t* shifted_encode,
                                                    int32_t* shifted_decode) {
  __shared__ int s_sum[32], s_kept[32], s_center;
  __shared__ int32_t s_encode[256];
  const int tid = threadIdx.x;
  const int32_t decode_row = shifted_decode != nullptr ? base_decode[tid] : 0;
  if (shifted_encode != nullptr && tid < 256) s_encode[tid] = base_encode[tid];
  int sum = 0, kept = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int exponent = raw[k] - 127;
    if (raw[k] >= 0 && exponent >= -120) { sum += exponent; ++kept; }
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) {
    sum += __shfl_down_sync(0xFFFFFFFFu, sum, d);
    kept += __shfl_down_sync(0xFFFFFFFFu, kept, d);
  }
  if ((tid & 31) == 0) { s_sum[tid >> 5] = sum; s_kept[tid >> 5] = kept; }
  __syncthreads();
  if (tid < 32) {
    int total = s_sum[tid], count = s_kept[tid];
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) {
      total += __shfl_down_sync(0xFFFFFFFFu, total, d);
      count += __shfl_down_sync(0xFFFFFFFFu, count, d);
    }
    if (tid == 0) {
      const int safe = count > 0 ? count : 1;
      int center = total >= 0 ? (total + safe / 2) / safe : -((-total + safe / 2) / safe);
      if (count == 0) center = 0;
      center = min(max(center, -128), 127);
      s_center = center;
      *center_out = center;
    }
  }
  __syncthreads();
  const int center = s_center;
  if (shifted_encode != nullptr && tid < 256)
    shifted_encode[tid] = shifted_encode_entry(s_encode, tid, center);
  if (shifted_decode != nullptr) shifted_decode[tid] = shifted_decode_entry(decode_row, center);
}

}  // namespace lct
