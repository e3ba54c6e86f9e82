// Codebook preparation kernels: exponent-center sampling, per-tensor shifted
// tables, and the per-codebook two-symbol lookup table.
#include "batch.cuh"
#include "center.cuh"
#include "common.cuh"
#include "lct_b200.h"

namespace lct {

// Shifted tables for a center: encode indexed by raw exponent byte, decode
// storing the unbiased exponent above the code length.
__device__ __forceinline__ void write_shifted_tables(const int32_t* __restrict__ base_encode,
                                                     const int32_t* __restrict__ base_decode,
                                                     int center, int32_t* shifted_encode,
                                                     int32_t* shifted_decode) {
  if (shifted_encode != nullptr) {
    for (int raw = threadIdx.x; raw < 256; raw += blockDim.x)
      shifted_encode[raw] = shifted_encode_entry(base_encode, raw, center);
  }
  if (shifted_decode != nullptr) {
    for (int i = threadIdx.x; i <= kFirstMask; i += blockDim.x)
      shifted_decode[i] = shifted_decode_entry(base_decode[i], center);
  }
}

// One CTA of 1024 threads.  Every thread takes four of the <= 4096 jittered
// sample positions; the mean exponent of the samples with exponent >= -120,
// rounded half away from zero, is the center.  The kernel is one chain of
// memory latencies, so everything independent is issued up front: the four
// sample loads together, and the base-table rows the shifted tables are made
// from before the samples come back.
template <bool kPrecomputed>
__device__ __forceinline__ void center_and_tables(const void* __restrict__ src, int64_t n,
                                                  const int32_t* __restrict__ base_encode,
                                                  const int32_t* __restrict__ base_decode,
                                                  int32_t* center_out, int32_t* shifted_encode,
                                                  int32_t* shifted_decode) {
  const int tid = threadIdx.x;
  const int64_t samples = n < kSampleCount ? n : kSampleCount;
  int raw[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int64_t idx = tid + k * kTableThreads;
    raw[k] = -1;
    if (idx < samples) {
      const int64_t pos = sample_position(idx, n);
      raw[k] = kPrecomputed ? (int)static_cast<const uint8_t*>(src)[pos]
                            : ((int)static_cast<const uint16_t*>(src)[pos] >> 7) & 0xFF;
    }
  }
  center_from_samples(raw, base_encode, base_decode, center_out, shifted_encode, shifted_decode);
}

template <bool kPrecomputed>
__global__ void __launch_bounds__(kTableThreads)
center_and_tables_kernel(const void* __restrict__ src, int64_t n,
                         const int32_t* __restrict__ base_encode,
                         const int32_t* __restrict__ base_decode, int32_t* center_out,
                         int32_t* shifted_encode, int32_t* shifted_decode) {
  // The samples may come from a kernel that was still running when this one was scheduled;
  // a dependent encoder may start its table-independent prologue right away.
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  center_and_tables<kPrecomputed>(src, n, base_encode, base_decode, center_out, shifted_encode,
                                  shifted_decode);
}

__global__ void __launch_bounds__(kTableThreads)
center_batch_kernel(const lct_encode_job* __restrict__ jobs, const int32_t* __restrict__ base_encode,
                    const int32_t* __restrict__ base_decode, int32_t* shifted_encode) {
  cudaTriggerProgrammaticLaunchCompletion();  // the encoder behind waits where it needs the tables
  const lct_encode_job& job = jobs[blockIdx.x];
  center_and_tables<false>(job.src, job.logical_numel, base_encode, base_decode, job.center,
                           shifted_encode + 256 * (int64_t)blockIdx.x, job.shifted_decode);
}

__global__ void __launch_bounds__(kTableThreads)
center_update_batch_kernel(const lct_update_job* __restrict__ jobs,
                           const int32_t* __restrict__ base_encode,
                           const int32_t* __restrict__ base_decode,
                           const uint8_t* __restrict__ samples, int32_t* shifted_encode) {
  // The samples come from the kernel in front; the fused kernel behind may start its
  // table-independent prologue right away.
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  const lct_update_job& job = jobs[blockIdx.x];
  const int64_t count = job.logical_numel < kSampleCount ? job.logical_numel : kSampleCount;
  center_and_tables<true>(samples + (int64_t)kSampleCount * blockIdx.x, count, base_encode,
                          base_decode, job.center, shifted_encode + 256 * (int64_t)blockIdx.x,
                          job.shifted_decode);
}

__global__ void __launch_bounds__(kTableThreads)
shift_tables_kernel(const int32_t* __restrict__ base_encode, const int32_t* __restrict__ base_decode,
                    const int32_t* __restrict__ center, int32_t* shifted_encode,
                    int32_t* shifted_decode) {
  write_shifted_tables(base_encode, base_decode, *center, shifted_encode, shifted_decode);
}

// Two symbols per lookup over 12 stream bits, one 4096-entry table per possible
// center (CTA c serves center c - 128), symbols stored as raw exponent bytes so
// a decoder copies the table of its tensor's center and uses it as it is.  The
// second symbol is present only when both codes are direct and fit in the 12
// bits together.  The entry for stream window i is stored at table_slot(i) = i.
__global__ void __launch_bounds__(kTableThreads)
pair_table_kernel(const int32_t* __restrict__ decode, int rare_length,
                  uint32_t* __restrict__ pair_table) {
  const int center = (int)blockIdx.x - 128;
  uint32_t* table = pair_table + (size_t)blockIdx.x * kPairEntries;
  for (int slot = threadIdx.x; slot < kPairEntries; slot += blockDim.x) {
    const int i = slot;  // table_slot is the identity on 12-bit windows
    const int32_t first = decode[i & kFirstMask];
    uint32_t entry;
    if (first == 0) {
      entry = make_single_entry((uint32_t)(rare_length + 8), 0u, true);  // prefix + 8-bit literal
    } else {
      const uint32_t len0 = (uint32_t)first & 255u;
      const uint32_t byte0 = index_to_exponent_byte(((uint32_t)first >> 8) & 255u, center);
      const int32_t second = decode[(i >> len0) & kFirstMask];
      const uint32_t len1 = (uint32_t)second & 255u;
      if (second != 0 && len0 + len1 <= (uint32_t)kPairBits) {
        const uint32_t byte1 = index_to_exponent_byte(((uint32_t)second >> 8) & 255u, center);
        entry = make_pair_entry(len0, byte0, len1, byte1);
      } else {
        entry = make_single_entry(len0, byte0, false);
      }
    }
    table[slot] = entry;
  }
}

int launch_center(const void* src, int64_t logical_numel, bool precomputed,
                  const int32_t* encode_table, const int32_t* decode_table, int32_t* center,
                  int32_t* shifted_encode, int32_t* shifted_decode, bool overlapped,
                  cudaStream_t stream) {
  auto kernel = precomputed ? center_and_tables_kernel<true> : center_and_tables_kernel<false>;
  if (overlapped)
    return launch_overlapped(kernel, 1, kTableThreads, 0, stream, src, logical_numel, encode_table,
                             decode_table, center, shifted_encode, shifted_decode);
  kernel<<<1, kTableThreads, 0, stream>>>(src, logical_numel, encode_table, decode_table, center,
                                          shifted_encode, shifted_decode);
  return (int)cudaGetLastError();
}

int launch_center_batch(const lct_encode_job* jobs, int n_jobs, const int32_t* encode_table,
                        const int32_t* decode_table, int32_t* shifted_encode, cudaStream_t stream) {
  center_batch_kernel<<<n_jobs, kTableThreads, 0, stream>>>(jobs, encode_table, decode_table,
                                                            shifted_encode);
  return (int)cudaGetLastError();
}

int launch_center_batch(const lct_update_job* jobs, int n_jobs, const int32_t* encode_table,
                        const int32_t* decode_table, const uint8_t* samples,
                        int32_t* shifted_encode, cudaStream_t stream) {
  return launch_overlapped(center_update_batch_kernel, (unsigned)n_jobs, kTableThreads, 0, stream,
                           jobs, encode_table, decode_table, samples, shifted_encode);
}

}  // namespace lct

extern "C" {

int lct_build_pair_table(const int32_t* decode_table, int rare_length, uint32_t* pair_table,
                         void* stream) {
  if (decode_table == nullptr || pair_table == nullptr) return LCT_E_NULL_POINTER;
  if (rare_length < 0 || rare_length > 8) return LCT_E_BAD_ARGUMENT;
  lct::pair_table_kernel<<<lct::kCenterValues, lct::kTableThreads, 0,
                           static_cast<cudaStream_t>(stream)>>>(decode_table, rare_length,
                                                                pair_table);
  return (int)cudaGetLastError();
}

int lct_center_and_tables(const void* src, int64_t logical_numel, int precomputed,
                          const int32_t* encode_table, const int32_t* decode_table,
                          int32_t* center, int32_t* shifted_encode, int32_t* shifted_decode,
                          void* stream) {
  if (encode_table == nullptr || decode_table == nullptr || center == nullptr)
    return LCT_E_NULL_POINTER;
  if (logical_numel < 0) return LCT_E_BAD_ARGUMENT;
  if (logical_numel > 0 && src == nullptr) return LCT_E_NULL_POINTER;
  return lct::launch_center(src, logical_numel, precomputed != 0, encode_table, decode_table, center,
                            shifted_encode, shifted_decode, false,
                            static_cast<cudaStream_t>(stream));
}

int lct_shift_tables(const int32_t* encode_table, const int32_t* decode_table,
                     const int32_t* center, int32_t* shifted_encode, int32_t* shifted_decode,
                     void* stream) {
  if (center == nullptr) return LCT_E_NULL_POINTER;
  if ((shifted_encode != nullptr && encode_table == nullptr) ||
      (shifted_decode != nullptr && decode_table == nullptr))
    return LCT_E_NULL_POINTER;
  lct::shift_tables_kernel<<<1, lct::kTableThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      encode_table, decode_table, center, shifted_encode, shifted_decode);
  return (int)cudaGetLastError();
}

}  // extern "C"
