// Launchers of kernels that live in other translation units (lct_compress and
// lct_compress_batch in encode.cu string them together), and the launch helper
// for a kernel that may start while its predecessor in the stream still runs.
#pragma once

#include <cuda_runtime.h>

#include "lct_b200.h"

namespace lct {

// tables.cu: one CTA per job samples the center and writes the shifted tables.
int launch_center_batch(const lct_encode_job* jobs, int n_jobs, const int32_t* encode_table,
                        const int32_t* decode_table, int32_t* shifted_encode, cudaStream_t stream);

// arena.cu: per-job summary scans, then the arena reservations in job order.
int launch_scan_batch(const lct_encode_job* jobs, int n_jobs, int32_t* summaries,
                      void* arena_storage, int max_free_regions, int block_symbols,
                      cudaStream_t stream);

// The same three steps for the jobs of a batched update (lct_update_batch in update.cu).
// tables.cu: job j's center from its sampled result exponents, samples + 4096 * j.
int launch_center_batch(const lct_update_job* jobs, int n_jobs, const int32_t* encode_table,
                        const int32_t* decode_table, const uint8_t* samples,
                        int32_t* shifted_encode, cudaStream_t stream);
int launch_scan_batch(const lct_update_job* jobs, int n_jobs, int32_t* summaries,
                      void* arena_storage, int max_free_regions, int block_symbols,
                      cudaStream_t stream);
// encode.cu: tails of all jobs from their spill arrays (raw result exponents).
int launch_compact_batch(const lct_update_job* jobs, int n_jobs, int64_t total_blocks,
                         uint8_t* arena_payload, const uint8_t* extra_starts,
                         const int32_t* summaries, int block_symbols, int steps, int fixed_words,
                         cudaStream_t stream);

// tables.cu: center sample + shifted tables of one tensor.
int launch_center(const void* src, int64_t logical_numel, bool precomputed,
                  const int32_t* encode_table, const int32_t* decode_table, int32_t* center,
                  int32_t* shifted_encode, int32_t* shifted_decode, bool overlapped,
                  cudaStream_t stream);

// encode.cu: overflow entries + raw tails of one tensor (argument checks included).
int launch_compact(const void* src, uint8_t* lanes, uint8_t* starts, uint8_t* tail,
                   const int32_t* descriptor, const int32_t* counts, int32_t* blocks_out,
                   const uint8_t* extra_starts, const int32_t* summaries, int64_t size,
                   int64_t logical_numel, int block_symbols, int steps, int precomputed,
                   bool overlapped, cudaStream_t stream);

// arena.cu: summary scan (+ arena reservation, + release of another region of the same arena
// right after it).  `overlapped`: see launch_overlapped.
int launch_scan_allocate(int32_t* summaries, int32_t* counts, int32_t* descriptor,
                         void* arena_storage, int64_t blocks, int max_free_regions,
                         bool overlapped, cudaStream_t stream,
                         int32_t* release_descriptor = nullptr, int32_t* release_status = nullptr);

// Launch with programmatic stream serialisation: the grid may be scheduled as soon as every
// CTA of the previous kernel in the stream has exited or called
// cudaTriggerProgrammaticLaunchCompletion(), and must call cudaGridDependencySynchronize()
// before it touches anything that kernel (or anything before it) wrote.  Everything the
// grid does ahead of that call overlaps the previous kernel's tail.
template <typename... Params, typename... Args>
int launch_overlapped(void (*kernel)(Params...), unsigned grid, unsigned threads, size_t shared,
                      cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(grid);
  config.blockDim = dim3(threads);
  config.dynamicSmemBytes = shared;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return (int)cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

}  // namespace lct
