// Launchers of the multi-tensor kernels that live in other translation units
// (lct_compress_batch in encode.cu strings them together).
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

}  // namespace lct
