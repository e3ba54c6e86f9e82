// Device-resident first-fit allocator for the shared overflow arena, and the
// per-tensor scan of block overflow summaries that feeds it.  Every launch is
// a single CTA; nothing here waits on another kernel, and the one lock wait is
// bounded (status 7 when it gives up).
#include "batch.cuh"
#include "common.cuh"
#include "lct_b200.h"

namespace lct {

constexpr int kArenaThreads = 256;
constexpr int kScanThreads = 1024;

__global__ void __launch_bounds__(kArenaThreads)
arena_reset_kernel(void* storage, int regions, int32_t capacity) {
  const Arena a = arena_of(storage, regions);
  for (int i = threadIdx.x; i < regions; i += blockDim.x) {
    a.starts[i] = 0;
    a.sizes[i] = i == 0 ? capacity : 0;
  }
  if (threadIdx.x == 0) {
    *a.count = 1;
    *a.generation = *a.generation + 1;
    __threadfence();
    atomicExch(a.lock, 0);
  }
}

__global__ void __launch_bounds__(kArenaThreads)
arena_allocate_kernel(void* storage, const int32_t* requested_bytes, const int32_t* item_count,
                      int item_bytes, int32_t* descriptor, int regions) {
  __shared__ int scratch[2];
  int32_t request = *requested_bytes;
  if (item_bytes != 0) request += *item_count * item_bytes;
  arena_allocate(arena_of(storage, regions), regions, request, descriptor, scratch);
}

// Return a region to the sorted free list, merging with its neighbours.  The caller holds
// the arena lock; `scratch` needs 2 ints.  Ends with every thread past a block barrier.
__device__ __forceinline__ void arena_free_locked(const Arena& a, int regions, int32_t* descriptor,
                                                  int32_t* status_out, int* scratch) {
  const int32_t offset = descriptor[0], size = descriptor[1];
  const bool valid = descriptor[2] == 0 && descriptor[3] == *a.generation && offset >= 0 && size > 0;
  const int count = *a.count;
  // Insert position = number of free regions that start below the freed one.
  if (threadIdx.x == 0) scratch[1] = 0;
  __syncthreads();
  int below = 0;
  for (int i = threadIdx.x; i < count; i += blockDim.x) below += a.starts[i] < offset ? 1 : 0;
  if (below) atomicAdd(&scratch[1], below);
  __syncthreads();
  const int insert = scratch[1];
  __syncthreads();
  bool merge_prev = false, merge_next = false;
  int32_t prev_size = 0, next_size = 0;
  if (valid) {
    if (insert > 0) {
      prev_size = a.sizes[insert - 1];
      merge_prev = a.starts[insert - 1] + prev_size == offset;
    }
    if (insert < count) {
      next_size = a.sizes[insert];
      merge_next = offset + size == a.starts[insert];
    }
  }
  __syncthreads();
  int status = valid ? 0 : 4;
  if (valid && merge_prev && merge_next) {
    if (threadIdx.x == 0) a.sizes[insert - 1] = prev_size + size + next_size;
    for (int base = insert; base + 1 < count; base += blockDim.x) {
      const int i = base + threadIdx.x;
      const bool move = i + 1 < count;
      int32_t ns = 0, nz = 0;
      if (move) { ns = a.starts[i + 1]; nz = a.sizes[i + 1]; }
      __syncthreads();
      if (move) { a.starts[i] = ns; a.sizes[i] = nz; }
      __syncthreads();
    }
    if (threadIdx.x == 0) *a.count = count - 1;
  } else if (valid && merge_prev) {
    if (threadIdx.x == 0) a.sizes[insert - 1] = prev_size + size;
  } else if (valid && merge_next) {
    if (threadIdx.x == 0) { a.starts[insert] = offset; a.sizes[insert] = next_size + size; }
  } else if (valid) {
    if (count >= regions) {
      status = 3;
    } else {
      // Open a slot: shift right from the top down, chunk by chunk.
      for (int top = count; top > insert; top -= blockDim.x) {
        const int i = top - 1 - (int)threadIdx.x;  // source index, moves to i + 1
        const bool move = i >= insert;
        int32_t ps = 0, pz = 0;
        if (move) { ps = a.starts[i]; pz = a.sizes[i]; }
        __syncthreads();
        if (move) { a.starts[i + 1] = ps; a.sizes[i + 1] = pz; }
        __syncthreads();
      }
      if (threadIdx.x == 0) {
        a.starts[insert] = offset;
        a.sizes[insert] = size;
        *a.count = count + 1;
      }
    }
  }
  if (threadIdx.x == 0) {
    if (status == 0) descriptor[2] = 5;
    *status_out = status;
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kArenaThreads)
arena_free_kernel(void* storage, int32_t* descriptor, int32_t* status_out, int regions) {
  __shared__ int scratch[2];
  const Arena a = arena_of(storage, regions);
  if (!arena_lock(a, scratch)) {
    if (threadIdx.x == 0) *status_out = kStatusLockTimeout;
    return;
  }
  arena_free_locked(a, regions, descriptor, status_out, scratch);
  arena_unlock(a);
}

// Many regions under one lock, in list order (the free list ends up as after one call each).
__global__ void __launch_bounds__(kArenaThreads)
arena_free_many_kernel(void* storage, int32_t* const* descriptors, int n, int32_t* status_out,
                       int regions) {
  __shared__ int scratch[2];
  const Arena a = arena_of(storage, regions);
  if (!arena_lock(a, scratch)) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) status_out[i] = kStatusLockTimeout;
    return;
  }
  for (int i = 0; i < n; ++i) arena_free_locked(a, regions, descriptors[i], status_out + i, scratch);
  arena_unlock(a);
}

// Exclusive scans of the per-block overflow counts and tail bytes, totals, and
// (for a shared arena) the reservation of this tensor's overflow region.
__global__ void __launch_bounds__(kScanThreads)
scan_allocate_kernel(int32_t* summaries, int32_t* counts, int32_t* descriptor, void* arena_storage,
                     int64_t blocks, int regions, int32_t* release_descriptor,
                     int32_t* release_status) {
  __shared__ int scratch[33];
  __shared__ int alloc_scratch[2];
  // The summaries come from the encoder in front of this kernel; the tail compaction behind
  // it may be scheduled now and waits for this kernel itself.
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  int running_count = 0, running_bytes = 0;
  for (int64_t base = 0; base < blocks; base += blockDim.x) {
    const int64_t i = base + threadIdx.x;
    const int c = i < blocks ? summaries[i] : 0;
    const int t = i < blocks ? summaries[blocks + i] : 0;
    int total_c, total_t;
    const int pc = block_exclusive_scan(c, scratch, &total_c);
    const int pt = block_exclusive_scan(t, scratch, &total_t);
    if (i < blocks) {
      summaries[2 * blocks + i] = running_count + pc;
      summaries[3 * blocks + i] = running_bytes + pt;
    }
    running_count += total_c;
    running_bytes += total_t;
  }
  if (threadIdx.x == 0) {
    counts[0] = running_count;
    counts[1] = running_bytes;
    counts[2] = 0;
    counts[3] = 0;
  }
  if (arena_storage != nullptr) {
    // Two metadata bytes per overflowing stream (lane, start) ahead of the tails.
    const Arena arena = arena_of(arena_storage, regions);
    const int32_t request = running_bytes + 2 * running_count;
    if (release_descriptor == nullptr) {
      arena_allocate(arena, regions, request, descriptor, alloc_scratch);
      return;
    }
    // An in-place update: the region of the value that was just replaced goes back after the
    // new one has been reserved (the order of a separate allocate and free), under one lock.
    if (!arena_lock(arena, alloc_scratch)) {
      arena_allocate_timed_out(arena, descriptor);
      if (threadIdx.x == 0) *release_status = kStatusLockTimeout;
      return;
    }
    arena_allocate_locked(arena, regions, request, descriptor, alloc_scratch);
    arena_free_locked(arena, regions, release_descriptor, release_status, alloc_scratch);
    arena_unlock(arena);
  }
}

// All jobs of a batch.  Phase 1: every warp takes jobs in turn and scans that
// job's block summaries with shuffles.  Phase 2: the reservations, strictly in
// job order, so the arena ends up exactly as after one call per job.  The lock
// is taken once and the free list is worked on in shared memory (one thread,
// no global round trips per job), then written back; arenas with more free-list
// slots than fit there take the per-job path.  Jobs without overflow get the
// "empty request" descriptor, which is what the allocator would have written.
constexpr int kListSlots = 1024;

template <typename Job>  // lct_encode_job or lct_update_job: size, first_block, counts, descriptor
__global__ void __launch_bounds__(kScanThreads)
scan_batch_kernel(const Job* __restrict__ jobs, int n_jobs, int32_t* summaries,
                  void* arena_storage, int regions, int block_symbols) {
  __shared__ int alloc_scratch[2];
  __shared__ int32_t list_starts[kListSlots], list_sizes[kListSlots];
  __shared__ int32_t job_request[kScanThreads], job_start[kScanThreads], job_size[kScanThreads];
  __shared__ int list_count;
  // Summaries come from the encoder in front; the compaction behind may be scheduled now.
  cudaGridDependencySynchronize();
  cudaTriggerProgrammaticLaunchCompletion();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  for (int j = warp; j < n_jobs; j += warps) {
    const Job& job = jobs[j];
    const int64_t blocks = job.size / block_symbols;
    int32_t* rows = summaries + 4 * job.first_block;
    int running_count = 0, running_bytes = 0;
    for (int64_t base = 0; base < blocks; base += 32) {
      const int64_t i = base + lane;
      const int c = i < blocks ? rows[i] : 0;
      const int t = i < blocks ? rows[blocks + i] : 0;
      int ic = c, it = t;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int uc = __shfl_up_sync(0xFFFFFFFFu, ic, d), ut = __shfl_up_sync(0xFFFFFFFFu, it, d);
        if (lane >= d) { ic += uc; it += ut; }
      }
      if (i < blocks) {
        rows[2 * blocks + i] = running_count + ic - c;
        rows[3 * blocks + i] = running_bytes + it - t;
      }
      running_count += __shfl_sync(0xFFFFFFFFu, ic, 31);
      running_bytes += __shfl_sync(0xFFFFFFFFu, it, 31);
    }
    if (lane == 0) {
      job.counts[0] = running_count;
      job.counts[1] = running_bytes;
      job.counts[2] = 0;
      job.counts[3] = 0;
    }
  }
  __threadfence_block();
  __syncthreads();
  const Arena arena = arena_of(arena_storage, regions);
  if (regions > kListSlots) {
    for (int j = 0; j < n_jobs; ++j) {
      const Job& job = jobs[j];
      const int32_t request = job.counts[1] + 2 * job.counts[0];  // uniform across the CTA
      if (request > 0) {
        arena_allocate(arena, regions, request, job.descriptor, alloc_scratch);
        __syncthreads();
      } else if (threadIdx.x == 0) {
        job.descriptor[0] = -1;
        job.descriptor[1] = 0;
        job.descriptor[2] = 2;
        job.descriptor[3] = *arena.generation;
      }
    }
    return;
  }
  const int32_t generation = *arena.generation;
  const bool locked = arena_lock(arena, alloc_scratch);
  const int first_count = locked ? *arena.count : 0;
  for (int i = threadIdx.x; i < first_count; i += blockDim.x) {
    list_starts[i] = arena.starts[i];
    list_sizes[i] = arena.sizes[i];
  }
  if (threadIdx.x == 0) list_count = first_count;
  for (int base = 0; base < n_jobs; base += blockDim.x) {
    const int j = base + threadIdx.x;
    if (j < n_jobs) job_request[threadIdx.x] = jobs[j].counts[1] + 2 * jobs[j].counts[0];
    __syncthreads();
    if (threadIdx.x == 0) {
      int count = list_count;
      const int chunk = min((int)blockDim.x, n_jobs - base);
      for (int k = 0; k < chunk; ++k) {
        const int32_t request = job_request[k];
        int32_t start = -1, size = 0;
        if (request > 0 && locked) {
          const int32_t wanted = (request + 15) / 16 * 16;
          int slot = 0;
          while (slot < count && list_sizes[slot] < wanted) ++slot;
          if (slot < count) {
            start = list_starts[slot];
            size = wanted;
            if (list_sizes[slot] == wanted) {  // exact fit: the region disappears
              for (int i = slot; i + 1 < count; ++i) {
                list_starts[i] = list_starts[i + 1];
                list_sizes[i] = list_sizes[i + 1];
              }
              --count;
            } else {
              list_starts[slot] = start + wanted;
              list_sizes[slot] -= wanted;
            }
          }
        }
        job_start[k] = start;
        job_size[k] = size;
      }
      list_count = count;
    }
    __syncthreads();
    if (j < n_jobs) {
      const int32_t request = job_request[threadIdx.x];
      int32_t* descriptor = jobs[j].descriptor;
      descriptor[0] = job_start[threadIdx.x];
      descriptor[1] = job_size[threadIdx.x];
      descriptor[2] = request <= 0 ? 2
                      : !locked    ? kStatusLockTimeout
                                   : (job_start[threadIdx.x] >= 0 ? 0 : 1);
      descriptor[3] = generation;
    }
    __syncthreads();
  }
  if (!locked) return;
  // Slots that left the list keep their last contents, as after per-job calls.
  for (int i = threadIdx.x; i < first_count; i += blockDim.x) {
    arena.starts[i] = list_starts[i];
    arena.sizes[i] = list_sizes[i];
  }
  if (threadIdx.x == 0) *arena.count = list_count;
  arena_unlock(arena);
}

int launch_scan_allocate(int32_t* summaries, int32_t* counts, int32_t* descriptor,
                         void* arena_storage, int64_t blocks, int max_free_regions,
                         bool overlapped, cudaStream_t stream, int32_t* release_descriptor,
                         int32_t* release_status) {
  if (release_descriptor != nullptr && (arena_storage == nullptr || release_status == nullptr))
    return LCT_E_NULL_POINTER;
  if (overlapped)
    return launch_overlapped(scan_allocate_kernel, 1, kScanThreads, 0, stream, summaries, counts,
                             descriptor, arena_storage, blocks, max_free_regions,
                             release_descriptor, release_status);
  scan_allocate_kernel<<<1, kScanThreads, 0, stream>>>(summaries, counts, descriptor, arena_storage,
                                                       blocks, max_free_regions,
                                                       release_descriptor, release_status);
  return (int)cudaGetLastError();
}

int launch_scan_batch(const lct_encode_job* jobs, int n_jobs, int32_t* summaries,
                      void* arena_storage, int max_free_regions, int block_symbols,
                      cudaStream_t stream) {
  return launch_overlapped(scan_batch_kernel<lct_encode_job>, 1, kScanThreads, 0, stream, jobs,
                           n_jobs, summaries, arena_storage, max_free_regions, block_symbols);
}

int launch_scan_batch(const lct_update_job* jobs, int n_jobs, int32_t* summaries,
                      void* arena_storage, int max_free_regions, int block_symbols,
                      cudaStream_t stream) {
  return launch_overlapped(scan_batch_kernel<lct_update_job>, 1, kScanThreads, 0, stream, jobs,
                           n_jobs, summaries, arena_storage, max_free_regions, block_symbols);
}

}  // namespace lct

extern "C" {

static bool power_of_two(int v) { return v > 0 && (v & (v - 1)) == 0; }

int lct_buffer_reset(void* storage, int max_free_regions, int32_t capacity_bytes, void* stream) {
  if (storage == nullptr) return LCT_E_NULL_POINTER;
  if (!power_of_two(max_free_regions) || capacity_bytes < 0) return LCT_E_BAD_ARGUMENT;
  lct::arena_reset_kernel<<<1, lct::kArenaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      storage, max_free_regions, capacity_bytes);
  return (int)cudaGetLastError();
}

int lct_buffer_allocate(void* storage, const int32_t* requested_bytes, const int32_t* item_count,
                        int item_bytes, int32_t* descriptor, int max_free_regions, void* stream) {
  if (storage == nullptr || requested_bytes == nullptr || descriptor == nullptr)
    return LCT_E_NULL_POINTER;
  if (item_bytes != 0 && item_count == nullptr) return LCT_E_NULL_POINTER;
  if (!power_of_two(max_free_regions) || item_bytes < 0) return LCT_E_BAD_ARGUMENT;
  lct::arena_allocate_kernel<<<1, lct::kArenaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      storage, requested_bytes, item_count, item_bytes, descriptor, max_free_regions);
  return (int)cudaGetLastError();
}

int lct_buffer_free(void* storage, int32_t* descriptor, int32_t* status, int max_free_regions,
                    void* stream) {
  if (storage == nullptr || descriptor == nullptr || status == nullptr) return LCT_E_NULL_POINTER;
  if (!power_of_two(max_free_regions)) return LCT_E_BAD_ARGUMENT;
  lct::arena_free_kernel<<<1, lct::kArenaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      storage, descriptor, status, max_free_regions);
  return (int)cudaGetLastError();
}

int lct_buffer_free_many(void* storage, int32_t* const* descriptors, int n, int32_t* status,
                         int max_free_regions, void* stream) {
  if (storage == nullptr || descriptors == nullptr || status == nullptr) return LCT_E_NULL_POINTER;
  if (!power_of_two(max_free_regions) || n <= 0) return LCT_E_BAD_ARGUMENT;
  lct::arena_free_many_kernel<<<1, lct::kArenaThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      storage, descriptors, n, status, max_free_regions);
  return (int)cudaGetLastError();
}

int lct_scan_allocate(int32_t* summaries, int32_t* counts, int32_t* descriptor,
                      void* arena_storage, int64_t blocks, int max_free_regions, void* stream) {
  if (summaries == nullptr || counts == nullptr) return LCT_E_NULL_POINTER;
  if (arena_storage != nullptr && descriptor == nullptr) return LCT_E_NULL_POINTER;
  if (blocks < 0) return LCT_E_BAD_ARGUMENT;
  if (arena_storage != nullptr && !power_of_two(max_free_regions)) return LCT_E_BAD_ARGUMENT;
  return lct::launch_scan_allocate(summaries, counts, descriptor, arena_storage, blocks,
                                   max_free_regions, false, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
