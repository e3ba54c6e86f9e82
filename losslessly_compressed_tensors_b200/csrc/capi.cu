// Library identity and error text.
#include <cuda_runtime.h>

#include "common.cuh"
#include "lct_b200.h"

namespace lct {

static int g_lane_mask = 254;

int lane_mask_now() { return g_lane_mask; }

}  // namespace lct

extern "C" {

int lct_set_lane_mapping(int linear) {
  if (linear != 0 && linear != 1) return LCT_E_BAD_ARGUMENT;
  lct::g_lane_mask = linear ? 0 : 254;
  return 0;
}

int lct_get_lane_mapping(void) { return lct::g_lane_mask == 0 ? 1 : 0; }

const char* lct_version(void) { return "lct-b200 0.1.0 sm_100a"; }

const char* lct_error_string(int code) {
  switch (code) {
    case 0: return "success";
    case LCT_E_BAD_GEOMETRY: return "unsupported stream geometry";
    case LCT_E_NULL_POINTER: return "required pointer is null";
    case LCT_E_ALIGNMENT: return "buffer is not aligned as required";
    case LCT_E_BAD_ARGUMENT: return "argument out of range";
    case LCT_E_TOO_LARGE: return "tensor has too many blocks for one launch";
    case LCT_E_SCRATCH_LIMIT:
      return "tensor exceeds the built-in scratch of lct_encode_noalloc (1024 codec blocks)";
    default: break;
  }
  if (code > 0) return cudaGetErrorString(static_cast<cudaError_t>(code));
  return "unknown lct error";
}

}  // extern "C"
