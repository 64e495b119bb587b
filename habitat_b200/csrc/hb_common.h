// Shared host-side helpers of the library: error text, CUDA call checking.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "habitat_b200.h"

namespace hb {

// Records the message hb_last_error() returns on this thread.
void set_error(const char* fmt, ...);

inline hb_status cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return HB_ERR_CUDA;
}

}  // namespace hb

#define HB_CUDA_TRY(expr)                                   \
  do {                                                      \
    cudaError_t hb_e_ = (expr);                             \
    if (hb_e_ != cudaSuccess) return hb::cuda_fail(hb_e_, #expr); \
  } while (0)
