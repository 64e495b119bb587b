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

// ---------------------------------------------------------------------------
// Programmatic dependent launch.  A kernel launched through hb::launch_overlapped
// may be scheduled while the kernel before it on the stream is still draining;
// its first statement must be hb_grid_dependency_wait(), which returns once that
// kernel has completed and its writes are visible, so the data dependences are
// those of an ordinary launch and only the launch latency and the block
// scheduling overlap.  Kernels that call hb_grid_dependency_wait() also allow the
// kernel after them to be scheduled early.  Set HB_NO_OVERLAPPED_LAUNCH=1 to
// launch the ordinary way.
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)
__device__ __forceinline__ void hb_grid_dependency_wait() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

namespace hb {
bool overlapped_launch_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlapped_launch_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace hb
#endif
