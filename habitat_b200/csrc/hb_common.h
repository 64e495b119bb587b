// Shared host-side helpers of the library: error text, CUDA call checking.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <mutex>

#include "habitat_b200.h"

namespace hb {

// Records the message hb_last_error() returns on this thread.
void set_error(const char* fmt, ...);

inline hb_status cuda_fail(cudaError_t e, const char* what) {
  set_error("%s: %s", what, cudaGetErrorString(e));
  return HB_ERR_CUDA;
}

}  // namespace hb

// ---------------------------------------------------------------------------
// Staging for the `_host` entry points: one device block per GPU that only ever
// grows, and one non-blocking stream per GPU, both kept for the life of the
// process.  A `_host` call holds the arena's mutex from its first copy to its
// final synchronise, so calls on one GPU run one after the other and the block
// can be re-carved (and, when too small, replaced) without anything in flight.
// ---------------------------------------------------------------------------
namespace hb {
struct HostArena {
  std::mutex mu;
  void* base = nullptr;
  size_t bytes = 0;
  cudaStream_t stream = nullptr;
};
// The arena of the current CUDA device (created, with its stream, on first use).
hb_status arena_for_current_device(HostArena** out);
// Makes the block at least `bytes` large.  Call with the arena's mutex held.
hb_status arena_reserve(HostArena* arena, size_t bytes);

// Hands out 256-byte aligned pieces of a block; with a null base it only adds up sizes.
class Carver {
 public:
  explicit Carver(void* base) : base_(static_cast<uint8_t*>(base)) {}
  template <typename T>
  T* take(size_t count) {
    const size_t at = off_;
    off_ += (count * sizeof(T) + 255) & ~static_cast<size_t>(255);
    return base_ ? reinterpret_cast<T*>(base_ + at) : nullptr;
  }
  size_t used() const { return off_; }

 private:
  uint8_t* base_;
  size_t off_ = 0;
};
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

// The same with the grid's blocks grouped into thread-block clusters of `cluster_x` consecutive
// blocks (grid.x must be a multiple of it); cluster_x == 1 is the plain launch above.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_overlapped_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, unsigned cluster_x,
                                             cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  if (overlapped_launch_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
}  // namespace hb
#endif
