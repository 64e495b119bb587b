// Trace-level totals and the special-operation ratio: small reduction and
// elementwise kernels that follow the two big ones on the same stream.
//
// hb_segment_sum stands in for Trace.run_time_ms / RunTimePrediction.run_time_ms
// (analyzer/habitat/analysis/trace.py:26-36, run_time.py:49-58) over many
// segments at once; hb_special_scale for the last line of
// Predictor._{conv2d,linear,bmm,lstm}_scale and the clamp in _special_scale
// (analysis/predictor.py:132-148, :182).
//
// Sums are accumulated in float64 with a fixed assignment of elements to lanes
// and a fixed reduction tree, so the result does not depend on grid size or
// scheduling (no floating-point atomics).
#include <mutex>

#include "hb_common.h"
#include "reduce_stage1.cuh"

namespace {

// One block per segment.
__global__ void __launch_bounds__(kSumThreads)
segment_sum_kernel(const float* __restrict__ values, const int64_t* __restrict__ offsets,
                   int64_t n_segments, double* __restrict__ out) {
  for (int64_t s = blockIdx.x; s < n_segments; s += gridDim.x) {
    const int64_t lo = offsets[s], hi = offsets[s + 1];
    double acc = 0.0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kSumThreads) acc += static_cast<double>(values[i]);
    const double t = block_sum(acc);
    if (threadIdx.x == 0) out[s] = t;
  }
}

template <int CLUSTER>
__global__ void __launch_bounds__(kFinalThreadsMax)
plane_final_kernel(const double* __restrict__ partial, int per_plane, double* __restrict__ out) {
  hb_grid_dependency_wait();
  const double t = plane_total<CLUSTER>(partial, per_plane);
  if (threadIdx.x == 0 && blockIdx.x % CLUSTER == 0) out[blockIdx.x / CLUSTER] = t;
}

__global__ void __launch_bounds__(256)
special_scale_kernel(const float* __restrict__ run_time_ms, const float* __restrict__ pred_dest,
                     const float* __restrict__ pred_orig, int64_t n, float* __restrict__ out_ms,
                     uint32_t* __restrict__ negative_count) {
  const int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  bool neg = false;
  if (i < n) {
    // predictor.py:182: run_time_ms * pred_dest / pred_orig, left to right
    // (float64 there; the two predictions are float32 values)
    double v = static_cast<double>(run_time_ms[i]) * static_cast<double>(pred_dest[i]) /
               static_cast<double>(pred_orig[i]);
    neg = v < 0;
    if (neg) v = 0.0;  // predictor.py:135-141
    out_ms[i] = static_cast<float>(v);
  }
  if (negative_count) {
    const unsigned m = __ballot_sync(0xFFFFFFFFu, neg);
    if ((threadIdx.x & 31) == 0 && m) atomicAdd(negative_count, __popc(m));
  }
}

// Per-GPU scratch of the two-stage sums.  A buffer that a launch may still be reading (or
// that a captured graph refers to) is never freed: when more room is needed a larger buffer
// is allocated and the old one is kept until the process ends.
constexpr int kMaxCudaDevices = 64;
struct SumScratch {
  double* plane = nullptr;      // [planes][kPlaneBlocks]
  size_t planes = 0;
  double* group = nullptr;      // [kMaxGroups][kGroupBlocks]
};
SumScratch g_scratch[kMaxCudaDevices];
std::mutex g_scratch_mu;

// Scratch of the current GPU with room for `planes` plane sums (0: leave as is) and, when
// `want_group`, for the group sum.  Allocates on the first call that needs more.
hb_status scratch_for_current_device(size_t planes, bool want_group, SumScratch* out) {
  int dev = 0;
  HB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxCudaDevices) {
    hb::set_error("device ordinal %d out of range", dev);
    return HB_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  SumScratch& sc = g_scratch[dev];
  if (planes > sc.planes) {
    // at least 64 planes, then doubling: a handful of allocations over the life of the process
    size_t want = sc.planes ? sc.planes : 64;
    while (want < planes) want *= 2;
    double* fresh = nullptr;
    HB_CUDA_TRY(cudaMalloc(&fresh, sizeof(double) * kPlaneBlocks * want));
    sc.plane = fresh;   // the previous buffer stays allocated: launches in flight and graphs may hold it
    sc.planes = want;
  }
  if (want_group && !sc.group) HB_CUDA_TRY(cudaMalloc(&sc.group, sizeof(double) * kMaxGroups * kGroupBlocks));
  *out = sc;
  return HB_OK;
}

}  // namespace

// Current size, in planes, of the plane-sum scratch of CUDA device `device` (0: none yet).
// For tests of the per-GPU bookkeeping; no reference counterpart.
extern "C" int64_t hb_plane_sum_scratch_planes(int32_t device) {
  if (device < 0 || device >= kMaxCudaDevices) return -1;
  std::lock_guard<std::mutex> lock(g_scratch_mu);
  return static_cast<int64_t>(g_scratch[device].planes);
}

extern "C" hb_status hb_segment_sum(const float* values, const int64_t* offsets,
                                    int64_t n_segments, double* out, void* stream) {
  if (n_segments < 0 || (n_segments > 0 && (!values || !offsets || !out))) {
    hb::set_error("hb_segment_sum: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n_segments == 0) return HB_OK;
  const int64_t blocks = n_segments < 148 * 8 * 8 ? n_segments : 148 * 8 * 8;
  segment_sum_kernel<<<static_cast<unsigned>(blocks), kSumThreads, 0,
                       static_cast<cudaStream_t>(stream)>>>(values, offsets, n_segments, out);
  HB_CUDA_TRY(cudaGetLastError());
  return HB_OK;
}

extern "C" hb_status hb_plane_sum(const float* values, int64_t plane_len, int32_t n_planes,
                                  double* out, void* stream) {
  if (plane_len < 0 || n_planes < 0 || n_planes > 65535 || (n_planes > 0 && (!values || !out))) {
    hb::set_error("hb_plane_sum: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n_planes == 0) return HB_OK;
  SumScratch sc;
  const hb_status st = scratch_for_current_device(static_cast<size_t>(n_planes), false, &sc);
  if (st != HB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  HB_CUDA_TRY(hb::launch_overlapped(plane_partial_kernel, dim3(n_planes, kPlaneBlocks), dim3(kSumThreads), 0, s,
                                    values, plane_len, sc.plane));
  HB_CUDA_TRY(hb::launch_overlapped(plane_final_kernel<1>, dim3(n_planes), dim3(kSumThreads), 0, s,
                                    static_cast<const double*>(sc.plane), kPlaneBlocks, out));
  return HB_OK;
}

extern "C" hb_status hb_partials_sum(const double* partials, int32_t per_plane, int32_t n_planes, double* out,
                                     void* stream) {
  if (per_plane < 0 || n_planes < 0 || n_planes > 65535 || (n_planes > 0 && (!out || (per_plane > 0 && !partials)))) {
    hb::set_error("hb_partials_sum: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n_planes == 0) return HB_OK;
  if (final_cluster(per_plane) == 1) {
    HB_CUDA_TRY(hb::launch_overlapped(plane_final_kernel<1>, dim3(n_planes), dim3(final_threads(per_plane)), 0,
                                      static_cast<cudaStream_t>(stream), partials, per_plane, out));
  } else {
    HB_CUDA_TRY(hb::launch_overlapped_cluster(plane_final_kernel<kFinalCluster>, dim3(n_planes * kFinalCluster),
                                              dim3(kFinalThreadsMax), kFinalCluster,
                                              static_cast<cudaStream_t>(stream), partials, per_plane, out));
  }
  return HB_OK;
}

extern "C" hb_status hb_group_sum(const float* values, const uint8_t* keys, int64_t n, int32_t n_groups,
                                  double* out, void* stream) {
  if (n < 0 || n_groups < 0 || n_groups > 256 || (n_groups > 0 && !out) || (n > 0 && (!values || !keys))) {
    hb::set_error("hb_group_sum: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n_groups == 0) return HB_OK;
  SumScratch sc;
  const hb_status st = scratch_for_current_device(0, true, &sc);
  if (st != HB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // eight groups per pass; the passes share the scratch and follow one another on the stream
  for (int32_t g0 = 0; g0 < n_groups; g0 += kMaxGroups) {
    const int32_t ng = n_groups - g0 < kMaxGroups ? n_groups - g0 : kMaxGroups;
    HB_CUDA_TRY(hb::launch_overlapped(group_partial_kernel, dim3(kGroupBlocks), dim3(kSumThreads), 0, s, values,
                                      keys, n, g0, ng, sc.group));
    static_assert(kGroupBlocks == kPlaneBlocks, "the final stage is shared with the plane sum");
    HB_CUDA_TRY(hb::launch_overlapped(plane_final_kernel<1>, dim3(ng), dim3(kSumThreads), 0, s,
                                      static_cast<const double*>(sc.group), kGroupBlocks, out + g0));
  }
  return HB_OK;
}

extern "C" hb_status hb_special_scale(const float* run_time_ms, const float* pred_dest,
                                      const float* pred_orig, int64_t n, float* out_ms,
                                      uint32_t* negative_count, void* stream) {
  if (n < 0 || (n > 0 && (!run_time_ms || !pred_dest || !pred_orig || !out_ms))) {
    hb::set_error("hb_special_scale: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n == 0) return HB_OK;
  const int64_t blocks = (n + 255) / 256;
  special_scale_kernel<<<static_cast<unsigned>(blocks), 256, 0,
                         static_cast<cudaStream_t>(stream)>>>(run_time_ms, pred_dest, pred_orig, n,
                                                              out_ms, negative_count);
  HB_CUDA_TRY(cudaGetLastError());
  return HB_OK;
}

// ---------------------------------------------------------------------------
// Plane sums for callers that must not allocate
// ---------------------------------------------------------------------------
// hb_plane_sum above keeps its stage-1 partial sums in a buffer it obtains with
// cudaMalloc on first use.  Some hosts cannot tolerate that: a serving process
// that hands the whole device to its own memory pool at start-up (a later
// driver allocation fails or fragments the pool), or one whose latency rules
// forbid driver allocations once initialisation is over.  For them the same two
// kernels run on a scratch array that is part of the library image: it occupies
// kStaticPlanes * kPlaneBlocks * 8 bytes = 128 KB on every GPU that loads the
// library, from load until the process exits.
constexpr int kStaticPlanes = 64;
static __device__ __align__(256) double g_static_partial[kStaticPlanes * kPlaneBlocks];

namespace {
// Device address of g_static_partial on each device, resolved on first use.  In
// host code the symbol's name is only a handle for the runtime, not an address a
// kernel could dereference, hence the look-up.
double* g_static_partial_ptr[kMaxCudaDevices] = {};
}  // namespace

extern "C" hb_status hb_plane_sum_static(const float* values, int64_t plane_len, int32_t n_planes,
                                         double* out, void* stream) {
  if (plane_len < 0 || n_planes < 0 || (n_planes > 0 && (!values || !out))) {
    hb::set_error("hb_plane_sum_static: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n_planes > kStaticPlanes) {
    hb::set_error("hb_plane_sum_static: %d planes requested, the built-in scratch holds %d "
                  "(use hb_plane_sum, or split the call)", n_planes, kStaticPlanes);
    return HB_ERR_TOO_LARGE;
  }
  if (n_planes == 0) return HB_OK;
  int dev = 0;
  HB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxCudaDevices) {
    hb::set_error("hb_plane_sum_static: device ordinal %d out of range", dev);
    return HB_ERR_UNSUPPORTED;
  }
  if (!g_static_partial_ptr[dev]) {
    // once per device, with that device current
    void* ptr = nullptr;
    HB_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_static_partial));
    g_static_partial_ptr[dev] = static_cast<double*>(ptr);
  }
  double* scratch = g_static_partial_ptr[dev];
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // Stage 1 writes every partial that stage 2 reads, so nothing in the scratch
  // has to start at zero; whatever the previous call left there is overwritten.
  plane_partial_kernel<<<dim3(n_planes, kPlaneBlocks), kSumThreads, 0, s>>>(values, plane_len, scratch);
  HB_CUDA_TRY(cudaGetLastError());
  plane_final_kernel<1><<<n_planes, kSumThreads, 0, s>>>(scratch, kPlaneBlocks, out);
  HB_CUDA_TRY(cudaGetLastError());
  return HB_OK;
}
