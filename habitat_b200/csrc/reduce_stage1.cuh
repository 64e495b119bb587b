// First stage of the two-stage float64 sums, shared by reduce.cu (local totals) and
// peer_exchange.cu (totals exchanged between GPUs): a fixed number of blocks, each summing a fixed
// contiguous chunk with a fixed assignment of elements to lanes and a fixed reduction tree, so the
// result does not depend on scheduling (no floating-point atomics) and is the same bits in both files.
#pragma once

#include <cooperative_groups.h>

#include "hb_common.h"

namespace {

constexpr int kSumThreads = 256;

__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xFFFFFFFFu, v, o);
  return v;
}

// Block-wide sum of one value per thread (blocks of 32..1024 threads); valid in thread 0.
__device__ __forceinline__ double block_sum(double v) {
  __shared__ double s[32];
  v = warp_sum(v);
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = v;
  __syncthreads();
  double t = 0.0;
  if (threadIdx.x < 32) {
    t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.0;
    t = warp_sum(t);
  }
  __syncthreads();
  return t;
}

// This thread's share of the `per_plane` first-stage sums of one plane: elements threadIdx.x,
// threadIdx.x + blockDim.x, ... in eight interleaved accumulators, eight loads in flight (a
// fixed assignment for a given block size, so the value does not depend on scheduling).  With
// per_plane <= blockDim.x it is the thread's own element.
__device__ __forceinline__ double partials_share(const double* __restrict__ q, int per_plane) {
  // eight ways: sixteen measured slower (accumulators plus loads in flight no longer fit the
  // 64 registers a thread of a 1024-thread block may have)
  constexpr int kWays = 8;
  double a[kWays];
#pragma unroll
  for (int u = 0; u < kWays; ++u) a[u] = 0.0;
  const int n = blockDim.x;
  int i = threadIdx.x;
  for (; i + (kWays - 1) * n < per_plane; i += kWays * n) {
#pragma unroll
    for (int u = 0; u < kWays; ++u) a[u] += q[i + u * n];
  }
#pragma unroll
  for (int u = 0; u < kWays - 1; ++u)
    if (i + u * n < per_plane) a[u] += q[i + u * n];
#pragma unroll
  for (int w = kWays / 2; w > 0; w >>= 1) {
#pragma unroll
    for (int u = 0; u < w; ++u) a[u] += a[u + w];
  }
  return a[0];
}

// Threads per block of a final stage over `per_plane` first-stage sums: the plane sums' own 256
// first-stage sums keep the block size their results were defined with; long lists (one sum per
// block of the wave-scaling kernel) get 1024 threads so that more loads are in flight, and very
// long ones a cluster of blocks per plane, each block adding one contiguous part of the list.
constexpr int kFinalThreadsMax = 1024;
constexpr int kFinalCluster = 8;
inline int final_threads(int per_plane) { return per_plane > 2 * kSumThreads ? kFinalThreadsMax : kSumThreads; }
inline int final_cluster(int per_plane) { return per_plane > 8 * kFinalThreadsMax ? kFinalCluster : 1; }

// Sum of the `per_plane` first-stage sums of plane blockIdx.x / CLUSTER, formed by the CLUSTER
// consecutive blocks that share the plane; valid in thread 0 of the first of them.  With
// CLUSTER > 1 the kernel must have been launched with that cluster dimension: block r adds part r
// of the list, stores its sum into slot r of the first block's shared memory, and the first block
// adds the slots in order, so the result is fixed by (per_plane, block size, CLUSTER).  The
// one-block form is an instantiation of its own: kernels that contain cluster code launched
// measurably slower (≈ 0.8 µs) even when they were not launched as clusters.
template <int CLUSTER>
__device__ __forceinline__ double plane_total(const double* __restrict__ partial, int per_plane) {
  constexpr int cluster = CLUSTER;
  const int plane = blockIdx.x / cluster, r = blockIdx.x % cluster;
  const int part = (per_plane + cluster - 1) / cluster;
  const int lo = r * part < per_plane ? r * part : per_plane;
  const int hi = lo + part < per_plane ? lo + part : per_plane;
  const double t = block_sum(partials_share(partial + static_cast<size_t>(plane) * per_plane + lo, hi - lo));
  if (cluster == 1) return t;
  __shared__ double slots[kFinalCluster];
  cooperative_groups::cluster_group c = cooperative_groups::this_cluster();
  c.sync();                                   // every block of the cluster runs: its shared memory may be written
  if (threadIdx.x == 0) c.map_shared_rank(slots, 0)[r] = t;
  c.sync();                                   // the slots are visible to the first block
  double total = 0.0;
  if (r == 0 && threadIdx.x == 0)
    for (int q = 0; q < cluster; ++q) total += slots[q];
  return total;
}

// Stage 1 of the plane sum: a fixed number of blocks per plane, each summing a
// fixed contiguous chunk; NaN entries (pairs the reference raises on) skipped.
constexpr int kPlaneBlocks = 256;

__global__ void __launch_bounds__(kSumThreads)
plane_partial_kernel(const float* __restrict__ values, int64_t plane_len,
                     double* __restrict__ partial) {
  hb_grid_dependency_wait();
  const int plane = blockIdx.x;     // grid (planes, chunks): the planes' ends are visited together
  const float* v = values + static_cast<int64_t>(plane) * plane_len;
  // Blocks take the chunks from the end of the plane backwards: the kernel that has just written the
  // plane wrote its end last, so that part is the likeliest to be still in L2.  The partial sum of a
  // chunk lands in the chunk's own slot, so the result does not depend on this order.
  const int chunk_id = kPlaneBlocks - 1 - static_cast<int>(blockIdx.y);
  const int64_t chunk = (plane_len + kPlaneBlocks - 1) / kPlaneBlocks;
  const int64_t lo = static_cast<int64_t>(chunk_id) * chunk;
  const int64_t hi = lo + chunk < plane_len ? lo + chunk : plane_len;
  // The bulk of a chunk goes through 16-byte loads with four independent accumulators (the
  // assignment of elements to accumulators is fixed, so the result is the same for every launch);
  // the ragged edges of a chunk are taken one element at a time.
  double acc = 0.0;
  int64_t head = lo;
  while (head < hi && (reinterpret_cast<uintptr_t>(v + head) & 15) != 0) ++head;
  const int64_t n4 = (hi - head) / 4;
  for (int64_t i = lo + threadIdx.x; i < head; i += kSumThreads) {
    const float x = v[i];
    if (x == x) acc += static_cast<double>(x);
  }
  double a0 = 0.0, a1 = 0.0, a2 = 0.0, a3 = 0.0;
  const float4* v4 = reinterpret_cast<const float4*>(v + head);
#pragma unroll 4
  for (int64_t i = threadIdx.x; i < n4; i += kSumThreads) {   // several 16-byte loads in flight per thread
    const float4 x = v4[i];
    if (x.x == x.x) a0 += static_cast<double>(x.x);
    if (x.y == x.y) a1 += static_cast<double>(x.y);
    if (x.z == x.z) a2 += static_cast<double>(x.z);
    if (x.w == x.w) a3 += static_cast<double>(x.w);
  }
  acc += (a0 + a1) + (a2 + a3);
  for (int64_t i = head + 4 * n4 + threadIdx.x; i < hi; i += kSumThreads) {
    const float x = v[i];
    if (x == x) acc += static_cast<double>(x);
  }
  const double t = block_sum(acc);
  if (threadIdx.x == 0) partial[plane * kPlaneBlocks + chunk_id] = t;
}

// Stage 1 of the group sum: values carry a small group key each (the device row of an MLP
// query); a block sums a fixed contiguous chunk into one accumulator per group.  Keys at or
// above n_groups and NaN values are skipped.
constexpr int kGroupBlocks = 256;
constexpr int kMaxGroups = 8;     // groups per pass; more groups take more passes

__global__ void __launch_bounds__(kSumThreads)
group_partial_kernel(const float* __restrict__ values, const uint8_t* __restrict__ keys, int64_t n,
                     int32_t group0, int32_t n_groups, double* __restrict__ partial) {
  hb_grid_dependency_wait();
  const int64_t chunk = (n + kGroupBlocks - 1) / kGroupBlocks;
  const int64_t lo = static_cast<int64_t>(blockIdx.x) * chunk;
  const int64_t hi = lo + chunk < n ? lo + chunk : n;
  double acc[kMaxGroups];
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g) acc[g] = 0.0;
  for (int64_t i = lo + threadIdx.x; i < hi; i += kSumThreads) {
    const float x = values[i];
    const int key = static_cast<int>(keys[i]) - group0;
    const double v = x == x ? static_cast<double>(x) : 0.0;
#pragma unroll
    for (int g = 0; g < kMaxGroups; ++g) acc[g] += key == g ? v : 0.0;
  }
#pragma unroll
  for (int g = 0; g < kMaxGroups; ++g) {
    const double t = block_sum(acc[g]);
    if (threadIdx.x == 0 && g < n_groups) partial[g * kGroupBlocks + blockIdx.x] = t;
  }
}

}  // namespace
