// C-ABI window onto the reference's own occupancy code -- TEST INFRASTRUCTURE ONLY.
//
// Compiled together with the reference's cpp/src/cuda/kernel.cpp (from where it
// lies in the reference tree; nothing is copied) into oracle/_ref/.  The first
// entry point goes through habitat::cuda::KernelMetadata::threadBlockOccupancy
// (cpp/src/cuda/kernel.cpp:33-56); the second repeats that call convention on
// the reference's vendored cuda_occupancy.h to also read the four block limits
// the calculator reports (cpp/src/cuda/cuda_occupancy.h:1410-1413).
#include <climits>
#include <cstdint>
#include <cstring>

#include "cuda/kernel.h"

namespace ref_occ {
#include "cuda/cuda_occupancy.h"
}

extern "C" {

struct ref_device {
  int32_t compute_major, compute_minor, max_threads_per_block,
      max_threads_per_multiprocessor, regs_per_block, regs_per_multiprocessor,
      warp_size, shared_mem_per_block, shared_mem_per_multiprocessor, num_sms,
      shared_mem_per_block_optin, reserved_shared_mem_per_block,
      mem_bandwidth_gb, base_clock_mhz, peak_gflops_per_second;
};

static habitat::cuda::DeviceProperties to_props(const ref_device* d) {
  return habitat::cuda::DeviceProperties(
      "dev", d->compute_major, d->compute_minor, d->max_threads_per_block,
      d->max_threads_per_multiprocessor, d->regs_per_block,
      d->regs_per_multiprocessor, d->warp_size, d->shared_mem_per_block,
      d->shared_mem_per_multiprocessor, d->num_sms,
      d->shared_mem_per_block_optin, d->mem_bandwidth_gb, d->base_clock_mhz,
      d->peak_gflops_per_second);
}

uint32_t ref_thread_block_occupancy(const ref_device* d, int32_t block_size,
                                    int32_t dynamic_smem, int32_t static_smem,
                                    int32_t regs) {
  habitat::cuda::KernelMetadata k("k", 1, block_size, dynamic_smem, static_smem,
                                  static_cast<uint16_t>(regs));
  return k.threadBlockOccupancy(to_props(d), static_cast<uint16_t>(regs));
}

void ref_thread_block_occupancy_batch(const ref_device* d, int64_t n,
                                      const int32_t* block_size,
                                      const int32_t* dynamic_smem,
                                      const int32_t* static_smem,
                                      const int32_t* regs, uint32_t* out) {
  habitat::cuda::DeviceProperties props = to_props(d);
  for (int64_t i = 0; i < n; ++i) {
    habitat::cuda::KernelMetadata k("k", 1, block_size[i], dynamic_smem[i],
                                    static_smem[i],
                                    static_cast<uint16_t>(regs[i]));
    out[i] = k.threadBlockOccupancy(props, static_cast<uint16_t>(regs[i]));
  }
}

// Same convention, reference header, limits exposed: {regs, warps, blocks, smem}.
void ref_header_limits_batch(const ref_device* d, int64_t n,
                             const int32_t* block_size,
                             const int32_t* dynamic_smem,
                             const int32_t* static_smem, const int32_t* regs,
                             int32_t* occ, int32_t* limits) {
  using namespace ref_occ;
  cudaOccDeviceProp p;
  p.computeMajor = d->compute_major;
  p.computeMinor = d->compute_minor;
  p.maxThreadsPerBlock = d->max_threads_per_block;
  p.maxThreadsPerMultiprocessor = d->max_threads_per_multiprocessor;
  p.regsPerBlock = d->regs_per_block;
  p.regsPerMultiprocessor = d->regs_per_multiprocessor;
  p.warpSize = d->warp_size;
  p.sharedMemPerBlock = d->shared_mem_per_block;
  p.sharedMemPerMultiprocessor = d->shared_mem_per_multiprocessor;
  p.numSms = d->num_sms;
  p.sharedMemPerBlockOptin = d->shared_mem_per_block_optin;
  for (int64_t i = 0; i < n; ++i) {
    cudaOccDeviceState state;
    cudaOccFuncAttributes attr;
    attr.maxThreadsPerBlock = INT_MAX;
    attr.maxDynamicSharedSizeBytes = INT_MAX;
    attr.numRegs = static_cast<uint16_t>(regs[i]);
    attr.sharedSizeBytes = static_smem[i];
    cudaOccResult r;
    if (cudaOccMaxActiveBlocksPerMultiprocessor(&r, &p, &attr, &state, block_size[i],
                                                dynamic_smem[i]) != CUDA_OCC_SUCCESS) {
      occ[i] = 0;
      limits[4 * i] = limits[4 * i + 1] = limits[4 * i + 2] = limits[4 * i + 3] = 0;
    } else {
      occ[i] = r.activeBlocksPerMultiprocessor;
      limits[4 * i + 0] = r.blockLimitRegs;
      limits[4 * i + 1] = r.blockLimitWarps;
      limits[4 * i + 2] = r.blockLimitBlocks;
      limits[4 * i + 3] = r.blockLimitSharedMem;
    }
  }
}

}  // extern "C"
