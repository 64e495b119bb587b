// C-ABI window onto the CUDA toolkit's cuda_occupancy.h -- TEST INFRASTRUCTURE ONLY.
//
// The header vendored by the reference rejects compute capability >= 8, so for
// those device rows the oracle is checked against the toolkit's newer header
// under the very same call convention Habitat uses
// (cpp/src/cuda/kernel.cpp:33-56: default device state, default-constructed
// function attributes with unlimited block size and dynamic shared memory),
// plus the reservedSharedMemPerBlock device field that header adds.
#include <climits>
#include <cstdint>
#include <cstring>

namespace tk_occ {
#include <cuda_occupancy.h>
}

extern "C" {

struct tk_device {
  int32_t compute_major, compute_minor, max_threads_per_block,
      max_threads_per_multiprocessor, regs_per_block, regs_per_multiprocessor,
      warp_size, shared_mem_per_block, shared_mem_per_multiprocessor, num_sms,
      shared_mem_per_block_optin, reserved_shared_mem_per_block,
      mem_bandwidth_gb, base_clock_mhz, peak_gflops_per_second;
};

void tk_header_limits_batch(const tk_device* d, int64_t n, const int32_t* block_size,
                            const int32_t* dynamic_smem, const int32_t* static_smem,
                            const int32_t* regs, int32_t* occ, int32_t* limits) {
  using namespace tk_occ;
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
  p.reservedSharedMemPerBlock = d->reserved_shared_mem_per_block;
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
