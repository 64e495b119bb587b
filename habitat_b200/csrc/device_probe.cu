// Device description and peak-throughput probe for a row of the device table.
//
// Stands in for two offline tools of the reference: cpp/src/device_info.cpp:16-30, which
// prints the cudaDeviceProp fields a devices.yml row consists of, and the pair
// cpp/src/cuda/diagnostics.cu:9-15 + tools/device-metadata/measure_peak_flops.py:10-18, which
// estimate the single-precision peak from a profiled kernel of dependent additions and
// its reported efficiency.  No profiler is involved here: the probe runs eight independent
// fused multiply-add chains per thread, enough resident warps to hide the pipeline latency,
// and reports what it achieved (2 flops per FMA), best of several launches.
#include <algorithm>

#include "hb_common.h"

namespace {

constexpr int kChains = 8;
constexpr int kIters = 4096;

__global__ void __launch_bounds__(256) fma_probe_kernel(float* sink, float seed) {
  float a[kChains];
#pragma unroll
  for (int c = 0; c < kChains; ++c) a[c] = seed + static_cast<float>(threadIdx.x + c);
  const float m = 0.999f, b = 1e-3f;
  for (int i = 0; i < kIters; ++i) {
#pragma unroll
    for (int c = 0; c < kChains; ++c) a[c] = fmaf(a[c], m, b);
  }
  float s = 0.f;
#pragma unroll
  for (int c = 0; c < kChains; ++c) s += a[c];
  // never true for the seeds used; keeps the chains alive
  if (s == 12345.678f) sink[blockIdx.x * blockDim.x + threadIdx.x] = s;
}

}  // namespace

extern "C" hb_status hb_device_info(int32_t device, hb_device_spec* out) {
  if (!out) {
    hb::set_error("hb_device_info: out is NULL");
    return HB_ERR_INVALID_ARGUMENT;
  }
  auto attr = [&](cudaDeviceAttr a, int* v) { return cudaDeviceGetAttribute(v, a, device); };
  int major = 0, minor = 0, tpb = 0, tpm = 0, rpb = 0, rpm = 0, warp = 0, spb = 0, spm = 0, sms = 0,
      optin = 0, reserved = 0, mem_khz = 0, bus_bits = 0, clock_khz = 0;
  HB_CUDA_TRY(attr(cudaDevAttrComputeCapabilityMajor, &major));
  HB_CUDA_TRY(attr(cudaDevAttrComputeCapabilityMinor, &minor));
  HB_CUDA_TRY(attr(cudaDevAttrMaxThreadsPerBlock, &tpb));
  HB_CUDA_TRY(attr(cudaDevAttrMaxThreadsPerMultiProcessor, &tpm));
  HB_CUDA_TRY(attr(cudaDevAttrMaxRegistersPerBlock, &rpb));
  HB_CUDA_TRY(attr(cudaDevAttrMaxRegistersPerMultiprocessor, &rpm));
  HB_CUDA_TRY(attr(cudaDevAttrWarpSize, &warp));
  HB_CUDA_TRY(attr(cudaDevAttrMaxSharedMemoryPerBlock, &spb));
  HB_CUDA_TRY(attr(cudaDevAttrMaxSharedMemoryPerMultiprocessor, &spm));
  HB_CUDA_TRY(attr(cudaDevAttrMultiProcessorCount, &sms));
  HB_CUDA_TRY(attr(cudaDevAttrMaxSharedMemoryPerBlockOptin, &optin));
  HB_CUDA_TRY(attr(cudaDevAttrReservedSharedMemoryPerBlock, &reserved));
  HB_CUDA_TRY(attr(cudaDevAttrMemoryClockRate, &mem_khz));
  HB_CUDA_TRY(attr(cudaDevAttrGlobalMemoryBusWidth, &bus_bits));
  HB_CUDA_TRY(attr(cudaDevAttrClockRate, &clock_khz));
  hb_device_spec s{};
  s.compute_major = major;
  s.compute_minor = minor;
  s.max_threads_per_block = tpb;
  s.max_threads_per_multiprocessor = tpm;
  s.regs_per_block = rpb;
  s.regs_per_multiprocessor = rpm;
  s.warp_size = warp;
  s.shared_mem_per_block = spb;
  s.shared_mem_per_multiprocessor = spm;
  s.num_sms = sms;
  s.shared_mem_per_block_optin = optin;
  s.reserved_shared_mem_per_block = reserved;
  // double data rate: two transfers per memory clock
  s.mem_bandwidth_gb = static_cast<int32_t>(2.0 * mem_khz * 1e3 * (bus_bits / 8.0) / 1e9 + 0.5);
  s.base_clock_mhz = clock_khz / 1000;
  // nominal: one FMA per lane and clock, 128 lanes per SM on every architecture since 6.1 except 7.x (64)
  const int lanes = (major == 7 || (major == 6 && minor == 0)) ? 64 : 128;
  s.peak_gflops_per_second = static_cast<int32_t>(2.0 * lanes * sms * (clock_khz / 1e6) + 0.5);
  *out = s;
  return HB_OK;
}

extern "C" hb_status hb_peak_flops_test(int32_t trials, double* gflops_per_second, void* stream) {
  if (!gflops_per_second || trials < 1 || trials > 1000) {
    hb::set_error("hb_peak_flops_test: need 1..1000 trials and an output pointer");
    return HB_ERR_INVALID_ARGUMENT;
  }
  int dev = 0, sms = 0;
  HB_CUDA_TRY(cudaGetDevice(&dev));
  HB_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int blocks = sms * 8, threads = 256;
  float* sink = nullptr;
  HB_CUDA_TRY(cudaMalloc(&sink, sizeof(float) * blocks * threads));
  cudaEvent_t e0 = nullptr, e1 = nullptr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  hb_status st = HB_OK;
  double best = 0.0;
  do {
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) {
      st = hb::cuda_fail(cudaGetLastError(), "cudaEventCreate");
      break;
    }
    fma_probe_kernel<<<blocks, threads, 0, s>>>(sink, 0.5f);   // warm-up
    for (int t = 0; t < trials; ++t) {
      cudaEventRecord(e0, s);
      fma_probe_kernel<<<blocks, threads, 0, s>>>(sink, 0.5f + t);
      cudaEventRecord(e1, s);
      const cudaError_t e = cudaEventSynchronize(e1);
      if (e != cudaSuccess) { st = hb::cuda_fail(e, "fma_probe_kernel"); break; }
      float ms = 0.f;
      cudaEventElapsedTime(&ms, e0, e1);
      const double flops = 2.0 * kChains * kIters * static_cast<double>(blocks) * threads;
      if (ms > 0.f) best = std::max(best, flops / (ms * 1e-3) / 1e9);
    }
  } while (false);
  if (e0) cudaEventDestroy(e0);
  if (e1) cudaEventDestroy(e1);
  cudaFree(sink);
  if (st == HB_OK) *gflops_per_second = best;
  return st;
}
