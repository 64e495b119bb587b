// Test-only: compiles the library's device occupancy code (occupancy.cuh) for the
// host so that its integer logic can be checked against the oracle without a GPU.
// Not part of the product library.
#include "occupancy.cuh"

extern "C" void harness_occupancy(const hb_device_spec* spec, long n, const int* block,
                                  const int* smem, const int* regs, int* occ, int* limits) {
  const hb_dev_pre pre = hb_fold_device(*spec);
  for (long i = 0; i < n; ++i) occ[i] = hb_occupancy(pre, block[i], smem[i], regs[i], limits + 4 * i);
}
