// Test-only: compiles the library's device occupancy code (occupancy.cuh) for the
// host so that its integer logic can be checked against the oracle without a GPU.
// Not part of the product library.
#include <initializer_list>

#include "occupancy.cuh"

extern "C" void harness_occupancy(const hb_device_spec* spec, long n, const int* block,
                                  const int* smem, const int* regs, int* occ, int* limits) {
  const hb_dev_pre pre = hb_fold_device(*spec);
  for (long i = 0; i < n; ++i) occ[i] = hb_occupancy(pre, block[i], smem[i], regs[i], limits + 4 * i);
}

// The division-free form used by the fast kernel; returns -1 per sample when the
// row does not qualify for it.
extern "C" void harness_fast_occupancy(const hb_device_spec* spec, long n, const int* block,
                                       const int* smem, const int* regs, int* occ) {
  const hb_dev_pre pre = hb_fold_device(*spec);
  static uint32_t magic[kMagicN];
  for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
  if (!fast_row_ok(*spec, pre)) {
    for (long i = 0; i < n; ++i) occ[i] = -1;
    return;
  }
  const FastDev d = fold_fast(*spec, pre);
  for (long i = 0; i < n; ++i) {
    FastKernel k;
    k.block_size = block[i];
    k.wpb = (k.block_size + 31) >> 5;
    k.regs = regs[i];
    k.rpw_units = (k.regs + 7) >> 3;
    k.smem = smem[i];
    k.m_wpb = magic[k.wpb < kMagicN - 1 ? k.wpb : kMagicN - 1];
    const uint32_t m_rpw = magic[k.rpw_units < kMagicN - 1 ? k.rpw_units : kMagicN - 1];
    occ[i] = fast_occupancy(d, k, k.regs, k.rpw_units, m_rpw, magic);
  }
}

// Magic-number division self-check over a grid of operands.
extern "C" long harness_magic_errors(void) {
  long bad = 0;
  for (uint32_t d = 1; d < 5000; ++d) {
    const uint32_t M = magic_of(d);
    for (uint32_t n : {0u, 1u, d - 1, d, d + 1, 1000u, 65535u, 1u << 20, (1u << 20) + 77u,
                       0x7FFFFFFFu, 0x7FFFFFFEu, 123456789u}) {
      if (udiv_magic_fix(n, d, M) != n / d) ++bad;
      if (static_cast<uint64_t>(n) * d < (1ull << 32) && udiv_magic(n, d, M) != n / d) ++bad;
    }
  }
  return bad;
}
