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


// The table kernel's occupancy and wave-count arithmetic, evaluated on the host from the
// tables the library builds for a device row: occ = min(P[index], S[index]) and
// floor(nb / (SMs * occ)) = umulhi(nb, M) >> shift.  Returns 0 when the row cannot be tabulated.
extern "C" int harness_lut(const hb_device_spec* spec, long n, const int* block, const unsigned* smem,
                           const int* regs, const int* num_blocks, int* occ, unsigned* waves) {
  const hb_dev_pre pre = hb_fold_device(*spec);
  if (!lut_row_ok(*spec, pre)) return 0;
  static uint32_t magic[kMagicN];
  for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
  static uint8_t pt[kLutP], st[kLutS];
  static LutOcc tt[kLutOcc];
  build_row_lut(*spec, fold_fast(*spec, pre), pt, st, tt, magic);
  for (long i = 0; i < n; ++i) {
    const uint32_t bs = static_cast<uint32_t>(block[i]) & 0xFFFFu, rg = static_cast<uint32_t>(regs[i]) & 0xFFFFu;
    const uint32_t p = pt[lut_p_index(bs, rg)], s = st[lut_s_index(smem[i])];
    const uint32_t o = p < s ? p : s;
    occ[i] = static_cast<int>(o);
    const LutOcc& e = tt[o];
    waves[i] = o ? (hb_umulhi(static_cast<uint32_t>(num_blocks[i]), e.magic) >> e.shift) : 0xFFFFFFFFu;
  }
  return 1;
}

// The three tables of a device row as the library builds them: P [34 * 34] bytes, S [2048] bytes,
// T [33][4] 32-bit words {multiplier, shift, A_hi bits, A_lo bits}.  Returns 0 when the row cannot
// be tabulated.
extern "C" int harness_tables(const hb_device_spec* spec, unsigned char* p_out, unsigned char* s_out,
                              unsigned* t_out) {
  const hb_dev_pre pre = hb_fold_device(*spec);
  if (!lut_row_ok(*spec, pre)) return 0;
  uint32_t magic[kMagicN];
  for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
  LutOcc tt[kLutOcc];
  build_row_lut(*spec, fold_fast(*spec, pre), p_out, s_out, tt, magic);
  static_assert(sizeof(LutOcc) == 16, "four 32-bit words per entry");
  for (int i = 0; i < kLutOcc; ++i) {
    t_out[4 * i] = tt[i].magic;
    t_out[4 * i + 1] = tt[i].shift;
    float f[2] = {tt[i].lg_hi, tt[i].lg_lo};
    unsigned u[2];
    __builtin_memcpy(u, f, 8);
    t_out[4 * i + 2] = u[0];
    t_out[4 * i + 3] = u[1];
  }
  return 1;
}

#if defined(HARNESS_MAIN)
// Stand-alone self-check for sanitizer builds: fuzzed device rows and records through every
// code path above; any out-of-bounds table access or undefined arithmetic aborts the run.
#include <cstdio>
#include <random>
#include <vector>
int main() {
  std::mt19937 g(12345);
  auto pick = [&](std::initializer_list<int> v) { return *(v.begin() + g() % v.size()); };
  long checked = 0, mismatched = 0;
  for (int row = 0; row < 400; ++row) {
    hb_device_spec s{};
    s.compute_major = pick({3, 5, 6, 7, 8, 9, 10, 12});
    s.compute_minor = pick({0, 1, 2, 5, 6, 7, 9});
    s.max_threads_per_block = pick({512, 768, 1000, 1024});
    s.max_threads_per_multiprocessor = pick({1024, 1536, 2048});
    s.regs_per_block = pick({32768, 65536});
    s.regs_per_multiprocessor = pick({65536, 131072});
    s.warp_size = 32;
    s.shared_mem_per_block = pick({48 * 1024, 99 * 1024, 163 * 1024, 227 * 1024});
    s.shared_mem_per_multiprocessor = pick({64 * 1024, 96 * 1024, 100 * 1024, 164 * 1024, 228 * 1024});
    s.num_sms = 1 + static_cast<int>(g() % 300);
    s.reserved_shared_mem_per_block = s.compute_major >= 8 ? pick({0, 1024}) : 0;
    s.mem_bandwidth_gb = 900; s.base_clock_mhz = 1 + static_cast<int>(g() % 3000); s.peak_gflops_per_second = 15000;
    const int n = 2000;
    std::vector<int> block(n), regs(n), nb(n), occ(n), ref(n), lim(4 * n);
    std::vector<unsigned> smem(n), waves(n);
    std::vector<int> smem_i(n);
    for (int i = 0; i < n; ++i) {
      block[i] = static_cast<int>(g() % 1200);
      regs[i] = static_cast<int>(g() % 300);
      smem[i] = g() % 4 == 0 ? g() : g() % (240 * 1024);
      smem_i[i] = smem[i] > 0x7FFF0000u ? -1 : static_cast<int>(smem[i]);
      nb[i] = static_cast<int>(g() % 0x7FFFFFFFu) + 1;
    }
    harness_occupancy(&s, n, block.data(), smem_i.data(), regs.data(), ref.data(), lim.data());
    if (!harness_lut(&s, n, block.data(), smem.data(), regs.data(), nb.data(), occ.data(), waves.data())) continue;
    for (int i = 0; i < n; ++i) {
      ++checked;
      if (occ[i] != ref[i]) ++mismatched;
      if (occ[i] > 0 && waves[i] != static_cast<unsigned>(nb[i]) / (static_cast<unsigned>(s.num_sms) * occ[i])) ++mismatched;
    }
  }
  std::printf("checked %ld mismatched %ld\n", checked, mismatched);
  return (checked > 100000 && mismatched == 0) ? 0 : 1;
}
#endif
