// Thread-block occupancy as Habitat computes it, for device (and host) code.
//
// Behavioural equivalent of KernelMetadata::threadBlockOccupancy
// (cpp/src/cuda/kernel.cpp:33-56 of the reference), which calls NVIDIA's
// standalone occupancy calculator with partitioned global caching off, the
// default shared-memory limit and carve-out, and unlimited per-function block
// size and dynamic shared memory.  Compute capability 3/5/6/7 follows the
// rules of the header the reference vendors; 8/9/10/12, which that header
// rejects, follow the CUDA 12 toolkit header with its per-block reserved
// shared memory.  All arithmetic is integer and must match bit for bit.
//
// Everything that depends only on the device row is folded once, on the host,
// into an hb_dev_pre; the per-kernel part is hb_occupancy().
#pragma once

#include <cmath>
#include <cstdint>

#include "habitat_b200.h"

#if defined(__CUDACC__)
#define HB_HD __host__ __device__ __forceinline__
#else
#define HB_HD inline
#endif

#define HB_INT_MAX 0x7FFFFFFF

// Per-device constants of the occupancy rules (one row of constant memory).
struct hb_dev_pre {
  int32_t valid;            // row passes the calculator's input checks
  int32_t warp_size;
  int32_t warp_shift;       // log2(warp_size) if a power of two, else -1
  int32_t parts;            // register-file sub-partitions per SM
  int32_t gp100;            // cc 6.0: re-check the register limit with 4 parts
  int32_t regs_per_block;
  int32_t regs_per_part;    // regs_per_multiprocessor / parts
  int32_t regs_per_part4;   // regs_per_multiprocessor / 4
  int32_t max_warps;        // max_threads_per_multiprocessor / warp_size
  int32_t max_threads_per_block;
  int32_t blocks_limit;
  int32_t smem_gran;        // allocation granularity, bytes
  int32_t smem_reserved;    // driver-reserved bytes per block (cc >= 8)
  int32_t smem_cap;         // per-block cap incl. the reserved bytes
  int32_t smem_pref;        // configured per-SM carve-out (snapped), < 0: error
  int32_t ladder_kind;      // which carve-out ladder applies (see hb_carveout_snap)
  int32_t smem_per_sm;
  int32_t num_sms;
};

// Ladder kinds: 0 none (cc < 7: fixed per-SM size), 1 Volta, 2 Turing,
// 3: {..64,100} KB, 4: {..64,100,132,164} KB, 5: {..64,100,...,228} KB.
HB_HD int32_t hb_carveout_snap(int32_t kind, int32_t smem_per_sm, int32_t size) {
  if (kind == 2) return size <= 32768 ? 32768 : smem_per_sm;
  if (size == 0) return 0;
  if (size <= 8192) return 8192;
  if (size <= 16384) return 16384;
  if (size <= 32768) return 32768;
  if (size <= 65536) return 65536;
  if (kind == 1) return smem_per_sm;
  if (size <= 100 * 1024) return 100 * 1024;
  if (kind == 3) return -1;
  if (size <= 132 * 1024) return 132 * 1024;
  if (size <= 164 * 1024) return 164 * 1024;
  if (kind == 4) return -1;
  if (size <= 196 * 1024) return 196 * 1024;
  if (size <= 228 * 1024) return 228 * 1024;
  return -1;
}

// Folds one device row.  Host only: runs when the table is uploaded.
inline hb_dev_pre hb_fold_device(const hb_device_spec& s) {
  hb_dev_pre p{};
  const int major = s.compute_major, minor = s.compute_minor;
  bool ok = s.max_threads_per_block > 0 && s.max_threads_per_multiprocessor > 0 &&
            s.regs_per_block > 0 && s.regs_per_multiprocessor > 0 && s.warp_size > 0 &&
            s.shared_mem_per_block > 0 && s.shared_mem_per_multiprocessor > 0 && s.num_sms > 0;
  ok = ok && (major == 3 || (major >= 5 && major <= 10) || major == 12);
  p.num_sms = s.num_sms;
  p.smem_per_sm = s.shared_mem_per_multiprocessor;
  if (!ok) return p;
  p.warp_size = s.warp_size;
  p.warp_shift = -1;
  for (int b = 0; b < 16; ++b)
    if (s.warp_size == (1 << b)) p.warp_shift = b;
  p.gp100 = (major == 6 && minor == 0) ? 1 : 0;
  p.parts = p.gp100 ? 2 : 4;
  p.regs_per_block = s.regs_per_block;
  p.regs_per_part = s.regs_per_multiprocessor / p.parts;
  p.regs_per_part4 = s.regs_per_multiprocessor / 4;
  p.max_warps = s.max_threads_per_multiprocessor / s.warp_size;
  p.max_threads_per_block = s.max_threads_per_block;
  switch (major) {
    case 3: p.blocks_limit = 16; break;
    case 5: case 6: p.blocks_limit = 32; break;
    case 7: p.blocks_limit = minor == 5 ? 16 : 32; break;
    case 8: p.blocks_limit = minor == 0 ? 32 : (minor == 9 ? 24 : 16); break;
    case 9: p.blocks_limit = 32; break;
    case 10: p.blocks_limit = minor == 1 ? 24 : 32; break;
    default: p.blocks_limit = 24; break;  // 12
  }
  p.smem_gran = major >= 8 ? 128 : 256;
  p.smem_reserved = major >= 8 ? s.reserved_shared_mem_per_block : 0;
  p.smem_cap = s.shared_mem_per_block + p.smem_reserved;
  if (major < 7) {
    p.ladder_kind = 0;
    p.smem_pref = s.shared_mem_per_multiprocessor;
  } else {
    int kind = -1;
    if (major == 7) kind = minor == 5 ? 2 : 1;
    else if (major == 8) kind = (minor == 0 || minor == 7) ? 4 : 3;
    else if (major == 9) kind = 5;
    else if (major == 10) kind = (minor == 0 || minor == 1 || minor == 3) ? 5 : -1;
    else if (major == 12) kind = (minor == 0 || minor == 1) ? 3 : -1;
    if (kind < 0) return p;  // the calculator reports an unknown device
    p.ladder_kind = kind;
    p.smem_pref = hb_carveout_snap(kind, s.shared_mem_per_multiprocessor,
                                   s.shared_mem_per_multiprocessor);
    if (p.smem_pref < 0) return p;
  }
  p.valid = 1;
  return p;
}

// Exact quotient n / d for n >= 0, d >= 1.  Below 2^22 the quotient comes from
// one reciprocal and a remainder fix-up instead of a full integer division.
HB_HD int32_t hb_div_small(int32_t n, int32_t d) {
#if defined(__CUDA_ARCH__)
  if (n >= (1 << 22)) return n / d;
  int32_t q = __float2int_rz(__int2float_rn(n) * __frcp_rn(__int2float_rn(d)));
  int32_t r = n - q * d;
  if (r < 0) --q;
  else if (r >= d) ++q;
  return q;
#else
  return n / d;
#endif
}

// Returns active blocks per SM; lim[4] = {regs, warps, blocks, smem} (all 0 on
// error).  `regs` may differ per device (kernel metadata look-up).
HB_HD int32_t hb_occupancy(const hb_dev_pre& d, int32_t block_size, int32_t smem, int32_t regs,
                           int32_t lim[4]) {
  lim[0] = lim[1] = lim[2] = lim[3] = 0;
  if (!d.valid || block_size <= 0 || regs < 0) return 0;

  const int32_t wpb = d.warp_shift >= 0 ? (block_size + d.warp_size - 1) >> d.warp_shift
                                        : (block_size + d.warp_size - 1) / d.warp_size;
  // registers
  int32_t lr = 0;
  if (regs <= 256) {
    const int32_t rpw = ((regs * d.warp_size + 255) >> 8) << 8;
    const int32_t wpb_up = ((wpb + d.parts - 1) / d.parts) * d.parts;
    const int64_t per_cta = (int64_t)rpw * wpb;
    const int64_t assumed = (int64_t)rpw * wpb_up;
    if (!(d.regs_per_block < assumed || d.regs_per_block < per_cta)) {
      if (rpw > 0) {
        lr = (hb_div_small(d.regs_per_part, rpw) * d.parts) / wpb;
        if (d.gp100 && lr != 0) {
          const int64_t assumed4 = (int64_t)rpw * (((wpb + 3) >> 2) << 2);
          if (d.regs_per_block < assumed4 || (d.regs_per_part4 / rpw) * 4 / wpb == 0) lr = 0;
        }
      } else {
        lr = HB_INT_MAX;
      }
    }
  }
  // warps
  const int32_t lw = block_size > d.max_threads_per_block ? 0 : d.max_warps / wpb;
  // shared memory
  int32_t ls = 0;
  if (smem >= 0) {
    const int32_t alloc = ((smem + d.smem_reserved + d.smem_gran - 1) / d.smem_gran) * d.smem_gran;
    if (alloc <= d.smem_cap) {
      int32_t budget = d.smem_pref;
      if (budget < alloc) {
        budget = d.ladder_kind == 0 ? d.smem_per_sm
                                    : hb_carveout_snap(d.ladder_kind, d.smem_per_sm, alloc);
        if (budget < 0) return 0;
      }
      ls = alloc > 0 ? budget / alloc : HB_INT_MAX;
    }
  }
  lim[0] = lr; lim[1] = lw; lim[2] = d.blocks_limit; lim[3] = ls;
  int32_t occ = lr < ls ? lr : ls;
  occ = occ < lw ? occ : lw;
  return occ < d.blocks_limit ? occ : d.blocks_limit;
}

// ---------------------------------------------------------------------------
// Division-free form for "ordinary" device rows (see wave_scale.cu, fast path)
// ---------------------------------------------------------------------------
HB_HD uint32_t hb_umulhi(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
  return __umulhi(a, b);
#else
  return static_cast<uint32_t>((static_cast<uint64_t>(a) * b) >> 32);
#endif
}

constexpr int kMagicN = 512;

struct FastDev {       // per destination (and origin), folded on the host
  int32_t regs_per_block;
  int32_t regs_units;        // (regs_per_multiprocessor / parts) >> 8
  int32_t parts_shift;       // log2(sub-partitions)
  int32_t gp100_units4;      // cc 6.0: (regs_per_multiprocessor / 4) >> 8, else -1
  int32_t max_warps;
  int32_t max_threads_per_block;
  int32_t blocks_limit;
  int32_t gran_shift;        // 7 or 8
  int32_t smem_reserved;
  int32_t smem_cap;
  int32_t smem_pref;
  int32_t ladder_kind;
  int32_t smem_per_sm;
  int32_t num_sms;
  uint32_t sms_magic;        // for ceil(num_blocks / num_sms) in the small-kernel branch
  float a_hi, a_lo, b_hi, b_lo;  // large branch exponent, split float64 constants
  double log2_clk;
};

struct FastParams {
  int32_t D;
  int64_t K;
  FastDev origin;
  FastDev dest[HB_MAX_DEVICES / 2];   // the fast path takes up to 32 destinations
};

// n / d for d >= 1 with M = floor(2^32 / d) + 1 (d >= 2); exact while n * d < 2^32.
HB_HD uint32_t udiv_magic(uint32_t n, uint32_t d, uint32_t M) {
  return d == 1u ? n : hb_umulhi(n, M);
}
// Same for any n < 2^32: the estimate is the quotient or one above it.
HB_HD uint32_t udiv_magic_fix(uint32_t n, uint32_t d, uint32_t M) {
  if (d == 1u) return n;
  uint32_t q = hb_umulhi(n, M);
  if (q * d > n) --q;
  return q;
}

struct FastKernel {   // per recorded kernel, device independent
  int32_t block_size, wpb, regs, rpw_units, smem;
  uint32_t m_wpb;
};

// The three device-dependent limits, each reading only "its" fields of the row,
// so that rows which agree on those fields can share one evaluation.
// Registers: allocation unit 256 per warp, checked against the per-block file
// with the warp count rounded up to the number of sub-partitions.
HB_HD int32_t fast_regs_limit(const FastDev& d, const FastKernel& k, int32_t regs,
                              int32_t rpw_units, uint32_t m_rpw) {
  if (regs > 256) return 0;
  if (rpw_units <= 0) return HB_INT_MAX;
  const int32_t pm = (1 << d.parts_shift) - 1;
  const int32_t wpb_up = (k.wpb + pm) & ~pm;
  if (d.regs_per_block < ((rpw_units * wpb_up) << 8)) return 0;
  const uint32_t warps_part = udiv_magic(d.regs_units, rpw_units, m_rpw);
  int32_t lr = static_cast<int32_t>(udiv_magic(warps_part << d.parts_shift, k.wpb, k.m_wpb));
  if (d.gp100_units4 >= 0 && lr != 0) {
    if (d.regs_per_block < ((rpw_units * ((k.wpb + 3) & ~3)) << 8) ||
        udiv_magic(udiv_magic(d.gp100_units4, rpw_units, m_rpw) << 2, k.wpb, k.m_wpb) == 0)
      lr = 0;
  }
  return lr;
}

HB_HD int32_t fast_warps_limit(const FastDev& d, const FastKernel& k) {
  if (k.block_size <= 0 || k.block_size > d.max_threads_per_block) return 0;
  return static_cast<int32_t>(udiv_magic(d.max_warps, k.wpb, k.m_wpb));
}

// 0 also stands for "the calculator reports an error" (occupancy 0 either way).
HB_HD int32_t fast_smem_limit(const FastDev& d, const FastKernel& k,
                              const uint32_t* __restrict__ s_magic) {
  if (k.smem < 0) return 0;
  const int32_t units = (k.smem + d.smem_reserved + (1 << d.gran_shift) - 1) >> d.gran_shift;
  const int32_t alloc = units << d.gran_shift;
  if (alloc > d.smem_cap) return 0;
  if (units <= 0) return HB_INT_MAX;
  int32_t budget = d.smem_pref;
  if (budget < alloc) {
    budget = d.ladder_kind == 0 ? d.smem_per_sm : hb_carveout_snap(d.ladder_kind, d.smem_per_sm, alloc);
    if (budget < 0) return 0;
  }
  return units < kMagicN
             ? static_cast<int32_t>(udiv_magic(budget >> d.gran_shift, units, s_magic[units]))
             : (budget >> d.gran_shift) / units;
}

HB_HD int32_t fast_occupancy(const FastDev& d, const FastKernel& k, int32_t regs, int32_t rpw_units,
                             uint32_t m_rpw, const uint32_t* __restrict__ s_magic) {
  // an invalid block size zeroes the warp limit, hence the result
  const int32_t lw = fast_warps_limit(d, k);
  if (lw == 0) return 0;
  const int32_t lr = fast_regs_limit(d, k, regs, rpw_units, m_rpw);
  const int32_t ls = fast_smem_limit(d, k, s_magic);
  int32_t occ = lr < ls ? lr : ls;
  occ = occ < lw ? occ : lw;
  return occ < d.blocks_limit ? occ : d.blocks_limit;
}

// Rows that agree on the fields one limit reads form a class for that limit.
inline bool same_regs_class(const FastDev& a, const FastDev& b) {
  return a.regs_per_block == b.regs_per_block && a.regs_units == b.regs_units &&
         a.parts_shift == b.parts_shift && a.gp100_units4 == b.gp100_units4;
}
inline bool same_warps_class(const FastDev& a, const FastDev& b) {
  return a.max_warps == b.max_warps && a.max_threads_per_block == b.max_threads_per_block;
}
inline bool same_smem_class(const FastDev& a, const FastDev& b) {
  return a.gran_shift == b.gran_shift && a.smem_reserved == b.smem_reserved &&
         a.smem_cap == b.smem_cap && a.smem_pref == b.smem_pref && a.ladder_kind == b.ladder_kind &&
         a.smem_per_sm == b.smem_per_sm;
}

// Whether a device row fits the fast path's assumptions.
inline bool fast_row_ok(const hb_device_spec& s, const hb_dev_pre& pre) {
  return pre.valid && s.warp_size == 32 && s.regs_per_multiprocessor <= (1 << 22) &&
         s.regs_per_block <= (1 << 22) && s.max_threads_per_multiprocessor <= (1 << 16) &&
         s.max_threads_per_block <= 16352 /* warps per block stay inside the magic table */ &&
         s.shared_mem_per_multiprocessor <= (1 << 24) && s.shared_mem_per_block <= (1 << 24) &&
         s.num_sms <= 4096 && pre.smem_reserved >= 0 && pre.smem_reserved <= (1 << 20);
}

inline uint32_t magic_of(uint32_t d) { return d >= 2 ? static_cast<uint32_t>((1ull << 32) / d) + 1u : 0u; }

inline FastDev fold_fast(const hb_device_spec& s, const hb_dev_pre& pre) {
  FastDev f{};
  f.regs_per_block = pre.regs_per_block;
  f.regs_units = pre.regs_per_part >> 8;
  f.parts_shift = pre.parts == 2 ? 1 : 2;
  f.gp100_units4 = pre.gp100 ? (pre.regs_per_part4 >> 8) : -1;
  f.max_warps = pre.max_warps;
  f.max_threads_per_block = pre.max_threads_per_block;
  f.blocks_limit = pre.blocks_limit;
  f.gran_shift = pre.smem_gran == 128 ? 7 : 8;
  f.smem_reserved = pre.smem_reserved;
  f.smem_cap = pre.smem_cap;
  f.smem_pref = pre.smem_pref;
  f.ladder_kind = pre.ladder_kind;
  f.smem_per_sm = pre.smem_per_sm;
  f.num_sms = s.num_sms;
  f.sms_magic = magic_of(static_cast<uint32_t>(s.num_sms));
  return f;
}

// ---------------------------------------------------------------------------
// Tables of the table kernel (wave_scale.cu: wave_scale_lut_kernel), built on the host
// ---------------------------------------------------------------------------
// Per device row, one byte each:
//   P[warps per block 0..33][256-register units per warp 0..33] = min(register, warp and
//     blocks-per-SM limit)          (index 33 = "more than 32 warps" / "more than 256 registers")
//   S[shared memory in 128-byte steps 0..2047] = shared-memory limit (last entry: above every cap)
// and per occupancy 0..32 an entry T = {M, sh, A_hi, A_lo}: floor(n / (SMs * occ)) =
// umulhi(n, M) >> sh for every 0 <= n < 2^31, A = log2(occ) - log2(clock MHz) as float hi + lo.
constexpr int kLutW = 34;
constexpr int kLutU = 34;
constexpr int kLutP = kLutW * kLutU;
constexpr int kLutS = 2048;
constexpr int kLutOcc = 33;

struct alignas(16) LutOcc {
  uint32_t magic, shift;
  float lg_hi, lg_lo;
};

// Whether a row can be tabulated.
inline bool lut_row_ok(const hb_device_spec& s, const hb_dev_pre& pre) {
  return fast_row_ok(s, pre) && s.num_sms >= 2 && pre.max_threads_per_block % 32 == 0 &&
         pre.max_threads_per_block <= 1024 && pre.smem_reserved % 128 == 0 &&
         pre.smem_cap <= (kLutS - 2) * 128 && pre.blocks_limit <= kLutOcc - 1 && s.base_clock_mhz > 0;
}

// Tabulates one device row.  `magic`: magic_of(i) for i < kMagicN.
inline void build_row_lut(const hb_device_spec& spec, const FastDev& f, uint8_t* pt, uint8_t* st, LutOcc* tt,
                          const uint32_t* magic) {
  auto clamp = [](int32_t v) { return v < 0 ? 0 : (v > 127 ? 127 : v); };
  for (int wpb = 0; wpb < kLutW; ++wpb) {
    FastKernel k{};
    k.block_size = wpb * 32;   // the largest block of this many warps; thread limits are multiples of 32
    k.wpb = wpb;
    k.m_wpb = magic_of(static_cast<uint32_t>(wpb));
    const int32_t lw = clamp(fast_warps_limit(f, k));
    for (int u = 0; u < kLutU; ++u) {
      k.regs = u * 8;          // any count with this many 256-register units per warp
      k.rpw_units = u;
      int32_t v = 0;
      if (wpb != 0) {
        v = clamp(fast_regs_limit(f, k, k.regs, u, magic_of(static_cast<uint32_t>(u))));
        v = v < lw ? v : lw;
        v = v < f.blocks_limit ? v : f.blocks_limit;
      }
      pt[wpb * kLutU + u] = static_cast<uint8_t>(v);
    }
  }
  for (int s = 0; s < kLutS; ++s) {
    FastKernel k{};
    k.smem = s * 128;          // the largest request of this 128-byte step
    st[s] = s == kLutS - 1 ? 0 : static_cast<uint8_t>(clamp(fast_smem_limit(f, k, magic)));
  }
  const double l_clk = std::log2(static_cast<double>(spec.base_clock_mhz));
  for (int occ = 0; occ < kLutOcc; ++occ) {
    LutOcc e{0u, 0u, 0.0f, 0.0f};
    if (occ > 0) {
      const uint64_t wave = static_cast<uint64_t>(spec.num_sms) * occ;   // >= 2
      int s = 0;
      while ((uint64_t{1} << s) < wave) ++s;                             // ceil(log2 wave) >= 1
      e.magic = static_cast<uint32_t>((uint64_t{1} << (31 + s)) / wave + 1);
      e.shift = static_cast<uint32_t>(s - 1);
      const double a = std::log2(static_cast<double>(occ)) - l_clk;
      e.lg_hi = static_cast<float>(a);
      e.lg_lo = static_cast<float>(a - static_cast<double>(e.lg_hi));
    }
    tt[occ] = e;
  }
}

// Indices the kernel forms from a record (shared with the host-side checks).
HB_HD uint32_t lut_p_index(uint32_t block_size, uint32_t regs) {
  const uint32_t wpb = (block_size + 31u) >> 5;
  const uint32_t units = (regs + 7u) >> 3;
  return (wpb < kLutW - 1 ? wpb : kLutW - 1) * kLutU + (units < kLutU - 1 ? units : kLutU - 1);
}
HB_HD uint32_t lut_s_index(uint32_t smem) {
  const uint32_t capped = smem < (static_cast<uint32_t>(kLutS - 1) << 7) ? smem : (static_cast<uint32_t>(kLutS - 1) << 7);
  return (capped + 127u) >> 7;
}
