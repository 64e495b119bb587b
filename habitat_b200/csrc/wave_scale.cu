// Wave scaling of recorded kernels: one fused elementwise kernel over
// (kernel x destination-device) pairs.
//
// Stands in for the per-kernel Python loop of the reference
// (analyzer/habitat/analysis/predictor.py:111-130 calling
// wave_scaling/roofline.py:8-65, resimplified.py:7-40, common.py:3-20 and,
// through pybind, cpp/src/cuda/kernel.cpp:33-56).
//
// Layout: kernels arrive as structure-of-arrays, results leave as
// destination-major planes.  One thread owns VEC consecutive kernels and walks
// all D destinations, so each record is read once and the origin-side
// occupancy is computed once.  Device rows live in constant memory; the
// per-launch (origin, destination) log2 ratios travel as a kernel parameter.
// The kernel is HBM-bound by design: 20 B read + 5 B written per kernel and
// 9 B written per pair.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "hb_common.h"
#include "occupancy.cuh"
#include "reduce_stage1.cuh"

namespace {

thread_local int32_t t_path = 0;   // kernel of the last launch, see hb_wave_scale_path

__constant__ hb_dev_pre c_dev[HB_MAX_DEVICES];

struct LaunchParams {
  int32_t D;
  int32_t origin_row;
  int64_t K;
  double origin_peak;          // origin peak GFLOP/s (metrics mode)
  uint8_t dest_row[HB_MAX_DEVICES];
  // large branch: log2 t' = log2 t + gamma * a + b, a = log2(bw) - b,
  // b = log2(clock ratio) + log2(SM ratio); small branch uses log2_clk.
  double a[HB_MAX_DEVICES];
  double b[HB_MAX_DEVICES];
  double log2_clk[HB_MAX_DEVICES];
  double ridge[HB_MAX_DEVICES];  // destination peak / bandwidth (metrics mode)
};

// log2(i) for the per-SM block counts of the small-kernel branch (<= 32
// because occupancy never exceeds the blocks-per-SM limit).
__constant__ double c_log2_int[65];

template <typename T, int N>
struct alignas(sizeof(T) * N) Vec {
  T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Vec<T, N> load_vec(const T* p) {
  return *reinterpret_cast<const Vec<T, N>*>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_vec(T* p, const Vec<T, N>& v) {
  *reinterpret_cast<Vec<T, N>*>(p) = v;
}

struct Ptrs {
  const int32_t* num_blocks;
  const uint16_t* block_size;
  const uint16_t* regs;
  const uint32_t* smem;
  const float* time_ns;
  const float* gamma;
  const double* flop_eff;
  const double* dram_read;
  const double* dram_write;
  const uint8_t* has_metrics;
  const int16_t* dest_regs;
  float* scaled_ns;
  uint8_t* dest_occ;
  uint32_t* dest_waves;
  uint8_t* origin_occ;
  uint32_t* origin_waves;
  uint8_t* status;
  int32_t* limits;
  double* block_sums;   // table kernel with fused totals: [D][blocks] sums of each block's results
};

// Per-SM block count ceil(nb / sms) for a kernel that fits in one wave.
__device__ __forceinline__ int32_t ceil_div_sms(int32_t nb, int32_t sms) {
  return hb_div_small(nb + sms - 1, sms);
}

template <int VEC, bool METRICS, bool EXTRA>
__global__ void __launch_bounds__(256)
wave_scale_kernel(const Ptrs p, const __grid_constant__ LaunchParams lp) {
  const int64_t K = lp.K;
  const int64_t k0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
  if (k0 >= K) return;

  const Vec<int32_t, VEC> nbv = load_vec<int32_t, VEC>(p.num_blocks + k0);
  const Vec<uint16_t, VEC> bsv = load_vec<uint16_t, VEC>(p.block_size + k0);
  const Vec<uint16_t, VEC> rgv = load_vec<uint16_t, VEC>(p.regs + k0);
  const Vec<uint32_t, VEC> smv = load_vec<uint32_t, VEC>(p.smem + k0);
  const Vec<float, VEC> tv = load_vec<float, VEC>(p.time_ns + k0);
  Vec<float, VEC> gv;
  if (!METRICS) gv = load_vec<float, VEC>(p.gamma + k0);

  const hb_dev_pre& od = c_dev[lp.origin_row];

  int32_t smem[VEC], wave_o[VEC], omax[VEC];
  double intensity[VEC];   // METRICS: GFLOP per GB, < 0 encodes the special cases
  Vec<uint8_t, VEC> oocc;
  Vec<uint32_t, VEC> owav;
  int32_t lim[4];

#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    smem[i] = smv.v[i] > 0x7FFF0000u ? -1 : static_cast<int32_t>(smv.v[i]);
    const int32_t occ = hb_occupancy(od, bsv.v[i], smem[i], rgv.v[i], lim);
    if (EXTRA && p.limits) {
#pragma unroll
      for (int j = 0; j < 4; ++j) p.limits[static_cast<int64_t>(j) * K + k0 + i] = lim[j];
    }
    wave_o[i] = od.num_sms * occ;
    oocc.v[i] = static_cast<uint8_t>(occ);
    const int32_t nb = nbv.v[i];
    owav.v[i] = (wave_o[i] > 0 && nb >= 1) ? static_cast<uint32_t>(nb / wave_o[i]) : 0xFFFFFFFFu;
    // only consulted when nb < wave_o, i.e. the value is <= occ <= 32
    omax[i] = (nb >= 1 && nb < wave_o[i]) ? ceil_div_sms(nb, od.num_sms) : 1;
    if (METRICS) {
      // wave_scaling/roofline.py:68-88, same operation order, fp64
      double g = -1.0;  // "no metrics": gamma = 1
      if (p.has_metrics[k0 + i]) {
        const double total_gb =
            (p.dram_read[k0 + i] + p.dram_write[k0 + i]) / 1024 / 1024 / 1024;
        const double gps = p.flop_eff[k0 + i] / 100 * lp.origin_peak;
        const double gf = gps * static_cast<double>(tv.v[i]) / 1e9;
        if (gf < 1e-9) g = -1.0;             // gamma = 1
        else if (total_gb == 0) g = -2.0;    // gamma = 0
        else g = gf / total_gb;
      }
      intensity[i] = g;
    }
  }
  store_vec<uint8_t, VEC>(p.origin_occ + k0, oocc);
  store_vec<uint32_t, VEC>(p.origin_waves + k0, owav);

  for (int d = 0; d < lp.D; ++d) {
    const hb_dev_pre& dd = c_dev[lp.dest_row[d]];
    const int64_t base = static_cast<int64_t>(d) * K + k0;
    Vec<float, VEC> outv;
    Vec<uint8_t, VEC> occv, stv;
    Vec<uint32_t, VEC> wavv;
    Vec<int16_t, VEC> drv;
    if (p.dest_regs) drv = load_vec<int16_t, VEC>(p.dest_regs + base);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int32_t nb = nbv.v[i];
      int32_t regs = rgv.v[i];
      if (p.dest_regs && drv.v[i] >= 0) regs = drv.v[i];
      const int32_t occ = hb_occupancy(dd, bsv.v[i], smem[i], regs, lim);
      if (EXTRA && p.limits) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          p.limits[(static_cast<int64_t>(d + 1) * 4 + j) * K + k0 + i] = lim[j];
      }
      const int32_t wave_d = dd.num_sms * occ;
      occv.v[i] = static_cast<uint8_t>(occ);
      wavv.v[i] = (wave_d > 0 && nb >= 1) ? static_cast<uint32_t>(nb / wave_d) : 0xFFFFFFFFu;

      double gamma;
      if (METRICS) {
        const double x = intensity[i];
        if (x == -1.0) gamma = 1.0;
        else if (x == -2.0) gamma = 0.0;
        else {
          const double r = lp.ridge[d];
          gamma = x > r ? 0.5 * r / x : -0.5 / r * x + 1.0;
        }
      } else {
        gamma = static_cast<double>(gv.v[i]);
      }

      // Mirrors the short-circuit of roofline.py:29-30: the destination wave
      // size is only examined when the kernel fits in one origin wave.
      int32_t st;
      double e = 0.0;  // log2 of the scale factor
      if (nb < 1) {
        st = HB_PAIR_BAD_INPUT;
      } else if (wave_o[i] == 0) {
        st = HB_PAIR_ZERO_WAVE;
      } else if (nb < wave_o[i]) {
        if (wave_d == 0) {
          st = HB_PAIR_ZERO_WAVE;
        } else if (nb < wave_d) {
          st = HB_PAIR_SMALL;
          const int32_t dmax = ceil_div_sms(nb, dd.num_sms);
          e = (1.0 - gamma) * (lp.log2_clk[d] + c_log2_int[dmax] - c_log2_int[omax[i]]);
        } else {
          st = HB_PAIR_LARGE;
        }
      } else {
        st = HB_PAIR_LARGE;
      }
      if (st == HB_PAIR_LARGE) e = fma(gamma, lp.a[d], lp.b[d]);
      outv.v[i] = st <= HB_PAIR_SMALL ? tv.v[i] * exp2f(static_cast<float>(e))
                                      : __int_as_float(0x7FC00000);
      stv.v[i] = static_cast<uint8_t>(st);
    }
    store_vec<float, VEC>(p.scaled_ns + base, outv);
    store_vec<uint8_t, VEC>(p.dest_occ + base, occv);
    store_vec<uint32_t, VEC>(p.dest_waves + base, wavv);
    if (EXTRA && p.status) store_vec<uint8_t, VEC>(p.status + base, stv);
  }
}


// ---------------------------------------------------------------------------
// Fast path.  The generic kernel above spends its time in the transcendental /
// conversion unit: every integer division compiles to reciprocal + conversion
// sequences, about ninety such operations per pair, and that unit issues sixteen
// lanes per clock.  When every row of the launch is "ordinary" (valid, warp size
// 32, fields small enough for 32-bit magic numbers - true of every real GPU) the
// divisions become multiply-high by magic numbers M[d] = floor(2^32 / d) + 1
// looked up in shared memory:
//   * divisors that depend on the kernel only (warps per block, register
//     allocation units, shared-memory allocation units) index one 512-entry
//     table loaded from global memory;
//   * the wave size of a pair is num_sms * occupancy with occupancy <= 32, so
//     each device gets a 33-entry table built at block start.
// ---------------------------------------------------------------------------
__device__ uint32_t g_magic[kMagicN];   // filled by hb_set_devices

template <int VEC, bool DEST_REGS>
__global__ void __launch_bounds__(256)
wave_scale_fast_kernel(const Ptrs p, const __grid_constant__ FastParams fp) {
  __shared__ uint32_t s_magic[kMagicN];
  __shared__ uint32_t s_wave_magic[HB_MAX_DEVICES / 2 + 1][33];
  __shared__ double s_log2[33];
  for (int i = threadIdx.x; i < kMagicN; i += blockDim.x) s_magic[i] = g_magic[i];
  for (int i = threadIdx.x; i < (fp.D + 1) * 33; i += blockDim.x) {
    const int d = i / 33, occ = i - d * 33;
    const uint32_t wave = static_cast<uint32_t>((d == 0 ? fp.origin.num_sms : fp.dest[d - 1].num_sms) * occ);
    s_wave_magic[d][occ] = wave >= 2u ? 0xFFFFFFFFu / wave + ((0xFFFFFFFFu % wave) + 1u == wave ? 1u : 0u) + 1u : 0u;
  }
  if (threadIdx.x < 33) s_log2[threadIdx.x] = c_log2_int[threadIdx.x];
  __syncthreads();

  const int64_t K = fp.K;
  const int64_t k0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
  if (k0 >= K) return;

  const Vec<int32_t, VEC> nbv = load_vec<int32_t, VEC>(p.num_blocks + k0);
  const Vec<uint16_t, VEC> bsv = load_vec<uint16_t, VEC>(p.block_size + k0);
  const Vec<uint16_t, VEC> rgv = load_vec<uint16_t, VEC>(p.regs + k0);
  const Vec<uint32_t, VEC> smv = load_vec<uint32_t, VEC>(p.smem + k0);
  const Vec<float, VEC> tv = load_vec<float, VEC>(p.time_ns + k0);
  const Vec<float, VEC> gv = load_vec<float, VEC>(p.gamma + k0);

  FastKernel fk[VEC];
  uint32_t m_rpw[VEC];
  int32_t wave_o[VEC], omax[VEC];
  Vec<uint8_t, VEC> oocc;
  Vec<uint32_t, VEC> owav;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    FastKernel& k = fk[i];
    k.block_size = bsv.v[i];
    k.wpb = (k.block_size + 31) >> 5;
    k.regs = rgv.v[i];
    k.rpw_units = (k.regs + 7) >> 3;               // roundup(regs * 32, 256) / 256
    k.smem = smv.v[i] > 0x7FFF0000u ? -1 : static_cast<int32_t>(smv.v[i]);
    k.m_wpb = s_magic[min(k.wpb, kMagicN - 1)];    // wpb <= 32 whenever the block can run
    m_rpw[i] = s_magic[min(k.rpw_units, kMagicN - 1)];
    const int32_t occ = fast_occupancy(fp.origin, k, k.regs, k.rpw_units, m_rpw[i], s_magic);
    const int32_t nb = nbv.v[i];
    wave_o[i] = fp.origin.num_sms * occ;
    oocc.v[i] = static_cast<uint8_t>(occ);
    owav.v[i] = (occ > 0 && nb >= 1)
                    ? udiv_magic_fix(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_o[i]),
                                     s_wave_magic[0][occ])
                    : 0xFFFFFFFFu;
    omax[i] = (nb >= 1 && nb < wave_o[i])
                  ? static_cast<int32_t>(udiv_magic(nb + fp.origin.num_sms - 1, fp.origin.num_sms,
                                                    fp.origin.sms_magic))
                  : 1;
  }
  store_vec<uint8_t, VEC>(p.origin_occ + k0, oocc);
  store_vec<uint32_t, VEC>(p.origin_waves + k0, owav);

  for (int d = 0; d < fp.D; ++d) {
    const FastDev& dd = fp.dest[d];
    const int64_t base = static_cast<int64_t>(d) * K + k0;
    Vec<float, VEC> outv;
    Vec<uint8_t, VEC> occv;
    Vec<uint32_t, VEC> wavv;
    Vec<int16_t, VEC> drv;
    if (DEST_REGS) drv = load_vec<int16_t, VEC>(p.dest_regs + base);
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int32_t nb = nbv.v[i];
      int32_t regs = fk[i].regs, units = fk[i].rpw_units;
      uint32_t m = m_rpw[i];
      if (DEST_REGS && drv.v[i] >= 0) {
        regs = drv.v[i];
        units = (regs + 7) >> 3;
        m = s_magic[min(units, kMagicN - 1)];
      }
      const int32_t occ = fast_occupancy(dd, fk[i], regs, units, m, s_magic);
      const int32_t wave_d = dd.num_sms * occ;
      occv.v[i] = static_cast<uint8_t>(occ);
      wavv.v[i] = (occ > 0 && nb >= 1)
                      ? udiv_magic_fix(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_d),
                                       s_wave_magic[d + 1][occ])
                      : 0xFFFFFFFFu;
      const float gamma = gv.v[i];
      float e;
      bool ok = nb >= 1 && wave_o[i] != 0;
      if (ok && nb < wave_o[i] && nb < wave_d) {
        // small kernel (roofline.py:32-45); both per-SM block counts are <= 32
        const int32_t dmax = static_cast<int32_t>(udiv_magic(nb + dd.num_sms - 1, dd.num_sms, dd.sms_magic));
        e = static_cast<float>((1.0 - static_cast<double>(gamma)) *
                               (dd.log2_clk + s_log2[dmax] - s_log2[omax[i]]));
      } else {
        ok = ok && !(nb < wave_o[i] && wave_d == 0);
        e = fmaf(gamma, dd.a_hi, dd.b_hi) + fmaf(gamma, dd.a_lo, dd.b_lo);
      }
      outv.v[i] = ok ? tv.v[i] * exp2f(e) : __int_as_float(0x7FC00000);
    }
    store_vec<float, VEC>(p.scaled_ns + base, outv);
    store_vec<uint8_t, VEC>(p.dest_occ + base, occv);
    store_vec<uint32_t, VEC>(p.dest_waves + base, wavv);
  }
}


bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

bool vec4_ok(const Ptrs& p, int64_t K, bool need_gamma) {
  // The 4-wide path needs every plane base (d * K elements in) and every input
  // to sit on a 16-byte boundary for its widest type.
  return (K % 4 == 0) && aligned16(p.num_blocks) && aligned16(p.smem) && aligned16(p.time_ns) &&
         (!need_gamma || aligned16(p.gamma)) && aligned16(p.scaled_ns) && aligned16(p.dest_waves) &&
         aligned16(p.origin_waves) && (reinterpret_cast<uintptr_t>(p.block_size) % 8 == 0) &&
         (reinterpret_cast<uintptr_t>(p.regs) % 8 == 0) &&
         (reinterpret_cast<uintptr_t>(p.dest_occ) % 4 == 0) &&
         (reinterpret_cast<uintptr_t>(p.origin_occ) % 4 == 0) &&
         (!p.status || reinterpret_cast<uintptr_t>(p.status) % 4 == 0) &&
         (!p.dest_regs || reinterpret_cast<uintptr_t>(p.dest_regs) % 8 == 0);
}

// ---------------------------------------------------------------------------
// Table kernel.  Every device-dependent limit of a record is a function of small
// integers, so hb_set_devices tabulates, per device row and one byte each:
//   P[warps per block 0..33][256-register units per warp 0..33] =
//       min(register limit, warp limit, blocks-per-SM limit)
//   S[shared memory in 128-byte steps 0..2047] = shared-memory limit
// and, per occupancy 0..32, a 16-byte entry T[occ] = {M, sh, A_hi, A_lo}:
//   * floor(n / (SMs * occ)) = umulhi(n, M) >> sh for every 0 <= n < 2^31
//     (M = floor(2^(31+s) / wave) + 1 with s = ceil(log2 wave), sh = s - 1: the
//     error term n e / 2^(31+s) stays below 1 / wave because e <= wave <= 2^s),
//     so a pair's wave count is one table load, one multiply-high and a shift,
//     and "the kernel fits in one wave" is the test quotient == 0;
//   * A = log2(occ) - log2(clock MHz) as float hi + lo: the exponent of the
//     small-kernel rule (roofline.py:32-45) is (1 - gamma) (A_dest[blocks per SM
//     on the destination] - A_origin[blocks per SM on the origin]).
// Rows that agree on everything P (or S) reads form a class; a launch carries at
// most four classes of each, a record loads one byte per class, and a
// destination picks its two bytes with a byte permute and takes one 16-bit-pair
// minimum for the two records a thread owns.  The tables a launch touches
// (a few KB) stay in L1.  The extended variant (EXT) reads every device's own P and S
// bytes per pair instead (no class limit) and adds, under launch-uniform branches,
// the status plane, per-destination register counts and gamma from raw metrics
// (one float64 intensity per record, a compare and a multiply-add per pair); it
// also serves launches with more than four classes.  The grid is persistent:
// blocks stride over the batch.
// Conditions (checked on the host, else wave_scale_fast_kernel or the generic
// kernel runs): D <= 32, D K < 2^31, and per row 2 <= SMs <= 4096,
// blocks-per-SM limit <= 32, thread limit per block a multiple of 32 and <= 1024,
// shared-memory reserve a multiple of 128, shared-memory cap below the table's
// last step.
// ---------------------------------------------------------------------------
constexpr int kMaxClasses = 4;   // table sizes, LutOcc and the table builder: occupancy.cuh

__device__ uint8_t g_lut_p[HB_MAX_DEVICES * kLutP];
__device__ uint8_t g_lut_s[HB_MAX_DEVICES * kLutS];
__device__ LutOcc g_lut_t[HB_MAX_DEVICES * kLutOcc];

struct alignas(16) LutDev {       // three 16-byte groups, each fetched with one constant load
  uint32_t sel_p, sel_s;          // permute selectors: class byte of record 0 -> low half, record 1 -> high half
  uint32_t t_off;                 // byte offset of the row's T entries
  uint32_t p_off;                 // byte offset of the row's own P table (per-destination register counts)
  float a_hi, a_lo, b_hi, b_lo;   // large-kernel exponent gamma a + b, split float64 constants
  uint32_t sms_m1, sms_magic;     // SMs - 1 and floor(2^32 / SMs) + 1, for ceil(blocks / SMs)
  uint32_t s_off;                 // byte offset of the row's own S table (extended variant)
  uint32_t pad;
};
struct LutDevRegs {               // LutDev as read by a thread
  uint4 sel;
  float4 ab;
  uint4 sm;
};
__device__ __forceinline__ LutDevRegs load_lut_dev(const LutDev& d) {
  LutDevRegs r;
  r.sel = *reinterpret_cast<const uint4*>(&d.sel_p);
  r.ab = *reinterpret_cast<const float4*>(&d.a_hi);
  r.sm = *reinterpret_cast<const uint4*>(&d.sms_m1);
  return r;
}

struct LutParams {
  uint32_t K;
  int32_t D;
  uint32_t off_p[kMaxClasses], off_s[kMaxClasses];   // byte offsets of the class tables
  double origin_peak;                                // metrics mode: origin peak GFLOP/s
  LutDev origin;
  LutDev dest[HB_MAX_DEVICES / 2];
  double ridge[HB_MAX_DEVICES / 2];                  // metrics mode: destination peak / bandwidth
  double slope[HB_MAX_DEVICES / 2];                  // -0.5 / ridge
};

constexpr int kLutThreads = 128;

// prmt.b32 in its default mode: selector nibble n picks byte (n & 7) of {b, a}; with bit 3 set
// the byte's sign bit is replicated instead (0x00 for the values below 128 used here).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#if defined(HB_BOUNDS_CHECK)
// Checked build: every table index and element index is compared with its bound; a violation is
// recorded (first one wins) and the access redirected to element 0.  Nothing traps.
__device__ uint32_t g_bounds_word = 0;
__device__ __forceinline__ uint32_t hb_checked(uint32_t idx, uint32_t limit, uint32_t site) {
  if (idx >= limit) {
    atomicCAS(&g_bounds_word, 0u, (site << 24) | (idx & 0xFFFFFFu) | 0x80000000u);
    return 0u;
  }
  return idx;
}
#define HB_IDX(idx, limit, site) hb_checked((idx), (limit), (site))
#else
#define HB_IDX(idx, limit, site) (idx)
#endif

// Two records per thread (VEC = 2) need the inputs on 8-byte boundaries; ALIGNED says that the
// output planes are too (K even), so results leave as 8-byte stores.  Otherwise (odd K: every
// other plane starts on an odd element) the same two-record arithmetic ends in scalar stores,
// and the thread that owns the last, single record loads it alone.
template <typename T, int VEC, bool ALIGNED>
__device__ __forceinline__ Vec<T, VEC> load_pair(const T* q, bool pair) {
  if (VEC == 1 || ALIGNED) return load_vec<T, VEC>(q);
  Vec<T, VEC> v;
  if (pair) {
    v = load_vec<T, VEC>(q);
  } else {
    v.v[0] = q[0];
    v.v[VEC - 1] = q[0];
  }
  return v;
}
template <typename T, int VEC, bool ALIGNED>
__device__ __forceinline__ void store_pair(T* q, const Vec<T, VEC>& v, bool pair) {
  if (VEC == 1 || ALIGNED) {
    store_vec<T, VEC>(q, v);
  } else {
    q[0] = v.v[0];
    if (pair) q[VEC - 1] = v.v[VEC - 1];
  }
}
// The low bytes of the two 16-bit halves of `pair_word` as one or two bytes at q.
template <int VEC, bool ALIGNED>
__device__ __forceinline__ void store_byte_pair(uint8_t* q, uint32_t pair_word, bool pair) {
  if (VEC == 2 && ALIGNED) {
    *reinterpret_cast<uint16_t*>(q) = static_cast<uint16_t>(__byte_perm(pair_word, 0u, 0x4420u));
  } else {
    q[0] = static_cast<uint8_t>(pair_word);
    if (VEC == 2 && pair) q[1] = static_cast<uint8_t>(pair_word >> 16);
  }
}

// TOT: every block also adds up its own results per destination (float64, fixed order, NaN results
// skipped like the plane sums do) and leaves the sums in p.block_sums[d * gridDim.x + block], so
// the totals of a launch need no second pass over the [D x K] plane.  A thread parks the float64
// sum of its two results per destination in shared memory; at the end sixteen lanes per
// destination add the block's 128 sums.  Needs a grid that covers the batch in one pass and
// D <= kTotMaxD.
constexpr int kTotMaxD = kLutThreads / 16;

template <int VEC, bool EXT, bool ALIGNED, int NP, int NS, bool TOT = false>
__global__ void __launch_bounds__(kLutThreads, EXT ? 8 : 12)
wave_scale_lut_kernel(const Ptrs p, const __grid_constant__ LutParams lp) {
  static_assert(!TOT || (VEC == 2 && ALIGNED && !EXT), "fused totals: aligned two-record variant only");
  __shared__ double s_tot[TOT ? kTotMaxD : 1][TOT ? kLutThreads : 1];
  hb_grid_dependency_wait();
  const uint32_t K = lp.K;
  const int D = lp.D;
  if (TOT && (blockIdx.x * kLutThreads + threadIdx.x) * VEC >= K) {
    for (int d = 0; d < D; ++d) s_tot[d][threadIdx.x] = 0.0;   // threads past the end
  }
  const uint8_t* __restrict__ tab_t = reinterpret_cast<const uint8_t*>(g_lut_t);
  const uint32_t stride = gridDim.x * (kLutThreads * VEC);
  const bool with_regs = EXT && p.dest_regs != nullptr;
  const bool with_metrics = EXT && p.has_metrics != nullptr;
  const bool with_status = EXT && p.status != nullptr;

  for (uint32_t k0 = (blockIdx.x * kLutThreads + threadIdx.x) * VEC; k0 < K; k0 += stride) {
    const bool pair = VEC == 2 && (ALIGNED || k0 + 1 < K);   // false: the last record of an odd batch
    const Vec<int32_t, VEC> nbv = load_pair<int32_t, VEC, ALIGNED>(p.num_blocks + k0, pair);
    const Vec<uint16_t, VEC> bsv = load_pair<uint16_t, VEC, ALIGNED>(p.block_size + k0, pair);
    const Vec<uint16_t, VEC> rgv = load_pair<uint16_t, VEC, ALIGNED>(p.regs + k0, pair);
    const Vec<uint32_t, VEC> smv = load_pair<uint32_t, VEC, ALIGNED>(p.smem + k0, pair);
    const Vec<float, VEC> tv = load_pair<float, VEC, ALIGNED>(p.time_ns + k0, pair);
    Vec<float, VEC> gv;
    if (!with_metrics) gv = load_pair<float, VEC, ALIGNED>(p.gamma + k0, pair);

    uint32_t P[2] = {0u, 0u}, S[2] = {0u, 0u};   // class bytes of the two records
    uint32_t wrow[2] = {0u, 0u};                 // EXT: warps per block x row length (P index base)
    float omg[2] = {0.0f, 0.0f};
    double xint[2] = {-1.0, -1.0}, xinv[2] = {0.0, 0.0};   // EXT: intensity (< 0: special case) and 1 / intensity
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const uint32_t wpb = min((static_cast<uint32_t>(bsv.v[i]) + 31u) >> 5, static_cast<uint32_t>(kLutW - 1));
      const uint32_t pidx = HB_IDX(lut_p_index(bsv.v[i], rgv.v[i]), kLutP, 1);
      const uint32_t steps = HB_IDX(lut_s_index(smv.v[i]), kLutS, 2);
      if (!EXT) {
        uint32_t pw = 0, sw = 0;
#pragma unroll
        for (int c = 0; c < NP; ++c) pw |= static_cast<uint32_t>(__ldg(g_lut_p + (lp.off_p[c] + pidx))) << (8 * c);
#pragma unroll
        for (int c = 0; c < NS; ++c) sw |= static_cast<uint32_t>(__ldg(g_lut_s + (lp.off_s[c] + steps))) << (8 * c);
        P[i] = pw; S[i] = sw;
      } else {
        // extended variant: every device's own tables are indexed directly (no class limit)
        P[i] = pidx; S[i] = steps;
        wrow[i] = wpb * kLutU;
      }
      if (!with_metrics) omg[i] = 1.0f - gv.v[i];
      if (with_metrics) {
        // wave_scaling/roofline.py:68-92, float64, same operation order
        double x = -1.0;   // "no metrics" or next to no floating-point work: gamma = 1
        const uint32_t ki = (i == 0 || pair) ? k0 + i : k0;   // the tail thread's second slot repeats the first
        if (p.has_metrics[ki]) {
          const double total_gb = (p.dram_read[ki] + p.dram_write[ki]) / 1024 / 1024 / 1024;
          const double gps = p.flop_eff[ki] / 100 * lp.origin_peak;
          const double gf = gps * static_cast<double>(tv.v[i]) / 1e9;
          if (gf < 1e-9) x = -1.0;
          else if (total_gb == 0) x = -2.0;   // gamma = 0
          else x = gf / total_gb;
        }
        xint[i] = x;
        xinv[i] = x > 0.0 ? 1.0 / x : 0.0;
      }
    }

    // origin: both records at once
    const LutDevRegs og = load_lut_dev(lp.origin);
    uint32_t o2;
    if (!EXT) {
      o2 = __vimin_s16x2_relu(prmt(P[0], P[1], og.sel.x), prmt(S[0], S[1], og.sel.y));
    } else {
      o2 = 0;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const uint32_t pb = __ldg(g_lut_p + (og.sel.w + P[i]));
        const uint32_t sb = __ldg(g_lut_s + (og.sm.z + S[i]));
        o2 |= min(pb, sb) << (16 * i);
      }
    }
    bool nbok[2] = {false, false}, live[2] = {false, false}, fits_o[2] = {false, false};
    float2 lg_o[2];
    Vec<uint32_t, VEC> owav;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const uint32_t occ = i == 0 ? (o2 & 0xFFFFu) : (o2 >> 16);
      const int32_t nb = nbv.v[i];
      const uint2 w = __ldg(reinterpret_cast<const uint2*>(tab_t + (og.sel.z + HB_IDX(occ, kLutOcc, 3) * 16u)));
      const uint32_t q = __umulhi(static_cast<uint32_t>(nb), w.x) >> w.y;
      nbok[i] = nb >= 1;
      live[i] = nbok[i] && occ != 0u;
      owav.v[i] = live[i] ? q : 0xFFFFFFFFu;
      fits_o[i] = live[i] && q == 0u;            // num_blocks < origin wave size
      // ceil(num_blocks / SMs) <= occupancy <= 32 whenever the small-kernel rule applies; otherwise
      // the entry read here is never used, and the clamp only keeps the index inside the table.  Not
      // selecting on fits_o keeps this load independent of the one above.
      const uint32_t om = min(__umulhi(static_cast<uint32_t>(nb) + og.sm.x, og.sm.y), static_cast<uint32_t>(kLutOcc - 1));
      lg_o[i] = __ldg(reinterpret_cast<const float2*>(tab_t + (og.sel.z + HB_IDX(om, kLutOcc, 4) * 16u + 8u)));
    }
    store_byte_pair<VEC, ALIGNED>(p.origin_occ + k0, o2, pair);
    store_pair<uint32_t, VEC, ALIGNED>(p.origin_waves + k0, owav, pair);

#pragma unroll 1
    for (int d = 0; d < D; ++d) {
      const LutDevRegs dd = load_lut_dev(lp.dest[d]);
      const uint32_t base = static_cast<uint32_t>(d) * K + k0;   // D K < 2^31
      uint32_t occ2;
      if (!EXT) {
        occ2 = __vimin_s16x2_relu(prmt(P[0], P[1], dd.sel.x), prmt(S[0], S[1], dd.sel.y));
      } else {
        Vec<int16_t, VEC> drv;
        if (with_regs) {
          if (VEC == 1 || ALIGNED) {
            drv = load_vec<int16_t, VEC>(p.dest_regs + base);
          } else {
            drv.v[0] = p.dest_regs[base];
            drv.v[VEC - 1] = pair ? p.dest_regs[base + 1] : static_cast<int16_t>(-1);
          }
        }
        occ2 = 0;
#pragma unroll
        for (int i = 0; i < VEC; ++i) {
          uint32_t pidx = P[i];
          if (with_regs && drv.v[i] >= 0) {
            // MetadataManager.kernel_registers_for gave another register count for this destination
            const uint32_t units = min((static_cast<uint32_t>(drv.v[i]) + 7u) >> 3, static_cast<uint32_t>(kLutU - 1));
            pidx = HB_IDX(wrow[i] + units, kLutP, 5);
          }
          const uint32_t pb = __ldg(g_lut_p + (dd.sel.w + pidx));
          const uint32_t sb = __ldg(g_lut_s + (dd.sm.z + S[i]));
          occ2 |= min(pb, sb) << (16 * i);
        }
      }
      Vec<float, VEC> outv;
      Vec<uint32_t, VEC> wavv;
      uint32_t st2 = 0;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const uint32_t occ = i == 0 ? (occ2 & 0xFFFFu) : (occ2 >> 16);
        const int32_t nb = nbv.v[i];
        const uint2 w = __ldg(reinterpret_cast<const uint2*>(tab_t + (dd.sel.z + HB_IDX(occ, kLutOcc, 6) * 16u)));
        const uint32_t q = __umulhi(static_cast<uint32_t>(nb), w.x) >> w.y;
        const bool has_wave = occ != 0u;
        wavv.v[i] = (nbok[i] && has_wave) ? q : 0xFFFFFFFFu;
        // roofline.py:29-30 with its short circuit: the destination is only looked at when the
        // kernel fits in one origin wave
        const bool small = fits_o[i] && has_wave && q == 0u;
        const bool ok = live[i] && !(fits_o[i] && !has_wave);
        // blocks per SM on the destination: meaningful (and <= occupancy) when `small`; computed from
        // the record alone so that this table load does not wait for the one above
        const uint32_t dm = min(__umulhi(static_cast<uint32_t>(nb) + dd.sm.x, dd.sm.y), static_cast<uint32_t>(kLutOcc - 1));
        const float2 lg_d = __ldg(reinterpret_cast<const float2*>(tab_t + (dd.sel.z + HB_IDX(dm, kLutOcc, 7) * 16u + 8u)));
        float gamma, one_minus;
        if (with_metrics) {
          const double x = xint[i];
          double gm;
          if (x < 0.0) gm = x == -1.0 ? 1.0 : 0.0;
          else gm = x > lp.ridge[d] ? 0.5 * lp.ridge[d] * xinv[i] : fma(lp.slope[d], x, 1.0);
          gamma = static_cast<float>(gm);
          one_minus = static_cast<float>(1.0 - gm);
        } else {
          gamma = gv.v[i];
          one_minus = omg[i];
        }
        const float e_small = one_minus * ((lg_d.x - lg_o[i].x) + (lg_d.y - lg_o[i].y));
        const float e_large = fmaf(gamma, dd.ab.x, dd.ab.z) + fmaf(gamma, dd.ab.y, dd.ab.w);
        const float e = small ? e_small : e_large;
        outv.v[i] = ok ? tv.v[i] * ex2_approx(e) : __int_as_float(0x7FC00000);
        if (with_status) {
          const uint32_t st = !nbok[i] ? HB_PAIR_BAD_INPUT
                                       : (!ok ? HB_PAIR_ZERO_WAVE : (small ? HB_PAIR_SMALL : HB_PAIR_LARGE));
          st2 |= st << (16 * i);
        }
      }
      store_pair<float, VEC, ALIGNED>(p.scaled_ns + base, outv, pair);
      store_pair<uint32_t, VEC, ALIGNED>(p.dest_waves + base, wavv, pair);
      store_byte_pair<VEC, ALIGNED>(p.dest_occ + base, occ2, pair);
      if (with_status) store_byte_pair<VEC, ALIGNED>(p.status + base, st2, pair);
      if (TOT) {
        const float g0 = outv.v[0] == outv.v[0] ? outv.v[0] : 0.0f;                     // NaN: no prediction
        const float g1 = outv.v[VEC - 1] == outv.v[VEC - 1] ? outv.v[VEC - 1] : 0.0f;
        s_tot[d][threadIdx.x] = static_cast<double>(g0) + static_cast<double>(g1);   // exact
      }
    }
  }
  if (TOT) {
    __syncthreads();
    const int d = threadIdx.x >> 4, j = threadIdx.x & 15;
    double acc = 0.0;
    if (d < D) {
      const double2* row = reinterpret_cast<const double2*>(s_tot[d]);
#pragma unroll
      for (int i = 0; i < kLutThreads / 32; ++i) {
        const double2 x = row[j + 16 * i];
        acc += x.x + x.y;
      }
    }
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) acc += __shfl_down_sync(0xFFFFFFFFu, acc, o, 16);
    if (j == 0 && d < D) p.block_sums[static_cast<size_t>(d) * gridDim.x + blockIdx.x] = acc;
  }
}

// ---------------------------------------------------------------------------
// Host side: device table, per-GPU upload, launch selection
// ---------------------------------------------------------------------------
// The table hb_set_devices receives is kept on the host; every GPU of the process gets its own
// copy (constant rows, tabulated limits) the first time it is used after a change, so one
// process may drive several GPUs.  All of it is guarded by one mutex; hb_wave_scale only takes
// the lock when the current GPU's copy is stale.
constexpr int kMaxCudaDevices = 64;

struct HostTable {
  int n = 0;
  hb_device_spec rows[HB_MAX_DEVICES];
  hb_dev_pre pre[HB_MAX_DEVICES];
  bool lut_ok[HB_MAX_DEVICES] = {};
  uint64_t row_version[HB_MAX_DEVICES] = {};   // bumped when a row's specification changes
  std::vector<uint8_t> lut_p = std::vector<uint8_t>(static_cast<size_t>(HB_MAX_DEVICES) * kLutP);
  std::vector<uint8_t> lut_s = std::vector<uint8_t>(static_cast<size_t>(HB_MAX_DEVICES) * kLutS);
  std::vector<LutOcc> lut_t = std::vector<LutOcc>(static_cast<size_t>(HB_MAX_DEVICES) * kLutOcc);
};
struct GpuCopy {
  std::atomic<bool> constants{false};          // row-independent tables uploaded (read without the lock)
  uint64_t row_version[HB_MAX_DEVICES] = {};   // version of each row this GPU holds
  int sm_count = 0;
};

std::mutex g_mu;
HostTable g_tab;
GpuCopy g_gpu[kMaxCudaDevices];
std::atomic<uint64_t> g_version{0};                       // bumped by every hb_set_devices that changed a row
std::atomic<uint64_t> g_gpu_version[kMaxCudaDevices];     // table version each GPU has seen

// Brings the current GPU's copy of the table up to date (rows that changed since its last
// upload, plus the row-independent tables on first use).  Synchronises the device when it
// uploads anything, so launches on any stream see the new rows.
hb_status sync_gpu(int* sm_count) {
  int dev = 0;
  HB_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxCudaDevices) {
    hb::set_error("hb_wave_scale: device ordinal %d out of range", dev);
    return HB_ERR_UNSUPPORTED;
  }
  if (g_gpu_version[dev].load(std::memory_order_acquire) == g_version.load(std::memory_order_acquire) &&
      g_gpu[dev].constants.load(std::memory_order_acquire)) {
    if (sm_count) *sm_count = g_gpu[dev].sm_count;
    return HB_OK;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  GpuCopy& gc = g_gpu[dev];
  bool uploaded = false;
  if (!gc.constants.load(std::memory_order_relaxed)) {
    HB_CUDA_TRY(cudaDeviceGetAttribute(&gc.sm_count, cudaDevAttrMultiProcessorCount, dev));
    double lg[65];
    lg[0] = 0.0;
    for (int i = 1; i <= 64; ++i) lg[i] = std::log2(static_cast<double>(i));
    HB_CUDA_TRY(cudaMemcpyToSymbol(c_log2_int, lg, sizeof(lg)));
    uint32_t magic[kMagicN];
    for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_magic, magic, sizeof(magic)));
    gc.constants.store(true, std::memory_order_release);
    uploaded = true;
  }
  for (int i = 0; i < g_tab.n; ++i) {
    if (gc.row_version[i] == g_tab.row_version[i]) continue;
    HB_CUDA_TRY(cudaMemcpyToSymbol(c_dev, &g_tab.pre[i], sizeof(hb_dev_pre), sizeof(hb_dev_pre) * i));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_p, &g_tab.lut_p[static_cast<size_t>(i) * kLutP], kLutP,
                                   static_cast<size_t>(i) * kLutP));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_s, &g_tab.lut_s[static_cast<size_t>(i) * kLutS], kLutS,
                                   static_cast<size_t>(i) * kLutS));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_t, &g_tab.lut_t[static_cast<size_t>(i) * kLutOcc],
                                   sizeof(LutOcc) * kLutOcc, sizeof(LutOcc) * kLutOcc * i));
    gc.row_version[i] = g_tab.row_version[i];
    uploaded = true;
  }
  if (uploaded) HB_CUDA_TRY(cudaDeviceSynchronize());
  g_gpu_version[dev].store(g_version.load(std::memory_order_acquire), std::memory_order_release);
  if (sm_count) *sm_count = gc.sm_count;
  return HB_OK;
}

uint32_t pair_selector(int c) {
  const uint32_t lo = static_cast<uint32_t>(c), hi = static_cast<uint32_t>(4 + c);
  return lo | ((8u | lo) << 4) | (hi << 8) | ((8u | hi) << 12);
}

bool same_p_class(const FastDev& a, const FastDev& b) {
  return same_regs_class(a, b) && same_warps_class(a, b) && a.blocks_limit == b.blocks_limit;
}

// Class (index into `rows`, which lists the first row of each class) of `row`; -1 when full.
template <typename Same>
int class_of(int* rows, int* n, int row, Same same) {
  for (int c = 0; c < *n; ++c)
    if (same(fold_fast(g_tab.rows[rows[c]], g_tab.pre[rows[c]]), fold_fast(g_tab.rows[row], g_tab.pre[row]))) return c;
  if (*n >= kMaxClasses) return -1;
  rows[*n] = row;
  return (*n)++;
}

template <int VEC, bool EXT, bool ALIGNED, int NP, int NS, bool TOT = false>
cudaError_t launch_lut(unsigned grid, cudaStream_t stream, const Ptrs& p, const LutParams& q) {
  return hb::launch_overlapped(wave_scale_lut_kernel<VEC, EXT, ALIGNED, NP, NS, TOT>, dim3(grid), dim3(kLutThreads),
                               0, stream, p, q);
}

template <int NP, bool TOT>
cudaError_t launch_lut_plain(int ns, unsigned grid, cudaStream_t stream, const Ptrs& p, const LutParams& q) {
  switch (ns) {
    case 1: return launch_lut<2, false, true, NP, 1, TOT>(grid, stream, p, q);
    case 2: return launch_lut<2, false, true, NP, 2, TOT>(grid, stream, p, q);
    case 3: return launch_lut<2, false, true, NP, 3, TOT>(grid, stream, p, q);
    default: return launch_lut<2, false, true, NP, 4, TOT>(grid, stream, p, q);
  }
}
template <bool TOT>
cudaError_t launch_lut_plain(int np, int ns, unsigned grid, cudaStream_t stream, const Ptrs& p, const LutParams& q) {
  switch (np) {
    case 1: return launch_lut_plain<1, TOT>(ns, grid, stream, p, q);
    case 2: return launch_lut_plain<2, TOT>(ns, grid, stream, p, q);
    case 3: return launch_lut_plain<3, TOT>(ns, grid, stream, p, q);
    default: return launch_lut_plain<4, TOT>(ns, grid, stream, p, q);
  }
}

// Launches wave_scale_lut_kernel when the launch qualifies; false = nothing launched.  *fused says
// whether the launch also wrote p.block_sums (one sum per destination and block of the grid).
bool try_launch_lut(const Ptrs& p, const LaunchParams& lp, int sm_count, cudaStream_t stream, hb_status* st,
                    bool* fused, unsigned* fused_blocks) {
  *fused = false;
  static const bool use_lut = [] { const char* e = std::getenv("HB_WAVE_LUT"); return !e || std::atoi(e) != 0; }();
  if (!use_lut || p.limits || lp.D > HB_MAX_DEVICES / 2) return false;
  const int64_t K = lp.K;
  if (static_cast<int64_t>(lp.D) * K >= (int64_t{1} << 31)) return false;   // 32-bit element indices
  LutParams q{};
  int rows_p[kMaxClasses] = {}, rows_s[kMaxClasses] = {}, n_p = 0, n_s = 0;
  bool many_classes = false;
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_tab.lut_ok[lp.origin_row]) return false;
    for (int d = 0; d < lp.D; ++d)
      if (!g_tab.lut_ok[lp.dest_row[d]]) return false;
    for (int d = -1; d < lp.D; ++d) {
      const int row = d < 0 ? lp.origin_row : lp.dest_row[d];
      const int pc = many_classes ? -1 : class_of(rows_p, &n_p, row, same_p_class);
      const int sc = many_classes ? -1 : class_of(rows_s, &n_s, row, same_smem_class);
      if (pc < 0 || sc < 0) many_classes = true;   // more than four classes: every row's own tables (extended variant)
      LutDev& o = d < 0 ? q.origin : q.dest[d];
      o.sel_p = pair_selector(pc < 0 ? 0 : pc);
      o.sel_s = pair_selector(sc < 0 ? 0 : sc);
      o.t_off = static_cast<uint32_t>(row * kLutOcc * sizeof(LutOcc));
      o.p_off = static_cast<uint32_t>(row * kLutP);
      o.s_off = static_cast<uint32_t>(row * kLutS);
      o.sms_m1 = static_cast<uint32_t>(g_tab.rows[row].num_sms - 1);
      o.sms_magic = magic_of(static_cast<uint32_t>(g_tab.rows[row].num_sms));
      if (d >= 0) {
        o.a_hi = static_cast<float>(lp.a[d]);
        o.a_lo = static_cast<float>(lp.a[d] - static_cast<double>(o.a_hi));
        o.b_hi = static_cast<float>(lp.b[d]);
        o.b_lo = static_cast<float>(lp.b[d] - static_cast<double>(o.b_hi));
        q.ridge[d] = lp.ridge[d];
        q.slope[d] = -0.5 / lp.ridge[d];
      }
    }
  }
  // class slots beyond the count repeat class 0 (the kernel variants are built for 1..4 classes,
  // the extended one always loads four)
  for (int c = 0; c < kMaxClasses; ++c) {
    q.off_p[c] = static_cast<uint32_t>(rows_p[c < n_p ? c : 0] * kLutP);   // unused by the extended variant
    q.off_s[c] = static_cast<uint32_t>(rows_s[c < n_s ? c : 0] * kLutS);
  }
  q.K = static_cast<uint32_t>(K);
  q.D = lp.D;
  q.origin_peak = lp.origin_peak;

  auto al = [](const void* ptr, uintptr_t a) { return (reinterpret_cast<uintptr_t>(ptr) & (a - 1)) == 0; };
  const bool metrics = p.has_metrics != nullptr;
  const bool ext = metrics || p.dest_regs != nullptr || p.status != nullptr || many_classes;
  // two records per thread when the inputs sit on 8-byte boundaries; 8-byte stores when the
  // output planes do too (K even)
  const bool vec2 = al(p.num_blocks, 8) && al(p.smem, 8) && al(p.time_ns, 8) && (metrics || al(p.gamma, 8)) &&
                    al(p.block_size, 4) && al(p.regs, 4) && K >= 2;
  const bool aligned = vec2 && K % 2 == 0 && al(p.scaled_ns, 8) && al(p.dest_waves, 8) && al(p.origin_waves, 8) &&
                       al(p.dest_occ, 2) && al(p.origin_occ, 2) && (!p.status || al(p.status, 2)) &&
                       (!p.dest_regs || al(p.dest_regs, 4));
  const int vec = vec2 ? 2 : 1;
  const int64_t blocks = ((K + vec - 1) / vec + kLutThreads - 1) / kLutThreads;
  // One block per 128 threads' worth of records measured fastest at every batch size (the block
  // scheduler balances the tail); HB_LUT_BLOCKS_PER_SM = n caps the grid at n blocks per SM, which
  // then stride over the batch.
  static const int per_sm = [] { const char* e = std::getenv("HB_LUT_BLOCKS_PER_SM"); return e ? std::atoi(e) : 0; }();
  const int64_t cap = per_sm > 0 ? static_cast<int64_t>(sm_count) * per_sm : blocks;
  const unsigned grid = static_cast<unsigned>(blocks < cap ? blocks : cap);
  cudaError_t le;
  if (ext) {
    le = !vec2 ? launch_lut<1, true, true, 1, 1>(grid, stream, p, q)
               : (aligned ? launch_lut<2, true, true, 1, 1>(grid, stream, p, q)
                          : launch_lut<2, true, false, 1, 1>(grid, stream, p, q));
  } else if (!vec2) {
    le = launch_lut<1, false, true, 4, 4>(grid, stream, p, q);
  } else if (!aligned) {
    le = launch_lut<2, false, false, 4, 4>(grid, stream, p, q);
  } else if (p.block_sums && lp.D <= kTotMaxD && grid == blocks) {
    le = launch_lut_plain<true>(n_p, n_s, grid, stream, p, q);
    *fused = true;
    *fused_blocks = grid;
  } else {
    le = launch_lut_plain<false>(n_p, n_s, grid, stream, p, q);
  }
  t_path = 4;
  const cudaError_t ce = le != cudaSuccess ? le : cudaGetLastError();
  *st = ce == cudaSuccess ? HB_OK : hb::cuda_fail(ce, "wave_scale_lut_kernel launch");
  return true;
}

// Division-free kernel when every row of the launch is ordinary and only the five standard
// outputs are wanted; returns false (nothing launched) otherwise.
bool try_launch_fast(const Ptrs& p, const LaunchParams& lp, cudaStream_t stream, hb_status* st) {
  if (p.status || p.limits || lp.D > HB_MAX_DEVICES / 2) return false;
  FastParams fp{};
  {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!fast_row_ok(g_tab.rows[lp.origin_row], g_tab.pre[lp.origin_row])) return false;
    for (int d = 0; d < lp.D; ++d)
      if (!fast_row_ok(g_tab.rows[lp.dest_row[d]], g_tab.pre[lp.dest_row[d]])) return false;
    fp.D = lp.D;
    fp.K = lp.K;
    fp.origin = fold_fast(g_tab.rows[lp.origin_row], g_tab.pre[lp.origin_row]);
    for (int d = 0; d < lp.D; ++d) {
      FastDev& f = fp.dest[d];
      f = fold_fast(g_tab.rows[lp.dest_row[d]], g_tab.pre[lp.dest_row[d]]);
      f.a_hi = static_cast<float>(lp.a[d]);
      f.a_lo = static_cast<float>(lp.a[d] - static_cast<double>(f.a_hi));
      f.b_hi = static_cast<float>(lp.b[d]);
      f.b_lo = static_cast<float>(lp.b[d] - static_cast<double>(f.b_hi));
      f.log2_clk = lp.log2_clk[d];
    }
  }
  const int64_t K = lp.K;
  const bool vec4 = vec4_ok(p, K, true);
  const int threads = 256, vec = vec4 ? 4 : 1;
  const int64_t blocks = ((K + vec - 1) / vec + threads - 1) / threads;
  if (blocks > 0x7FFFFFFF) {
    hb::set_error("hb_wave_scale: K too large for one launch");
    *st = HB_ERR_TOO_LARGE;
    return true;
  }
  const dim3 grid(static_cast<unsigned>(blocks));
  if (vec4) {
    if (p.dest_regs) wave_scale_fast_kernel<4, true><<<grid, threads, 0, stream>>>(p, fp);
    else wave_scale_fast_kernel<4, false><<<grid, threads, 0, stream>>>(p, fp);
  } else {
    if (p.dest_regs) wave_scale_fast_kernel<1, true><<<grid, threads, 0, stream>>>(p, fp);
    else wave_scale_fast_kernel<1, false><<<grid, threads, 0, stream>>>(p, fp);
  }
  t_path = 2;
  const cudaError_t e = cudaGetLastError();
  *st = e == cudaSuccess ? HB_OK : hb::cuda_fail(e, "wave_scale_fast_kernel launch");
  return true;
}

template <bool METRICS>
hb_status launch_kernel(const Ptrs& p, const LaunchParams& lp, cudaStream_t stream, bool* fused,
                        unsigned* fused_blocks) {
  int sm_count = 0;
  const hb_status sync_st = sync_gpu(&sm_count);
  if (sync_st != HB_OK) return sync_st;
  const int64_t K = lp.K;
  const bool extra = p.status != nullptr || p.limits != nullptr;
  hb_status fast_st = HB_OK;
  *fused = false;
  if (try_launch_lut(p, lp, sm_count, stream, &fast_st, fused, fused_blocks)) return fast_st;
  if (!METRICS && try_launch_fast(p, lp, stream, &fast_st)) return fast_st;
  const bool vec4 = vec4_ok(p, K, !METRICS);
  const int threads = 256;
  const int vec = vec4 ? 4 : 1;
  const int64_t nthreads = (K + vec - 1) / vec;
  const int64_t blocks = (nthreads + threads - 1) / threads;
  if (blocks > 0x7FFFFFFF) {
    hb::set_error("hb_wave_scale: K too large for one launch");
    return HB_ERR_TOO_LARGE;
  }
  const dim3 grid(static_cast<unsigned>(blocks));
  if (vec4) {
    if (extra) wave_scale_kernel<4, METRICS, true><<<grid, threads, 0, stream>>>(p, lp);
    else wave_scale_kernel<4, METRICS, false><<<grid, threads, 0, stream>>>(p, lp);
  } else {
    if (extra) wave_scale_kernel<1, METRICS, true><<<grid, threads, 0, stream>>>(p, lp);
    else wave_scale_kernel<1, METRICS, false><<<grid, threads, 0, stream>>>(p, lp);
  }
  t_path = 1;
  HB_CUDA_TRY(cudaGetLastError());
  return HB_OK;
}

// The wave-scaling kernel the launch qualifies for; with p.block_sums also the first stage of the
// per-destination totals: inside the table kernel when it can (per_plane = blocks of its grid),
// else by the plane-sum kernel over the results just written (per_plane = kPlaneBlocks).
template <bool METRICS>
hb_status launch(const Ptrs& p, const LaunchParams& lp, cudaStream_t stream, int32_t* per_plane = nullptr) {
  bool fused = false;
  unsigned fused_blocks = 0;
  const hb_status st = launch_kernel<METRICS>(p, lp, stream, &fused, &fused_blocks);
  if (st != HB_OK || !p.block_sums) return st;
  if (fused) {
    *per_plane = static_cast<int32_t>(fused_blocks);
    return HB_OK;
  }
  HB_CUDA_TRY(hb::launch_overlapped(plane_partial_kernel, dim3(lp.D, kPlaneBlocks), dim3(kSumThreads), 0, stream,
                                    static_cast<const float*>(p.scaled_ns), static_cast<int64_t>(lp.K),
                                    p.block_sums));
  *per_plane = kPlaneBlocks;
  return HB_OK;
}

hb_status fill_params(LaunchParams* lp, int64_t K, int32_t origin_row, const int32_t* dest_rows,
                      int32_t D) {
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_tab.n == 0) {
    hb::set_error("hb_wave_scale: no device table (call hb_set_devices first)");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (K < 0 || D < 1 || D > HB_MAX_DEVICES || !dest_rows || origin_row < 0 ||
      origin_row >= g_tab.n) {
    hb::set_error("hb_wave_scale: bad K/D/origin_row");
    return HB_ERR_INVALID_ARGUMENT;
  }
  std::memset(lp, 0, sizeof(*lp));
  lp->D = D;
  lp->K = K;
  lp->origin_row = origin_row;
  const hb_device_spec& o = g_tab.rows[origin_row];
  lp->origin_peak = static_cast<double>(o.peak_gflops_per_second);
  for (int d = 0; d < D; ++d) {
    const int r = dest_rows[d];
    if (r < 0 || r >= g_tab.n) {
      hb::set_error("hb_wave_scale: destination row %d out of range", r);
      return HB_ERR_INVALID_ARGUMENT;
    }
    const hb_device_spec& t = g_tab.rows[r];
    lp->dest_row[d] = static_cast<uint8_t>(r);
    // wave_scaling/roofline.py:48-57: ratios of the integer device fields
    const double l_bw = std::log2(static_cast<double>(o.mem_bandwidth_gb) / t.mem_bandwidth_gb);
    const double l_clk = std::log2(static_cast<double>(o.base_clock_mhz) / t.base_clock_mhz);
    const double l_sm = std::log2(static_cast<double>(o.num_sms) / t.num_sms);
    lp->b[d] = l_clk + l_sm;
    lp->a[d] = l_bw - lp->b[d];
    lp->log2_clk[d] = l_clk;
    lp->ridge[d] = static_cast<double>(t.peak_gflops_per_second) / t.mem_bandwidth_gb;
  }
  return HB_OK;
}

hb_status check_io(const hb_kernel_soa* k, const hb_wave_out* out, bool need_gamma, int64_t K) {
  if (K == 0 && k && out) return HB_OK;  // nothing to read or write: pointers may be NULL
  if (!k || !out || !k->num_blocks || !k->block_size || !k->regs_per_thread || !k->smem_bytes ||
      !k->run_time_ns || (need_gamma && !k->gamma) || !out->scaled_ns || !out->dest_occupancy ||
      !out->dest_waves || !out->origin_occupancy || !out->origin_waves) {
    hb::set_error("hb_wave_scale: required pointer is NULL");
    return HB_ERR_INVALID_ARGUMENT;
  }
  return HB_OK;
}

Ptrs make_ptrs(const hb_kernel_soa* k, const hb_kernel_metrics* m, const int16_t* dest_regs,
               const hb_wave_out* out) {
  Ptrs p{};
  p.num_blocks = k->num_blocks;
  p.block_size = k->block_size;
  p.regs = k->regs_per_thread;
  p.smem = k->smem_bytes;
  p.time_ns = k->run_time_ns;
  p.gamma = k->gamma;
  if (m) {
    p.flop_eff = m->flop_efficiency_pct;
    p.dram_read = m->dram_read_bytes;
    p.dram_write = m->dram_write_bytes;
    p.has_metrics = m->has_metrics;
  }
  p.dest_regs = dest_regs;
  p.scaled_ns = out->scaled_ns;
  p.dest_occ = out->dest_occupancy;
  p.dest_waves = out->dest_waves;
  p.origin_occ = out->origin_occupancy;
  p.origin_waves = out->origin_waves;
  p.status = out->status;
  p.limits = out->limits;
  return p;
}

}  // namespace

extern "C" int32_t hb_wave_scale_path(void) { return t_path; }

extern "C" hb_status hb_set_devices(const hb_device_spec* rows, int32_t n) {
  if (!rows || n < 1 || n > HB_MAX_DEVICES) {
    hb::set_error("hb_set_devices: need 1..%d rows", HB_MAX_DEVICES);
    return HB_ERR_INVALID_ARGUMENT;
  }
  for (int i = 0; i < n; ++i) {
    if (rows[i].mem_bandwidth_gb <= 0 || rows[i].base_clock_mhz <= 0 || rows[i].num_sms <= 0 ||
        rows[i].peak_gflops_per_second <= 0) {
      hb::set_error("hb_set_devices: row %d has a non-positive bandwidth/clock/SM/peak field", i);
      return HB_ERR_INVALID_ARGUMENT;
    }
  }
  {
    std::lock_guard<std::mutex> lock(g_mu);
    uint32_t magic[kMagicN];
    for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
    bool changed = n != g_tab.n;
    for (int i = 0; i < n; ++i) {
      // a row is folded and tabulated again only when its specification changed (callers append
      // rows one at a time and pass the whole table); rows already on a GPU are left alone
      if (i < g_tab.n && g_tab.row_version[i] != 0 &&
          std::memcmp(&g_tab.rows[i], &rows[i], sizeof(hb_device_spec)) == 0)
        continue;
      g_tab.rows[i] = rows[i];
      g_tab.pre[i] = hb_fold_device(rows[i]);
      g_tab.lut_ok[i] = lut_row_ok(g_tab.rows[i], g_tab.pre[i]);
      uint8_t* pt = &g_tab.lut_p[static_cast<size_t>(i) * kLutP];
      uint8_t* st = &g_tab.lut_s[static_cast<size_t>(i) * kLutS];
      LutOcc* tt = &g_tab.lut_t[static_cast<size_t>(i) * kLutOcc];
      if (g_tab.lut_ok[i]) {
        build_row_lut(g_tab.rows[i], fold_fast(g_tab.rows[i], g_tab.pre[i]), pt, st, tt, magic);
      } else {
        std::memset(pt, 0, kLutP);
        std::memset(st, 0, kLutS);
        std::memset(tt, 0, sizeof(LutOcc) * kLutOcc);
      }
      ++g_tab.row_version[i];
      changed = true;
    }
    g_tab.n = n;
    if (changed) g_version.fetch_add(1, std::memory_order_acq_rel);
  }
  // the current GPU gets its copy now; the others on their first launch.  A process without a
  // GPU keeps the host table only (hb_thread_block_occupancy needs no more).
  int count = 0;
  if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
    cudaGetLastError();   // not an error of this call
    return HB_OK;
  }
  return sync_gpu(nullptr);
}

extern "C" hb_status hb_wave_scale(const hb_kernel_soa* kernels, int64_t K, int32_t origin_row,
                                   const int32_t* dest_rows_host, int32_t D,
                                   const int16_t* dest_regs, const hb_wave_out* out,
                                   void* stream) {
  hb_status st = check_io(kernels, out, true, K);
  if (st != HB_OK) return st;
  LaunchParams lp;
  st = fill_params(&lp, K, origin_row, dest_rows_host, D);
  if (st != HB_OK) return st;
  if (K == 0) return HB_OK;
  return launch<false>(make_ptrs(kernels, nullptr, dest_regs, out), lp,
                       static_cast<cudaStream_t>(stream));
}

extern "C" int64_t hb_wave_scale_partials_len(int64_t K) {
  if (K < 0) return -1;
  const int64_t blocks = ((K + 1) / 2 + kLutThreads - 1) / kLutThreads;
  return blocks > kPlaneBlocks ? blocks : kPlaneBlocks;
}

extern "C" hb_status hb_wave_scale_partials(const hb_kernel_soa* kernels, int64_t K, int32_t origin_row,
                                            const int32_t* dest_rows_host, int32_t D,
                                            const int16_t* dest_regs, const hb_wave_out* out,
                                            double* partials, int32_t* per_plane, void* stream) {
  hb_status st = check_io(kernels, out, true, K);
  if (st != HB_OK) return st;
  if (!per_plane || (K > 0 && !partials)) {
    hb::set_error("hb_wave_scale_partials: partials / per_plane is NULL");
    return HB_ERR_INVALID_ARGUMENT;
  }
  LaunchParams lp;
  st = fill_params(&lp, K, origin_row, dest_rows_host, D);
  if (st != HB_OK) return st;
  *per_plane = 0;
  if (K == 0) return HB_OK;
  Ptrs p = make_ptrs(kernels, nullptr, dest_regs, out);
  p.block_sums = partials;
  return launch<false>(p, lp, static_cast<cudaStream_t>(stream), per_plane);
}

extern "C" hb_status hb_wave_scale_metrics(const hb_kernel_soa* kernels,
                                           const hb_kernel_metrics* metrics, int64_t K,
                                           int32_t origin_row, const int32_t* dest_rows_host,
                                           int32_t D, const int16_t* dest_regs,
                                           const hb_wave_out* out, void* stream) {
  hb_status st = check_io(kernels, out, false, K);
  if (st != HB_OK) return st;
  if (!metrics || (K > 0 && (!metrics->flop_efficiency_pct || !metrics->dram_read_bytes ||
                             !metrics->dram_write_bytes || !metrics->has_metrics))) {
    hb::set_error("hb_wave_scale_metrics: metrics pointer is NULL");
    return HB_ERR_INVALID_ARGUMENT;
  }
  LaunchParams lp;
  st = fill_params(&lp, K, origin_row, dest_rows_host, D);
  if (st != HB_OK) return st;
  if (K == 0) return HB_OK;
  return launch<true>(make_ptrs(kernels, metrics, dest_regs, out), lp,
                      static_cast<cudaStream_t>(stream));
}

extern "C" hb_status hb_wave_scale_host(const hb_kernel_soa* kernels, int64_t K,
                                        int32_t origin_row, const int32_t* dest_rows_host,
                                        int32_t D, const int16_t* dest_regs,
                                        const hb_wave_out* out) {
  hb_status st = check_io(kernels, out, true, K);
  if (st != HB_OK) return st;
  LaunchParams lp;
  st = fill_params(&lp, K, origin_row, dest_rows_host, D);
  if (st != HB_OK) return st;
  if (K == 0) return HB_OK;
  const size_t k = static_cast<size_t>(K), kd = k * D;
  // one staging block per GPU, kept between calls, and the library's own stream
  hb::HostArena* arena = nullptr;
  st = hb::arena_for_current_device(&arena);
  if (st != HB_OK) return st;
  std::lock_guard<std::mutex> lock(arena->mu);
  const size_t lim_bytes = out->limits ? static_cast<size_t>(D + 1) * 4 * k * 4 : 0;
  hb::Carver sizes(nullptr);
  sizes.take<uint8_t>(k * 4); sizes.take<uint8_t>(k * 2); sizes.take<uint8_t>(k * 2); sizes.take<uint8_t>(k * 4);
  sizes.take<uint8_t>(k * 4); sizes.take<uint8_t>(k * 4); sizes.take<uint8_t>(kd * 4); sizes.take<uint8_t>(kd);
  sizes.take<uint8_t>(kd * 4); sizes.take<uint8_t>(k); sizes.take<uint8_t>(k * 4); sizes.take<uint8_t>(kd * 2);
  sizes.take<uint8_t>(kd); sizes.take<uint8_t>(lim_bytes);
  st = hb::arena_reserve(arena, sizes.used());
  if (st != HB_OK) return st;
  hb::Carver c(arena->base);
  int32_t* nb = c.take<int32_t>(k);
  uint16_t* bs = c.take<uint16_t>(k);
  uint16_t* rg = c.take<uint16_t>(k);
  uint32_t* sm = c.take<uint32_t>(k);
  float* tm = c.take<float>(k);
  float* gm = c.take<float>(k);
  float* o_ns = c.take<float>(kd);
  uint8_t* o_occ = c.take<uint8_t>(kd);
  uint32_t* o_wav = c.take<uint32_t>(kd);
  uint8_t* o_oocc = c.take<uint8_t>(k);
  uint32_t* o_owav = c.take<uint32_t>(k);
  int16_t* dr = c.take<int16_t>(kd);
  uint8_t* o_st = c.take<uint8_t>(kd);
  int32_t* o_lim = reinterpret_cast<int32_t*>(c.take<uint8_t>(lim_bytes));
  cudaStream_t s = arena->stream;
  const cudaMemcpyKind h2d = cudaMemcpyHostToDevice, d2h = cudaMemcpyDeviceToHost;
  HB_CUDA_TRY(cudaMemcpyAsync(nb, kernels->num_blocks, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(bs, kernels->block_size, k * 2, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(rg, kernels->regs_per_thread, k * 2, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(sm, kernels->smem_bytes, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(tm, kernels->run_time_ns, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(gm, kernels->gamma, k * 4, h2d, s));
  if (dest_regs) HB_CUDA_TRY(cudaMemcpyAsync(dr, dest_regs, kd * 2, h2d, s));
  hb_kernel_soa dk{nb, bs, rg, sm, tm, gm};
  hb_wave_out dout{o_ns, o_occ, o_wav, o_oocc, o_owav, out->status ? o_st : nullptr,
                   out->limits ? o_lim : nullptr};
  st = launch<false>(make_ptrs(&dk, nullptr, dest_regs ? dr : nullptr, &dout), lp, s);
  if (st != HB_OK) return st;
  HB_CUDA_TRY(cudaMemcpyAsync(out->scaled_ns, o_ns, kd * 4, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->dest_occupancy, o_occ, kd, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->dest_waves, o_wav, kd * 4, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->origin_occupancy, o_oocc, k, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->origin_waves, o_owav, k * 4, d2h, s));
  if (out->status) HB_CUDA_TRY(cudaMemcpyAsync(out->status, o_st, kd, d2h, s));
  if (out->limits) HB_CUDA_TRY(cudaMemcpyAsync(out->limits, o_lim, lim_bytes, d2h, s));
  HB_CUDA_TRY(cudaStreamSynchronize(s));
  return HB_OK;
}

// The occupancy rules are plain integer code that also compiles for the host
// (occupancy.cuh), so a single record needs no GPU: no allocation, no launch, no
// synchronisation, and the call is legal during a stream capture.
extern "C" hb_status hb_thread_block_occupancy(int32_t device_row, int32_t block_size,
                                               uint32_t smem_bytes, int32_t regs_per_thread,
                                               int32_t* occupancy, int32_t limits[4]) {
  if (!occupancy || block_size < 0 || block_size > 0xFFFF || regs_per_thread < 0 ||
      regs_per_thread > 0xFFFF) {
    hb::set_error("hb_thread_block_occupancy: argument out of range");
    return HB_ERR_INVALID_ARGUMENT;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (device_row < 0 || device_row >= g_tab.n) {
    hb::set_error("hb_thread_block_occupancy: device row %d is not in the table (hb_set_devices)", device_row);
    return HB_ERR_INVALID_ARGUMENT;
  }
  int32_t lim[4];
  const int32_t smem = smem_bytes > 0x7FFF0000u ? -1 : static_cast<int32_t>(smem_bytes);
  *occupancy = hb_occupancy(g_tab.pre[device_row], block_size, smem, regs_per_thread, lim);
  if (limits) for (int j = 0; j < 4; ++j) limits[j] = lim[j];
  return HB_OK;
}

#if defined(HB_BOUNDS_CHECK)
extern "C" hb_status hb_bounds_check_word(uint32_t* word, int32_t reset) {
  if (!word) return HB_ERR_INVALID_ARGUMENT;
  HB_CUDA_TRY(cudaDeviceSynchronize());
  HB_CUDA_TRY(cudaMemcpyFromSymbol(word, g_bounds_word, sizeof(uint32_t)));
  if (reset) {
    const uint32_t zero = 0;
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_bounds_word, &zero, sizeof(uint32_t)));
  }
  return HB_OK;
}
#else
extern "C" hb_status hb_bounds_check_word(uint32_t* word, int32_t reset) {
  (void)word; (void)reset;
  hb::set_error("hb_bounds_check_word: this build has no index checks (build with -DHB_BOUNDS_CHECK)");
  return HB_ERR_UNSUPPORTED;
}
#endif
