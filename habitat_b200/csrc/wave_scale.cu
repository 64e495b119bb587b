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
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "hb_common.h"
#include "occupancy.cuh"

namespace {

thread_local int32_t t_path = 0;   // kernel of the last launch, see hb_wave_scale_path

__constant__ hb_dev_pre c_dev[HB_MAX_DEVICES];

// Host mirror of the uploaded table (ratios are formed from the raw rows).
hb_device_spec g_rows[HB_MAX_DEVICES];
hb_dev_pre g_pre[HB_MAX_DEVICES];
int g_n_rows = 0;

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
// Class kernel.  Device rows usually differ in only a few of the fields the
// occupancy rules read (all six benchmark rows share one register file shape,
// two warp budgets and three shared-memory budgets).  The host groups the rows
// of a launch into classes per limit; a thread evaluates each class once per
// kernel record and a destination only picks its three limits and takes the
// minimum.  Up to four classes per limit, no per-destination register
// overrides; anything else takes wave_scale_fast_kernel.
// ---------------------------------------------------------------------------
constexpr int kMaxClasses = 4;

struct ClassDev {
  int32_t num_sms;
  uint32_t sms_magic;
  float a_hi, a_lo, b_hi, b_lo;
  float clk_hi, clk_lo;     // log2 of the clock ratio, split
  uint8_t rc, wc, sc, blocks_limit;
};

struct ClassParams {
  int32_t D, n_rc, n_wc, n_sc;
  int64_t K;
  FastDev cls_r[kMaxClasses], cls_w[kMaxClasses], cls_s[kMaxClasses];
  ClassDev origin;
  ClassDev dest[HB_MAX_DEVICES / 2];
};

// Byte c of a packed word (one permute instruction).
__device__ __forceinline__ int32_t pick_byte(uint32_t packed, uint32_t c) {
  return static_cast<int32_t>(__byte_perm(packed, 0u, 0x4440u | c));
}
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

template <int VEC>
__global__ void __launch_bounds__(128)
wave_scale_class_kernel(const Ptrs p, const __grid_constant__ ClassParams cp) {
  __shared__ uint32_t s_magic[kMagicN];
  __shared__ uint32_t s_wave_magic[HB_MAX_DEVICES / 2 + 1][33];
  __shared__ float2 s_log2[33];   // log2(i) as float hi + lo
  for (int i = threadIdx.x; i < kMagicN; i += blockDim.x) s_magic[i] = g_magic[i];
  for (int i = threadIdx.x; i < (cp.D + 1) * 33; i += blockDim.x) {
    const int d = i / 33, occ = i - d * 33;
    const uint32_t wave = static_cast<uint32_t>((d == 0 ? cp.origin.num_sms : cp.dest[d - 1].num_sms) * occ);
    s_wave_magic[d][occ] = wave >= 2u ? 0xFFFFFFFFu / wave + ((0xFFFFFFFFu % wave) + 1u == wave ? 1u : 0u) + 1u : 0u;
  }
  if (threadIdx.x < 33) {
    const double l = c_log2_int[threadIdx.x];
    const float hi = static_cast<float>(l);
    s_log2[threadIdx.x] = make_float2(hi, static_cast<float>(l - static_cast<double>(hi)));
  }
  __syncthreads();

  const int64_t K = cp.K;
  const int64_t k0 = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) * VEC;
  if (k0 >= K) return;

  const Vec<int32_t, VEC> nbv = load_vec<int32_t, VEC>(p.num_blocks + k0);
  const Vec<uint16_t, VEC> bsv = load_vec<uint16_t, VEC>(p.block_size + k0);
  const Vec<uint16_t, VEC> rgv = load_vec<uint16_t, VEC>(p.regs + k0);
  const Vec<uint32_t, VEC> smv = load_vec<uint32_t, VEC>(p.smem + k0);
  const Vec<float, VEC> tv = load_vec<float, VEC>(p.time_ns + k0);
  const Vec<float, VEC> gv = load_vec<float, VEC>(p.gamma + k0);

  // the class limits of a record, one byte each (values above 255 cannot win the
  // minimum against the blocks-per-SM limit, which is at most 32)
  uint32_t lr[VEC], lw[VEC], ls[VEC];
  int32_t wave_o[VEC];
  float2 lg_o[VEC];   // log2 of the origin's per-SM block count (small-kernel branch)
  Vec<uint8_t, VEC> oocc;
  Vec<uint32_t, VEC> owav;
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    FastKernel k;
    k.block_size = bsv.v[i];
    k.wpb = (k.block_size + 31) >> 5;
    k.regs = rgv.v[i];
    k.rpw_units = (k.regs + 7) >> 3;
    k.smem = smv.v[i] > 0x7FFF0000u ? -1 : static_cast<int32_t>(smv.v[i]);
    k.m_wpb = s_magic[min(k.wpb, kMagicN - 1)];
    const uint32_t m_rpw = s_magic[min(k.rpw_units, kMagicN - 1)];
    lr[i] = lw[i] = ls[i] = 0;
#pragma unroll
    for (int c = 0; c < kMaxClasses; ++c) {
      if (c < cp.n_rc) lr[i] |= static_cast<uint32_t>(min(fast_regs_limit(cp.cls_r[c], k, k.regs, k.rpw_units, m_rpw), 255)) << (8 * c);
      if (c < cp.n_wc) lw[i] |= static_cast<uint32_t>(min(fast_warps_limit(cp.cls_w[c], k), 255)) << (8 * c);
      if (c < cp.n_sc) ls[i] |= static_cast<uint32_t>(min(fast_smem_limit(cp.cls_s[c], k, s_magic), 255)) << (8 * c);
    }
    const int32_t occ = min(min(pick_byte(lr[i], cp.origin.rc), pick_byte(ls[i], cp.origin.sc)),
                            min(pick_byte(lw[i], cp.origin.wc), static_cast<int32_t>(cp.origin.blocks_limit)));
    const int32_t nb = nbv.v[i];
    wave_o[i] = cp.origin.num_sms * occ;
    oocc.v[i] = static_cast<uint8_t>(occ);
    owav.v[i] = (occ > 0 && nb >= 1)
                    ? udiv_magic_fix(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_o[i]),
                                     s_wave_magic[0][occ])
                    : 0xFFFFFFFFu;
    // ceil(nb / num_sms) <= occupancy <= 32 whenever the small-kernel branch is taken
    const uint32_t om = (nb >= 1 && nb < wave_o[i])
                            ? udiv_magic(nb + cp.origin.num_sms - 1, cp.origin.num_sms, cp.origin.sms_magic)
                            : 1u;
    lg_o[i] = s_log2[om];
  }
  store_vec<uint8_t, VEC>(p.origin_occ + k0, oocc);
  store_vec<uint32_t, VEC>(p.origin_waves + k0, owav);

  for (int d = 0; d < cp.D; ++d) {
    const ClassDev& dd = cp.dest[d];
    const int64_t base = static_cast<int64_t>(d) * K + k0;
    const uint32_t rc = dd.rc, wc = dd.wc, sc = dd.sc;
    const int32_t bl = dd.blocks_limit;
    Vec<float, VEC> outv;
    Vec<uint8_t, VEC> occv;
    Vec<uint32_t, VEC> wavv;
#pragma unroll
    for (int i = 0; i < VEC; ++i) {
      const int32_t nb = nbv.v[i];
      const int32_t occ = min(min(pick_byte(lr[i], rc), pick_byte(ls[i], sc)), min(pick_byte(lw[i], wc), bl));
      const int32_t wave_d = dd.num_sms * occ;
      occv.v[i] = static_cast<uint8_t>(occ);
      wavv.v[i] = (occ > 0 && nb >= 1)
                      ? udiv_magic_fix(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_d),
                                       s_wave_magic[d + 1][occ])
                      : 0xFFFFFFFFu;
      const float gamma = gv.v[i];
      const bool live = nb >= 1 && wave_o[i] != 0;
      const bool small = live && nb < wave_o[i] && nb < wave_d;
      const bool ok = live && !(nb < wave_o[i] && wave_d == 0);
      // small kernel (roofline.py:32-45): exponent (1 - gamma) (log2 clk + log2 dmax - log2 omax),
      // both per-SM block counts <= 32; log2 values carried as float hi + lo
      const uint32_t dm = small ? udiv_magic(nb + dd.num_sms - 1, dd.num_sms, dd.sms_magic) : 1u;
      const float2 lg_d = s_log2[dm];
      const float e_small = (1.0f - gamma) * ((lg_d.x - lg_o[i].x) + ((lg_d.y - lg_o[i].y) + dd.clk_lo) + dd.clk_hi);
      const float e_large = fmaf(gamma, dd.a_hi, dd.b_hi) + fmaf(gamma, dd.a_lo, dd.b_lo);
      const float e = small ? e_small : e_large;
      outv.v[i] = ok ? tv.v[i] * ex2_approx(e) : __int_as_float(0x7FC00000);
    }
    store_vec<float, VEC>(p.scaled_ns + base, outv);
    store_vec<uint8_t, VEC>(p.dest_occ + base, occv);
    store_vec<uint32_t, VEC>(p.dest_waves + base, wavv);
  }
}

// ---------------------------------------------------------------------------
// Table kernel.  The three class limits of a record are functions of small
// integers: the register limit of (warps per block, 256-register units per
// warp), the warp limit of the warps per block, the shared-memory limit of the
// request in 128-byte steps.  hb_set_devices tabulates them per device row (one
// byte each: anything above 127 cannot win against the blocks-per-SM limit) in
// global memory; a launch reads the rows that represent its classes through
// L1 (a few KB), so a record costs one byte load per class instead of the limit
// arithmetic, and the kernel needs no shared memory and no block prologue.  The
// reciprocals of the wave sizes (SMs x occupancy) and the log2 pairs of the
// small-kernel branch are tabulated the same way.  A thread owns two consecutive
// records and forms both occupancies of a destination with 16-bit-pair minimum
// instructions.
// Conditions (checked on the host, else the class kernel runs): the class
// kernel's own, plus K even, D K < 2^31, and per row 16 <= SMs, SMs x
// blocks-per-SM limit inside the reciprocal table, thread limit per block a
// multiple of 32 and <= 1024, shared-memory reserve a multiple of 128,
// shared-memory cap below the table's last step, blocks-per-SM limit <= 127.
// ---------------------------------------------------------------------------
constexpr int kLutW = 34;      // warps per block 0..32, 33 = more
constexpr int kLutU = 34;      // register units per warp 0..32, 33 = more than 256 registers
constexpr int kLutS = 2048;    // shared memory in 128-byte steps, last entry = above every cap
constexpr int kLutWPad = 36;

__device__ uint8_t g_lut_r[HB_MAX_DEVICES][kLutW * kLutU];
__device__ uint8_t g_lut_w[HB_MAX_DEVICES][kLutWPad];
__device__ uint8_t g_lut_s[HB_MAX_DEVICES][kLutS];
bool g_lut_ok[HB_MAX_DEVICES];   // host: row tabulated

struct alignas(16) LutDev {       // three 16-byte groups, each fetched with one constant load
  uint32_t sel_r, sel_w, sel_s;   // permute selectors: class byte of record 0 -> low half, record 1 -> high half
  uint32_t bl2;                   // blocks-per-SM limit in both halves
  float a_hi, a_lo, b_hi, b_lo;
  int32_t num_sms;
  uint32_t sms_magic;
  float clk_hi, clk_lo;
};
struct LutDevRegs {               // LutDev as read by a thread
  uint4 sel;                      // sel_r, sel_w, sel_s, bl2
  float4 ab;                      // a_hi, a_lo, b_hi, b_lo
  uint4 sm;                       // num_sms, sms_magic, clk_hi, clk_lo (bits)
};
__device__ __forceinline__ LutDevRegs load_lut_dev(const LutDev& d) {
  LutDevRegs r;
  r.sel = *reinterpret_cast<const uint4*>(&d.sel_r);
  r.ab = *reinterpret_cast<const float4*>(&d.a_hi);
  r.sm = *reinterpret_cast<const uint4*>(&d.num_sms);
  return r;
}

struct LutParams {
  int32_t D, n_rc, n_wc, n_sc;
  int64_t K;
  int32_t row_r[kMaxClasses], row_w[kMaxClasses], row_s[kMaxClasses];   // table rows of the classes
  LutDev origin;
  LutDev dest[HB_MAX_DEVICES / 2];
};

constexpr int kLutThreads = 128;

__device__ float2 g_log2_pair[33];     // log2(i) as float hi + lo; filled by hb_set_devices
constexpr int kWaveMagicN = 8192;      // wave sizes (SMs x occupancy) below this have a tabulated reciprocal
__device__ uint32_t g_wave_magic[kWaveMagicN];

// floor(n / d) for d >= 2 with M = floor(2^32 / d) + 1 and any n < 2^32.
__device__ __forceinline__ uint32_t udiv_fix_ge2(uint32_t n, uint32_t d, uint32_t M) {
  uint32_t q = __umulhi(n, M);
  if (q * d > n) --q;
  return q;
}

// 12 blocks of 128 threads per SM (40 registers) measured fastest (8, 10 and 16 were slower), and
// so did the run-time destination loop against instances unrolled for a known destination count.
__global__ void __launch_bounds__(kLutThreads, 12)
wave_scale_lut_kernel(const Ptrs p, const __grid_constant__ LutParams lp) {
  hb_grid_dependency_wait();
  const int D = lp.D;
  const int64_t K = lp.K;
  const int64_t k0 = (static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x) * 2;
  if (k0 >= K) return;

  const Vec<int32_t, 2> nbv = load_vec<int32_t, 2>(p.num_blocks + k0);
  const Vec<uint16_t, 2> bsv = load_vec<uint16_t, 2>(p.block_size + k0);
  const Vec<uint16_t, 2> rgv = load_vec<uint16_t, 2>(p.regs + k0);
  const Vec<uint32_t, 2> smv = load_vec<uint32_t, 2>(p.smem + k0);
  const Vec<float, 2> tv = load_vec<float, 2>(p.time_ns + k0);
  const Vec<float, 2> gv = load_vec<float, 2>(p.gamma + k0);

  uint32_t lr[2], lw[2], ls[2];
  int32_t wave_o[2];
  float2 lg_o[2];
  float omg[2];
  bool live[2], lt_o[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t wpb = min((static_cast<uint32_t>(bsv.v[i]) + 31u) >> 5, static_cast<uint32_t>(kLutW - 1));
    const uint32_t units = min((static_cast<uint32_t>(rgv.v[i]) + 7u) >> 3, static_cast<uint32_t>(kLutU - 1));
    const uint32_t steps = min((min(smv.v[i], static_cast<uint32_t>(kLutS) << 7) + 127u) >> 7,
                               static_cast<uint32_t>(kLutS - 1));
    uint32_t r = 0, w = 0, sm = 0;
#pragma unroll
    for (int c = 0; c < kMaxClasses; ++c) {
      if (c < lp.n_rc) r |= static_cast<uint32_t>(__ldg(&g_lut_r[lp.row_r[c]][wpb * kLutU + units])) << (8 * c);
      if (c < lp.n_wc) w |= static_cast<uint32_t>(__ldg(&g_lut_w[lp.row_w[c]][wpb])) << (8 * c);
      if (c < lp.n_sc) sm |= static_cast<uint32_t>(__ldg(&g_lut_s[lp.row_s[c]][steps])) << (8 * c);
    }
    lr[i] = r; lw[i] = w; ls[i] = sm;
    omg[i] = 1.0f - gv.v[i];
  }
  // origin: both records at once
  const LutDevRegs og = load_lut_dev(lp.origin);
  const int32_t o_sms = static_cast<int32_t>(og.sm.x);
  const uint32_t o2 = __vimin3_s16x2(
      __vimin3_s16x2(prmt(lr[0], lr[1], og.sel.x), prmt(ls[0], ls[1], og.sel.z), prmt(lw[0], lw[1], og.sel.y)),
      og.sel.w, og.sel.w);
  Vec<uint32_t, 2> owav;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const uint32_t occ = i == 0 ? (o2 & 0xFFFFu) : (o2 >> 16);
    const int32_t nb = nbv.v[i];
    wave_o[i] = o_sms * static_cast<int32_t>(occ);
    owav.v[i] = (occ > 0 && nb >= 1)
                    ? udiv_fix_ge2(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_o[i]),
                                   __ldg(&g_wave_magic[wave_o[i]]))
                    : 0xFFFFFFFFu;
    live[i] = nb >= 1 && occ != 0;
    lt_o[i] = nb < wave_o[i];
    // ceil(nb / num_sms) <= occupancy <= 32 whenever the small-kernel branch is taken
    const uint32_t om = (nb >= 1 && lt_o[i]) ? __umulhi(nb + o_sms - 1, og.sm.y) : 1u;
    lg_o[i] = __ldg(&g_log2_pair[om]);
  }
  *reinterpret_cast<uint16_t*>(p.origin_occ + k0) = static_cast<uint16_t>(__byte_perm(o2, 0u, 0x4420u));
  store_vec<uint32_t, 2>(p.origin_waves + k0, owav);

#pragma unroll 1
  for (int d = 0; d < D; ++d) {
    const LutDevRegs dd = load_lut_dev(lp.dest[d]);
    const int32_t d_sms = static_cast<int32_t>(dd.sm.x);
    const float clk_hi = __uint_as_float(dd.sm.z), clk_lo = __uint_as_float(dd.sm.w);
    const uint32_t base = static_cast<uint32_t>(d) * static_cast<uint32_t>(K) + static_cast<uint32_t>(k0);   // D K < 2^31
    const uint32_t occ2 = __vimin3_s16x2(
        __vimin3_s16x2(prmt(lr[0], lr[1], dd.sel.x), prmt(ls[0], ls[1], dd.sel.z), prmt(lw[0], lw[1], dd.sel.y)),
        dd.sel.w, dd.sel.w);
    Vec<float, 2> outv;
    Vec<uint32_t, 2> wavv;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint32_t occ = i == 0 ? (occ2 & 0xFFFFu) : (occ2 >> 16);
      const int32_t nb = nbv.v[i];
      const int32_t wave_d = d_sms * static_cast<int32_t>(occ);
      wavv.v[i] = (occ > 0 && nb >= 1)
                      ? udiv_fix_ge2(static_cast<uint32_t>(nb), static_cast<uint32_t>(wave_d),
                                     __ldg(&g_wave_magic[wave_d]))
                      : 0xFFFFFFFFu;
      const float gamma = gv.v[i];
      const bool small = live[i] && lt_o[i] && nb < wave_d;
      const bool ok = live[i] && !(lt_o[i] && occ == 0);
      // small kernel (roofline.py:32-45): exponent (1 - gamma) (log2 clk + log2 dmax - log2 omax),
      // both per-SM block counts <= 32; log2 values carried as float hi + lo
      const uint32_t dm = small ? __umulhi(nb + d_sms - 1, dd.sm.y) : 1u;
      const float2 lg_d = __ldg(&g_log2_pair[dm]);
      const float e_small = omg[i] * ((lg_d.x - lg_o[i].x) + ((lg_d.y - lg_o[i].y) + clk_lo) + clk_hi);
      const float e_large = fmaf(gamma, dd.ab.x, dd.ab.z) + fmaf(gamma, dd.ab.y, dd.ab.w);
      const float e = small ? e_small : e_large;
      outv.v[i] = ok ? tv.v[i] * ex2_approx(e) : __int_as_float(0x7FC00000);
    }
    store_vec<float, 2>(p.scaled_ns + base, outv);
    *reinterpret_cast<uint16_t*>(p.dest_occ + base) = static_cast<uint16_t>(__byte_perm(occ2, 0u, 0x4420u));
    store_vec<uint32_t, 2>(p.dest_waves + base, wavv);
  }
}

// Finds (or appends) the class of `f` under `same`; returns -1 when full.
template <typename Same>
int class_of(FastDev* classes, int32_t* n, const FastDev& f, Same same) {
  for (int c = 0; c < *n; ++c)
    if (same(classes[c], f)) return c;
  if (*n >= kMaxClasses) return -1;
  classes[*n] = f;
  return (*n)++;
}

bool build_class_params(const FastParams& fp, ClassParams* cp) {
  std::memset(cp, 0, sizeof(*cp));
  cp->D = fp.D;
  cp->K = fp.K;
  for (int d = -1; d < fp.D; ++d) {
    const FastDev& f = d < 0 ? fp.origin : fp.dest[d];
    ClassDev& c = d < 0 ? cp->origin : cp->dest[d];
    const int rc = class_of(cp->cls_r, &cp->n_rc, f, same_regs_class);
    const int wc = class_of(cp->cls_w, &cp->n_wc, f, same_warps_class);
    const int sc = class_of(cp->cls_s, &cp->n_sc, f, same_smem_class);
    if (rc < 0 || wc < 0 || sc < 0 || f.blocks_limit > 255) return false;
    c.rc = static_cast<uint8_t>(rc);
    c.wc = static_cast<uint8_t>(wc);
    c.sc = static_cast<uint8_t>(sc);
    c.blocks_limit = static_cast<uint8_t>(f.blocks_limit);
    c.num_sms = f.num_sms;
    c.sms_magic = f.sms_magic;
    c.a_hi = f.a_hi; c.a_lo = f.a_lo; c.b_hi = f.b_hi; c.b_lo = f.b_lo;
    c.clk_hi = static_cast<float>(f.log2_clk);
    c.clk_lo = static_cast<float>(f.log2_clk - static_cast<double>(c.clk_hi));
  }
  return true;
}

// Whether a row can be tabulated for wave_scale_lut_kernel.
bool lut_row_ok(const hb_device_spec& s, const hb_dev_pre& pre) {
  return fast_row_ok(s, pre) && s.num_sms >= 16 && s.num_sms * pre.blocks_limit < kWaveMagicN && pre.max_threads_per_block % 32 == 0 &&
         pre.max_threads_per_block <= 1024 && pre.smem_reserved % 128 == 0 &&
         pre.smem_cap <= (kLutS - 2) * 128 && pre.blocks_limit <= 127;
}

// Tabulates the three limits of one device row (host side of hb_set_devices).
void build_row_lut(const FastDev& f, uint8_t* r, uint8_t* w, uint8_t* sm, const uint32_t* magic) {
  auto clamp = [](int32_t v) { return static_cast<uint8_t>(v < 0 ? 0 : (v > 127 ? 127 : v)); };
  for (int wpb = 0; wpb < kLutW; ++wpb) {
    FastKernel k{};
    k.block_size = wpb * 32;
    k.wpb = wpb;
    k.m_wpb = magic_of(static_cast<uint32_t>(wpb));
    w[wpb] = clamp(fast_warps_limit(f, k));
    for (int u = 0; u < kLutU; ++u) {
      k.regs = u * 8;          // any count with this many 256-register units per warp
      k.rpw_units = u;
      r[wpb * kLutU + u] = wpb == 0 ? 0 : clamp(fast_regs_limit(f, k, k.regs, u, magic_of(static_cast<uint32_t>(u))));
    }
  }
  for (int i = kLutW; i < kLutWPad; ++i) w[i] = 0;
  for (int st = 0; st < kLutS; ++st) {
    FastKernel k{};
    k.smem = st * 128;         // the largest request of this 128-byte step
    sm[st] = st == kLutS - 1 ? 0 : clamp(fast_smem_limit(f, k, magic));
  }
}

uint32_t pair_selector(int c) {
  const uint32_t lo = static_cast<uint32_t>(c), hi = static_cast<uint32_t>(4 + c);
  return lo | ((8u | lo) << 4) | (hi << 8) | ((8u | hi) << 12);
}

// Launches wave_scale_lut_kernel when the launch qualifies; false = nothing launched.
bool try_launch_lut(const Ptrs& p, const FastParams& fp, const ClassParams& cp, const LaunchParams& lp,
                    cudaStream_t stream, hb_status* st) {
  const int64_t K = fp.K;
  auto al = [](const void* q, uintptr_t a) { return (reinterpret_cast<uintptr_t>(q) & (a - 1)) == 0; };
  if (K % 2 != 0 || !al(p.num_blocks, 8) || !al(p.smem, 8) || !al(p.time_ns, 8) || !al(p.gamma, 8) ||
      !al(p.block_size, 4) || !al(p.regs, 4) || !al(p.scaled_ns, 8) || !al(p.dest_waves, 8) ||
      !al(p.origin_waves, 8) || !al(p.dest_occ, 2) || !al(p.origin_occ, 2))
    return false;
  if (static_cast<int64_t>(lp.D) * K >= (int64_t{1} << 31)) return false;   // 32-bit element indices
  if (!g_lut_ok[lp.origin_row]) return false;
  for (int d = 0; d < lp.D; ++d)
    if (!g_lut_ok[lp.dest_row[d]]) return false;

  LutParams q{};
  q.D = cp.D; q.K = K; q.n_rc = cp.n_rc; q.n_wc = cp.n_wc; q.n_sc = cp.n_sc;
  // a class is represented by the first row of the launch that belongs to it
  bool have_r[kMaxClasses] = {}, have_w[kMaxClasses] = {}, have_s[kMaxClasses] = {};
  for (int d = -1; d < lp.D; ++d) {
    const ClassDev& c = d < 0 ? cp.origin : cp.dest[d];
    const int row = d < 0 ? lp.origin_row : lp.dest_row[d];
    if (!have_r[c.rc]) { have_r[c.rc] = true; q.row_r[c.rc] = row; }
    if (!have_w[c.wc]) { have_w[c.wc] = true; q.row_w[c.wc] = row; }
    if (!have_s[c.sc]) { have_s[c.sc] = true; q.row_s[c.sc] = row; }
    LutDev& o = d < 0 ? q.origin : q.dest[d];
    o.num_sms = c.num_sms; o.sms_magic = c.sms_magic;
    o.a_hi = c.a_hi; o.a_lo = c.a_lo; o.b_hi = c.b_hi; o.b_lo = c.b_lo;
    o.clk_hi = c.clk_hi; o.clk_lo = c.clk_lo;
    o.sel_r = pair_selector(c.rc); o.sel_w = pair_selector(c.wc); o.sel_s = pair_selector(c.sc);
    o.bl2 = static_cast<uint32_t>(c.blocks_limit) * 0x00010001u;
  }

  const int64_t blocks = (K / 2 + kLutThreads - 1) / kLutThreads;
  if (blocks > 0x7FFFFFFF || blocks < 1) return false;
  const unsigned grid = static_cast<unsigned>(blocks);
  // 12 blocks of 128 threads per SM (40 registers) measured fastest; 8, 10 and 16 were slower
  const cudaError_t le = hb::launch_overlapped(wave_scale_lut_kernel, dim3(grid), dim3(kLutThreads), 0, stream, p, q);
  t_path = 4;
  const cudaError_t ce = le != cudaSuccess ? le : cudaGetLastError();
  *st = ce == cudaSuccess ? HB_OK : hb::cuda_fail(ce, "wave_scale_lut_kernel launch");
  return true;
}

// Fast path when every row of the launch qualifies and only the five standard
// outputs are wanted; returns false (nothing launched) otherwise.
bool try_launch_fast(const Ptrs& p, const LaunchParams& lp, cudaStream_t stream, hb_status* st) {
  if (p.status || p.limits || lp.D > HB_MAX_DEVICES / 2) return false;
  if (!fast_row_ok(g_rows[lp.origin_row], g_pre[lp.origin_row])) return false;
  for (int d = 0; d < lp.D; ++d)
    if (!fast_row_ok(g_rows[lp.dest_row[d]], g_pre[lp.dest_row[d]])) return false;
  FastParams fp{};
  fp.D = lp.D;
  fp.K = lp.K;
  fp.origin = fold_fast(g_rows[lp.origin_row], g_pre[lp.origin_row]);
  for (int d = 0; d < lp.D; ++d) {
    FastDev& f = fp.dest[d];
    f = fold_fast(g_rows[lp.dest_row[d]], g_pre[lp.dest_row[d]]);
    f.a_hi = static_cast<float>(lp.a[d]);
    f.a_lo = static_cast<float>(lp.a[d] - static_cast<double>(f.a_hi));
    f.b_hi = static_cast<float>(lp.b[d]);
    f.b_lo = static_cast<float>(lp.b[d] - static_cast<double>(f.b_hi));
    f.log2_clk = lp.log2_clk[d];
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
  ClassParams cp;
  if (!p.dest_regs && build_class_params(fp, &cp)) {
    static const bool use_lut = [] { const char* e = std::getenv("HB_WAVE_LUT"); return !e || std::atoi(e) != 0; }();
    if (use_lut && try_launch_lut(p, fp, cp, lp, stream, st)) return true;
    const int cthreads = 128;
    static const int vec_pref = [] { const char* e = std::getenv("HB_WAVE_VEC"); return e ? std::atoi(e) : 2; }();
    // two records per thread measured fastest (more resident warps than four per thread)
    const int cvec = vec4 ? (vec_pref == 4 ? 4 : (vec_pref == 1 ? 1 : 2)) : 1;
    const int64_t cblocks = ((K + cvec - 1) / cvec + cthreads - 1) / cthreads;
    if (cblocks <= 0x7FFFFFFF) {
      if (cvec == 4) wave_scale_class_kernel<4><<<static_cast<unsigned>(cblocks), cthreads, 0, stream>>>(p, cp);
      else if (cvec == 2) wave_scale_class_kernel<2><<<static_cast<unsigned>(cblocks), cthreads, 0, stream>>>(p, cp);
      else wave_scale_class_kernel<1><<<static_cast<unsigned>(cblocks), cthreads, 0, stream>>>(p, cp);
      t_path = 3;
      const cudaError_t ce = cudaGetLastError();
      *st = ce == cudaSuccess ? HB_OK : hb::cuda_fail(ce, "wave_scale_class_kernel launch");
      return true;
    }
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
hb_status launch(const Ptrs& p, const LaunchParams& lp, cudaStream_t stream) {
  const int64_t K = lp.K;
  const bool extra = p.status != nullptr || p.limits != nullptr;
  if (!METRICS) {
    hb_status fast_st = HB_OK;
    if (try_launch_fast(p, lp, stream, &fast_st)) return fast_st;
  }
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

hb_status fill_params(LaunchParams* lp, int64_t K, int32_t origin_row, const int32_t* dest_rows,
                      int32_t D) {
  if (g_n_rows == 0) {
    hb::set_error("hb_wave_scale: no device table (call hb_set_devices first)");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (K < 0 || D < 1 || D > HB_MAX_DEVICES || !dest_rows || origin_row < 0 ||
      origin_row >= g_n_rows) {
    hb::set_error("hb_wave_scale: bad K/D/origin_row");
    return HB_ERR_INVALID_ARGUMENT;
  }
  std::memset(lp, 0, sizeof(*lp));
  lp->D = D;
  lp->K = K;
  lp->origin_row = origin_row;
  const hb_device_spec& o = g_rows[origin_row];
  lp->origin_peak = static_cast<double>(o.peak_gflops_per_second);
  for (int d = 0; d < D; ++d) {
    const int r = dest_rows[d];
    if (r < 0 || r >= g_n_rows) {
      hb::set_error("hb_wave_scale: destination row %d out of range", r);
      return HB_ERR_INVALID_ARGUMENT;
    }
    const hb_device_spec& t = g_rows[r];
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
    g_rows[i] = rows[i];
    g_pre[i] = hb_fold_device(rows[i]);
  }
  g_n_rows = n;
  HB_CUDA_TRY(cudaMemcpyToSymbol(c_dev, g_pre, sizeof(hb_dev_pre) * n));
  double lg[65];
  lg[0] = 0.0;
  for (int i = 1; i <= 64; ++i) lg[i] = std::log2(static_cast<double>(i));
  HB_CUDA_TRY(cudaMemcpyToSymbol(c_log2_int, lg, sizeof(lg)));
  uint32_t magic[kMagicN];
  for (int i = 0; i < kMagicN; ++i) magic[i] = magic_of(static_cast<uint32_t>(i));
  HB_CUDA_TRY(cudaMemcpyToSymbol(g_magic, magic, sizeof(magic)));
  {
    // Host copies of the tables persist between calls: a row is tabulated again only when its
    // specification changed (callers append rows one at a time and upload the whole table).
    static std::vector<uint8_t> r(static_cast<size_t>(HB_MAX_DEVICES) * kLutW * kLutU),
        w(static_cast<size_t>(HB_MAX_DEVICES) * kLutWPad), sm(static_cast<size_t>(HB_MAX_DEVICES) * kLutS);
    static hb_device_spec built[HB_MAX_DEVICES];
    static bool have[HB_MAX_DEVICES] = {};
    for (int i = 0; i < n; ++i) {
      if (have[i] && std::memcmp(&built[i], &g_rows[i], sizeof(hb_device_spec)) == 0) continue;
      built[i] = g_rows[i];
      have[i] = true;
      g_lut_ok[i] = lut_row_ok(g_rows[i], g_pre[i]);
      uint8_t* ri = &r[static_cast<size_t>(i) * kLutW * kLutU];
      uint8_t* wi = &w[static_cast<size_t>(i) * kLutWPad];
      uint8_t* si = &sm[static_cast<size_t>(i) * kLutS];
      if (g_lut_ok[i]) {
        build_row_lut(fold_fast(g_rows[i], g_pre[i]), ri, wi, si, magic);
      } else {
        std::memset(ri, 0, kLutW * kLutU);
        std::memset(wi, 0, kLutWPad);
        std::memset(si, 0, kLutS);
      }
    }
    float2 lp2[33];
    for (int i = 0; i < 33; ++i) {
      const float hi = static_cast<float>(lg[i]);
      lp2[i] = make_float2(hi, static_cast<float>(lg[i] - static_cast<double>(hi)));
    }
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_log2_pair, lp2, sizeof(lp2)));
    std::vector<uint32_t> wm(kWaveMagicN);
    for (int i = 0; i < kWaveMagicN; ++i) wm[i] = magic_of(static_cast<uint32_t>(i));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_wave_magic, wm.data(), wm.size() * sizeof(uint32_t)));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_r, r.data(), static_cast<size_t>(n) * kLutW * kLutU));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_w, w.data(), static_cast<size_t>(n) * kLutWPad));
    HB_CUDA_TRY(cudaMemcpyToSymbol(g_lut_s, sm.data(), static_cast<size_t>(n) * kLutS));
  }
  return HB_OK;
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

namespace {

// Scoped device buffer for the host-buffer entry points.
struct DevBuf {
  void* p = nullptr;
  ~DevBuf() { if (p) cudaFree(p); }
  cudaError_t alloc(size_t n) { return cudaMalloc(&p, n ? n : 1); }
  template <typename T> T* as() { return static_cast<T*>(p); }
};

}  // namespace

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
  cudaStream_t s = nullptr;
  DevBuf nb, bs, rg, sm, tm, gm, dr, o_ns, o_occ, o_wav, o_oocc, o_owav, o_st, o_lim;
  HB_CUDA_TRY(nb.alloc(k * 4)); HB_CUDA_TRY(bs.alloc(k * 2)); HB_CUDA_TRY(rg.alloc(k * 2));
  HB_CUDA_TRY(sm.alloc(k * 4)); HB_CUDA_TRY(tm.alloc(k * 4)); HB_CUDA_TRY(gm.alloc(k * 4));
  HB_CUDA_TRY(o_ns.alloc(kd * 4)); HB_CUDA_TRY(o_occ.alloc(kd)); HB_CUDA_TRY(o_wav.alloc(kd * 4));
  HB_CUDA_TRY(o_oocc.alloc(k)); HB_CUDA_TRY(o_owav.alloc(k * 4));
  if (dest_regs) HB_CUDA_TRY(dr.alloc(kd * 2));
  if (out->status) HB_CUDA_TRY(o_st.alloc(kd));
  if (out->limits) HB_CUDA_TRY(o_lim.alloc(static_cast<size_t>(D + 1) * 4 * k * 4));
  const cudaMemcpyKind h2d = cudaMemcpyHostToDevice, d2h = cudaMemcpyDeviceToHost;
  HB_CUDA_TRY(cudaMemcpyAsync(nb.p, kernels->num_blocks, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(bs.p, kernels->block_size, k * 2, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(rg.p, kernels->regs_per_thread, k * 2, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(sm.p, kernels->smem_bytes, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(tm.p, kernels->run_time_ns, k * 4, h2d, s));
  HB_CUDA_TRY(cudaMemcpyAsync(gm.p, kernels->gamma, k * 4, h2d, s));
  if (dest_regs) HB_CUDA_TRY(cudaMemcpyAsync(dr.p, dest_regs, kd * 2, h2d, s));
  hb_kernel_soa dk{nb.as<int32_t>(), bs.as<uint16_t>(), rg.as<uint16_t>(), sm.as<uint32_t>(),
                   tm.as<float>(), gm.as<float>()};
  hb_wave_out dout{o_ns.as<float>(), o_occ.as<uint8_t>(), o_wav.as<uint32_t>(),
                   o_oocc.as<uint8_t>(), o_owav.as<uint32_t>(),
                   out->status ? o_st.as<uint8_t>() : nullptr,
                   out->limits ? o_lim.as<int32_t>() : nullptr};
  st = launch<false>(make_ptrs(&dk, nullptr, dest_regs ? dr.as<int16_t>() : nullptr, &dout), lp, s);
  if (st != HB_OK) return st;
  HB_CUDA_TRY(cudaMemcpyAsync(out->scaled_ns, o_ns.p, kd * 4, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->dest_occupancy, o_occ.p, kd, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->dest_waves, o_wav.p, kd * 4, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->origin_occupancy, o_oocc.p, k, d2h, s));
  HB_CUDA_TRY(cudaMemcpyAsync(out->origin_waves, o_owav.p, k * 4, d2h, s));
  if (out->status) HB_CUDA_TRY(cudaMemcpyAsync(out->status, o_st.p, kd, d2h, s));
  if (out->limits)
    HB_CUDA_TRY(cudaMemcpyAsync(out->limits, o_lim.p, static_cast<size_t>(D + 1) * 4 * k * 4, d2h, s));
  HB_CUDA_TRY(cudaStreamSynchronize(s));
  return HB_OK;
}

extern "C" hb_status hb_thread_block_occupancy(int32_t device_row, int32_t block_size,
                                               uint32_t smem_bytes, int32_t regs_per_thread,
                                               int32_t* occupancy, int32_t limits[4]) {
  if (!occupancy || block_size < 0 || block_size > 0xFFFF || regs_per_thread < 0 ||
      regs_per_thread > 0xFFFF) {
    hb::set_error("hb_thread_block_occupancy: argument out of range");
    return HB_ERR_INVALID_ARGUMENT;
  }
  // One record through the batched kernel, with the queried row as origin.
  int32_t nb = 1;
  uint16_t bs = static_cast<uint16_t>(block_size), rg = static_cast<uint16_t>(regs_per_thread);
  float t = 1.0f, g = 1.0f;
  hb_kernel_soa k{&nb, &bs, &rg, &smem_bytes, &t, &g};
  float ns;
  uint8_t docc, oocc;
  uint32_t dw, ow;
  int32_t lim[8];
  hb_wave_out out{&ns, &docc, &dw, &oocc, &ow, nullptr, lim};
  const int32_t dest = device_row;
  hb_status st = hb_wave_scale_host(&k, 1, device_row, &dest, 1, nullptr, &out);
  if (st != HB_OK) return st;
  *occupancy = oocc;
  if (limits) for (int j = 0; j < 4; ++j) limits[j] = lim[j];
  return HB_OK;
}
