/*
 * CPU oracle for Habitat's batched prediction path -- TEST INFRASTRUCTURE ONLY.
 * See habitat_oracle.h for what this file is and how it is pinned.
 *
 * The occupancy routine restates, in its own words, the behaviour of NVIDIA's
 * standalone occupancy calculator under the fixed call convention Habitat uses
 * (cpp/src/cuda/kernel.cpp:33-56): partitioned global caching off, default
 * shared-memory limit (no opt-in), default carve-out and cache preference,
 * unlimited per-function block size and dynamic shared memory.
 *   - compute capability 3/5/6/7 follows the header vendored by the reference
 *     (cpp/src/cuda/cuda_occupancy.h: limits :1016-1282, constants :573-746,
 *     per-block cap :866-897, driver :1288-1420);
 *   - compute capability 8/9/10/12, which that header rejects, follows the
 *     CUDA 12.9 toolkit header (include/cuda_occupancy.h) under the same
 *     convention, with its reservedSharedMemPerBlock device field.
 */
#include "habitat_oracle.h"

#include <limits.h>
#include <math.h>
#include <stddef.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static int div_up(int x, int y) { return (x + (y - 1)) / y; }
static int round_up(int x, int y) { return y * div_up(x, y); }
static int imin(int a, int b) { return b < a ? b : a; }

#define KB(x) ((int64_t)(x) * 1024)

/* Shared memory carve-out sizes an SM can be configured to; returns -1 when
 * the request is beyond the largest size (an error in the calculator). */
static int64_t carveout_snap(const hbo_device* d, int64_t size) {
  static const int64_t volta_like[] = {0, 8, 16, 32, 64};
  int major = d->compute_major, minor = d->compute_minor;
  if (major == 7) {
    /* cuda_occupancy.h:699-746 (reference): anything above the ladder snaps to
     * the device's own per-SM figure, never an error. */
    if (minor == 5) return size <= KB(32) ? KB(32) : d->shared_mem_per_multiprocessor;
    for (int i = 0; i < 5; ++i)
      if (size <= KB(volta_like[i])) return KB(volta_like[i]);
    return d->shared_mem_per_multiprocessor;
  }
  int64_t top[6];
  int ntop = 0;
  if (major == 8) {
    top[ntop++] = 100;
    if (minor == 0 || minor == 7) { top[ntop++] = 132; top[ntop++] = 164; }
  } else if (major == 9 || (major == 10 && (minor == 0 || minor == 1 || minor == 3))) {
    top[ntop++] = 100; top[ntop++] = 132; top[ntop++] = 164;
    top[ntop++] = 196; top[ntop++] = 228;
  } else if (major == 12 && (minor == 0 || minor == 1)) {
    top[ntop++] = 100;
  } else {
    return -1;
  }
  for (int i = 0; i < 5; ++i)
    if (size <= KB(volta_like[i])) return KB(volta_like[i]);
  for (int i = 0; i < ntop; ++i)
    if (size <= KB(top[i])) return KB(top[i]);
  return -1;
}

static int max_blocks_per_sm(const hbo_device* d) {
  switch (d->compute_major) {
    case 3: return 16;
    case 5: case 6: return 32;
    case 7: return d->compute_minor == 5 ? 16 : 32;
    case 8: return d->compute_minor == 0 ? 32 : (d->compute_minor == 9 ? 24 : 16);
    case 9: return 32;
    case 10: return d->compute_minor == 1 ? 24 : 32;
    case 12: return 24;
    default: return -1;
  }
}

static int regs_limit(const hbo_device* d, int block_size, int regs, int parts) {
  /* 256 registers per thread is the cap on every supported part: in the
   * reference header the 3/5/6 case falls through into the 7/8 case
   * (cuda_occupancy.h:600-608).  Tested first so that the products below
   * cannot overflow; the reference's three conditions are or-ed. */
  if (regs > 256) return 0;
  int wpb = div_up(block_size, d->warp_size);
  int rpw = round_up(regs * d->warp_size, 256);
  int64_t per_cta = (int64_t)rpw * wpb;
  int64_t assumed = (int64_t)rpw * round_up(wpb, parts);
  if (d->regs_per_block < assumed || d->regs_per_block < per_cta) return 0;
  if (rpw <= 0) return INT_MAX;
  int warps_per_part = (d->regs_per_multiprocessor / parts) / rpw;
  return (warps_per_part * parts) / wpb;
}

int hbo_occupancy(const hbo_device* d, int block_size, int64_t smem_total,
                  int regs, int limits[4]) {
  int lim[4] = {0, 0, 0, 0};
  int occ = 0;
  int major = d->compute_major;
  int known = major == 3 || (major >= 5 && major <= 10) || major == 12;
  if (limits) { limits[0] = limits[1] = limits[2] = limits[3] = 0; }

  if (block_size <= 0 || regs < 0) return 0;
  if (d->max_threads_per_block <= 0 || d->max_threads_per_multiprocessor <= 0 ||
      d->regs_per_block <= 0 || d->regs_per_multiprocessor <= 0 ||
      d->warp_size <= 0 || d->shared_mem_per_block <= 0 ||
      d->shared_mem_per_multiprocessor <= 0 || d->num_sms <= 0)
    return 0;
  if (!known) return 0;

  /* registers (cuda_occupancy.h:1164-1282; GP100 re-check :1344-1361) */
  int parts = (major == 6 && d->compute_minor == 0) ? 2 : 4;
  lim[0] = regs_limit(d, block_size, regs, parts);
  if (major == 6 && d->compute_minor == 0 && lim[0] != 0) {
    if (regs_limit(d, block_size, regs, 4) == 0) lim[0] = 0;
  }

  /* warps (cuda_occupancy.h:1016-1062) */
  int wpb = div_up(block_size, d->warp_size);
  lim[1] = block_size > d->max_threads_per_block
               ? 0
               : (d->max_threads_per_multiprocessor / d->warp_size) / wpb;

  /* blocks (cuda_occupancy.h:670-694) */
  lim[2] = max_blocks_per_sm(d);

  /* shared memory (cuda_occupancy.h:1066-1162) */
  {
    int gran = major >= 8 ? 128 : 256;
    int64_t reserved = major >= 8 ? d->reserved_shared_mem_per_block : 0;
    /* The calculator rounds in `int`; requests near 2 GiB wrap negative there
     * and end up above the cap, so they are cut off here instead. */
    int64_t alloc = smem_total > 0x7FFF0000LL ? INT64_MAX
                                              : round_up((int)(smem_total + reserved), gran);
    int64_t cap = (int64_t)d->shared_mem_per_block + reserved;
    /* The configured carve-out is resolved before anything else; a device whose
     * per-SM size is beyond its architecture's ladder is an error outright. */
    int64_t pref = major >= 7 ? carveout_snap(d, d->shared_mem_per_multiprocessor) : 0;
    if (pref < 0) return 0;
    if (smem_total < 0 || alloc > cap) {
      lim[3] = 0;
    } else {
      int64_t budget;
      if (major >= 7) {
        if (pref >= alloc) {
          budget = pref;
        } else {
          budget = carveout_snap(d, alloc);
          if (budget < 0) return 0;
        }
      } else {
        budget = d->shared_mem_per_multiprocessor;
      }
      lim[3] = alloc > 0 ? (int)(budget / alloc) : INT_MAX;
    }
  }

  occ = imin(lim[0], imin(lim[3], imin(lim[1], lim[2])));
  if (limits) { limits[0] = lim[0]; limits[1] = lim[1]; limits[2] = lim[2]; limits[3] = lim[3]; }
  return occ;
}

double hbo_roofline_gamma(double flop_efficiency, double dram_read_bytes,
                          double dram_write_bytes, double run_time_ns,
                          const hbo_device* origin, const hbo_device* dest) {
  /* wave_scaling/roofline.py:68-104, same operation order */
  double total_gb = (dram_read_bytes + dram_write_bytes) / 1024 / 1024 / 1024;
  double gflops_per_second = flop_efficiency / 100 * (double)origin->peak_gflops_per_second;
  double num_gflops = gflops_per_second * run_time_ns / 1e9;
  if (num_gflops < 1e-9) return 1.0;
  if (total_gb == 0) return 0.0;
  double intensity = num_gflops / total_gb;
  double ridge = (double)dest->peak_gflops_per_second / (double)dest->mem_bandwidth_gb;
  if (intensity > ridge) return 0.5 * ridge / intensity;
  return -0.5 / ridge * intensity + 1.0;
}

int hbo_wave_scale_pair(const hbo_device* origin, const hbo_device* dest,
                        int32_t num_blocks, int block_size, int64_t smem_total,
                        int regs, int dest_regs, double run_time_ns,
                        double gamma, double* scaled_ns, int* origin_occ,
                        int* dest_occ, int64_t* origin_waves,
                        int64_t* dest_waves) {
  /* wave_scaling/common.py:3-20 */
  int occ_o = hbo_occupancy(origin, block_size, smem_total, regs, NULL);
  int occ_d = hbo_occupancy(dest, block_size, smem_total,
                            dest_regs >= 0 ? dest_regs : regs, NULL);
  int64_t wave_o = (int64_t)origin->num_sms * occ_o;
  int64_t wave_d = (int64_t)dest->num_sms * occ_d;
  double gamma_compl = 1.0 - gamma;
  int status;
  double out = NAN;

  if (origin_occ) *origin_occ = occ_o;
  if (dest_occ) *dest_occ = occ_d;
  if (origin_waves) *origin_waves = wave_o > 0 && num_blocks >= 1 ? num_blocks / wave_o : -1;
  if (dest_waves) *dest_waves = wave_d > 0 && num_blocks >= 1 ? num_blocks / wave_d : -1;

  if (num_blocks < 1) {
    status = HBO_ERR_INPUT;
  } else if (wave_o == 0) {
    /* `kernel.num_blocks // origin_wave_size` divides by zero (roofline.py:29) */
    status = HBO_ERR_ZERO_WAVE;
  } else if (num_blocks / wave_o == 0) {
    /* the `and` short-circuit reaches the second division (roofline.py:30) */
    if (wave_d == 0) {
      status = HBO_ERR_ZERO_WAVE;
    } else if (num_blocks / wave_d == 0) {
      /* roofline.py:32-45 */
      double origin_max = ceil((double)num_blocks / (double)origin->num_sms);
      double dest_max = ceil((double)num_blocks / (double)dest->num_sms);
      double partial = ((double)origin->base_clock_mhz / (double)dest->base_clock_mhz) *
                       (dest_max / origin_max);
      out = run_time_ns * pow(partial, gamma_compl);
      status = HBO_OK_SMALL;
    } else {
      status = HBO_OK_LARGE;
    }
  } else {
    status = HBO_OK_LARGE;
  }

  if (status == HBO_OK_LARGE) {
    /* roofline.py:48-65 */
    double bw = (double)origin->mem_bandwidth_gb / (double)dest->mem_bandwidth_gb;
    double clk = (double)origin->base_clock_mhz / (double)dest->base_clock_mhz;
    double sm = (double)origin->num_sms / (double)dest->num_sms;
    out = run_time_ns * pow(bw, gamma) * pow(clk, gamma_compl) * pow(sm, gamma_compl);
  }
  if (scaled_ns) *scaled_ns = out;
  return status;
}

int hbo_wave_scale_batch(const hbo_device* devices, int origin_row,
                         const int32_t* dest_rows, int D, int64_t K,
                         const int32_t* num_blocks, const uint16_t* block_size,
                         const uint16_t* regs, const uint32_t* smem_total,
                         const double* run_time_ns, const float* gamma,
                         const int16_t* dest_regs, double* scaled_ns,
                         uint8_t* dest_occ, uint32_t* dest_waves,
                         uint8_t* origin_occ, uint32_t* origin_waves,
                         uint8_t* status, int32_t* limits) {
  const hbo_device* origin = &devices[origin_row];
  int nthreads = 1;
#ifdef _OPENMP
  nthreads = omp_get_max_threads();
#endif
#pragma omp parallel for schedule(static)
  for (int64_t k = 0; k < K; ++k) {
    int lim[4];
    if (limits) {
      hbo_occupancy(origin, block_size[k], smem_total[k], regs[k], lim);
      for (int j = 0; j < 4; ++j) limits[(0 * 4 + j) * K + k] = lim[j];
    }
    for (int d = 0; d < D; ++d) {
      const hbo_device* dest = &devices[dest_rows[d]];
      int dr = dest_regs ? dest_regs[(int64_t)d * K + k] : -1;
      double out;
      int oo, od;
      int64_t wo, wd;
      int st = hbo_wave_scale_pair(origin, dest, num_blocks[k], block_size[k],
                                   smem_total[k], regs[k], dr, run_time_ns[k],
                                   (double)gamma[k], &out, &oo, &od, &wo, &wd);
      int64_t p = (int64_t)d * K + k;
      if (scaled_ns) scaled_ns[p] = out;
      if (dest_occ) dest_occ[p] = (uint8_t)od;
      if (dest_waves) dest_waves[p] = wd < 0 ? 0xFFFFFFFFu : (uint32_t)wd;
      if (status) status[p] = (uint8_t)st;
      if (d == 0) {
        if (origin_occ) origin_occ[k] = (uint8_t)oo;
        if (origin_waves) origin_waves[k] = wo < 0 ? 0xFFFFFFFFu : (uint32_t)wo;
      }
      if (limits) {
        hbo_occupancy(dest, block_size[k], smem_total[k], dr >= 0 ? dr : regs[k], lim);
        for (int j = 0; j < 4; ++j) limits[((int64_t)(d + 1) * 4 + j) * K + k] = lim[j];
      }
    }
  }
  return nthreads;
}
