/*
 * habitat_b200 -- C ABI of the B200 (sm_100a) batched prediction library.
 *
 * Every entry point takes plain pointers and sizes, returns an hb_status and
 * never throws or aborts.  Unless an entry point's name ends in `_host`, its
 * data pointers are DEVICE pointers owned by the caller, the work is queued on
 * the caller's CUDA stream (passed as an opaque `void*` cudaStream_t; NULL is
 * the default stream) and the call does not synchronise.  `_host` entry
 * points take host buffers, do their own transfers and return when the result
 * is in the caller's buffer.
 *
 * Each declaration cites the reference interface it stands in for (paths are
 * relative to the geoffxy/habitat tree).
 */
#ifndef HABITAT_B200_H
#define HABITAT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t hb_status;
enum {
  HB_OK = 0,
  HB_ERR_INVALID_ARGUMENT = 1,
  HB_ERR_CUDA = 2,          /* a CUDA runtime call failed; see hb_last_error() */
  HB_ERR_UNSUPPORTED = 3,   /* shape outside what the kernels handle          */
  HB_ERR_DEVICE_TIMEOUT = 4,/* a bounded device-side wait ran out             */
  HB_ERR_TOO_LARGE = 5      /* size beyond a fixed-capacity entry point       */
};

/* Text of the most recent error on the calling thread ("" if none). */
const char* hb_last_error(void);

/* Library version, "major.minor.patch". */
const char* hb_version(void);

/* ------------------------------------------------------------------------ */
/* Device table                                                             */
/* ------------------------------------------------------------------------ */

#define HB_MAX_DEVICES 64

/* Numeric fields of habitat::cuda::DeviceProperties
 * (cpp/src/cuda/kernel.h:14-62; bound at cpp/src/frontend/model_bindings.cpp:17-55)
 * plus the driver-reserved shared memory per block used for compute
 * capability >= 8 (0 otherwise). */
typedef struct {
  int32_t compute_major;
  int32_t compute_minor;
  int32_t max_threads_per_block;
  int32_t max_threads_per_multiprocessor;
  int32_t regs_per_block;
  int32_t regs_per_multiprocessor;
  int32_t warp_size;
  int32_t shared_mem_per_block;
  int32_t shared_mem_per_multiprocessor;
  int32_t num_sms;
  int32_t shared_mem_per_block_optin;
  int32_t reserved_shared_mem_per_block;
  int32_t mem_bandwidth_gb;
  int32_t base_clock_mhz;
  int32_t peak_gflops_per_second;
} hb_device_spec;

/* Replaces the per-call `hc.DeviceProperties` arguments of
 * KernelInstance.thread_block_occupancy (cpp/src/frontend/model_bindings.cpp:75-82):
 * rows are referred to by index afterwards.  n <= HB_MAX_DEVICES.
 * The table is kept on the host and copied to a GPU (constant rows plus the
 * tabulated limits of each row) when that GPU is current in this call or in the
 * first hb_wave_scale after it; only rows whose specification changed are
 * written again, and the copy ends with a device synchronise, so launches on any
 * stream see it.  That copy is a set-up step: make it (on every GPU used) before
 * a stream capture begins.  A row that kernels in flight are reading must not be
 * given a new specification.  Calls may come from several threads (one mutex
 * guards the table). */
hb_status hb_set_devices(const hb_device_spec* rows, int32_t n);

/* Fills a device-table row for CUDA device `device` from the driver's attributes: the eleven
 * fields cpp/src/device_info.cpp:16-30 prints, the shared memory the driver reserves per block,
 * and nominal figures for bandwidth (memory clock x bus width, double data rate), clock and
 * single-precision peak (FMA lanes x SMs x clock) where the reference's devices.yml holds
 * numbers from data sheets and from measure_peak_flops.py. */
hb_status hb_device_info(int32_t device, hb_device_spec* out);

/* Achieved single-precision GFLOP/s of a fused multiply-add kernel on the current device, best
 * of `trials` launches on `stream`: a value for peak_gflops_per_second measured on the machine.
 * Replaces cpp/src/cuda/diagnostics.cu:9-15 + tools/device-metadata/measure_peak_flops.py:10-18
 * (which profile a kernel of dependent additions and divide by its reported efficiency).
 * Synchronises; allocates and frees a small buffer. */
hb_status hb_peak_flops_test(int32_t trials, double* gflops_per_second, void* stream);

/* ------------------------------------------------------------------------ */
/* Wave scaling                                                             */
/* ------------------------------------------------------------------------ */

/* Structure-of-arrays view of K recorded kernels: the fields of
 * habitat::cuda::KernelMetadata / KernelInstance (cpp/src/cuda/kernel.h:64-151)
 * that the prediction path reads.  smem_bytes is static + dynamic shared
 * memory (only the sum enters the occupancy calculation under Habitat's call
 * convention, cpp/src/cuda/kernel.cpp:37-51).  gamma is the memory-bound
 * fraction of wave_scaling/roofline.py:14; pass gamma = 1 for kernels without
 * metrics (that is wave_scaling/resimplified.py:7-40). */
typedef struct {
  const int32_t* num_blocks;      /* [K] >= 1                      */
  const uint16_t* block_size;     /* [K] threads per block         */
  const uint16_t* regs_per_thread;/* [K]                           */
  const uint32_t* smem_bytes;     /* [K] static + dynamic          */
  const float* run_time_ns;       /* [K] measured time             */
  const float* gamma;             /* [K] in [0, 1]                 */
} hb_kernel_soa;

/* Raw metrics form of gamma (wave_scaling/roofline.py:68-104): when passed to
 * hb_wave_scale_metrics, gamma is computed per (kernel, destination) pair from
 * these instead of being read from hb_kernel_soa.gamma.  has_metrics[k] == 0
 * selects the no-metrics rule (gamma = 1, wave_scaling/unified.py:26-35). */
typedef struct {
  const double* flop_efficiency_pct; /* [K] Metric.SinglePrecisionFLOPEfficiency */
  const double* dram_read_bytes;     /* [K] Metric.DRAMReadBytes                 */
  const double* dram_write_bytes;    /* [K] Metric.DRAMWriteBytes                */
  const uint8_t* has_metrics;        /* [K] all three present                    */
} hb_kernel_metrics;

/* Outputs.  Planes are destination-major: element (d, k) is at d*K + k.
 * scaled_ns is NaN exactly where the Python reference would raise.  Any
 * pointer from `status` down may be NULL to skip that output. */
typedef struct {
  float* scaled_ns;        /* [D][K] predicted time on destination d          */
  uint8_t* dest_occupancy; /* [D][K] thread blocks per SM                     */
  uint32_t* dest_waves;    /* [D][K] num_blocks // (num_sms * occupancy);
                                     0xFFFFFFFF where the wave size is 0      */
  uint8_t* origin_occupancy; /* [K]                                           */
  uint32_t* origin_waves;    /* [K]                                           */
  uint8_t* status;         /* [D][K] hb_pair_status                           */
  int32_t* limits;         /* [(D+1)][4][K] block limits {regs, warps, blocks,
                                     smem}; plane 0 is the origin             */
} hb_wave_out;

enum {
  HB_PAIR_LARGE = 0,     /* wave_scaling/roofline.py:48-65                    */
  HB_PAIR_SMALL = 1,     /* wave_scaling/roofline.py:29-45                    */
  HB_PAIR_ZERO_WAVE = 2, /* the reference raises ZeroDivisionError            */
  HB_PAIR_BAD_INPUT = 3  /* num_blocks < 1                                    */
};

/* Replaces the per-kernel loop of Predictor._wave_scale
 * (analyzer/habitat/analysis/predictor.py:111-130) over
 * roofline_wave_scaling / resimplified_wave_scaling
 * (wave_scaling/roofline.py:8-65, resimplified.py:7-40) and
 * calculate_wave_info (wave_scaling/common.py:3-20), for K kernels and D
 * destination rows at once.  dest_regs ([D][K], may be NULL) carries the
 * result of MetadataManager.kernel_registers_for (wave_scaling/metadata.py:12-37),
 * -1 meaning "no entry: use the kernel's own register count". */
hb_status hb_wave_scale(const hb_kernel_soa* kernels, int64_t K, int32_t origin_row,
                        const int32_t* dest_rows_host, int32_t D,
                        const int16_t* dest_regs, const hb_wave_out* out, void* stream);

/* Same, with gamma computed on the device from raw metrics
 * (wave_scaling/roofline.py:68-104, wave_scaling/unified.py:8-35). */
hb_status hb_wave_scale_metrics(const hb_kernel_soa* kernels, const hb_kernel_metrics* metrics,
                                int64_t K, int32_t origin_row, const int32_t* dest_rows_host,
                                int32_t D, const int16_t* dest_regs, const hb_wave_out* out,
                                void* stream);

/* Which kernel the calling thread's most recent hb_wave_scale / hb_wave_scale_metrics call
 * launched: 0 none yet, 1 generic (any device row, block-limit planes, more than 32
 * destinations), 2 division-free (ordinary rows that cannot be tabulated), 4 tabulated
 * limits (status plane, per-destination registers and metrics included).  For tests and
 * for naming the measured kernel; no reference counterpart. */
int32_t hb_wave_scale_path(void);

/* Host-buffer form of hb_wave_scale: all pointers in `kernels`, `dest_regs`
 * and `out` are HOST pointers; transfers happen inside the call, through a
 * staging block and a stream the library keeps per GPU (the block grows when a
 * larger batch arrives and is never shrunk; `_host` calls on one GPU run one
 * after the other). */
hb_status hb_wave_scale_host(const hb_kernel_soa* kernels, int64_t K, int32_t origin_row,
                             const int32_t* dest_rows_host, int32_t D,
                             const int16_t* dest_regs, const hb_wave_out* out);

/* Single-kernel occupancy with the four block limits.  Stands in for
 * KernelInstance.thread_block_occupancy(device, registers_per_thread)
 * (cpp/src/frontend/model_bindings.cpp:75-82).  Evaluated on the host with the
 * same integer code the kernels run (as the reference evaluates its header on
 * the host): no allocation, no launch, no synchronisation. */
hb_status hb_thread_block_occupancy(int32_t device_row, int32_t block_size, uint32_t smem_bytes,
                                    int32_t regs_per_thread, int32_t* occupancy,
                                    int32_t limits[4]);

/* ------------------------------------------------------------------------ */
/* MLP runtime predictors                                                   */
/* ------------------------------------------------------------------------ */

typedef struct hb_mlp hb_mlp;

enum { HB_PRECISION_BF16 = 0, HB_PRECISION_BF16X3 = 1 };

/* Builds the device-side weight pack of one runtime predictor: the module
 * RuntimePredictor owns (analyzer/habitat/analysis/mlp/mlp.py:113-131;
 * topology mlp.py:17-109: fc1 (F+4 -> width) + ReLU, `layers` x [width ->
 * width + ReLU], fc2 (width -> 1)) together with its mu/sigma
 * (mlp.py:133-137).  All pointers are HOST pointers, weights row-major
 * [out][in] as in torch.nn.Linear:
 *   fc1_w [width][F+4], fc1_b [width], hidden_w [layers][width][width],
 *   hidden_b [layers][width], fc2_w [width], fc2_b [1], mu/sigma [F+4].
 * device_features is [n_device_rows][4] = (mem, mem_bw, num_sm, single), the
 * columns RuntimePredictor.predict reads from devices.csv
 * (analysis/mlp/devices.py:5-10, mlp.py:125).  1 <= width <= 1024 (the shipped
 * predictors are 1024 wide; a narrower network is zero-padded to 1024 inside the
 * pack and costs as much), 1 <= layers <= 64. */
hb_status hb_mlp_create(hb_mlp** handle, int32_t n_op_features, int32_t layers, int32_t width,
                        const float* fc1_w, const float* fc1_b, const float* hidden_w,
                        const float* hidden_b, const float* fc2_w, const float* fc2_b,
                        const double* mu, const double* sigma, const double* device_features,
                        int32_t n_device_rows, int32_t precision);

void hb_mlp_destroy(hb_mlp* handle);

/* Replaces RuntimePredictor.predict (analysis/mlp/mlp.py:252-267) for Q
 * queries at once: op_features [Q][F] float32 row-major, device_row [Q]
 * indexes device_features, out [Q] float32 (milliseconds, un-clamped).
 * The GPU the handle was created on must be current
 * (HB_ERR_INVALID_ARGUMENT otherwise). */
hb_status hb_mlp_predict(hb_mlp* handle, const float* op_features, const uint8_t* device_row,
                         int64_t Q, float* out, void* stream);

/* Synchronises with the device and reports whether any launch on this handle
 * gave up on a bounded device-side wait (HB_ERR_DEVICE_TIMEOUT; *device_status
 * names the waiting role and site) since the last call that reported one: the
 * word is cleared once it has been reported, so later launches are judged on
 * their own.  No reference counterpart: the reference's predict() is host code. */
hb_status hb_mlp_status(hb_mlp* handle, int32_t* device_status);

/* Writes the handle's device status word from the host, as a kernel that gave up
 * on a wait would.  Host-side fault injection for tests of the error path (no
 * kernel is made to wait or fail).  No reference counterpart. */
hb_status hb_mlp_inject_status(hb_mlp* handle, int32_t device_status);

/* Profiling aid (bf16 kernel): SM cycle counters of the first cluster's leader CTA
 * for the most recent launch.  out[0..3] first epilogue group: waiting for its
 * output blocks, draining them, fc2, layers counted.  out[4..8] MMA issuer:
 * waiting for activations, for weights, for TMEM blocks to be read out, issuing,
 * ring slots counted.  out[9..11] first producer: waiting for a free slot, copy
 * latency, copies counted.  out[12], out[13]: the MMA issuer's whole loop in SM
 * cycles and in nanoseconds (their ratio is the SM clock under load).
 * out[14], out[15] first epilogue group: hand-over of a drained block, stores
 * into the peer CTA.  Synchronises.  No reference counterpart. */
hb_status hb_mlp_phase_cycles(hb_mlp* handle, int64_t out[16]);

/* Host-buffer form of hb_mlp_predict; also checks hb_mlp_status. */
hb_status hb_mlp_predict_host(hb_mlp* handle, const float* op_features,
                              const uint8_t* device_row, int64_t Q, float* out);

/* Replaces the last line of Predictor._{conv2d,linear,bmm,lstm}_scale and the
 * clamp of Predictor._special_scale (analysis/predictor.py:132-148, :182):
 * out_ms[i] = max(0, run_time_ms[i] * pred_dest[i] / pred_orig[i]);
 * *negative_count (device, may be NULL) is incremented per clamped value. */
hb_status hb_special_scale(const float* run_time_ms, const float* pred_dest,
                           const float* pred_orig, int64_t n, float* out_ms,
                           uint32_t* negative_count, void* stream);

/* ------------------------------------------------------------------------ */
/* Trace-level totals                                                       */
/* ------------------------------------------------------------------------ */

/* Replaces Trace.run_time_ms (analyzer/habitat/analysis/trace.py:26-36) and
 * RunTimePrediction.run_time_ms (analysis/run_time.py:49-58) for many
 * segments at once: out[s] = sum(values[offsets[s] : offsets[s+1]]) in
 * float64, fixed summation order (results do not depend on the launch). */
hb_status hb_segment_sum(const float* values, const int64_t* offsets, int64_t n_segments,
                         double* out, void* stream);

/* Sum of each of n_planes contiguous planes of plane_len float32 values,
 * skipping NaN entries (pairs the reference would have raised on); used for
 * per-destination totals of hb_wave_out.scaled_ns.  out [n_planes] float64.
 * The partial sums of all calls on one GPU share a scratch buffer the library
 * keeps for that GPU: calls on one GPU must be ordered, on one stream or by
 * events.  The buffer is allocated by the first call on a GPU (room for 64
 * planes) and replaced by a larger one when a call needs more; a replaced buffer
 * is kept allocated until the process ends, so launches in flight and captured
 * graphs that hold its address stay valid.  The allocating call is a set-up step:
 * make it before a stream capture begins. */
hb_status hb_plane_sum(const float* values, int64_t plane_len, int32_t n_planes, double* out,
                       void* stream);

/* Planes the plane-sum scratch of CUDA device `device` has room for (0 before the
 * first call there, -1 for an ordinal out of range).  For tests of the per-GPU
 * bookkeeping; no reference counterpart. */
int64_t hb_plane_sum_scratch_planes(int32_t device);

/* Sums of values grouped by a small key: out[g] = sum of values[i] with
 * keys[i] == g, g < n_groups <= 256, float64, fixed order, NaN skipped.  With
 * keys = the device row of each MLP query this gives the per-device totals of a
 * batch of predictions (what summing Trace.run_time_ms per destination,
 * analysis/trace.py:26-36, gives the reference).  Scratch and ordering as for
 * hb_plane_sum (a buffer of its own, so the two may overlap). */
hb_status hb_group_sum(const float* values, const uint8_t* keys, int64_t n, int32_t n_groups,
                       double* out, void* stream);

/* hb_wave_scale that also leaves the first stage of the per-destination totals
 * (Trace.run_time_ms per destination, analysis/trace.py:26-36) in a buffer of the
 * caller: partials [D][*per_plane] float64, partials[d * *per_plane + i] = the sum,
 * NaN results skipped, of one fixed part of destination d's predicted times.
 * hb_partials_sum (or hb_partials_sum_allreduce across GPUs) turns them into the D
 * totals.  When the launch takes the table kernel with two records per thread
 * (every real device row, even K, 8-byte aligned arrays, no dest_regs / status /
 * limits, D <= 8) each block adds up its own 256 results per destination before
 * they leave the SM, so the [D x K] plane is not read a second time
 * (*per_plane = ceil(K / 256)); any other launch runs the first stage of
 * hb_plane_sum over the results (*per_plane = 256).  Either way a fixed assignment
 * of records to partial sums and a fixed order: the same inputs give the same bits.
 * `partials` must hold D * hb_wave_scale_partials_len(K) float64 values; *per_plane
 * is written on the host before the call returns (0 when K == 0).  Allocates
 * nothing. */
int64_t hb_wave_scale_partials_len(int64_t K);
hb_status hb_wave_scale_partials(const hb_kernel_soa* kernels, int64_t K, int32_t origin_row,
                                 const int32_t* dest_rows_host, int32_t D, const int16_t* dest_regs,
                                 const hb_wave_out* out, double* partials, int32_t* per_plane,
                                 void* stream);
/* out[p] = sum of partials[p * per_plane .. (p + 1) * per_plane), float64, fixed order. */
hb_status hb_partials_sum(const double* partials, int32_t per_plane, int32_t n_planes, double* out,
                          void* stream);

/* hb_plane_sum for callers that must not allocate device memory after start-up
 * (a process that gave the whole GPU to its own memory pool, or one that
 * forbids driver allocations once it is serving).  Same arguments and results
 * as hb_plane_sum, but the partial sums live in a 128 KB array built into the
 * library image (held on every GPU that loads the library until the process
 * exits) and the call performs no cudaMalloc / cudaFree.
 *   - n_planes <= 64; more is refused with HB_ERR_TOO_LARGE.
 *   - The first call on each device resolves the array's device address (the
 *     device must be current); make that call during set-up, before any stream
 *     capture is begun.
 *   - All calls on a device share the one array: calls whose kernels may run
 *     at the same time (different streams) race; serialise them.
 * It has no counterpart in the reference, whose totals are host-side sums. */
hb_status hb_plane_sum_static(const float* values, int64_t plane_len, int32_t n_planes, double* out,
                              void* stream);

/* ------------------------------------------------------------------------ */
/* Totals across the GPUs of one box                                        */
/* ------------------------------------------------------------------------ */

/* Kernels and queries shard across GPUs with nothing to exchange but totals (a
 * few float64 numbers per batch).  hb_plane_sum_allreduce / hb_group_sum_allreduce
 * are hb_plane_sum / hb_group_sum whose final stage also exchanges the results:
 * it stores them into a mailbox in every peer GPU's memory (plain stores through
 * peer-mapped pointers, no multicast), waits for the peers' values in its own
 * mailbox and adds them in rank order, so `out` holds the same sum, bit for bit,
 * on every GPU.  One process per GPU; every rank makes the same calls in the same
 * order, and the calls of a handle are ordered on its GPU (one stream, or events).
 * At most 64 values per call (hb_group_sum_allreduce: 8 groups).
 * Every device-side wait is bounded (1 s unless hb_peer_set_wait_ns says
 * otherwise): when a peer does not show up the value becomes NaN, the kernel
 * returns and hb_peer_status reports HB_ERR_DEVICE_TIMEOUT with the rank and value
 * waited for; ranks should therefore meet on the host once before their first
 * exchange.  Set-up: hb_peer_create on every rank (allocates the mailbox and the
 * scratch; before any stream capture), hb_peer_export -> 64 bytes that every
 * other rank passes, in rank order, to hb_peer_connect (CUDA IPC; the bytes
 * travel by whatever channel the host has).  The reference has no counterpart:
 * its totals are sums in one host process (analyzer/habitat/analysis/trace.py:26-36). */
typedef struct hb_peer hb_peer;

hb_status hb_peer_create(hb_peer** handle, int32_t rank, int32_t world);
hb_status hb_peer_export(hb_peer* handle, uint8_t out[64]);
/* handles: world x 64 bytes in rank order (this rank's own entry is ignored). */
hb_status hb_peer_connect(hb_peer* handle, const uint8_t* handles);
/* Same with device pointers that already address the peers' mailboxes from this
 * GPU (mailboxes[r] = hb_peer_mailbox of rank r, mapped by the caller; handles
 * that live in one process on one GPU, as in single-GPU tests). */
hb_status hb_peer_connect_pointers(hb_peer* handle, void* const* mailboxes);
void* hb_peer_mailbox(hb_peer* handle);
hb_status hb_peer_set_wait_ns(hb_peer* handle, int64_t wait_ns);
/* Frees the mailbox.  Peers store into it during their exchanges: destroy only after
 * every rank has finished its last exchange (meet on the host first). */
void hb_peer_destroy(hb_peer* handle);
/* Synchronises; HB_ERR_DEVICE_TIMEOUT (reported once, then cleared) when a wait ran out. */
hb_status hb_peer_status(hb_peer* handle, int32_t* device_status);

hb_status hb_plane_sum_allreduce(hb_peer* handle, const float* values, int64_t plane_len,
                                 int32_t n_planes, double* out, void* stream);
hb_status hb_group_sum_allreduce(hb_peer* handle, const float* values, const uint8_t* keys, int64_t n,
                                 int32_t n_groups, double* out, void* stream);
/* hb_partials_sum whose final stage also exchanges the totals (as above). */
hb_status hb_partials_sum_allreduce(hb_peer* handle, const double* partials, int32_t per_plane,
                                    int32_t n_planes, double* out, void* stream);
/* The exchange alone, in place on n device values.  phase 3 publishes and gathers in
 * one kernel; phases 1 (publish) and 2 (gather what the last publish of every rank
 * left) exist so that several ranks can be walked through one after the other on a
 * single GPU, where kernels must not wait for one another. */
hb_status hb_peer_allreduce(hb_peer* handle, double* values, int32_t n, int32_t phase, void* stream);

/* Builds made with -DHB_BOUNDS_CHECK compare every table and element index of the
 * wave-scaling kernels with its bound; the first violation is recorded in a device
 * word (site << 24 | index, top bit set) and the access redirected, nothing traps.
 * Synchronises, returns the word (0: none) and optionally clears it.  Ordinary
 * builds return HB_ERR_UNSUPPORTED.  No reference counterpart. */
hb_status hb_bounds_check_word(uint32_t* word, int32_t reset);

#ifdef __cplusplus
}
#endif
#endif
