// Fused inference of Habitat's per-operation MLP runtime predictors on sm_100a.
//
// Stands in for RuntimePredictor.predict (analyzer/habitat/analysis/mlp/mlp.py:252-267
// of the reference) over a whole batch of queries: feature normalisation
// (mlp.py:258-261), fc1 + ReLU, `layers` x [Linear(1024,1024) + ReLU] and fc2
// (mlp.py:17-109) run as ONE persistent kernel; activations never leave the SM.
//
// Formulation.  Two CTAs of a cluster own a tile of queries and compute every layer
// transposed, H^T = W . X^T, so that
//   A (M = 256 output features x K) = weight tiles, streamed from global/L2 into a
//                                     shared-memory ring by tiled TMA loads (mbarrier
//                                     completion), half of the rows in each CTA;
//   B (N = 128 columns x K)         = the activations, resident in shared memory
//                                     (MN-major, 128-byte swizzle), half of the columns
//                                     in each CTA;
//   D (128 lanes x 128 columns)     = fp32 accumulators in tensor memory, one column
//                                     block per 256-feature block, so the whole layer
//                                     output lives in TMEM until it is drained.
// tcgen05.mma.cta_group::2 (kind::f16, bf16 inputs, fp32 accumulate) is issued by one
// elected lane of a warp that walks the issue loop as a whole; the epilogue warps read TMEM
// with tcgen05.ld, add the bias, apply ReLU, round to bf16 and overwrite the activation
// buffer in place while the tensor core works on the remaining blocks of the layer.  fc2 is
// a dot product over features (= TMEM lanes), reduced through shared memory.
//
// fc1 has K = F + 4 <= 12.  Its inputs are the normalised features, which need
// more than bf16's 8 bits, so both x and w are split into bf16 hi + lo parts and
// the three products hi.hi + lo.hi + hi.lo are laid side by side along K
// (3 (F+4) <= 36 of the 64 columns of one K block).
//
// Precision modes: HB_PRECISION_BF16 rounds hidden activations and weights to bf16 (128
// queries per tile); HB_PRECISION_BF16X3 keeps hi + lo parts of both (64 queries per tile,
// the two parts of an activation side by side along N, the two parts of a weight tile in
// one ring slot: see the comment at the kernel).
//
// Warp roles: warp 0 = TMEM allocation, warp 1 = barrier set-up + MMA issuer (leader CTA),
// warps 2-5 and 12-15 = two epilogue groups (one TMEM lane quadrant per warp), warps 6-11 =
// weight producers.  Bulk copies issued by one thread complete one after the other (measured:
// about 750 cycles each whatever their size), so each ring slot has its own issuing warp.
// Every mbarrier wait is bounded: when a wait runs out the kernel records a status word, all
// roles leave their loops, outstanding bulk copies are waited for (bounded) and TMEM is released.
#include <cuda.h>
#include <cuda_bf16.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "hb_common.h"

namespace {

constexpr int kWidth = 1024;            // layer_size of every Habitat predictor
constexpr int kMTile = 128;             // output features per MMA (TMEM lanes)
constexpr int kKBlk = 64;               // bf16 per 128-byte swizzle row
constexpr int kNumMT = kWidth / kMTile; // 8
constexpr int kNumKB = kWidth / kKBlk;  // 16
constexpr int kTileBytes = kMTile * 128;// one weight tile image: 16 KB
constexpr int kMaxInFeat = 12;          // F + 4 (conv2d: 8 + 4)

struct MlpParams {
  const uint8_t* wpack;      // weight tile images, producer order
  const float* bias;         // [layers + 1][1024]: fc1, hidden...
  const float* fc2_w;        // [1024]
  float fc2_b;
  const double* mu;          // [F + 4]
  const double* sigma;       // [F + 4]
  const double* dev_feat;    // [n_dev][4]
  int32_t n_dev;
  int32_t n_op_feat;         // F
  int32_t layers;            // hidden layers
  const float* feats;        // [Q][F]
  const uint8_t* dev_row;    // [Q]
  int64_t Q;
  float* out;                // [Q]
  int32_t num_tiles;
  int32_t* status;           // device word: 0 ok, else (role << 8 | site)
  long long* phase_cycles;   // [16] cluster 0: cycle counters of the roles (diagnostic), or null
  CUtensorMap tmap_slot;     // pair kernel: the pack as [rows][128 B], box of two tile images (32 KB)
  CUtensorMap tmap_tile;     // same tensor, box of one tile image (16 KB, fc1)
  uint64_t unit_order;       // pair kernel: the 16 (block, K quarter) units of a hidden layer, 4 bits each
  uint32_t unit_gates;       // pair kernel: 4 bits per block j: the block whose completion frees K quarter j
};

// ---------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(pred)::"memory");
  return pred;
}
__device__ __forceinline__ void tc_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp gets lane
// (quadrant base + t), registers = columns.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 64 consecutive 32-bit columns in one instruction: halves the number of
// load round trips of the epilogue (each tcgen05.ld + wait costs several hundred cycles).
__device__ __forceinline__ void tc_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]),
        "=r"(r[38]), "=r"(r[39]), "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]),
        "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]), "=r"(r[48]), "=r"(r[49]),
        "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]),
        "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}

// Byte offset of element (row, col) inside a K-major 128-byte-swizzled block of
// 128-byte rows: 16-byte chunks are permuted by the row index modulo 8.
__host__ __device__ __forceinline__ uint32_t swz_off(uint32_t row, uint32_t col) {
  return row * 128u + ((((col >> 3) ^ row) & 7u) << 4) + ((col & 7u) << 1);
}

constexpr long long kWaitCycles = 4000000000LL;  // about two seconds

// Bounded wait.  Returns false when the wait ran out or another role gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          int32_t* status, int code) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The kernel.  A single CTA can only keep 64 queries on chip,
// and an M = 128 MMA with N = 64 occupies the tensor core for the same 64 cycles
// as one with N = 128, so the one-CTA kernel tops out at half rate.  Here two
// CTAs of a cluster share one tile of 128 queries:
//   * tcgen05.mma.cta_group::2 with M = 256, N = 128: CTA c supplies the A rows
//     (weights) of features 256 j + 128 c .. and the B rows (activations) of
//     queries 64 c .. 64 c + 63; its TMEM receives the D rows of its features
//     for all 128 queries.  Each weight byte is fetched once per pair.
//   * The leader CTA (rank 0) issues every MMA.  A ring slot is ready when the
//     leader's weight box and the peer's have landed: both are tiled TMA loads
//     (cp.async.bulk.tensor with .cta_group::2, no multicast) whose bytes are
//     counted on the leader's barrier, so no thread of the peer has to forward
//     anything.  tcgen05.commit multicasts "slot free" and "output block j
//     accumulated" to both CTAs.
//   * The activations are the MN-major B operand here (one 128-byte row of 64
//     queries per K index): an epilogue thread owns one feature = one K row
//     and writes eight queries per 16-byte store.
//   * The epilogue of CTA c holds features x all 128 queries, but the next
//     layer needs, in each CTA, all features x its 64 queries: half of the
//     bf16 results are stored into the peer's shared memory (st.async, counted
//     in bytes on a barrier of the peer).
//   * Epilogue and tensor core overlap: a hidden layer is issued as 16 units
//     (output block, K quarter) in the order kPairOrder, so that output blocks
//     finish one after the other and each frees the K quarter it will replace.
//     The leader waits per K quarter (bar_actq) and per TMEM block (bar_tfree)
//     instead of per layer; only the drain of the last block is exposed.
//   * fc2: each CTA reduces its 512 features to 128 partial sums, hands the 64
//     that belong to the peer's queries over through the peer's shared memory,
//     and finishes its own 64 queries.
// ---------------------------------------------------------------------------
constexpr int kPairQ = 128;                 // queries per cluster tile
constexpr int kPairHalfQ = 64;              // activation rows resident per CTA
constexpr int kPairMT = kWidth / 256;       // 4 MMA row blocks per layer
constexpr int kPairSlotKb = 2;               // weight tiles (K blocks of 64) per ring slot
constexpr int kPairStages = 6 / kPairSlotKb; // ring slots: 96 KB in all
constexpr int kPairStageBytes = kPairSlotKb * kTileBytes;
static_assert(kPairStages <= 6, "one producer warp per ring slot, warps 6-11");
constexpr int kPairActKb = kPairHalfQ * 128;          // 8 KB per K block
constexpr int kPairActBytes = kNumKB * kPairActKb;    // 128 KB
// Order of the 16 (output block j, K quarter q) units of a hidden layer, four bits each
// (4 j + q), first unit in the low bits:
//   (0,0) (1,0) (2,0) (3,0) | (0,1) (0,2) (0,3) | (1,1) (2,1) (3,1) | (1,2) (1,3) | (2,2) (3,2) | (2,3) | (3,3)
// Block j completes after 7, 12, 15, 16 units, and by then no later unit reads quarter j,
// so the epilogue of block j can replace quarter j of the activations in place while the
// tensor core works on the remaining blocks; the next layer consumes the quarters in the
// same order.
constexpr uint64_t kPairOrder = 0xFBEA76D95321C840ull;
constexpr uint32_t kPairGates = 0x3210u;
__device__ __forceinline__ int pair_unit_j(uint64_t order, int u) { return static_cast<int>((order >> (4 * u + 2)) & 3u); }
__device__ __forceinline__ int pair_unit_q(uint64_t order, int u) { return static_cast<int>((order >> (4 * u)) & 3u); }
constexpr int kPairThreads = 512;              // warps: 0 alloc, 1 MMA, 2-5 + 12-15 epilogue, 6-11 producers
constexpr int kPairSmemBytes = kPairActBytes + kPairStages * kPairStageBytes + 1024 + 1024;
static_assert(kPairSmemBytes <= 232448, "over the 227 KB shared-memory limit");

__device__ __forceinline__ void pair_epi_bar_sync() {
  asm volatile("bar.sync 1, 256;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
  return r;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr)
               : "memory");
}
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_cluster(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag, int32_t* status,
                                                  int code) {
  if (mbar_try_wait_cluster(bar, parity)) return true;
  const long long t0 = clock64();
  for (uint32_t i = 1;; ++i) {
    if (mbar_try_wait_cluster(bar, parity)) return true;
    if ((i & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitCycles) {
        *abort_flag = 1;
        atomicCAS(status, 0, code);
        return false;
      }
    }
  }
}
// Asynchronous 16-byte store into a peer CTA's shared memory; completion is counted
// in bytes on an mbarrier of that CTA.  Unlike st.shared::cluster the issuing
// thread does not wait for the store to be acknowledged.
__device__ __forceinline__ void st_async_v4(uint32_t cluster_addr, uint32_t a, uint32_t b, uint32_t c,
                                            uint32_t d, uint32_t cluster_mbar) {
  asm volatile(
      "st.async.weak.shared::cluster.mbarrier::complete_tx::bytes.v4.b32 [%0], {%1, %2, %3, %4}, [%5];"
      ::"r"(cluster_addr), "r"(a), "r"(b), "r"(c), "r"(d), "r"(cluster_mbar)
      : "memory");
}
// Byte offset of element (K row k, query n) of an MN-major, 128-byte-swizzled B
// operand holding 64 queries per row: rows are 128 B apart, the eight 16-byte
// groups of a row are permuted by the row index modulo 8.
__device__ __forceinline__ uint32_t mn_off(uint32_t k, uint32_t n) {
  return k * 128u + ((((n >> 3) ^ k) & 7u) << 4) + ((n & 7u) << 1);
}
__device__ __forceinline__ void st_cluster_f32(uint32_t cluster_addr, float v) {
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::
                   : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Tiled TMA load of a box of 128-byte rows into this CTA's shared memory.  With
// .cta_group::2 the completion may be counted on a barrier of the other CTA of the pair
// (given as a shared::cluster address): both CTAs' weight copies report to the leader's
// barrier directly.  No multicast: each CTA fetches its own half of the weights.
__device__ __forceinline__ void tma_rows_2sm(uint32_t dst, const CUtensorMap* map, int32_t row,
                                             uint32_t cluster_mbar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(cluster_mbar), "r"(0), "r"(row)
      : "memory");
}
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(bar),
      "h"(static_cast<uint16_t>(3))
      : "memory");
}
__device__ __forceinline__ void tc_mma_pair_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                                 uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// SPLIT = false: bf16 operands, 128 queries per cluster tile (64 per CTA).
// SPLIT = true (the 1e-4 mode): activations and weights are kept as bf16 hi + lo parts.  A CTA
// holds 32 queries and lays the hi and lo parts of an activation side by side along N (the 128-byte
// B row of K index k is [hi of 32 queries | lo of 32 queries]), so the same M = 256, N = 128 MMA
// multiplies a weight tile with both parts at once, at full rate; a ring slot carries the hi and the
// lo image of one K block of weights and both accumulate into the same TMEM columns:
// D = (W_hi + W_lo) [x_hi | x_lo], and the epilogue adds the two column halves of a query (all four
// partial products, fp32 accumulation).  Two MMAs per K step and 64 queries instead of one and 128:
// a quarter of the bf16 rate.
template <bool SPLIT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kPairThreads, 1)
mlp_chain_pair_kernel(const __grid_constant__ MlpParams p) {
  constexpr int kTileQ = SPLIT ? kPairQ / 2 : kPairQ;          // queries per cluster tile
  constexpr int kHalfQ = kTileQ / 2;                           // queries per CTA
  constexpr int kLoadsPerUnit = SPLIT ? 4 : 4 / kPairSlotKb;   // ring slots per (block, K quarter) unit
  constexpr int kRowsPerImage = (SPLIT ? 2 : 1) * (kTileBytes / 128);   // 128-byte rows per packed K block
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);

  const uint32_t act = base;
  const uint32_t stage0 = base + kPairActBytes;
  const uint32_t bars = stage0 + kPairStages * kPairStageBytes;
  uint8_t* bars_ptr = base_ptr + (bars - base);
  // barrier block (same offsets in both CTAs)
  const uint32_t bar_full = bars;            // [stages <= 8] leader only: both CTAs' weight boxes landed
  const uint32_t bar_empty = bars + 64;      // [stages <= 8] slot consumed (multicast commit)
  const uint32_t bar_accj = bars + 128;      // [4] output block j accumulated (multicast commit)
  const uint32_t bar_actq = bars + 160;      // [4] leader only: K quarter q of the activations ready in both CTAs
  const uint32_t bar_inq = bars + 192;       // [4] peer's half of K quarter q landed here (bytes)
  const uint32_t bar_tfree = bars + 224;     // [4] leader only: TMEM block j read out in both CTAs (8 warps)
  const uint32_t bar_fc2 = bars + 256;       // peer's fc2 partial sums arrived
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars_ptr + 264);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 268);
  volatile int* epi_ok = reinterpret_cast<volatile int*>(bars_ptr + 272);   // [2], one per epilogue group
  float* fc2_mine = reinterpret_cast<float*>(bars_ptr + 512);    // [64] own queries, own features
  float* fc2_peer = reinterpret_cast<float*>(bars_ptr + 768);    // [64] own queries, peer's features

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t peer = rank ^ 1u;

  if (threadIdx.x == 32) {
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(bar_full + 8 * s, 1);   // used in the leader only: its producer's arrive.expect_tx
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int q = 0; q < 4; ++q) {
      mbar_init(bar_accj + 8 * q, 1);
      mbar_init(bar_actq + 8 * q, 2);   // one arrive per CTA
      mbar_init(bar_inq + 8 * q, 1);
      mbar_init(bar_tfree + 8 * q, 8);  // one arrive per epilogue warp of the block, both CTAs
    }
    mbar_init(bar_fc2, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(tmem_slot)),
                 "r"(512u)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n_layers = p.layers + 1;
  const int n_pairs = static_cast<int>(gridDim.x >> 1);
  const int pair_id = static_cast<int>(blockIdx.x >> 1);
  int my_tiles = 0;
  if (pair_id < p.num_tiles) my_tiles = (p.num_tiles - 1 - pair_id) / n_pairs + 1;

  uint32_t issued = 0;

  if (warp >= 6 && warp < 12) {
    // ------------------------------ producers -----------------------------
    // One producer per ring slot.  The pack is laid out per 128-feature block
    // (layer -> block -> K block); this CTA streams blocks 2 j + rank.
    if (lane == 0 && warp - 6 < kPairStages) {
      const uint32_t w = static_cast<uint32_t>(warp - 6);
      uint32_t it = 0;
      bool ok = true;
      const bool ptimed = p.phase_cycles != nullptr && blockIdx.x == 0 && w == 0;
      const uint32_t peer_full_leader = map_to_cta(bar_full + 8 * w, 0);
      long long pc_empty = 0, pc_copy = 0, pc_n = 0;
      for (int t = 0; t < my_tiles && ok; ++t) {
        size_t layer_base = 0;   // in tile images
        for (int L = 0; L < n_layers && ok; ++L) {
          const int nkb = L == 0 ? 1 : kNumKB;
          // A ring slot takes two consecutive K blocks of one output block (fc1 has only one);
          // a hidden layer is streamed as 16 (block, K quarter) units of two slots each.
          const int n_units = nkb == 1 ? kPairMT : 16;
          const int n_loads = nkb == 1 ? 1 : kLoadsPerUnit;
          const uint32_t load_bytes = nkb == 1 ? kTileBytes : kPairStageBytes;
          {
            for (int u = 0; u < n_units && ok; ++u) {
              const int j = nkb == 1 ? u : pair_unit_j(p.unit_order, u);
              const int kq = nkb == 1 ? 0 : pair_unit_q(p.unit_order, u);
              const size_t blk = layer_base + static_cast<size_t>(2 * j + rank) * nkb + kq * 4;
              for (int g = 0; g < n_loads; ++g, ++it) {
                if (it % kPairStages != w) continue;
                const uint32_t ph = (it / kPairStages) & 1u;
                const long long q0 = ptimed ? clock64() : 0;
                if (!mbar_wait(bar_empty + 8 * w, ph ^ 1u, abort_flag, p.status, 0x111)) { ok = false; break; }
                const long long q1 = ptimed ? clock64() : 0;
                // both CTAs' boxes are counted on the leader's barrier
                if (rank == 0) mbar_expect_tx(bar_full + 8 * w, 2 * load_bytes);
                // bf16: a slot takes two consecutive K blocks (16 KB images); split: the hi and lo
                // image of one K block (stored back to back)
                tma_rows_2sm(stage0 + w * kPairStageBytes, nkb == 1 ? &p.tmap_tile : &p.tmap_slot,
                             static_cast<int32_t>((blk + (SPLIT ? 1 : kPairSlotKb) * g) * kRowsPerImage),
                             peer_full_leader);
                issued = it + 1;
                if (ptimed) {
                  mbar_wait(bar_full + 8 * w, ph, abort_flag, p.status, 0x112);
                  pc_empty += q1 - q0; pc_copy += clock64() - q1; ++pc_n;
                }
              }
            }
          }
          layer_base += static_cast<size_t>(kNumMT) * nkb;
        }
      }
      if (ptimed) { p.phase_cycles[9] = pc_empty; p.phase_cycles[10] = pc_copy; p.phase_cycles[11] = pc_n; }
    }
  } else if (warp == 1) {
    if (rank == 0) {
      // ------------------------------ MMA issuer (leader) -------------------
      // The whole warp walks the loop and one elected lane issues: the operands of
      // tcgen05.mma live in uniform registers, and a loop that only one lane of a
      // diverged warp executes was measured at 645 cycles per eight MMAs against
      // 512 (the tensor pipe's own rate) for the warp-uniform form.
      // D fp32, A/B bf16, A K-major, B MN-major (bit 16), N = 128, M = 256
      constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 16) |
                                 (static_cast<uint32_t>(kPairQ >> 3) << 17) |
                                 (static_cast<uint32_t>(256 >> 4) << 24);
      const uint64_t desc_hi = (static_cast<uint64_t>(1024 >> 4) << 32) | (static_cast<uint64_t>(1) << 46) |
                               (static_cast<uint64_t>(2) << 61) | (static_cast<uint64_t>(1) << 16);
      const uint32_t a_lo0 = (stage0 & 0x3FFFF) >> 4;
      const uint32_t b_lo0 = (act & 0x3FFFF) >> 4;
      // par: bits 0-3 = parity of the next wait on bar_actq[q], bits 4-7 on bar_tfree[j]
      uint32_t s = 0, ph = 0, par = 0;
      bool ok = true;
      const bool mtimed = p.phase_cycles != nullptr && blockIdx.x == 0;
      long long mc_act = 0, mc_full = 0, mc_tfree = 0, mc_issue = 0, mc_n = 0;
      auto wait_flip = [&](uint32_t bar0, uint32_t idx, uint32_t bit, long long& acc, int code) -> bool {
        const long long m0 = mtimed ? clock64() : 0;
        const bool got = mbar_wait_cluster(bar0 + 8 * idx, (par >> bit) & 1u, abort_flag, p.status, code);
        par ^= 1u << bit;
        tc_fence_after();
        if (mtimed) acc += clock64() - m0;
        return got;
      };
      const long long k0 = clock64();
      const unsigned long long g0 = global_timer_ns();
      for (int t = 0; t < my_tiles && ok; ++t) {
        for (int L = 0; L < n_layers && ok; ++L) {
          const int nkb = L == 0 ? 1 : kNumKB;
          const int n_units = nkb == 1 ? kPairMT : 16;
          const int n_loads = nkb == 1 ? 1 : kLoadsPerUnit;
          // fc1 reads K block 0, written after the previous tile's TMEM was read out
          if (nkb == 1 && !wait_flip(bar_actq, 0, 0, mc_act, 0x211)) { ok = false; break; }
          uint32_t seen = 0;   // bits 0-3: K quarters used, bits 4-7: blocks written, bits 8-15: units done per block
          for (int u = 0; u < n_units && ok; ++u) {
            const int j = nkb == 1 ? u : pair_unit_j(p.unit_order, u);
            const int kq = nkb == 1 ? 0 : pair_unit_q(p.unit_order, u);
            const bool first_of_block = ((seen >> (4 + j)) & 1u) == 0u;
            if (nkb > 1) {
              // first write into TMEM block j of this layer: the previous layer's values must be out
              if (first_of_block && !wait_flip(bar_tfree, j, 4 + j, mc_tfree, 0x213)) { ok = false; break; }
              // first use of K quarter kq
              if (((seen >> kq) & 1u) == 0u && !wait_flip(bar_actq, kq, kq, mc_act, 0x211)) { ok = false; break; }
            }
            seen |= (1u << kq) | (16u << j);
            // two-bit count of the block's earlier units; the fourth unit completes the block
            const bool last_of_block = nkb == 1 || ((seen >> (8 + 2 * j)) & 3u) == 3u;
            if (!last_of_block) seen += 1u << (8 + 2 * j);
            const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(j * kPairQ);
            for (int g = 0; g < n_loads; ++g) {
              const long long m1 = mtimed ? clock64() : 0;
              if (!mbar_wait_cluster(bar_full + 8 * s, ph, abort_flag, p.status, 0x212)) { ok = false; break; }
              const long long m2 = mtimed ? clock64() : 0;
              const uint64_t a0 = desc_hi | (a_lo0 + s * (kPairStageBytes >> 4));
              const uint64_t b0 = desc_hi | (b_lo0 + static_cast<uint32_t>(kq * 4 + (SPLIT ? 1 : kPairSlotKb) * g) *
                                                         (kPairActKb >> 4));
              if (elect_one()) {
                // a K step of 16: 32 bytes along an A row, 16 K rows (2 KB) of B
                tc_mma_pair_bf16(d_tmem, a0, b0, idesc, (first_of_block && g == 0) ? 0u : 1u);
                tc_mma_pair_bf16(d_tmem, a0 + 2, b0 + 128, idesc, 1u);
                tc_mma_pair_bf16(d_tmem, a0 + 4, b0 + 256, idesc, 1u);
                tc_mma_pair_bf16(d_tmem, a0 + 6, b0 + 384, idesc, 1u);
                if (kPairSlotKb == 2 && nkb > 1) {
                  // second image of the slot (16 KB on): bf16: the next K block, i.e. the next 64 K rows
                  // of the activations (8 KB on); split: the lo part of the same K block, same activations
                  const uint64_t a1 = a0 + (kTileBytes >> 4), b1 = SPLIT ? b0 : b0 + (kPairActKb >> 4);
                  tc_mma_pair_bf16(d_tmem, a1, b1, idesc, 1u);
                  tc_mma_pair_bf16(d_tmem, a1 + 2, b1 + 128, idesc, 1u);
                  tc_mma_pair_bf16(d_tmem, a1 + 4, b1 + 256, idesc, 1u);
                  tc_mma_pair_bf16(d_tmem, a1 + 6, b1 + 384, idesc, 1u);
                }
                tc_commit_pair(bar_empty + 8 * s);
                if (last_of_block && g == n_loads - 1) tc_commit_pair(bar_accj + 8 * j);
              }
              __syncwarp();
              if (mtimed) { mc_full += m2 - m1; mc_issue += clock64() - m2; ++mc_n; }
              if (++s == kPairStages) { s = 0; ph ^= 1u; }
            }
          }
        }
      }
      if (mtimed && lane == 0) {
        p.phase_cycles[4] = mc_act; p.phase_cycles[5] = mc_full; p.phase_cycles[6] = mc_tfree;
        p.phase_cycles[7] = mc_issue; p.phase_cycles[8] = mc_n;
        p.phase_cycles[12] = clock64() - k0;
        p.phase_cycles[13] = static_cast<long long>(global_timer_ns() - g0);
      }
    }
  } else if (warp >= 2) {
    // ------------------------------ epilogue ------------------------------
    // Two groups of four warps (warps 2-5 and 12-15); a warp may only read the
    // TMEM lane quadrant (warp id mod 4).  Group g drains the 256-feature blocks
    // g and g + 2 of a hidden layer (2 g and 2 g + 1 under fc2).
    const int grp = warp >= 12 ? 1 : 0;
    const int e = (warp - (grp ? 12 : 2)) * 32 + lane;   // 0..127 inside the group
    const int T = grp * 128 + e;                         // 0..255 over both groups
    const int quad = warp & 3;
    const int r = quad * 32 + lane;            // feature row inside this CTA's 128-row block
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const int C_in = p.n_op_feat + 4;
    const uint32_t act_peer = map_to_cta(act, peer);
    uint32_t in_phase = 0, lay = 0, tile_no = 0;
    bool ok = true;
    float* red = reinterpret_cast<float*>(base_ptr);   // [256][33], aliases activations
    const bool timed = p.phase_cycles != nullptr && blockIdx.x == 0 && T == 0;
    long long c_wait = 0, c_epi = 0, c_fc2 = 0, c_layers = 0, c_ld = 0, c_bias = 0, c_sync = 0, c_loc = 0, c_rem = 0;
    // named barrier of this group alone (ids 2 and 3; id 1 joins both groups)
    auto group_sync = [&]() { asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory"); };
    auto publish = [&](uint32_t q) {   // "this CTA's share of K quarter q is in place"
      const uint32_t bar = bar_actq + 8 * q;
      if (rank == 0) mbar_arrive(bar);
      else mbar_arrive_remote(map_to_cta(bar, 0));
    };

    for (int t = 0; t < my_tiles && ok; ++t, ++tile_no) {
      const int tile = pair_id + t * n_pairs;
      const int64_t q0 = static_cast<int64_t>(tile) * kTileQ + static_cast<int64_t>(rank) * kHalfQ;

      if (T < kPairHalfQ) {
        // one B column per thread: a query's split features (SPLIT: columns 32..63 are the lo parts
        // of the hidden layers; fc1 carries its own hi/lo expansion along K, so they are zero here)
        const int64_t q = q0 + T;
        __nv_bfloat16 row[kKBlk];
#pragma unroll
        for (int c = 0; c < kKBlk; ++c) row[c] = __float2bfloat16_rn(0.0f);
        if (T < kHalfQ && q < p.Q) {
          int dr = p.dev_row[q];
          dr = dr < p.n_dev ? dr : p.n_dev - 1;
          for (int c = 0; c < C_in; ++c) {
            const double x = c < p.n_op_feat
                                 ? static_cast<double>(p.feats[q * p.n_op_feat + c])
                                 : p.dev_feat[dr * 4 + (c - p.n_op_feat)];
            const float xn = static_cast<float>((x - p.mu[c]) / p.sigma[c]);
            const __nv_bfloat16 hi = __float2bfloat16_rn(xn);
            const __nv_bfloat16 lo = __float2bfloat16_rn(xn - __bfloat162float(hi));
            row[c] = hi;
            row[C_in + c] = lo;
            row[2 * C_in + c] = hi;
          }
        }
        // column T of K rows 0..63 (row k, query n: 128 k + 16 ((n / 8) xor (k mod 8)) + 2 (n mod 8))
#pragma unroll
        for (int c = 0; c < kKBlk; ++c)
          *reinterpret_cast<__nv_bfloat16*>(base_ptr + mn_off(static_cast<uint32_t>(c), static_cast<uint32_t>(T))) = row[c];
      }
      fence_proxy_async();
      pair_epi_bar_sync();
      if (T == 0) publish(0);

      for (int L = 0; L < n_layers && ok; ++L, ++lay) {
        const float* bias = p.bias + L * kWidth;
        const bool last = (L == n_layers - 1);
        if (!last) {
          // Group g drains output blocks g and g + 2.  Block j becomes K quarter j of the next
          // layer and is written over the current activations in place: in the unit order of a
          // hidden layer nothing reads quarter j once block j is complete.  Under fc1 the input
          // sits in quarter 0 until the last block is done, so everything waits for that.
#pragma unroll 1
          for (int jj = 0; jj < 2; ++jj) {
            const int j = grp + 2 * jj;
            const int gate = L == 0 ? 3 : static_cast<int>((p.unit_gates >> (4 * j)) & 3u);
            const long long c0 = timed ? clock64() : 0;
            if (e == 0) {
              epi_ok[grp] = mbar_wait(bar_accj + 8 * gate, lay & 1u, abort_flag, p.status, 0x311) ? 1 : 0;
              // the peer sends 128 K rows x 128 B of this quarter into this CTA
              mbar_expect_tx(bar_inq + 8 * j, 128u * 128u);
            }
            group_sync();
            if (epi_ok[grp] == 0) { ok = false; break; }
            tc_fence_after();
            const long long c1 = timed ? clock64() : 0;
            const int f = j * 256 + static_cast<int>(rank) * 128 + r;   // feature = next layer's K index
            const long long d0 = timed ? clock64() : 0;
            const float b = __ldg(bias + f);
            if (timed) { c_bias += clock64() - d0 + static_cast<long long>(b == 12345.0f); }
            const uint32_t row_off = static_cast<uint32_t>(f) * 128u;   // K row f of the next layer's B operand
            const uint32_t sw = static_cast<uint32_t>(f) & 7u;
            const uint32_t bar_in_peer = map_to_cta(bar_inq + 8 * j, peer);
            const uint32_t bar_tfree_leader = map_to_cta(bar_tfree + 8 * j, 0);
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {         // 64 queries = one CTA's share per load
              // the peer's half first: it has the longer way to go
              const bool mine = hh == 1;
              const uint32_t h = mine ? rank : peer;
              float v[64];
              const long long d1 = timed ? clock64() : 0;
              tc_ld64(t_lane + static_cast<uint32_t>(j * kPairQ) + h * 64u, v);
              if (timed) c_ld += clock64() - d1;
              if (mine) {
                // this warp has read all of its lanes of block j: the next layer may overwrite them
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                  if (rank == 0) mbar_arrive(bar_tfree + 8 * j);
                  else mbar_arrive_remote(bar_tfree_leader);
                }
              }
              if (SPLIT) {
                // columns 0..31 hold W x_hi, 32..63 W x_lo of the same 32 queries: add them, then split
                // the activation into bf16 hi (columns 0..31 of the new row) and lo (32..63)
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                  const float x = fmaxf((v[i] + v[32 + i]) + b, 0.0f);
                  const float hi = __bfloat162float(__float2bfloat16_rn(x));
                  v[i] = hi;
                  v[32 + i] = x - hi;
                }
              } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) v[i] = fmaxf(v[i] + b, 0.0f);
              }
#pragma unroll
              for (int g = 0; g < 8; ++g) {          // eight values per 16-byte store
                uint32_t w4[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const __nv_bfloat162 pk = __floats2bfloat162_rn(v[g * 8 + 2 * u], v[g * 8 + 2 * u + 1]);
                  w4[u] = *reinterpret_cast<const uint32_t*>(&pk);
                }
                const uint32_t off = row_off + ((static_cast<uint32_t>(g) ^ sw) << 4);
                if (mine) *reinterpret_cast<uint4*>(base_ptr + off) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
                else st_async_v4(act_peer + off, w4[0], w4[1], w4[2], w4[3], bar_in_peer);
              }
              if (timed) { if (mine) c_loc += clock64() - d1; else c_rem += clock64() - d1; }
            }
            const long long d2 = timed ? clock64() : 0;
            tc_fence_before();
            asm volatile("fence.proxy.async;" ::: "memory");   // local and peer shared memory
            group_sync();
            if (e == 0) {
              // own stores are fenced above; the peer's arrive as counted bytes
              if (mbar_wait_cluster(bar_inq + 8 * j, in_phase, abort_flag, p.status, 0x313))
                publish(static_cast<uint32_t>(j));
            }
            if (timed) { c_wait += c1 - c0; c_epi += clock64() - c1; c_sync += clock64() - d2; }
          }
          in_phase ^= 1u;
          if (timed) ++c_layers;
        } else {
          const long long c0 = timed ? clock64() : 0;
          if (T == 0) epi_ok[0] = mbar_wait(bar_accj + 8 * 3, lay & 1u, abort_flag, p.status, 0x311) ? 1 : 0;
          pair_epi_bar_sync();
          if (epi_ok[0] == 0) { ok = false; break; }
          tc_fence_after();
          const long long c1 = timed ? clock64() : 0;
          // fc2 over this CTA's 512 features, 32 queries at a time (bf16: the four column quarters
          // of the 128 queries; split: the two CTAs' 32 queries, hi and lo columns added first)
#pragma unroll 1
          for (int qd = 0; qd < (SPLIT ? 2 : 4); ++qd) {
            float acc[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) acc[i] = 0.0f;
#pragma unroll 1
            for (int jj = 0; jj < 2; ++jj) {
              const int j = grp * 2 + jj;
              const int f = j * 256 + static_cast<int>(rank) * 128 + r;
              const float b = __ldg(bias + f);
              const float w = __ldg(p.fc2_w + f);
              if (SPLIT) {
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  float vh[16], vl[16];
                  tc_ld16(t_lane + static_cast<uint32_t>(j * kPairQ + qd * 64 + h * 16), vh);
                  tc_ld16(t_lane + static_cast<uint32_t>(j * kPairQ + qd * 64 + 32 + h * 16), vl);
#pragma unroll
                  for (int i = 0; i < 16; ++i)
                    acc[h * 16 + i] = fmaf(w, fmaxf((vh[i] + vl[i]) + b, 0.0f), acc[h * 16 + i]);
                }
              } else {
                float v[32];
                tc_ld32(t_lane + static_cast<uint32_t>(j * kPairQ + qd * 32), v);
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] = fmaf(w, fmaxf(v[i] + b, 0.0f), acc[i]);
              }
            }
            const int row = grp * 128 + r;
#pragma unroll
            for (int i = 0; i < 32; ++i) red[row * 33 + i] = acc[i];
            pair_epi_bar_sync();
            const int n = T & 31, part = T >> 5;       // 8 parts of 32 feature rows each
            float sum = 0.0f;
            for (int k2 = 0; k2 < 32; ++k2) sum += red[(part * 32 + k2) * 33 + n];
            pair_epi_bar_sync();
            red[part * 32 + n] = sum;
            pair_epi_bar_sync();
            if (T < 32) {
              float tot = 0.0f;
#pragma unroll
              for (int k2 = 0; k2 < 8; ++k2) tot += red[k2 * 32 + T];
              // index among the owner's queries, and which CTA owns them
              const int slot = SPLIT ? T : (qd & 1) * 32 + T;
              const uint32_t owner = static_cast<uint32_t>(SPLIT ? qd : qd >> 1);
              if (owner == rank) fc2_mine[slot] = tot;
              else st_cluster_f32(map_to_cta(smem_u32(fc2_peer + slot), peer), tot);
            }
            pair_epi_bar_sync();
          }
          tc_fence_before();
          // hand-over of the partial sums, then the owner finishes its 64 queries
          if (T == 0) {
            mbar_arrive_remote(map_to_cta(bar_fc2, peer));
            epi_ok[0] = mbar_wait_cluster(bar_fc2, tile_no & 1u, abort_flag, p.status, 0x312) ? 1 : 0;
          }
          pair_epi_bar_sync();
          if (epi_ok[0] == 0) { ok = false; break; }
          if (T < kHalfQ) {
            const int64_t q = q0 + T;
            if (q < p.Q) p.out[q] = fc2_mine[T] + fc2_peer[T] + p.fc2_b;
          }
          pair_epi_bar_sync();
          if (timed) { c_wait += c1 - c0; c_fc2 += clock64() - c1; ++c_layers; }
        }
      }
    }
    if (timed) {
      p.phase_cycles[0] = c_wait; p.phase_cycles[1] = c_epi;
      p.phase_cycles[2] = c_fc2; p.phase_cycles[3] = c_layers;
      p.phase_cycles[14] = c_sync; p.phase_cycles[15] = c_rem;
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before();
  __syncthreads();
  if (rank == 0 && warp >= 6 && warp < 12 && lane == 0 && *abort_flag && warp - 6 < kPairStages && issued > 0) {
    const uint32_t j = issued - 1;
    const uint32_t ph = (j / kPairStages) & 1u;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar_full + 8 * (warp - 6), ph)) {
      if (clock64() - t0 > kWaitCycles) break;
    }
  }
  __syncthreads();
  cluster_sync_all();   // neither CTA leaves while the other may still touch its memory
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u)
                 : "memory");
  }
}

// ---------------------------------------------------------------------------
// Host side: weight packing and launch
// ---------------------------------------------------------------------------
uint16_t f32_to_bf16(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) return static_cast<uint16_t>((u >> 16) | 0x40);
  const uint32_t lsb = (u >> 16) & 1u;
  u += 0x7FFFu + lsb;
  return static_cast<uint16_t>(u >> 16);
}
float bf16_to_f32(uint16_t h) {
  const uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

void put(uint8_t* tile, int row, int col, uint16_t v) {
  std::memcpy(tile + swz_off(static_cast<uint32_t>(row), static_cast<uint32_t>(col)), &v, 2);
}

}  // namespace

struct hb_mlp {
  int32_t n_op_feat = 0, layers = 0, precision = 0, n_dev = 0, sm_count = 0, device = 0;
  float fc2_b = 0.f;
  uint8_t* wpack = nullptr;
  CUtensorMap tmap_slot{}, tmap_tile{};
  float* bias = nullptr;
  float* fc2_w = nullptr;
  double* mu = nullptr;
  double* sigma = nullptr;
  double* dev_feat = nullptr;
  int32_t* status = nullptr;
  long long* phase_cycles = nullptr;
};

extern "C" void hb_mlp_destroy(hb_mlp* h) {
  if (!h) return;
  cudaFree(h->wpack); cudaFree(h->bias); cudaFree(h->fc2_w); cudaFree(h->mu);
  cudaFree(h->sigma); cudaFree(h->dev_feat); cudaFree(h->status); cudaFree(h->phase_cycles);
  delete h;
}

extern "C" hb_status hb_mlp_create(hb_mlp** handle, int32_t n_op_features, int32_t layers,
                                   int32_t width, const float* fc1_w, const float* fc1_b,
                                   const float* hidden_w, const float* hidden_b,
                                   const float* fc2_w, const float* fc2_b, const double* mu,
                                   const double* sigma, const double* device_features,
                                   int32_t n_device_rows, int32_t precision) {
  if (!handle || !fc1_w || !fc1_b || (layers > 0 && (!hidden_w || !hidden_b)) || !fc2_w || !fc2_b ||
      !mu || !sigma || !device_features) {
    hb::set_error("hb_mlp_create: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (width < 1 || width > kWidth || layers < 1 || layers > 64 || n_op_features < 1 ||
      n_op_features + 4 > kMaxInFeat || n_device_rows < 1 || n_device_rows > 256 ||
      (precision != HB_PRECISION_BF16 && precision != HB_PRECISION_BF16X3)) {
    hb::set_error("hb_mlp_create: unsupported shape (1 <= width <= 1024, 1 <= F <= 8, 1 <= layers <= 64)");
    return HB_ERR_UNSUPPORTED;
  }
  // The kernel is built for 1024-wide layers.  A narrower network runs as a 1024-wide one whose
  // extra features have zero weights and zero bias: they stay 0 through every ReLU and add
  // nothing to any sum, so the results are those of the narrow network.
  std::vector<float> pad_fc1_w, pad_fc1_b, pad_hidden_w, pad_hidden_b, pad_fc2_w;
  if (width < kWidth) {
    const int C = n_op_features + 4;
    pad_fc1_w.assign(static_cast<size_t>(kWidth) * C, 0.0f);
    pad_fc1_b.assign(kWidth, 0.0f);
    pad_hidden_w.assign(static_cast<size_t>(layers) * kWidth * kWidth, 0.0f);
    pad_hidden_b.assign(static_cast<size_t>(layers) * kWidth, 0.0f);
    pad_fc2_w.assign(kWidth, 0.0f);
    std::memcpy(pad_fc1_w.data(), fc1_w, sizeof(float) * width * C);
    std::memcpy(pad_fc1_b.data(), fc1_b, sizeof(float) * width);
    std::memcpy(pad_fc2_w.data(), fc2_w, sizeof(float) * width);
    for (int L = 0; L < layers; ++L) {
      std::memcpy(&pad_hidden_b[static_cast<size_t>(L) * kWidth], hidden_b + static_cast<size_t>(L) * width,
                  sizeof(float) * width);
      for (int r = 0; r < width; ++r)
        std::memcpy(&pad_hidden_w[(static_cast<size_t>(L) * kWidth + r) * kWidth],
                    hidden_w + (static_cast<size_t>(L) * width + r) * width, sizeof(float) * width);
    }
    fc1_w = pad_fc1_w.data(); fc1_b = pad_fc1_b.data();
    hidden_w = pad_hidden_w.data(); hidden_b = pad_hidden_b.data();
    fc2_w = pad_fc2_w.data();
  }
  const bool split = precision == HB_PRECISION_BF16X3;
  const int C_in = n_op_features + 4;
  const size_t img = split ? 2 * kTileBytes : kTileBytes;
  const size_t n_img = kNumMT + static_cast<size_t>(layers) * kNumMT * kNumKB;
  std::vector<uint8_t> pack(n_img * img, 0);
  uint8_t* dst = pack.data();
  // fc1: [w_hi | w_hi | w_lo] along K, matching the activations' [x_hi | x_lo | x_hi]
  for (int mt = 0; mt < kNumMT; ++mt, dst += img) {
    for (int rr = 0; rr < kMTile; ++rr) {
      const float* wrow = fc1_w + static_cast<size_t>(mt * kMTile + rr) * C_in;
      for (int c = 0; c < C_in; ++c) {
        const uint16_t hi = f32_to_bf16(wrow[c]);
        const uint16_t lo = f32_to_bf16(wrow[c] - bf16_to_f32(hi));
        put(dst, rr, c, hi);
        put(dst, rr, C_in + c, hi);
        put(dst, rr, 2 * C_in + c, lo);
      }
    }
  }
  for (int L = 0; L < layers; ++L) {
    const float* W = hidden_w + static_cast<size_t>(L) * kWidth * kWidth;
    for (int mt = 0; mt < kNumMT; ++mt) {
      for (int kb = 0; kb < kNumKB; ++kb, dst += img) {
        for (int rr = 0; rr < kMTile; ++rr) {
          const float* wrow = W + static_cast<size_t>(mt * kMTile + rr) * kWidth + kb * kKBlk;
          for (int c = 0; c < kKBlk; ++c) {
            const uint16_t hi = f32_to_bf16(wrow[c]);
            put(dst, rr, c, hi);
            if (split) put(dst + kTileBytes, rr, c, f32_to_bf16(wrow[c] - bf16_to_f32(hi)));
          }
        }
      }
    }
  }

  hb_mlp* h = new hb_mlp();
  h->n_op_feat = n_op_features;
  h->layers = layers;
  h->precision = precision;
  h->n_dev = n_device_rows;
  h->fc2_b = fc2_b[0];
  auto fail = [&](cudaError_t e, const char* what) {
    hb_status st = hb::cuda_fail(e, what);
    hb_mlp_destroy(h);
    return st;
  };
  cudaError_t e;
  if ((e = cudaGetDevice(&h->device)) != cudaSuccess) return fail(e, "cudaGetDevice");
  if ((e = cudaDeviceGetAttribute(&h->sm_count, cudaDevAttrMultiProcessorCount, h->device)) != cudaSuccess)
    return fail(e, "cudaDeviceGetAttribute");
  std::vector<float> bias(static_cast<size_t>(layers + 1) * kWidth);
  std::memcpy(bias.data(), fc1_b, sizeof(float) * kWidth);
  std::memcpy(bias.data() + kWidth, hidden_b, sizeof(float) * kWidth * layers);
#define HB_UP(field, src, bytes)                                                        \
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->field), (bytes))) != cudaSuccess)    \
    return fail(e, "cudaMalloc " #field);                                               \
  if ((e = cudaMemcpy(h->field, (src), (bytes), cudaMemcpyHostToDevice)) != cudaSuccess) \
    return fail(e, "cudaMemcpy " #field);
  HB_UP(wpack, pack.data(), pack.size());
  HB_UP(bias, bias.data(), bias.size() * sizeof(float));
  HB_UP(fc2_w, fc2_w, sizeof(float) * kWidth);
  HB_UP(mu, mu, sizeof(double) * C_in);
  HB_UP(sigma, sigma, sizeof(double) * C_in);
  HB_UP(dev_feat, device_features, sizeof(double) * 4 * n_device_rows);
#undef HB_UP
  {
    // The pack as a 2-D tensor of 128-byte rows for the tiled TMA loads of the pair kernel.  The
    // tile images are stored already swizzled, so the maps use no swizzle of their own.
    using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if ((e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres)) != cudaSuccess)
      return fail(e, "cudaGetDriverEntryPoint(cuTensorMapEncodeTiled)");
    if (fn == nullptr || qres != cudaDriverEntryPointSuccess) {
      hb::set_error("hb_mlp_create: the driver does not export cuTensorMapEncodeTiled");
      hb_mlp_destroy(h);
      return HB_ERR_CUDA;
    }
    const cuuint64_t dims[2] = {128, static_cast<cuuint64_t>(pack.size() / 128)};
    const cuuint64_t strides[1] = {128};
    const cuuint32_t elem[2] = {1, 1};
    for (int which = 0; which < 2; ++which) {
      const cuuint32_t box[2] = {128, static_cast<cuuint32_t>((which == 0 ? kPairStageBytes : kTileBytes) / 128)};
      const CUresult r = reinterpret_cast<EncodeFn>(fn)(
          which == 0 ? &h->tmap_slot : &h->tmap_tile, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, h->wpack, dims, strides,
          box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
      if (r != CUDA_SUCCESS) {
        hb::set_error("hb_mlp_create: cuTensorMapEncodeTiled failed (CUresult %d)", static_cast<int>(r));
        hb_mlp_destroy(h);
        return HB_ERR_CUDA;
      }
    }
  }
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->status), sizeof(int32_t))) != cudaSuccess)
    return fail(e, "cudaMalloc status");
  if ((e = cudaMemset(h->status, 0, sizeof(int32_t))) != cudaSuccess) return fail(e, "cudaMemset");
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->phase_cycles), 16 * sizeof(long long))) != cudaSuccess)
    return fail(e, "cudaMalloc phase_cycles");
  if ((e = cudaMemset(h->phase_cycles, 0, 16 * sizeof(long long))) != cudaSuccess) return fail(e, "cudaMemset");
  e = cudaFuncSetAttribute(mlp_chain_pair_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kPairSmemBytes);
  if (e != cudaSuccess) return fail(e, "cudaFuncSetAttribute");
  e = cudaFuncSetAttribute(mlp_chain_pair_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           kPairSmemBytes);
  if (e != cudaSuccess) return fail(e, "cudaFuncSetAttribute");
  *handle = h;
  return HB_OK;
}

extern "C" hb_status hb_mlp_predict(hb_mlp* h, const float* op_features, const uint8_t* device_row,
                                    int64_t Q, float* out, void* stream) {
  if (!h || Q < 0 || (Q > 0 && (!op_features || !device_row || !out))) {
    hb::set_error("hb_mlp_predict: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (Q == 0) return HB_OK;
  int cur = -1;
  HB_CUDA_TRY(cudaGetDevice(&cur));
  if (cur != h->device) {
    // the weight pack, the tensor maps and the status word live on the GPU the handle was created on
    hb::set_error("hb_mlp_predict: the handle belongs to CUDA device %d but device %d is current", h->device, cur);
    return HB_ERR_INVALID_ARGUMENT;
  }
  const bool split = h->precision == HB_PRECISION_BF16X3;
  const int tile_q = split ? kPairQ / 2 : kPairQ;
  const int64_t tiles = (Q + tile_q - 1) / tile_q;
  if (tiles > 0x7FFFFFFF) {
    hb::set_error("hb_mlp_predict: Q too large for one launch");
    return HB_ERR_TOO_LARGE;
  }
  MlpParams p{};
  p.wpack = h->wpack; p.bias = h->bias; p.fc2_w = h->fc2_w; p.fc2_b = h->fc2_b;
  p.mu = h->mu; p.sigma = h->sigma; p.dev_feat = h->dev_feat; p.n_dev = h->n_dev;
  p.n_op_feat = h->n_op_feat; p.layers = h->layers; p.feats = op_features;
  p.dev_row = device_row; p.Q = Q; p.out = out; p.num_tiles = static_cast<int32_t>(tiles);
  p.status = h->status;
  p.phase_cycles = h->phase_cycles;
  p.tmap_slot = h->tmap_slot; p.tmap_tile = h->tmap_tile;
  p.unit_order = kPairOrder;
  p.unit_gates = kPairGates;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // one cluster of two CTAs per tile (128 queries, 64 in split precision), at most one cluster per SM pair
  const int pairs = static_cast<int>(tiles < h->sm_count / 2 ? tiles : h->sm_count / 2);
  if (split) mlp_chain_pair_kernel<true><<<2 * pairs, kPairThreads, kPairSmemBytes, s>>>(p);
  else mlp_chain_pair_kernel<false><<<2 * pairs, kPairThreads, kPairSmemBytes, s>>>(p);
  HB_CUDA_TRY(cudaGetLastError());
  return HB_OK;
}

extern "C" hb_status hb_mlp_status(hb_mlp* h, int32_t* device_status) {
  if (!h || !device_status) {
    hb::set_error("hb_mlp_status: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  HB_CUDA_TRY(cudaDeviceSynchronize());   // launches on non-blocking streams included
  HB_CUDA_TRY(cudaMemcpy(device_status, h->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (*device_status != 0) {
    // reported once: the word is cleared so that later launches are judged on their own
    HB_CUDA_TRY(cudaMemset(h->status, 0, sizeof(int32_t)));
    hb::set_error("mlp kernel: a bounded device-side wait ran out (site 0x%x)", *device_status);
    return HB_ERR_DEVICE_TIMEOUT;
  }
  return HB_OK;
}

extern "C" hb_status hb_mlp_inject_status(hb_mlp* h, int32_t device_status) {
  if (!h) {
    hb::set_error("hb_mlp_inject_status: NULL handle");
    return HB_ERR_INVALID_ARGUMENT;
  }
  HB_CUDA_TRY(cudaMemcpy(h->status, &device_status, sizeof(int32_t), cudaMemcpyHostToDevice));
  return HB_OK;
}

extern "C" hb_status hb_mlp_phase_cycles(hb_mlp* h, int64_t out[16]) {
  if (!h || !out) {
    hb::set_error("hb_mlp_phase_cycles: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  long long v[16];
  HB_CUDA_TRY(cudaMemcpy(v, h->phase_cycles, sizeof(v), cudaMemcpyDeviceToHost));
  for (int i = 0; i < 16; ++i) out[i] = v[i];
  return HB_OK;
}

extern "C" hb_status hb_mlp_predict_host(hb_mlp* h, const float* op_features,
                                         const uint8_t* device_row, int64_t Q, float* out) {
  if (!h || Q < 0 || (Q > 0 && (!op_features || !device_row || !out))) {
    hb::set_error("hb_mlp_predict_host: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (Q == 0) return HB_OK;
  // staged through the per-GPU block and stream the `_host` entry points share
  hb::HostArena* arena = nullptr;
  hb_status st = hb::arena_for_current_device(&arena);
  if (st != HB_OK) return st;
  std::lock_guard<std::mutex> lock(arena->mu);
  const size_t q = static_cast<size_t>(Q);
  hb::Carver sizes(nullptr);
  sizes.take<float>(q * h->n_op_feat); sizes.take<uint8_t>(q); sizes.take<float>(q);
  st = hb::arena_reserve(arena, sizes.used());
  if (st != HB_OK) return st;
  hb::Carver c(arena->base);
  float* d_f = c.take<float>(q * h->n_op_feat);
  uint8_t* d_r = c.take<uint8_t>(q);
  float* d_o = c.take<float>(q);
  cudaStream_t s = arena->stream;
  HB_CUDA_TRY(cudaMemcpyAsync(d_f, op_features, sizeof(float) * q * h->n_op_feat, cudaMemcpyHostToDevice, s));
  HB_CUDA_TRY(cudaMemcpyAsync(d_r, device_row, q, cudaMemcpyHostToDevice, s));
  st = hb_mlp_predict(h, d_f, d_r, Q, d_o, s);
  if (st != HB_OK) return st;
  HB_CUDA_TRY(cudaMemcpyAsync(out, d_o, sizeof(float) * q, cudaMemcpyDeviceToHost, s));
  HB_CUDA_TRY(cudaStreamSynchronize(s));
  int32_t code = 0;
  return hb_mlp_status(h, &code);
}
