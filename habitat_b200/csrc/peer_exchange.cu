// All-reduce of a handful of float64 totals between the GPUs of one box, fused into the last
// stage of the reductions that produce them.
//
// The prediction path shards kernels and queries across GPUs and exchanges nothing but totals
// (per-destination sums: 6 to 64 numbers).  A library all-reduce of that size costs tens of
// microseconds of launch and protocol latency, which is more than the sharded wave-scaling
// kernel itself takes on eight GPUs.  Here the final stage of the plane / group sum writes
// its results straight into a mailbox in every peer's memory (plain 8-byte stores over NVLink
// through peer-mapped pointers), then reads the peers' values from its own mailbox and adds
// them in rank order, so every GPU ends with the same bits.  One kernel does the last
// reduction step and the exchange.  The reference has no counterpart (its totals are host
// sums in one process, analyzer/habitat/analysis/trace.py:26-36).
//
// Mailbox of one GPU: slots[2 parities][world ranks][kPeerSlots] of {value, sequence}.  A call
// with sequence number s writes value then s (release) into slot [s & 1][my rank][i] of every
// peer and waits (acquire) for s in [s & 1][r][i] of its own mailbox for every rank r.  The
// parity keeps call s + 1 from overwriting values a slower peer is still reading for call s;
// slot [s & 1] is reused by call s + 2, which a rank can only start after every peer has
// written its flag of call s + 1, i.e. has finished reading call s.  That argument needs the
// calls of a handle to be ordered on each GPU (one stream, or events), and every rank to make
// the same calls in the same order.
//
// Every wait is bounded (one second unless hb_peer_set_wait_ns says otherwise): when it runs out the kernel records which (rank, slot)
// it gave up on in the handle's status word, writes NaN and returns; nothing traps.  No
// multicast of any kind is used: stores go to each peer in turn.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <mutex>
#include <vector>

#include "hb_common.h"
#include "reduce_stage1.cuh"

namespace {

constexpr int kPeerSlots = 64;            // values per call
constexpr int kPeerMaxWorld = 16;

struct PeerSlot {
  double value;
  unsigned long long seq;
};

struct PeerView {                          // what a kernel needs of a handle
  PeerSlot* boxes[kPeerMaxWorld];          // mailbox of every rank (peer-mapped; [rank] is the local one)
  int32_t rank, world;
  unsigned long long seq;
  unsigned long long wait_ns;
  int32_t* status;                         // device word: 0 ok, else 0x40000000 | rank << 8 | slot
};

__device__ __forceinline__ PeerSlot* slot_of(PeerSlot* box, unsigned long long seq, int world, int src, int i) {
  return box + ((static_cast<int>(seq & 1ull) * world + src) * kPeerSlots + i);
}
__device__ __forceinline__ void store_release_sys(unsigned long long* p, unsigned long long v) {
  asm volatile("st.global.release.sys.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long load_acquire_sys(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.global.acquire.sys.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Thread r < world publishes `mine` as element i of this call into rank r's mailbox.
__device__ __forceinline__ void peer_push(const PeerView& pv, int i, double mine) {
  const int r = threadIdx.x;
  if (r < pv.world) {
    PeerSlot* s = slot_of(pv.boxes[r], pv.seq, pv.world, pv.rank, i);
    s->value = mine;                                  // plain store into the peer's memory
    store_release_sys(&s->seq, pv.seq);               // orders the value before the flag
  }
}

// Thread r < world waits for rank r's element i; then thread 0 adds the values in rank order.
// Returns the sum in thread 0 (NaN when a wait ran out).  `sh` holds kPeerMaxWorld doubles.
__device__ __forceinline__ double peer_collect(const PeerView& pv, int i, double* sh) {
  const int r = threadIdx.x;
  if (r < pv.world) {
    PeerSlot* s = slot_of(pv.boxes[pv.rank], pv.seq, pv.world, r, i);
    double v = __longlong_as_double(0x7FF8000000000000ll);
    const unsigned long long t0 = now_ns();
    for (unsigned spins = 0;; ++spins) {
      if (load_acquire_sys(&s->seq) == pv.seq) {
        v = *reinterpret_cast<volatile double*>(&s->value);
        break;
      }
      if ((spins & 63u) == 63u && now_ns() - t0 > pv.wait_ns) {
        atomicCAS(pv.status, 0, 0x40000000 | (r << 8) | i);
        break;
      }
    }
    sh[r] = v;
  }
  __syncthreads();
  double total = 0.0;
  if (threadIdx.x == 0)
    for (int q = 0; q < pv.world; ++q) total += sh[q];
  __syncthreads();
  return total;
}

// Final stage + exchange: block i adds the `per_plane` partial sums of value i, publishes the result
// to every rank and gathers the ranks' results.  phase: 1 publish only, 2 gather only (of a
// value published by an earlier launch: `out` holds it), 3 both (the normal, fused call).
// CLUSTER consecutive blocks share a value when its list of partial sums is long (the launch
// then carries that cluster dimension); the first of them does the exchange.
template <int CLUSTER>
__global__ void __launch_bounds__(kFinalThreadsMax)
peer_final_exchange_kernel(const double* __restrict__ partial, int per_plane, double* __restrict__ out,
                           const PeerView pv, int phase) {
  hb_grid_dependency_wait();
  __shared__ double sh[kPeerMaxWorld];
  const int i = blockIdx.x / CLUSTER;
  double mine = 0.0;
  if (phase & 1) {
    const double t = partial ? plane_total<CLUSTER>(partial, per_plane) : 0.0;
    if (CLUSTER > 1 && blockIdx.x % CLUSTER != 0) return;   // helped with the sum; past the cluster's last barrier
    if (threadIdx.x == 0) sh[0] = partial ? t : out[i];
    __syncthreads();
    mine = sh[0];
    __syncthreads();
    peer_push(pv, i, mine);
  }
  if (phase & 2) {
    const double total = peer_collect(pv, i, sh);
    if (threadIdx.x == 0) out[i] = total;
  }
}

}  // namespace

struct hb_peer {
  int32_t rank = 0, world = 1, device = 0;
  PeerSlot* local = nullptr;                   // this GPU's mailbox (cudaMalloc)
  PeerSlot* boxes[kPeerMaxWorld] = {};
  bool opened[kPeerMaxWorld] = {};             // mapped with cudaIpcOpenMemHandle
  bool connected = false;
  double* partial = nullptr;                   // [kPeerSlots][256] stage-1 sums
  int32_t* status = nullptr;
  unsigned long long seq = 0;
  unsigned long long wait_ns = 1000000000ull;  // one second
};

namespace {
size_t mailbox_bytes(int world) { return sizeof(PeerSlot) * 2 * world * kPeerSlots; }

hb_status check_call(hb_peer* h, const char* who, int32_t n) {
  if (!h || !h->connected) {
    hb::set_error("%s: the handle is not connected", who);
    return HB_ERR_INVALID_ARGUMENT;
  }
  if (n > kPeerSlots) {
    hb::set_error("%s: %d values per call requested, a mailbox holds %d", who, n, kPeerSlots);
    return HB_ERR_TOO_LARGE;
  }
  int cur = -1;
  HB_CUDA_TRY(cudaGetDevice(&cur));
  if (cur != h->device) {
    hb::set_error("%s: the handle belongs to CUDA device %d but device %d is current", who, h->device, cur);
    return HB_ERR_INVALID_ARGUMENT;
  }
  return HB_OK;
}

PeerView view_of(hb_peer* h) {
  PeerView pv{};
  for (int r = 0; r < h->world; ++r) pv.boxes[r] = h->boxes[r];
  pv.rank = h->rank;
  pv.world = h->world;
  pv.seq = h->seq;
  pv.wait_ns = h->wait_ns;
  pv.status = h->status;
  return pv;
}
}  // namespace

extern "C" hb_status hb_peer_create(hb_peer** handle, int32_t rank, int32_t world) {
  if (!handle || world < 1 || world > kPeerMaxWorld || rank < 0 || rank >= world) {
    hb::set_error("hb_peer_create: need 0 <= rank < world <= %d", kPeerMaxWorld);
    return HB_ERR_INVALID_ARGUMENT;
  }
  hb_peer* h = new hb_peer();
  h->rank = rank;
  h->world = world;
  auto fail = [&](cudaError_t e, const char* what) {
    const hb_status st = hb::cuda_fail(e, what);
    cudaFree(h->local); cudaFree(h->partial); cudaFree(h->status);
    delete h;
    return st;
  };
  cudaError_t e;
  if ((e = cudaGetDevice(&h->device)) != cudaSuccess) return fail(e, "cudaGetDevice");
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->local), mailbox_bytes(world))) != cudaSuccess)
    return fail(e, "cudaMalloc mailbox");
  if ((e = cudaMemset(h->local, 0, mailbox_bytes(world))) != cudaSuccess) return fail(e, "cudaMemset mailbox");
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->partial), sizeof(double) * kPeerSlots * kPlaneBlocks)) != cudaSuccess)
    return fail(e, "cudaMalloc partial");
  if ((e = cudaMalloc(reinterpret_cast<void**>(&h->status), sizeof(int32_t))) != cudaSuccess)
    return fail(e, "cudaMalloc status");
  if ((e = cudaMemset(h->status, 0, sizeof(int32_t))) != cudaSuccess) return fail(e, "cudaMemset status");
  if ((e = cudaDeviceSynchronize()) != cudaSuccess) return fail(e, "cudaDeviceSynchronize");
  h->boxes[rank] = h->local;
  if (world == 1) h->connected = true;
  *handle = h;
  return HB_OK;
}

extern "C" hb_status hb_peer_export(hb_peer* h, uint8_t out[64]) {
  if (!h || !out) {
    hb::set_error("hb_peer_export: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "an IPC memory handle is 64 bytes");
  cudaIpcMemHandle_t ipc;
  HB_CUDA_TRY(cudaIpcGetMemHandle(&ipc, h->local));
  std::memcpy(out, &ipc, 64);
  return HB_OK;
}

extern "C" hb_status hb_peer_connect(hb_peer* h, const uint8_t* handles) {
  if (!h || !handles) {
    hb::set_error("hb_peer_connect: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  for (int r = 0; r < h->world; ++r) {
    if (r == h->rank || h->boxes[r]) continue;
    cudaIpcMemHandle_t ipc;
    std::memcpy(&ipc, handles + 64 * r, 64);
    void* p = nullptr;
    HB_CUDA_TRY(cudaIpcOpenMemHandle(&p, ipc, cudaIpcMemLazyEnablePeerAccess));
    h->boxes[r] = static_cast<PeerSlot*>(p);
    h->opened[r] = true;
  }
  h->connected = true;
  return HB_OK;
}

extern "C" hb_status hb_peer_connect_pointers(hb_peer* h, void* const* mailboxes) {
  if (!h || !mailboxes) {
    hb::set_error("hb_peer_connect_pointers: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  for (int r = 0; r < h->world; ++r) {
    if (r == h->rank) continue;
    if (!mailboxes[r]) {
      hb::set_error("hb_peer_connect_pointers: no mailbox for rank %d", r);
      return HB_ERR_INVALID_ARGUMENT;
    }
    h->boxes[r] = static_cast<PeerSlot*>(mailboxes[r]);
  }
  h->connected = true;
  return HB_OK;
}

extern "C" void* hb_peer_mailbox(hb_peer* h) { return h ? h->local : nullptr; }

extern "C" hb_status hb_peer_set_wait_ns(hb_peer* h, int64_t wait_ns) {
  if (!h || wait_ns < 1000 || wait_ns > 10000000000ll) {
    hb::set_error("hb_peer_set_wait_ns: need a handle and 1 us <= wait <= 10 s");
    return HB_ERR_INVALID_ARGUMENT;
  }
  h->wait_ns = static_cast<unsigned long long>(wait_ns);
  return HB_OK;
}

extern "C" void hb_peer_destroy(hb_peer* h) {
  if (!h) return;
  cudaDeviceSynchronize();
  for (int r = 0; r < h->world; ++r)
    if (h->opened[r]) cudaIpcCloseMemHandle(h->boxes[r]);
  cudaFree(h->local);
  cudaFree(h->partial);
  cudaFree(h->status);
  delete h;
}

extern "C" hb_status hb_peer_status(hb_peer* h, int32_t* device_status) {
  if (!h || !device_status) {
    hb::set_error("hb_peer_status: NULL argument");
    return HB_ERR_INVALID_ARGUMENT;
  }
  HB_CUDA_TRY(cudaDeviceSynchronize());
  HB_CUDA_TRY(cudaMemcpy(device_status, h->status, sizeof(int32_t), cudaMemcpyDeviceToHost));
  if (*device_status != 0) {
    HB_CUDA_TRY(cudaMemset(h->status, 0, sizeof(int32_t)));   // reported once
    hb::set_error("peer exchange: gave up waiting for rank %d, value %d (status 0x%x)",
                  (*device_status >> 8) & 0xFF, *device_status & 0xFF, *device_status);
    return HB_ERR_DEVICE_TIMEOUT;
  }
  return HB_OK;
}

extern "C" hb_status hb_plane_sum_allreduce(hb_peer* h, const float* values, int64_t plane_len,
                                            int32_t n_planes, double* out, void* stream) {
  if (plane_len < 0 || n_planes < 1 || !values || !out) {
    hb::set_error("hb_plane_sum_allreduce: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  const hb_status st = check_call(h, "hb_plane_sum_allreduce", n_planes);
  if (st != HB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ++h->seq;
  HB_CUDA_TRY(hb::launch_overlapped(plane_partial_kernel, dim3(n_planes, kPlaneBlocks), dim3(kSumThreads), 0, s,
                                    values, plane_len, h->partial));
  HB_CUDA_TRY(hb::launch_overlapped(peer_final_exchange_kernel<1>, dim3(n_planes), dim3(kSumThreads), 0, s,
                                    static_cast<const double*>(h->partial), kPlaneBlocks, out, view_of(h), 3));
  return HB_OK;
}

extern "C" hb_status hb_partials_sum_allreduce(hb_peer* h, const double* partials, int32_t per_plane,
                                               int32_t n_planes, double* out, void* stream) {
  if (per_plane < 0 || n_planes < 1 || !out || (per_plane > 0 && !partials)) {
    hb::set_error("hb_partials_sum_allreduce: bad arguments");
    return HB_ERR_INVALID_ARGUMENT;
  }
  const hb_status st = check_call(h, "hb_partials_sum_allreduce", n_planes);
  if (st != HB_OK) return st;
  ++h->seq;
  // an empty shard (per_plane 0) still takes part in the exchange, with zeros
  const double* list = per_plane > 0 ? partials : h->partial;
  if (final_cluster(per_plane) == 1) {
    HB_CUDA_TRY(hb::launch_overlapped(peer_final_exchange_kernel<1>, dim3(n_planes), dim3(final_threads(per_plane)), 0,
                                      static_cast<cudaStream_t>(stream), list, per_plane, out, view_of(h), 3));
  } else {
    HB_CUDA_TRY(hb::launch_overlapped_cluster(peer_final_exchange_kernel<kFinalCluster>,
                                              dim3(n_planes * kFinalCluster), dim3(kFinalThreadsMax), kFinalCluster,
                                              static_cast<cudaStream_t>(stream), list, per_plane, out, view_of(h), 3));
  }
  return HB_OK;
}

extern "C" hb_status hb_group_sum_allreduce(hb_peer* h, const float* values, const uint8_t* keys, int64_t n,
                                            int32_t n_groups, double* out, void* stream) {
  if (n < 0 || n_groups < 1 || n_groups > kMaxGroups || !out || (n > 0 && (!values || !keys))) {
    hb::set_error("hb_group_sum_allreduce: bad arguments (1 <= n_groups <= %d)", kMaxGroups);
    return HB_ERR_INVALID_ARGUMENT;
  }
  const hb_status st = check_call(h, "hb_group_sum_allreduce", n_groups);
  if (st != HB_OK) return st;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  ++h->seq;
  HB_CUDA_TRY(hb::launch_overlapped(group_partial_kernel, dim3(kGroupBlocks), dim3(kSumThreads), 0, s, values,
                                    keys, n, 0, n_groups, h->partial));
  HB_CUDA_TRY(hb::launch_overlapped(peer_final_exchange_kernel<1>, dim3(n_groups), dim3(kSumThreads), 0, s,
                                    static_cast<const double*>(h->partial), kGroupBlocks, out, view_of(h), 3));
  return HB_OK;
}

extern "C" hb_status hb_peer_allreduce(hb_peer* h, double* values, int32_t n, int32_t phase, void* stream) {
  if (!values || n < 1 || phase < 1 || phase > 3) {
    hb::set_error("hb_peer_allreduce: bad arguments (phase 1 publish, 2 gather, 3 both)");
    return HB_ERR_INVALID_ARGUMENT;
  }
  const hb_status st = check_call(h, "hb_peer_allreduce", n);
  if (st != HB_OK) return st;
  if (phase & 1) ++h->seq;      // a gather-only call belongs to the publish before it
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  HB_CUDA_TRY(hb::launch_overlapped(peer_final_exchange_kernel<1>, dim3(n), dim3(kSumThreads), 0, s,
                                    static_cast<const double*>(nullptr), 0, values, view_of(h), phase));
  return HB_OK;
}
