// Error text and version of the library.
#include <cstdlib>

#include "hb_common.h"

namespace {
thread_local char t_error[512] = "";
}

namespace hb {
void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}
bool overlapped_launch_enabled() {
  static const bool on = [] {
    const char* e = std::getenv("HB_NO_OVERLAPPED_LAUNCH");
    return !(e && e[0] && e[0] != '0');
  }();
  return on;
}

namespace {
constexpr int kArenaDevices = 64;
HostArena g_arena[kArenaDevices];
std::mutex g_arena_mu;
}  // namespace

hb_status arena_for_current_device(HostArena** out) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return cuda_fail(e, "cudaGetDevice");
  if (dev < 0 || dev >= kArenaDevices) {
    set_error("device ordinal %d out of range", dev);
    return HB_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_arena_mu);
  HostArena& a = g_arena[dev];
  if (!a.stream) {
    e = cudaStreamCreateWithFlags(&a.stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) return cuda_fail(e, "cudaStreamCreateWithFlags");
  }
  *out = &a;
  return HB_OK;
}

hb_status arena_reserve(HostArena* a, size_t bytes) {
  if (bytes <= a->bytes) return HB_OK;
  // nothing of an earlier call is in flight: every `_host` call ends with a synchronise
  if (a->base) cudaFree(a->base);
  a->base = nullptr;
  a->bytes = 0;
  const size_t want = bytes + bytes / 4;   // head room, so that slowly growing batches do not reallocate each time
  cudaError_t e = cudaMalloc(&a->base, want);
  if (e != cudaSuccess) {
    e = cudaMalloc(&a->base, bytes);
    if (e != cudaSuccess) return cuda_fail(e, "cudaMalloc (host-entry staging)");
    a->bytes = bytes;
    return HB_OK;
  }
  a->bytes = want;
  return HB_OK;
}
}  // namespace hb

extern "C" const char* hb_last_error(void) { return t_error; }
extern "C" const char* hb_version(void) { return "0.1.0"; }
