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
}  // namespace hb

extern "C" const char* hb_last_error(void) { return t_error; }
extern "C" const char* hb_version(void) { return "0.1.0"; }
