// Error text and version of the library.
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
}  // namespace hb

extern "C" const char* hb_last_error(void) { return t_error; }
extern "C" const char* hb_version(void) { return "0.1.0"; }
