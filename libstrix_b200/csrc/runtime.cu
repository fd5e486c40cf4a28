// Error reporting and version query of the C-ABI.
#include "common.cuh"

namespace strix {

char* error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

}  // namespace strix

extern "C" const char* strix_last_error(void) { return strix::error_buffer(); }

extern "C" int strix_version(void) { return 1000; }
