// Error reporting of the C ABI: a thread-local message behind epsb_last_error().
#include "common.cuh"

namespace epsb {

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return code;
}

int gemm_cta_limit(int want) {
  const int all = sm_count();
  return want > 0 && want < all ? want : all;
}

}  // namespace epsb

extern "C" const char* epsb_last_error(void) { return epsb::last_error_buffer(); }
extern "C" int epsb_version(void) { return 2; }
