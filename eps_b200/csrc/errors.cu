// Error reporting of the C ABI: a thread-local message behind epsb_last_error().
#include <atomic>

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

namespace {
std::atomic<int> g_gemm_sm_count{0};
}

int gemm_cta_limit() {
  const int all = sm_count();
  const int want = g_gemm_sm_count.load(std::memory_order_relaxed);
  return want > 0 && want < all ? want : all;
}

}  // namespace epsb

extern "C" int epsb_gemm_set_sm_count(int sm_count) {
  if (sm_count < 0) return epsb::fail(EPSB_ERR_INVALID, "sm_count %d is negative", sm_count);
  epsb::g_gemm_sm_count.store(sm_count, std::memory_order_relaxed);
  return EPSB_OK;
}

extern "C" const char* epsb_last_error(void) { return epsb::last_error_buffer(); }
extern "C" int epsb_version(void) { return 1; }
