// Error reporting and version of the rfa_b200 C ABI.
#include <stdarg.h>
#include <stdio.h>

#include "common.cuh"

namespace rfa {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) return 0;
  snprintf(g_err, sizeof(g_err), "%s: launch failed: %s", what, cudaGetErrorString(e));
  return (int)e;
}

}  // namespace rfa

extern "C" int rfa_version(void) { return RFA_B200_VERSION; }
extern "C" const char* rfa_last_error(void) { return rfa::g_err; }
