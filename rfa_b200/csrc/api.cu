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

int tc_status_causal_fwd();
int tc_status_causal_bwd();
int tc_status_causal_bwd_kv();
int tc_status_cross();
int tc_status_feature_map();

}  // namespace rfa

// Sticky device-side status of the tensor-core kernels: 0 = no bounded wait ever ran out;
// otherwise 100 * kernel family + the site code of the first wait that did.  Synchronises
// the device and clears the flags.
extern "C" int rfa_debug_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1000;
  const int f = rfa::tc_status_causal_fwd(), b = rfa::tc_status_causal_bwd();
  if (f) return f < 0 ? f : 100 + f;
  if (b) return b < 0 ? b : 200 + b;
  if (const int kv = rfa::tc_status_causal_bwd_kv()) return kv < 0 ? kv : 300 + kv;
  if (const int x = rfa::tc_status_cross()) return x < 0 ? x : 400 + x;
  if (const int f2 = rfa::tc_status_feature_map()) return f2 < 0 ? f2 : 500 + f2;
  return 0;
}

extern "C" int rfa_version(void) { return RFA_B200_VERSION; }
extern "C" const char* rfa_last_error(void) { return rfa::g_err; }
