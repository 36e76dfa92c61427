// Error reporting and version of the rfa_b200 C ABI.
#include <stdarg.h>
#include <stdio.h>

#include <mutex>

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

// per kernel family (one translation unit each): read-and-clear of the device status word, and the setter of the
// mapped host word its kernels mirror a failure into
#define RFA_TC_FAMILIES(X) X(causal_fwd, 1) X(causal_bwd, 2) X(causal_bwd_kv, 3) X(cross, 4) X(feature_map, 5) X(causal_bwd_saved, 6) X(stream_probe, 7) \
  X(causal_fwd_fused, 8)
#define RFA_DECLARE(name, id) int tc_status_##name(); int tc_mirror_##name(int*);
RFA_TC_FAMILIES(RFA_DECLARE)
#undef RFA_DECLARE

static std::mutex g_mirror_mu;
static int* g_mirror_word = nullptr;            // one word of mapped, portable host memory per process
static bool g_mirror_on[64] = {};               // per device ordinal: kernels there know the word

}  // namespace rfa

// Sticky device-side status of the tensor-core kernels: 0 = no bounded wait ever ran out;
// otherwise 100 * kernel family + the site code of the first wait that did.  Synchronises
// the device and clears the flags.
extern "C" int rfa_debug_status(void) {
  if (cudaDeviceSynchronize() != cudaSuccess) return -1000;
  int first = 0;
#define RFA_READ(name, id)                                   \
  {                                                          \
    const int v = rfa::tc_status_##name();                   \
    if (v && !first) first = v < 0 ? v : 100 * id + v;       \
  }
  RFA_TC_FAMILIES(RFA_READ)
#undef RFA_READ
  if (rfa::g_mirror_word) *reinterpret_cast<volatile int*>(rfa::g_mirror_word) = 0;
  return first;
}

extern "C" int rfa_status_mirror_enable(void) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return rfa::fail((int)e, "status_mirror_enable: cudaGetDevice: %s", cudaGetErrorString(e));
  RFA_REQUIRE(dev >= 0 && dev < 64, RFA_EUNSUPPORTED, "status_mirror_enable: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(rfa::g_mirror_mu);
  if (rfa::g_mirror_on[dev]) return 0;
  if (!rfa::g_mirror_word) {
    void* p = nullptr;
    e = cudaHostAlloc(&p, 64, cudaHostAllocMapped | cudaHostAllocPortable);
    if (e != cudaSuccess) return rfa::fail((int)e, "status_mirror_enable: cudaHostAlloc: %s", cudaGetErrorString(e));
    *static_cast<int*>(p) = 0;
    rfa::g_mirror_word = static_cast<int*>(p);
  }
  int* devp = nullptr;
  e = cudaHostGetDevicePointer(reinterpret_cast<void**>(&devp), rfa::g_mirror_word, 0);
  if (e != cudaSuccess) return rfa::fail((int)e, "status_mirror_enable: cudaHostGetDevicePointer: %s", cudaGetErrorString(e));
#define RFA_SET(name, id) \
  if (int r = rfa::tc_mirror_##name(devp)) return rfa::fail(r, "status_mirror_enable: cannot set the mirror of " #name);
  RFA_TC_FAMILIES(RFA_SET)
#undef RFA_SET
  rfa::g_mirror_on[dev] = true;
  return 0;
}

extern "C" int rfa_status_peek(void) {
  return rfa::g_mirror_word ? *reinterpret_cast<volatile int*>(rfa::g_mirror_word) : 0;
}

extern "C" int rfa_version(void) { return RFA_B200_VERSION; }
extern "C" const char* rfa_last_error(void) { return rfa::g_err; }
