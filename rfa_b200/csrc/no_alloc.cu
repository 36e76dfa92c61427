// Causal backward for callers that cannot provide (or allocate) scratch memory.
//
// The regular backward needs a caller-supplied workspace for two per-token scalars
// that its first sweep hands to its second.  Some hosts have no buffer to give: a
// plugin inside a serving process that split all device memory among its own pools
// at start-up and forbids cudaMalloc afterwards (it stalls every stream of the device
// and can fail once the pools own the memory), or a plain C caller with no device
// allocator of its own.  For them this file keeps that scratch in a fixed array that
// is part of the library image on every GPU that loads it.
#include <mutex>

#include "common.cuh"

namespace rfa {

// launchers of the two sweeps (causal_bwd_tc.cu)
int launch_causal_bwd_q_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq,
                           const float* s_seg, const float* z_seg, float* ws_den, float* ws_gz, float* ds_seg,
                           float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);
int launch_causal_bwd_kv_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                            const float* ws_den, const float* ws_gz, const float* ds_seg, const float* dz_seg,
                            int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);

// Largest T * BH the fixed scratch serves: two fp32 scalars per (token, head) = 4 MiB per GPU.
constexpr int64_t kNoAllocMaxTokenHeads = 512 * 1024;

static __device__ __align__(256) float g_noalloc_scratch[2 * kNoAllocMaxTokenHeads];

constexpr int kMaxDevices = 64;
static std::mutex g_noalloc_mu;
static float* g_noalloc_ptr[kMaxDevices];   // device address of the array, per device, filled on first use

// Device address of the scratch array on the current device.  The symbol name is only a
// host-side handle; the address a kernel can use comes from cudaGetSymbolAddress, looked
// up once per device with that device current.
static int noalloc_scratch(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "causal_bwd_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  RFA_REQUIRE(dev >= 0 && dev < kMaxDevices, RFA_EUNSUPPORTED, "causal_bwd_noalloc: device ordinal %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mu);
  if (!g_noalloc_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || !p)
      return fail(e != cudaSuccess ? (int)e : RFA_EDEVICE, "causal_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_noalloc_ptr[dev] = static_cast<float*>(p);
  }
  *out = g_noalloc_ptr[dev];
  return 0;
}

}  // namespace rfa

using namespace rfa;

extern "C" int64_t rfa_causal_bwd_noalloc_max_token_heads(void) { return kNoAllocMaxTokenHeads; }

extern "C" int rfa_causal_bwd_noalloc(const void* q, const void* k, const void* v, const void* g,
                                      void* gq, void* gk, void* gv,
                                      int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(T >= 0 && BH > 0, RFA_EINVAL, "causal_bwd_noalloc: T=%lld BH=%d", (long long)T, BH);
  RFA_REQUIRE(K == kK && d == kD, RFA_EUNSUPPORTED, "causal_bwd_noalloc: only K=%d, d=%d is built (got K=%d d=%d)", kK, kD, K, d);
  RFA_REQUIRE(BH <= 65535, RFA_EUNSUPPORTED, "causal_bwd_noalloc: BH=%d exceeds 65535", BH);
  RFA_REQUIRE(q && k && v && g && gq && gk && gv, RFA_EINVAL, "causal_bwd_noalloc: null pointer");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) && aligned16(gq) && aligned16(gk) && aligned16(gv),
              RFA_EALIGN, "causal_bwd_noalloc: 16-byte alignment required");
  RFA_REQUIRE(T <= kNoAllocMaxTokenHeads / BH, RFA_EWORKSPACE,      // a division: T * BH could overflow for absurd T
              "causal_bwd_noalloc: T=%lld x BH=%d exceeds the built-in scratch (max %lld token-heads); "
              "use rfa_causal_bwd with a caller workspace", (long long)T, BH, (long long)kNoAllocMaxTokenHeads);
  if (T == 0) return 0;
  float* scratch = nullptr;
  if (int e = noalloc_scratch(&scratch)) return e;
  float* den = scratch;                      // [BH][T], fully written by the first sweep before the second reads it
  float* gz = scratch + (size_t)T * BH;
  const int64_t tseg = (T + 127) / 128 * 128;   // one segment per (batch, head): no boundary-state scratch needed
  cudaStream_t st = as_stream(stream);
  if (int e = launch_causal_bwd_q_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g, (__half*)gq,
                                     nullptr, nullptr, den, gz, nullptr, nullptr, T, BH, 1, tseg, st))
    return e;
  return launch_causal_bwd_kv_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g, (__half*)gk,
                                 (__half*)gv, den, gz, nullptr, nullptr, T, BH, 1, tseg, st);
}
