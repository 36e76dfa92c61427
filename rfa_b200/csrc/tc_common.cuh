// Pieces shared by the tensor-core (tcgen05) kernels: chunk geometry, the sticky
// device status word of this translation unit, small epilogue helpers.
#pragma once

#include "sm100.cuh"
#include "tiles.cuh"

namespace rfa {

using namespace sm100;

constexpr int kTC = 128;                       // tokens per chunk
constexpr uint32_t kBox = 128 * 128;           // bytes of one [128 rows][64 halves] swizzled box

// Sticky per-translation-unit status: code of the first bounded wait that ran out (0 = none).
static __device__ int g_tc_status;

__device__ __forceinline__ void tc_fail(int code) { atomicCAS(&g_tc_status, 0, code); }

// Host: read and clear this translation unit's status word (device must be idle).
static int tc_status_read_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1001;
  cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  return v;
}

#ifdef __CUDACC__
// Barrier among the 128 epilogue threads built on an mbarrier so that it, too, is bounded.
__device__ __forceinline__ bool epi_sync(uint64_t* bar, uint32_t& phase) {
  mbar_arrive(bar);
  const bool ok = mbar_wait(bar, phase);
  phase ^= 1u;
  return ok;
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_half2(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}
#endif

}  // namespace rfa
