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
// Optional event trace of CTA (0,0) for tuning (compile with -DRFA_TRACE): each record is
// (event id, chunk, globaltimer ns).  Not part of normal builds.
#ifdef RFA_TRACE
// four roles x 1024 records, store-only (no atomics, nothing waits on the stores)
static __device__ unsigned long long g_trace[4 * 1024 * 2];
__device__ __forceinline__ void trace_ev(int role, int& n, int id, int chunk) {
  if (blockIdx.x == 0 && blockIdx.y == 0 && n < 1024) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    g_trace[(role * 1024 + n) * 2] = ((unsigned long long)id << 32) | (unsigned int)chunk;
    g_trace[(role * 1024 + n) * 2 + 1] = t;
    ++n;
  }
}
#define RFA_TRACE_DECL(role) const int trace_role_ = (role); int trace_n_ = 0;
#define RFA_TRACE_EV(id, chunk) trace_ev(trace_role_, trace_n_, (id), (chunk))
// defines  extern "C" int NAME(unsigned long long* out)  copying this translation unit's records (4*1024 pairs)
#define RFA_TRACE_DUMP_FN(NAME)                                      \
  extern "C" int NAME(unsigned long long* out) {                     \
    static unsigned long long zeros[4 * 1024 * 2];                   \
    cudaDeviceSynchronize();                                         \
    cudaMemcpyFromSymbol(out, g_trace, sizeof(g_trace));             \
    cudaMemcpyToSymbol(g_trace, zeros, sizeof(zeros));               \
    return 4 * 1024;                                                 \
  }
#else
#define RFA_TRACE_DUMP_FN(NAME)
#define RFA_TRACE_DECL(role)
#define RFA_TRACE_EV(id, chunk) ((void)0)
#endif

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

// byte offset of 16-byte chunk `ch` (0..15) of row r in a two-box [128][128] fp16 tile
__device__ __forceinline__ uint32_t row_chunk2(int r, int ch) {
  return (uint32_t)(ch >> 3) * kBox + (uint32_t)r * 128u + ((uint32_t)((ch & 7) ^ (r & 7)) << 4);
}
// same for a one-box [128][64] tile, ch in 0..7
__device__ __forceinline__ uint32_t row_chunk1(int r, int ch) {
  return (uint32_t)r * 128u + ((uint32_t)(ch ^ (r & 7)) << 4);
}

// fp32 state row (64 values in registers as bit patterns) -> fp16 row r of the swizzled state tile
__device__ __forceinline__ void store_state_row(unsigned char* tile, int r, const uint32_t* v) {
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
    uint4 p;
    p.x = pack_half2(__uint_as_float(v[ch * 8 + 0]), __uint_as_float(v[ch * 8 + 1]));
    p.y = pack_half2(__uint_as_float(v[ch * 8 + 2]), __uint_as_float(v[ch * 8 + 3]));
    p.z = pack_half2(__uint_as_float(v[ch * 8 + 4]), __uint_as_float(v[ch * 8 + 5]));
    p.w = pack_half2(__uint_as_float(v[ch * 8 + 6]), __uint_as_float(v[ch * 8 + 7]));
    *reinterpret_cast<uint4*>(tile + row_chunk1(r, ch)) = p;
  }
}

// sum over the chunk's rows s of X[s][col] * w[s]  (w == nullptr -> 1) for a two-box tile
__device__ __forceinline__ float column_sum2(const unsigned char* tile, int col, const float* w) {
  const unsigned char* base = tile + (col >> 6) * kBox + ((col & 7) << 1);
  const int cc = (col & 63) >> 3;
  float a = 0.f;
#pragma unroll 8
  for (int s = 0; s < 128; ++s) {
    const float x = __half2float(*reinterpret_cast<const __half*>(base + s * 128 + ((cc ^ (s & 7)) << 4)));
    a = w ? fmaf(x, w[s], a) : a + x;
  }
  return a;
}

#endif

}  // namespace rfa
