// Shared host/device helpers of the rfa_b200 kernels (sm_100a only).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rfa_b200.h"

namespace rfa {

// ---- host side: per-thread error text + uniform return codes ---------------
int fail(int code, const char* fmt, ...);   // records text, returns code
int check_launch(const char* what);         // cudaGetLastError -> 0 or cudaError_t (text recorded)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline cudaStream_t as_stream(rfa_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

#define RFA_REQUIRE(cond, code, ...)                      \
  do {                                                    \
    if (!(cond)) return ::rfa::fail((code), __VA_ARGS__); \
  } while (0)

// Geometry of the attention kernels: feature width K = 2 * proj_dim = 128, head dim d = 64.
constexpr int kK = 128;        // width of phi
constexpr int kD = 64;         // head dim

constexpr float kEps = 1.0f;       // denominator clamp (upstream rfa.py:17, cuda/utils.cu:20)
constexpr float kNormEps = 1e-3f;  // x / (|x| + 1e-3)   (upstream utils.py:102)

// ---- device side ------------------------------------------------------------
#ifdef __CUDACC__

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// 4 consecutive elements <-> float4 (16-byte access for float, 8-byte for half)
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __half* p) {
  uint2 r = *reinterpret_cast<const uint2*>(p);
  float2 a = __half22float2(*reinterpret_cast<__half2*>(&r.x));
  float2 b = __half22float2(*reinterpret_cast<__half2*>(&r.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void store4(__half* p, float4 v) {
  __half2 a = __floats2half2_rn(v.x, v.y), b = __floats2half2_rn(v.z, v.w);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&a);
  r.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = r;
}

// 8 consecutive halves (16 bytes) -> 8 floats
__device__ __forceinline__ void load8(const __half* p, float* f) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __half22float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ void store8(__half* p, const float* f) {
  uint4 r;
  __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = r;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Block-wide register-tiled product over shared-memory operands:
//   C(i,j) = sum_{l<L} A(i,l) * B(l,j),  i < M, j < N
// Each thread owns TM x TN outputs with interleaved rows/columns
// (i = tm + ii*M/TM, j = tn + jj*N/TN) so neighbouring threads touch neighbouring
// shared-memory words.  la/lb read one operand element, st receives (i, j, value).
template <int TM, int TN, class LA, class LB, class ST>
__device__ __forceinline__ void tile_gemm(int M, int N, int L, LA la, LB lb, ST st) {
  const int tiles_m = M / TM, tiles_n = N / TN;
  for (int tile = threadIdx.x; tile < tiles_m * tiles_n; tile += blockDim.x) {
    const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
    float acc[TM][TN];
#pragma unroll
    for (int ii = 0; ii < TM; ++ii)
#pragma unroll
      for (int jj = 0; jj < TN; ++jj) acc[ii][jj] = 0.f;
#pragma unroll 4
    for (int l = 0; l < L; ++l) {
      float a[TM], b[TN];
#pragma unroll
      for (int ii = 0; ii < TM; ++ii) a[ii] = la(tm + ii * tiles_m, l);
#pragma unroll
      for (int jj = 0; jj < TN; ++jj) b[jj] = lb(l, tn + jj * tiles_n);
#pragma unroll
      for (int ii = 0; ii < TM; ++ii)
#pragma unroll
        for (int jj = 0; jj < TN; ++jj) acc[ii][jj] = fmaf(a[ii], b[jj], acc[ii][jj]);
    }
#pragma unroll
    for (int ii = 0; ii < TM; ++ii)
#pragma unroll
      for (int jj = 0; jj < TN; ++jj) st(tm + ii * tiles_m, tn + jj * tiles_n, acc[ii][jj]);
  }
}

#endif  // __CUDACC__

}  // namespace rfa
