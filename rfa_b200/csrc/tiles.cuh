// Shared-memory tile helpers for the chunked attention kernels (K = 128, d = 64).
//
// A chunk is C = 64 consecutive tokens of one (batch, head).  Its q, k rows (K
// halves) and v, g rows (d halves) are staged as fp32 tiles with odd row strides
// so that both row-wise and column-wise walks are bank-conflict free.
#pragma once

#include "common.cuh"

namespace rfa {

constexpr int kK = 128;        // width of phi
constexpr int kD = 64;         // head dim
constexpr int kC = 64;         // tokens per chunk
constexpr int kLK = kK + 1;    // row stride of [*][K] tiles
constexpr int kLD = kD + 1;    // row stride of [*][d] and [*][C] tiles
constexpr int kThreads = 256;

#ifdef __CUDACC__

// Stage `valid` rows (of kC) of a time-major fp16 array into a fp32 tile; rows past
// `valid` are zero.  src points at element 0 of the chunk's first row for this
// (batch, head); consecutive tokens are row_stride elements apart.
template <int COLS>
__device__ __forceinline__ void stage_rows(float* dst, int ld, const __half* __restrict__ src,
                                           size_t row_stride, int valid) {
  constexpr int G = COLS / 8;
  for (int idx = threadIdx.x; idx < kC * G; idx += kThreads) {
    const int r = idx / G, c = (idx % G) * 8;
    float f[8];
    if (r < valid) {
      load8(src + (size_t)r * row_stride + c, f);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) dst[r * ld + c + e] = f[e];
  }
}

// Write `valid` rows of a fp32 tile back as fp16, 16 bytes per access.
template <int COLS>
__device__ __forceinline__ void unstage_rows(__half* __restrict__ dst, size_t row_stride,
                                             const float* src, int ld, int valid) {
  constexpr int G = COLS / 8;
  for (int idx = threadIdx.x; idx < kC * G; idx += kThreads) {
    const int r = idx / G, c = (idx % G) * 8;
    if (r >= valid) continue;
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = src[r * ld + c + e];
    store8(dst + (size_t)r * row_stride + c, f);
  }
}

// Load (or zero) a [K][d] fp32 state and its [K] companion into shared memory.
__device__ __forceinline__ void load_state(float* St, float* zs, const float* __restrict__ s_src,
                                           const float* __restrict__ z_src) {
  for (int i = threadIdx.x; i < kK * kD; i += kThreads)
    St[(i / kD) * kLD + (i % kD)] = s_src ? s_src[i] : 0.f;
  for (int i = threadIdx.x; i < kK; i += kThreads) zs[i] = z_src ? z_src[i] : 0.f;
}

__device__ __forceinline__ void store_state(float* __restrict__ s_dst, float* __restrict__ z_dst,
                                            const float* St, const float* zs) {
  for (int i = threadIdx.x; i < kK * kD; i += kThreads) s_dst[i] = St[(i / kD) * kLD + (i % kD)];
  for (int i = threadIdx.x; i < kK; i += kThreads) z_dst[i] = zs[i];
}

// St[k][j] += sum_r Ks[r][k] * Vs[r][j];  zs[k] += sum_r Ks[r][k] * wt[r]  (wt == nullptr -> 1)
// i.e. the rank-C update of the running state by one chunk.
__device__ __forceinline__ void accumulate_state(float* St, float* zs, const float* Ks, const float* Vs,
                                                 const float* wt) {
  tile_gemm<4, 8>(kK, kD, kC,
                  [&](int k, int r) { return Ks[r * kLK + k]; },
                  [&](int r, int j) { return Vs[r * kLD + j]; },
                  [&](int k, int j, float v) { St[k * kLD + j] += v; });
  if (threadIdx.x < kK) {
    float a = 0.f;
    for (int r = 0; r < kC; ++r) a = fmaf(Ks[r * kLK + threadIdx.x], wt ? wt[r] : 1.f, a);
    zs[threadIdx.x] += a;
  }
}

#endif  // __CUDACC__

}  // namespace rfa
