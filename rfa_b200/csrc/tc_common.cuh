// Pieces shared by the tensor-core (tcgen05) kernels: chunk geometry, the sticky
// device status word of this translation unit, small epilogue helpers.
#pragma once

#include "common.cuh"
#include "sm100.cuh"

namespace rfa {

using namespace sm100;

constexpr int kTC = 128;                       // tokens per chunk
constexpr uint32_t kBox = 128 * 128;           // bytes of one [128 rows][64 halves] swizzled box

// Sticky per-translation-unit status: code of the first bounded wait that ran out (0 = none).  A wait gives up after
// kSpinLimit (2^20) mbarrier.try_wait attempts, each of which suspends the thread for up to a few microseconds:
// about four seconds of wall-clock time, far beyond any legitimate wait inside these kernels (a chunk takes
// microseconds).  The kernel then leaves early and its outputs are invalid; besides the device word, the code
// (100 * RFA_TC_FAMILY + site) is written to a word of mapped host memory when the host has enabled one
// (rfa_status_mirror_enable), which the host can look at after any later call without synchronising.
#ifndef RFA_TC_FAMILY
#error "define RFA_TC_FAMILY (1..9) before including tc_common.cuh"
#endif
static __device__ int g_tc_status;
static __device__ int* g_tc_mirror;

__device__ __forceinline__ void tc_fail(int code) {
  if (atomicCAS(&g_tc_status, 0, code) == 0) {
    int* m = g_tc_mirror;
    if (m) {
      *reinterpret_cast<volatile int*>(m) = 100 * RFA_TC_FAMILY + code;
      __threadfence_system();
    }
  }
}

// Host: read and clear this translation unit's status word (device must be idle).
static int tc_status_read_clear() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1001;
  cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int));
  return v;
}
// Host: point this translation unit's kernels (on the current device) at the mapped host word.
static int tc_mirror_set(int* host_word) {
  return (int)cudaMemcpyToSymbol(g_tc_mirror, &host_word, sizeof(host_word));
}
// defines the two host hooks of a kernel family that api.cu calls
#define RFA_TC_UNIT(name)                                        \
  int tc_status_##name() { return tc_status_read_clear(); }      \
  int tc_mirror_##name(int* w) { return tc_mirror_set(w); }

#ifdef __CUDACC__
// The k-steps of one product, issued by the whole MMA warp (see umma_ss_w).  Operand k-step j sits at
// base + (j & 3) * step + (j >> 2) * block  (descriptor units of 16 bytes): K-major two-box tiles use
// (kStepK, kBlockK), MN-major tiles (kStepMN, kBlockMN); a packed fp16 operand in tensor memory advances
// by 8 columns per k-step.
constexpr uint32_t kStepK = 2, kBlockK = kBox >> 4;      // K-major operand of two 64-wide boxes
constexpr uint32_t kStepMN = 128, kBlockMN = 512;        // MN-major operand (k-step = 16 rows of 128 bytes)
template <int NSTEPS, uint32_t ASTEP, uint32_t ABLOCK, uint32_t BSTEP, uint32_t BBLOCK>
__device__ __forceinline__ void umma_chain_ss(uint32_t lead, uint32_t d_tmem, uint64_t a, uint64_t b, uint32_t idesc, uint32_t acc_first) {
#pragma unroll
  for (int j = 0; j < NSTEPS; ++j)
    umma_ss_w(lead, d_tmem, a + (uint64_t)((j & 3) * ASTEP + (j >> 2) * ABLOCK), b + (uint64_t)((j & 3) * BSTEP + (j >> 2) * BBLOCK), idesc,
              (j > 0) ? 1u : acc_first);
}
template <int NSTEPS, uint32_t BSTEP, uint32_t BBLOCK>
__device__ __forceinline__ void umma_chain_ts(uint32_t lead, uint32_t d_tmem, uint32_t a_tmem, uint64_t b, uint32_t idesc, uint32_t acc_first) {
#pragma unroll
  for (int j = 0; j < NSTEPS; ++j)
    umma_ts_w(lead, d_tmem, a_tmem + j * 8, b + (uint64_t)((j & 3) * BSTEP + (j >> 2) * BBLOCK), idesc, (j > 0) ? 1u : acc_first);
}

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

// Column sums of a two-box [128 rows][128 cols] fp16 tile: returns sum_s X[s][col] * w[s]
// (w == nullptr -> 1) for col = quarter * 32 + lane.  Warp-cooperative: a warp covers 32 columns;
// lane = 8 * c4 + rg reads the 16-byte chunk (4 * quarter + c4) of rows rg, rg + 8, ... (conflict-free,
// 16 loads of 8 values), the 8 row groups are then combined with shuffles.
__device__ __forceinline__ float column_sum2(const unsigned char* tile, int quarter, int lane, const float* w) {
  const int rg = lane & 7, cc = 4 * quarter + (lane >> 3);
  const unsigned char* base = tile + (cc >> 3) * kBox + (((cc & 7) ^ rg) << 4) + rg * 128;
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll 4
  for (int j = 0; j < 16; ++j) {
    const uint4 u = *reinterpret_cast<const uint4*>(base + j * 1024);
    const float wv = w ? w[rg + 8 * j] : 1.f;
    const float2 f0 = unpack_half2(u.x), f1 = unpack_half2(u.y), f2 = unpack_half2(u.z), f3 = unpack_half2(u.w);
    acc[0] = fmaf(f0.x, wv, acc[0]); acc[1] = fmaf(f0.y, wv, acc[1]);
    acc[2] = fmaf(f1.x, wv, acc[2]); acc[3] = fmaf(f1.y, wv, acc[3]);
    acc[4] = fmaf(f2.x, wv, acc[4]); acc[5] = fmaf(f2.y, wv, acc[5]);
    acc[6] = fmaf(f3.x, wv, acc[6]); acc[7] = fmaf(f3.y, wv, acc[7]);
  }
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 1);
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 2);
    acc[e] += __shfl_xor_sync(0xffffffffu, acc[e], 4);
  }
  float r = acc[0];                      // column 8 * cc + rg  ==  32 * quarter + lane
#pragma unroll
  for (int e = 1; e < 8; ++e) r = (rg == e) ? acc[e] : r;
  return r;
}
#endif

}  // namespace rfa
