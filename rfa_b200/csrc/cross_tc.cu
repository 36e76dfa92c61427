// Cross RFA on tcgen05 tensor cores (upstream cross_attention.py:97-104 and :254-270), and the
// state reduction that the segmented / sequence-sharded causal path uses for its boundary states.
//
//   state   S = sum_s phi_k[s] (x) v[s],  z = sum_s phi_k[s]      over unpadded keys
//   query   out_t = phi_q[t] . S / max(|phi_q[t] . z|, 1)
//   and the gradients of both.  All four kernels walk one (batch, head) in chunks of 128 rows with a
//   two-stage TMA ring; the products are tcgen05.mma with fp32 accumulators in TMEM:
//     state fwd   S  += K^T V                      (A, B MN-major)        z by CUDA-core column sums
//     query fwd   N   = Q [S|z]                    (B = state tile, MN-major, N = 80)
//     query bwd   N as above -> gs, gr;  dQ = gs S^T;  dS += Q^T gs;  dz by column sums
//     state bwd   dK  = V dS^T,  dV = K dS
// Warp roles (192 threads): warp 0 TMA producer, warp 1 MMA issuer, warps 2..5 epilogue
// (thread <-> TMEM lane <-> row).  All waits are bounded.
#define RFA_TC_FAMILY 4
#include "tc_common.cuh"

namespace rfa {

constexpr int kXThreads = 192;

// every kernel: prologue shared by all roles
#define RFA_X_PROLOGUE(NBARS, TMEM_COLS)                                                                          \
  extern __shared__ unsigned char x_raw[];                                                                       \
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(x_raw) + 1023) & ~uintptr_t(1023)); \
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBarOff);                                                    \
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + (NBARS));                                             \
  const uint32_t sbase = smem_u32(sm);                                                                           \
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;                                                 \
  (void)sbase; (void)lane;

// same, for kernels that use every byte two CTAs per SM may have: no slack to align the base, which is checked instead
#define RFA_X_PROLOGUE_ALIGNED(NBARS)                                                                            \
  extern __shared__ __align__(1024) unsigned char x_raw[];                                                       \
  unsigned char* sm = x_raw;                                                                                     \
  if (smem_u32(sm) & 1023u) {                                                                                    \
    if (threadIdx.x == 0) tc_fail(99);                                                                           \
    return;                                                                                                      \
  }                                                                                                              \
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBarOff);                                                    \
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + (NBARS));                                             \
  const uint32_t sbase = smem_u32(sm);                                                                           \
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;                                                 \
  (void)sbase; (void)lane;

#define RFA_X_START(TMEM_COLS)                                            \
  if (warp == 1) { tmem_alloc(tmem_slot, (TMEM_COLS)); tmem_relinquish(); } \
  tc_fence_before_sync();                                                 \
  __syncthreads();                                                        \
  tc_fence_after_sync();                                                  \
  const uint32_t tmem = *tmem_slot;                                       \
  pdl_wait(); /* nothing above touches global memory: all of it overlaps the previous kernel's tail */ \
  pdl_launch_dependents();

#define RFA_X_FINISH(TMEM_COLS)                          \
  tc_fence_before_sync();                                \
  __syncthreads();                                       \
  if (warp == 1) tmem_dealloc(tmem, (TMEM_COLS));

// fp32 state (S [128][64] rows, z [128]) -> fp16 operand tile: box 0 = S, box 1 = [z | 0 ...]
__device__ __forceinline__ void build_state_tile(unsigned char* tile, int row, const float* __restrict__ s_row, float zval) {
  uint32_t r[64];
#pragma unroll
  for (int n = 0; n < 64; n += 4) {
    const float4 f = *reinterpret_cast<const float4*>(s_row + n);
    r[n] = __float_as_uint(f.x); r[n + 1] = __float_as_uint(f.y); r[n + 2] = __float_as_uint(f.z); r[n + 3] = __float_as_uint(f.w);
  }
  store_state_row(tile, row, r);
#pragma unroll
  for (int ch = 1; ch < 8; ++ch) *reinterpret_cast<uint4*>(tile + kBox + row_chunk1(row, ch)) = make_uint4(0, 0, 0, 0);
  *reinterpret_cast<uint4*>(tile + kBox + row_chunk1(row, 0)) = make_uint4(pack_half2(zval, 0.f), 0, 0, 0);
}

__device__ __forceinline__ void zero_row2(unsigned char* tile, int row) {     // one row of a two-box [128][128] tile
#pragma unroll
  for (int ch = 0; ch < 16; ++ch) *reinterpret_cast<uint4*>(tile + row_chunk2(row, ch)) = make_uint4(0, 0, 0, 0);
}

// ===========================================================================
// state reduction.  grid (BH, nseg)
// ===========================================================================
namespace xs {
constexpr uint32_t kK_ = 0, kV_ = 2 * kBox, kStage = 3 * kBox;
// NS stages of 48 KB: two let two CTAs share an SM (many short sequences: cross attention), four give one CTA per SM
// enough loads in flight to run a long sequence at the memory's rate (segment / shard boundary states)
template <int NS> struct L {
  static constexpr uint32_t kBarOff = NS * kStage, kSmem = kBarOff + 128 + 1024;
  enum { bFull = 0, bReady = NS, bEmpty = 2 * NS, bDone = 3 * NS, bEpi = 3 * NS + 1, bNum = 3 * NS + 2 };
};
}

template <int NS>
__global__ void __launch_bounds__(kXThreads, 1)
cross_state_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const uint8_t* __restrict__ pad_mask, float* __restrict__ s_out, float* __restrict__ z_out,
                          int64_t T, int BH, int H, int nseg, int64_t tseg) {
  using namespace xs;
  constexpr uint32_t kBarOff = L<NS>::kBarOff;
  constexpr int bFull = L<NS>::bFull, bReady = L<NS>::bReady, bEmpty = L<NS>::bEmpty, bDone = L<NS>::bDone, bEpi = L<NS>::bEpi, bNum = L<NS>::bNum;
  RFA_X_PROLOGUE(bNum, 64)
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  const int nchunk = (int)((t_end - t_begin + kTC - 1) / kTC);
  if (tid == 0) {
    // a stage is free again once the product has read it (commit) and the epilogue warps have summed its K columns
    for (int i = 0; i < NS; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bReady + i], 128); mbar_init(&bars[bEmpty + i], 129); }
    mbar_init(&bars[bDone], 1); mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
  }
  RFA_X_START(64)
  if (warp == 0) {
    if (lane == 0)
      for (int c = 0; c < nchunk; ++c) {
        const int st = c % NS;
        if (c >= NS && !mbar_wait(&bars[bEmpty + st], ((c / NS) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * kStage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        mbar_arrive_expect_tx(&bars[bFull + st], kStage);
        tma_load_3d(base + kK_, &tm_k, &bars[bFull + st], 0, bh, t0);
        tma_load_3d(base + kK_ + kBox, &tm_k, &bars[bFull + st], 64, bh, t0);
        tma_load_3d(base + kV_, &tm_v, &bars[bFull + st], 0, bh, t0);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idMM = umma_idesc_f16(128, 64, true, true);
      const uint64_t dK = umma_smem_desc(sbase + kK_, kBox, 1024, kSwizzle128B), dV = umma_smem_desc(sbase + kV_, kBox, 1024, kSwizzle128B);
      bool ok = true;
#pragma unroll 1
      for (int c = 0; c < nchunk; ++c) {
        const int st = c % NS;
        // with a padding mask the epilogue warps first zero the padded rows of the staged K tile
        if (!mbar_wait(&bars[(pad_mask ? bReady : bFull) + st], (c / NS) & 1)) { tc_fail(2); ok = false; break; }
        tc_fence_after_sync();
        const uint64_t so = (uint64_t)st * (kStage >> 4);
        umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(1u, tmem, dK + so, dV + so, idMM, c > 0 ? 1u : 0u);
        umma_commit(&bars[bEmpty + st]);
      }
      if (ok) umma_commit(&bars[bDone]);
    }
  } else {
    const int quarter = warp & 3, row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint8_t* mrow = pad_mask ? pad_mask + (size_t)(bh / H) * T : nullptr;
    float z_acc = 0.f;
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c % NS;
      unsigned char* stage = sm + st * kStage;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      if (!mbar_wait(&bars[bFull + st], (c / NS) & 1)) { tc_fail(3); ok = false; break; }
      if (mrow) {                                   // padded keys contribute nothing: zero their feature rows
        if (t0 + row < t_end && mrow[t0 + row]) zero_row2(stage + kK_, row);
        fence_async_smem();
        if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(4); ok = false; break; }
        mbar_arrive(&bars[bReady + st]);
      }
      z_acc += column_sum2(stage + kK_, quarter, lane, nullptr);
      mbar_arrive(&bars[bEmpty + st]);
    }
    if (ok) {
      uint32_t r[64];
      if (nchunk > 0) {
        if (!mbar_wait(&bars[bDone], 0)) { tc_fail(5); ok = false; }
        tc_fence_after_sync();
        if (ok) { tmem_ld32(tmem + lane_addr, r); tmem_ld32(tmem + lane_addr + 32, r + 32); tmem_ld_wait(); }
      } else {
#pragma unroll
        for (int n = 0; n < 64; ++n) r[n] = 0u;
      }
      if (ok) {
        const size_t slot = (size_t)bh * nseg + seg;
        float4* dst = reinterpret_cast<float4*>(s_out + (slot * kK + row) * kD);
#pragma unroll
        for (int n = 0; n < 16; ++n)
          dst[n] = make_float4(__uint_as_float(r[4 * n]), __uint_as_float(r[4 * n + 1]), __uint_as_float(r[4 * n + 2]), __uint_as_float(r[4 * n + 3]));
        z_out[slot * kK + row] = z_acc;
      }
    }
  }
  RFA_X_FINISH(64)
}

// ===========================================================================
// query forward.  grid (BH)
// ===========================================================================
namespace xq {
constexpr uint32_t kQ_ = 0, kStage = 2 * kBox, kS_ = 2 * kStage, kBarOff = kS_ + 2 * kBox, kSmem = kBarOff + 128 + 1024;
enum { bFull = 0, bEmpty = 2, bNFull = 4, bNFree = 6, bSt = 8, bEpi = 9, bNum = 10 };
}

__global__ void __launch_bounds__(kXThreads, 2)
cross_query_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_o,
                          const float* __restrict__ s, const float* __restrict__ z, int64_t T, int BH) {
  using namespace xq;
  RFA_X_PROLOGUE(bNum, 256)
  const int bh = blockIdx.x;
  const int nchunk = (int)((T + kTC - 1) / kTC);
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 1); mbar_init(&bars[bNFull + i], 1); mbar_init(&bars[bNFree + i], 128); }
    mbar_init(&bars[bSt], 128); mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_o);
  }
  RFA_X_START(256)
  if (warp == 0) {
    if (lane == 0)
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[bEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(11); break; }
        unsigned char* base = sm + st * kStage;
        mbar_arrive_expect_tx(&bars[bFull + st], kStage);
        tma_load_3d(base + kQ_, &tm_q, &bars[bFull + st], 0, bh, c * kTC);
        tma_load_3d(base + kQ_ + kBox, &tm_q, &bars[bFull + st], 64, bh, c * kTC);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idQS = umma_idesc_f16(128, 80, false, true);
      const uint64_t dQ = umma_smem_desc(sbase + kQ_, 0, 1024, kSwizzle128B), dS = umma_smem_desc(sbase + kS_, kBox, 1024, kSwizzle128B);
      bool ok = mbar_wait(&bars[bSt], 0);
      if (!ok) tc_fail(12);
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(13); break; }
        if (c >= 2 && !mbar_wait(&bars[bNFree + st], ((c >> 1) + 1) & 1)) { tc_fail(14); break; }
        tc_fence_after_sync();
        const uint64_t so = (uint64_t)st * (kStage >> 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_ss(tmem + st * 128, dQ + so + kstep_kmajor(j, kBox), dS + kstep_mnmajor(j), idQS, j > 0);
        umma_commit(&bars[bNFull + st]);
      }
    }
  } else {
    const int quarter = warp & 3, row = quarter * 32 + lane, etid = tid - 64;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    build_state_tile(sm + kS_, row, s + ((size_t)bh * kK + row) * kD, z[(size_t)bh * kK + row]);
    fence_async_smem();
    mbar_arrive(&bars[bSt]);
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      unsigned char* stage = sm + st * kStage;
      if (!mbar_wait(&bars[bNFull + st], (c >> 1) & 1)) { tc_fail(15); ok = false; break; }
      tc_fence_after_sync();
      uint32_t nn[64], nz[16];
      tmem_ld32(tmem + lane_addr + st * 128, nn);
      tmem_ld32(tmem + lane_addr + st * 128 + 32, nn + 32);
      tmem_ld16(tmem + lane_addr + st * 128 + 64, nz);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bNFree + st]);
      const float inv = 1.f / fmaxf(fabsf(__uint_as_float(nz[0])), kEps);        // abs, then clamp (cross_attention.py:267)
#pragma unroll
      for (int i = 0; i < 64; ++i) nn[i] = __float_as_uint(__uint_as_float(nn[i]) * inv);
      store_state_row(stage + kQ_, row, nn);          // the MMA is done with this stage's Q: its first box is the staging tile
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(16); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(&tm_o, stage + kQ_, 0, bh, c * kTC);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&bars[bEmpty + st]);
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  RFA_X_FINISH(256)
}

// ===========================================================================
// query backward.  grid (BH)
// ===========================================================================
namespace xb {
// 113 KB and 256 TMEM columns exactly, so that two CTAs share an SM: the state tile is one box (q . z is formed on CUDA
// cores in fp32 instead of as a 65th column of the numerator product) and z itself is read through the L1 cache
constexpr uint32_t kQ_ = 0, kG_ = 2 * kBox, kStage = 3 * kBox, kS_ = 2 * kStage, kGr_ = kS_ + kBox,
                   kBarOff = kGr_ + 512, kSmem = 113 * 1024;
static_assert(kBarOff + 128 <= kSmem, "cross_query_bwd: shared memory map exceeds half an SM");
constexpr uint32_t cN = 0, cDQ = 64, cDS = 192;
enum { bFull = 0, bEmpty = 2, bN = 4, bG = 5, bDQ = 6, bDQFree = 7, bSt = 8, bEpi = 9, bNum = 10 };
}

__global__ void __launch_bounds__(kXThreads, 2)
cross_query_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_g,
                          const __grid_constant__ CUtensorMap tm_gq, const float* __restrict__ s, const float* __restrict__ z,
                          float* __restrict__ d_s, float* __restrict__ d_z, int64_t T, int BH) {
  using namespace xb;
  RFA_X_PROLOGUE_ALIGNED(bNum)
  float* grs = reinterpret_cast<float*>(sm + kGr_);
  const int bh = blockIdx.x;
  const int nchunk = (int)((T + kTC - 1) / kTC);
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 1); }
    mbar_init(&bars[bN], 1); mbar_init(&bars[bG], 128); mbar_init(&bars[bDQ], 1); mbar_init(&bars[bDQFree], 128);
    mbar_init(&bars[bSt], 128); mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_g); tma_prefetch_desc(&tm_gq);
  }
  RFA_X_START(256)
  if (warp == 0) {
    if (lane == 0)
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[bEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(21); break; }
        unsigned char* base = sm + st * kStage;
        mbar_arrive_expect_tx(&bars[bFull + st], kStage);
        tma_load_3d(base + kQ_, &tm_q, &bars[bFull + st], 0, bh, c * kTC);
        tma_load_3d(base + kQ_ + kBox, &tm_q, &bars[bFull + st], 64, bh, c * kTC);
        tma_load_3d(base + kG_, &tm_g, &bars[bFull + st], 0, bh, c * kTC);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idQS = umma_idesc_f16(128, 64, false, true);     // Q S
      constexpr uint32_t idKK = umma_idesc_f16(128, 128, false, false);   // gs S^T
      constexpr uint32_t idMM = umma_idesc_f16(128, 64, true, true);      // Q^T gs
      const uint64_t dQk = umma_smem_desc(sbase + kQ_, 0, 1024, kSwizzle128B), dQm = umma_smem_desc(sbase + kQ_, kBox, 1024, kSwizzle128B);
      const uint64_t dGk = umma_smem_desc(sbase + kG_, 0, 1024, kSwizzle128B), dGm = umma_smem_desc(sbase + kG_, kBox, 1024, kSwizzle128B);
      const uint64_t dSm = umma_smem_desc(sbase + kS_, kBox, 1024, kSwizzle128B), dSk = umma_smem_desc(sbase + kS_, 0, 1024, kSwizzle128B);
      bool ok = mbar_wait(&bars[bSt], 0);
      if (!ok) tc_fail(22);
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * (kStage >> 4);
        if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(23); break; }
        if (c > 0 && !mbar_wait(&bars[bG], (c - 1) & 1)) { tc_fail(24); break; }     // N of the previous chunk has been read
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_ss(tmem + cN, dQk + so + kstep_kmajor(j, kBox), dSm + kstep_mnmajor(j), idQS, j > 0);
        umma_commit(&bars[bN]);
        if (!mbar_wait(&bars[bG], c & 1)) { tc_fail(25); break; }
        if (c > 0 && !mbar_wait(&bars[bDQFree], (c - 1) & 1)) { tc_fail(26); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_ss(tmem + cDQ, dGk + so + kstep_kmajor(j, kBox), dSk + kstep_kmajor(j, kBox), idKK, j > 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_ss(tmem + cDS, dQm + so + kstep_mnmajor(j), dGm + so + kstep_mnmajor(j), idMM, (c > 0 || j > 0) ? 1u : 0u);
        umma_commit(&bars[bDQ]);
      }
    }
  } else {
    const int quarter = warp & 3, row = quarter * 32 + lane, etid = tid - 64;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float* zs = z + (size_t)bh * kK;         // 512 bytes every thread reads whole, every chunk: served by L1
    {
      uint32_t r[64];
      const float* src = s + ((size_t)bh * kK + row) * kD;
#pragma unroll
      for (int n = 0; n < 64; n += 4) {
        const float4 f = *reinterpret_cast<const float4*>(src + n);
        r[n] = __float_as_uint(f.x); r[n + 1] = __float_as_uint(f.y); r[n + 2] = __float_as_uint(f.z); r[n + 3] = __float_as_uint(f.w);
      }
      store_state_row(sm + kS_, row, r);
    }
    fence_async_smem();
    mbar_arrive(&bars[bSt]);
    uint32_t epi_phase = 0;
    float dz_acc = 0.f;
    bool ok = true;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t ph = c & 1;
      unsigned char* stage = sm + st * kStage;
      // ---- q . z in fp32 from this thread's own row of the staged Q tile while the tensor pipe forms N = phi_q S
      if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(32); ok = false; break; }
      float qz0 = 0.f, qz1 = 0.f, qz2 = 0.f, qz3 = 0.f;
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const uint4 u = *reinterpret_cast<const uint4*>(stage + kQ_ + row_chunk2(row, ch));
        const float4 z0 = __ldg(reinterpret_cast<const float4*>(zs + ch * 8)), z1 = __ldg(reinterpret_cast<const float4*>(zs + ch * 8 + 4));
        float2 f;
        f = unpack_half2(u.x); qz0 = fmaf(f.x, z0.x, qz0); qz1 = fmaf(f.y, z0.y, qz1);
        f = unpack_half2(u.y); qz2 = fmaf(f.x, z0.z, qz2); qz3 = fmaf(f.y, z0.w, qz3);
        f = unpack_half2(u.z); qz0 = fmaf(f.x, z1.x, qz0); qz1 = fmaf(f.y, z1.y, qz1);
        f = unpack_half2(u.w); qz2 = fmaf(f.x, z1.z, qz2); qz3 = fmaf(f.y, z1.w, qz3);
      }
      // ---- den, gs, gr
      if (!mbar_wait(&bars[bN], ph)) { tc_fail(27); ok = false; break; }
      tc_fence_after_sync();
      float gr;
      {
        uint32_t nn[64];
        tmem_ld32(tmem + lane_addr + cN, nn);
        tmem_ld32(tmem + lane_addr + cN + 32, nn + 32);
        tmem_ld_wait();
        const float raw = (qz0 + qz1) + (qz2 + qz3);
        const float dn = fmaxf(fabsf(raw), kEps), inv = 1.f / dn;
        float go = 0.f;
        unsigned char* grow = stage + kG_;
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          uint4* p = reinterpret_cast<uint4*>(grow + row_chunk1(row, ch));
          uint4 u = *p;
          float2 f0 = unpack_half2(u.x), f1 = unpack_half2(u.y), f2 = unpack_half2(u.z), f3 = unpack_half2(u.w);
          go = fmaf(f0.x, __uint_as_float(nn[ch * 8 + 0]), go); go = fmaf(f0.y, __uint_as_float(nn[ch * 8 + 1]), go);
          go = fmaf(f1.x, __uint_as_float(nn[ch * 8 + 2]), go); go = fmaf(f1.y, __uint_as_float(nn[ch * 8 + 3]), go);
          go = fmaf(f2.x, __uint_as_float(nn[ch * 8 + 4]), go); go = fmaf(f2.y, __uint_as_float(nn[ch * 8 + 5]), go);
          go = fmaf(f3.x, __uint_as_float(nn[ch * 8 + 6]), go); go = fmaf(f3.y, __uint_as_float(nn[ch * 8 + 7]), go);
          u.x = pack_half2(f0.x * inv, f0.y * inv); u.y = pack_half2(f1.x * inv, f1.y * inv);
          u.z = pack_half2(f2.x * inv, f2.y * inv); u.w = pack_half2(f3.x * inv, f3.y * inv);
          *p = u;
        }
        go *= inv;                                                        // g . out
        gr = fabsf(raw) > kEps ? (raw > 0.f ? -go * inv : go * inv) : 0.f; // d/d raw of 1/max(|raw|,1)
        grs[row] = gr;
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[bG]);
      if (!mbar_wait(&bars[bG], ph)) { tc_fail(28); ok = false; break; }   // gr of every row is in shared memory
      dz_acc += column_sum2(stage + kQ_, quarter, lane, grs);
      // ---- g_phi_q = dQ + gr z^T -> fp16 over the Q tile -> TMA store
      if (!mbar_wait(&bars[bDQ], ph)) { tc_fail(29); ok = false; break; }
      tc_fence_after_sync();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(30); ok = false; break; }   // every column sum over Q is done
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        tmem_ld32(tmem + lane_addr + cDQ + piece * 32, a);
        tmem_ld_wait();
        if (piece == 3) { tc_fence_before_sync(); mbar_arrive(&bars[bDQFree]); }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k0 = piece * 32 + j * 8;
          const float4 z0 = __ldg(reinterpret_cast<const float4*>(zs + k0)), z1 = __ldg(reinterpret_cast<const float4*>(zs + k0 + 4));
          uint4 u;
          u.x = pack_half2(fmaf(gr, z0.x, __uint_as_float(a[j * 8 + 0])), fmaf(gr, z0.y, __uint_as_float(a[j * 8 + 1])));
          u.y = pack_half2(fmaf(gr, z0.z, __uint_as_float(a[j * 8 + 2])), fmaf(gr, z0.w, __uint_as_float(a[j * 8 + 3])));
          u.z = pack_half2(fmaf(gr, z1.x, __uint_as_float(a[j * 8 + 4])), fmaf(gr, z1.y, __uint_as_float(a[j * 8 + 5])));
          u.w = pack_half2(fmaf(gr, z1.z, __uint_as_float(a[j * 8 + 6])), fmaf(gr, z1.w, __uint_as_float(a[j * 8 + 7])));
          *reinterpret_cast<uint4*>(stage + kQ_ + row_chunk2(row, piece * 4 + j)) = u;
        }
      }
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(31); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(&tm_gq, stage + kQ_, 0, bh, c * kTC);
        tma_store_3d(&tm_gq, stage + kQ_ + kBox, 64, bh, c * kTC);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&bars[bEmpty + st]);
      }
    }
    if (ok) {       // state gradients out (the last wait on bDQ ordered the dS accumulator)
      uint32_t r[64];
      if (nchunk > 0) { tmem_ld32(tmem + lane_addr + cDS, r); tmem_ld32(tmem + lane_addr + cDS + 32, r + 32); tmem_ld_wait(); }
      else {
#pragma unroll
        for (int n = 0; n < 64; ++n) r[n] = 0u;
      }
      float4* dst = reinterpret_cast<float4*>(d_s + ((size_t)bh * kK + row) * kD);
#pragma unroll
      for (int n = 0; n < 16; ++n)
        dst[n] = make_float4(__uint_as_float(r[4 * n]), __uint_as_float(r[4 * n + 1]), __uint_as_float(r[4 * n + 2]), __uint_as_float(r[4 * n + 3]));
      d_z[(size_t)bh * kK + row] = dz_acc;
    }
    if (etid == 0) tma_store_wait<0>();
  }
  RFA_X_FINISH(256)
}

// ===========================================================================
// state backward.  grid (BH)
// ===========================================================================
namespace xk {
// 113 KB exactly: two CTAs share an SM (256 sequences are then one wave instead of 148 + 108, and one CTA's ramp and
// drain hide behind the other's chunks)
constexpr uint32_t kK_ = 0, kV_ = 2 * kBox, kStage = 3 * kBox, kS_ = 2 * kStage, kDz_ = kS_ + kBox, kBarOff = kDz_ + 512,
                   kSmem = 113 * 1024;
static_assert(kBarOff + 128 <= kSmem, "cross_state_bwd: shared memory map exceeds half an SM");
constexpr uint32_t cDK = 0, cDV = 128;
enum { bFull = 0, bEmpty = 2, bReady = 4, bOut = 6, bFree = 7, bSt = 8, bEpi = 9, bNum = 10 };
}

__global__ void __launch_bounds__(kXThreads, 2)
cross_state_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                          const __grid_constant__ CUtensorMap tm_gk, const __grid_constant__ CUtensorMap tm_gv,
                          const uint8_t* __restrict__ pad_mask, const float* __restrict__ d_s, const float* __restrict__ d_z,
                          int64_t T, int BH, int H) {
  using namespace xk;
  RFA_X_PROLOGUE_ALIGNED(bNum)
  float* dzs = reinterpret_cast<float*>(sm + kDz_);
  const int bh = blockIdx.x;
  const int nchunk = (int)((T + kTC - 1) / kTC);
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 1); mbar_init(&bars[bReady + i], 128); }
    mbar_init(&bars[bOut], 1); mbar_init(&bars[bFree], 128); mbar_init(&bars[bSt], 128); mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_gk); tma_prefetch_desc(&tm_gv);
  }
  RFA_X_START(256)
  if (warp == 0) {
    if (lane == 0)
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[bEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(41); break; }
        unsigned char* base = sm + st * kStage;
        mbar_arrive_expect_tx(&bars[bFull + st], kStage);
        tma_load_3d(base + kK_, &tm_k, &bars[bFull + st], 0, bh, c * kTC);
        tma_load_3d(base + kK_ + kBox, &tm_k, &bars[bFull + st], 64, bh, c * kTC);
        tma_load_3d(base + kV_, &tm_v, &bars[bFull + st], 0, bh, c * kTC);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idKK = umma_idesc_f16(128, 128, false, false);   // V dS^T
      constexpr uint32_t idKM = umma_idesc_f16(128, 64, false, true);     // K dS
      const uint64_t dKk = umma_smem_desc(sbase + kK_, 0, 1024, kSwizzle128B), dVk = umma_smem_desc(sbase + kV_, 0, 1024, kSwizzle128B);
      const uint64_t dSk = umma_smem_desc(sbase + kS_, 0, 1024, kSwizzle128B), dSm = umma_smem_desc(sbase + kS_, kBox, 1024, kSwizzle128B);
      bool ok = mbar_wait(&bars[bSt], 0);
      if (!ok) tc_fail(42);
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * (kStage >> 4);
        if (!mbar_wait(&bars[bReady + st], (c >> 1) & 1)) { tc_fail(43); break; }
        if (c > 0 && !mbar_wait(&bars[bFree], (c - 1) & 1)) { tc_fail(44); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_ss(tmem + cDK, dVk + so + kstep_kmajor(j, kBox), dSk + kstep_kmajor(j, kBox), idKK, j > 0);
#pragma unroll
        for (int j = 0; j < 8; ++j) umma_ss(tmem + cDV, dKk + so + kstep_kmajor(j, kBox), dSm + kstep_mnmajor(j), idKM, j > 0);
        umma_commit(&bars[bOut]);
      }
    }
  } else {
    const int quarter = warp & 3, row = quarter * 32 + lane, etid = tid - 64;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint8_t* mrow = pad_mask ? pad_mask + (size_t)(bh / H) * T : nullptr;
    {
      uint32_t r[64];
      const float* src = d_s + ((size_t)bh * kK + row) * kD;
#pragma unroll
      for (int n = 0; n < 64; n += 4) {
        const float4 f = *reinterpret_cast<const float4*>(src + n);
        r[n] = __float_as_uint(f.x); r[n + 1] = __float_as_uint(f.y); r[n + 2] = __float_as_uint(f.z); r[n + 3] = __float_as_uint(f.w);
      }
      store_state_row(sm + kS_, row, r);
      dzs[row] = d_z[(size_t)bh * kK + row];
      fence_async_smem();
      mbar_arrive(&bars[bSt]);
    }
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      unsigned char* stage = sm + st * kStage;
      const int64_t t0 = (int64_t)c * kTC;
      if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(45); ok = false; break; }
      const bool keep = (t0 + row < T) && !(mrow && mrow[t0 + row]);
      if (mrow && !keep) zero_row2(stage + kK_, row);      // masked phi_k multiplies dS: its row of grad_v is zero
      fence_async_smem();
      mbar_arrive(&bars[bReady + st]);
      if (!mbar_wait(&bars[bOut], c & 1)) { tc_fail(46); ok = false; break; }
      tc_fence_after_sync();
      if (c == 0 && !epi_sync(&bars[bEpi], epi_phase)) { tc_fail(47); ok = false; break; }   // dzs complete
      {
        uint32_t r[64];
        tmem_ld32(tmem + lane_addr + cDV, r);
        tmem_ld32(tmem + lane_addr + cDV + 32, r + 32);
        tmem_ld_wait();
        store_state_row(stage + kV_, row, r);
      }
      const float kf = keep ? 1.f : 0.f;                    // masked_fill blocks the gradient at padded keys
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        tmem_ld32(tmem + lane_addr + cDK + piece * 32, a);
        tmem_ld_wait();
        if (piece == 3) { tc_fence_before_sync(); mbar_arrive(&bars[bFree]); }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k0 = piece * 32 + j * 8;
          const float4 z0 = *reinterpret_cast<const float4*>(dzs + k0), z1 = *reinterpret_cast<const float4*>(dzs + k0 + 4);
          uint4 u;
          u.x = pack_half2(kf * (__uint_as_float(a[j * 8 + 0]) + z0.x), kf * (__uint_as_float(a[j * 8 + 1]) + z0.y));
          u.y = pack_half2(kf * (__uint_as_float(a[j * 8 + 2]) + z0.z), kf * (__uint_as_float(a[j * 8 + 3]) + z0.w));
          u.z = pack_half2(kf * (__uint_as_float(a[j * 8 + 4]) + z1.x), kf * (__uint_as_float(a[j * 8 + 5]) + z1.y));
          u.w = pack_half2(kf * (__uint_as_float(a[j * 8 + 6]) + z1.z), kf * (__uint_as_float(a[j * 8 + 7]) + z1.w));
          *reinterpret_cast<uint4*>(stage + kK_ + row_chunk2(row, piece * 4 + j)) = u;
        }
      }
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(48); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(&tm_gk, stage + kK_, 0, bh, c * kTC);
        tma_store_3d(&tm_gk, stage + kK_ + kBox, 64, bh, c * kTC);
        tma_store_3d(&tm_gv, stage + kV_, 0, bh, c * kTC);
        tma_store_commit();
        tma_store_wait_read<0>();
        mbar_arrive(&bars[bEmpty + st]);
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  RFA_X_FINISH(256)
}

// ---------------------------------------------------------------------------
template <class Kern>
static int x_opt_in(Kern kern, uint32_t bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail((int)e, "%s: cannot reserve %u bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared);   // a hint only
  return 0;
}

int launch_cross_state_fwd_tc(const __half* k, const __half* v, const uint8_t* pad_mask, float* s, float* z, int64_t T, int BH,
                              int H, int nseg, int64_t tseg, cudaStream_t st) {
  CUtensorMap tk, tv;
  const int r1 = make_tmap_rows(&tk, k, T, BH, kK, kTC), r2 = make_tmap_rows(&tv, v, T, BH, kD, kTC);
  if (r1 || r2)
    return fail(RFA_EDEVICE, "cross_state_fwd: cuTensorMapEncodeTiled failed or is unavailable (%d, %d; k=%p v=%p T=%lld BH=%d)", r1, r2,
                (const void*)k, (const void*)v, (long long)T, BH);
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if ((int64_t)BH * nseg > sms) {            // more CTAs than SMs: two per SM, two stages each
    if (int e = x_opt_in(cross_state_fwd_tc_kernel<2>, xs::L<2>::kSmem, "cross_state_fwd")) return e;
    launch_pdl(cross_state_fwd_tc_kernel<2>, dim3(BH, nseg), kXThreads, xs::L<2>::kSmem, st, tk, tv, pad_mask, s, z, T, BH, H, nseg, tseg);
  } else {
    if (int e = x_opt_in(cross_state_fwd_tc_kernel<4>, xs::L<4>::kSmem, "cross_state_fwd")) return e;
    launch_pdl(cross_state_fwd_tc_kernel<4>, dim3(BH, nseg), kXThreads, xs::L<4>::kSmem, st, tk, tv, pad_mask, s, z, T, BH, H, nseg, tseg);
  }
  return check_launch("rfa_cross_state_fwd");
}

int launch_cross_query_fwd_tc(const __half* q, const float* s, const float* z, __half* out, int64_t T, int BH, cudaStream_t st) {
  CUtensorMap tq, to;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&to, out, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "cross_query_fwd: cuTensorMapEncodeTiled failed or is unavailable");
  if (int e = x_opt_in(cross_query_fwd_tc_kernel, xq::kSmem, "cross_query_fwd")) return e;
  launch_pdl(cross_query_fwd_tc_kernel, dim3(BH), kXThreads, xq::kSmem, st, tq, to, s, z, T, BH);
  return check_launch("rfa_cross_query_fwd");
}

int launch_cross_query_bwd_tc(const __half* q, const float* s, const float* z, const __half* g, __half* gq, float* d_s, float* d_z,
                              int64_t T, int BH, cudaStream_t st) {
  CUtensorMap tq, tg, tgq;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tg, g, T, BH, kD, kTC) || make_tmap_rows(&tgq, gq, T, BH, kK, kTC))
    return fail(RFA_EDEVICE, "cross_query_bwd: cuTensorMapEncodeTiled failed or is unavailable");
  if (int e = x_opt_in(cross_query_bwd_tc_kernel, xb::kSmem, "cross_query_bwd")) return e;
  launch_pdl(cross_query_bwd_tc_kernel, dim3(BH), kXThreads, xb::kSmem, st, tq, tg, tgq, s, z, d_s, d_z, T, BH);
  return check_launch("rfa_cross_query_bwd");
}

int launch_cross_state_bwd_tc(const __half* k, const __half* v, const uint8_t* pad_mask, const float* d_s, const float* d_z,
                              __half* gk, __half* gv, int64_t T, int BH, int H, cudaStream_t st) {
  CUtensorMap tk, tv, tgk, tgv;
  if (make_tmap_rows(&tk, k, T, BH, kK, kTC) || make_tmap_rows(&tv, v, T, BH, kD, kTC) ||
      make_tmap_rows(&tgk, gk, T, BH, kK, kTC) || make_tmap_rows(&tgv, gv, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "cross_state_bwd: cuTensorMapEncodeTiled failed or is unavailable");
  if (int e = x_opt_in(cross_state_bwd_tc_kernel, xk::kSmem, "cross_state_bwd")) return e;
  launch_pdl(cross_state_bwd_tc_kernel, dim3(BH), kXThreads, xk::kSmem, st, tk, tv, tgk, tgv, pad_mask, d_s, d_z, T, BH, H);
  return check_launch("rfa_cross_state_bwd");
}

RFA_TC_UNIT(cross)

}  // namespace rfa
