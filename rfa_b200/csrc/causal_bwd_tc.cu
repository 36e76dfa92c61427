// Causal RFA backward on tcgen05 tensor cores: the two sweeps of upstream's
// rfa_backward (cuda/backward.cu:453-527; math in rfa.py:79-101), chunked by 128 tokens.
//
// Sweep 1 (forward in time, one CTA per (batch, head[, segment])), per chunk:
//     A  = Q K^T                    P = mask(A) fp16 (TMEM), rowsum
//     N  = P V + Q S_prev           den = max(rowsum + q.z_prev, 1), out = N/den
//     gs = g/den  (fp16, written over the staged g tile),  gz = -(g.out)/den * [raw > 1]
//     dA = mask(gs V^T + gz)        fp16 (TMEM, over P)
//     dQ = dA K + gs S_prev^T + gz z_prev^T          -> grad_q
//     S += K^T V,  z += colsum(K);  optionally  dSseg += Q^T gs, dzseg += Q^T gz
//   den and gz per token go to the workspace for sweep 2.
// Sweep 2 (reverse in time), per chunk, with the transposed score matrices computed
// directly so that they can stay in TMEM as A operands:
//     At  = K Q^T  -> Pt = mask fp16          dAt = V gs^T  -> mask(dAt + gz_t) fp16
//     dK  = dAt Q + V dS_next^T + dz_next^T   -> grad_k
//     dV  = Pt gs + K dS_next                 -> grad_v
//     dS += Q^T gs,  dz += Q^T gz
// All running states (S, dS) are fp32 TMEM accumulators; their fp16 copies in shared
// memory serve as B operands.  z, dz stay fp32 in shared memory (CUDA-core updates).
#include "tc_common.cuh"

namespace rfa {

constexpr int kBwThreads = 192;    // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue

// shared memory map: two stages of {Q, K (2 boxes each), V, G (1 box each)}, then the fp16 state tile
constexpr uint32_t kBwQ = 0, kBwK = 2 * kBox, kBwV = 4 * kBox, kBwG = 5 * kBox, kBwStage = 6 * kBox;   // 98304
constexpr uint32_t kBwS = 2 * kBwStage;            // [128 k][64 n] fp16, swizzled: the running state as an operand
constexpr uint32_t kBwZ = kBwS + kBox;             // fp32 [128]  z (sweep 1) / dz (sweep 2)
constexpr uint32_t kBwGz = kBwZ + 512;             // fp32 [2][128]  gz of the chunk's rows (two chunks in flight)
constexpr uint32_t kBwBar = kBwGz + 1024;
constexpr uint32_t kBwSmem = kBwBar + 256 + 1024;

enum { bFull = 0, bEmpty = 2, bA = 4, bP = 5, bN = 6, bG = 7, bDA = 8, bDA16 = 9, bDQ = 10, bS = 11, bSt = 12, bEpi = 13, bNum = 14 };

// ===========================================================================
// sweep 1
// ===========================================================================
constexpr uint32_t q1ColA = 0, q1ColDQ = 128, q1ColN = 256, q1ColS = 320, q1ColDS = 384;

__global__ void __launch_bounds__(kBwThreads, 1)
causal_bwd_q_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                       const __grid_constant__ CUtensorMap tm_gq,
                       const float* __restrict__ s_seg, const float* __restrict__ z_seg,
                       float* __restrict__ ws_den, float* __restrict__ ws_gz,
                       float* __restrict__ ds_seg, float* __restrict__ dz_seg,
                       int64_t T, int BH, int nseg, int64_t tseg) {
  extern __shared__ unsigned char bw_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(bw_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBwBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bNum);
  float* zs = reinterpret_cast<float*>(sm + kBwZ);
  float* gzs = reinterpret_cast<float*>(sm + kBwGz);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  const int nchunk = (int)((t_end - t_begin + kTC - 1) / kTC);
  const size_t slot = (size_t)bh * nseg + seg;
  const float* s_in = s_seg ? s_seg + slot * kK * kD : nullptr;
  const float* z_in = z_seg ? z_seg + slot * kK : nullptr;
  const bool want_dseg = ds_seg != nullptr;

  if (tid == 0) {
    mbar_init(&bars[bFull], 1); mbar_init(&bars[bFull + 1], 1);
    mbar_init(&bars[bEmpty], 129); mbar_init(&bars[bEmpty + 1], 129);
    mbar_init(&bars[bA], 1); mbar_init(&bars[bP], 128); mbar_init(&bars[bN], 1); mbar_init(&bars[bG], 128);
    mbar_init(&bars[bDA], 1); mbar_init(&bars[bDA16], 128); mbar_init(&bars[bDQ], 1); mbar_init(&bars[bS], 1);
    mbar_init(&bars[bSt], 128); mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_g);
    tma_prefetch_desc(&tm_gq);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[bEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * kBwStage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        uint64_t* fb = &bars[bFull + st];
        mbar_arrive_expect_tx(fb, kBwStage);
        tma_load_3d(base + kBwQ, &tm_q, fb, 0, bh, t0);
        tma_load_3d(base + kBwQ + kBox, &tm_q, fb, 64, bh, t0);
        tma_load_3d(base + kBwK, &tm_k, fb, 0, bh, t0);
        tma_load_3d(base + kBwK + kBox, &tm_k, fb, 64, bh, t0);
        tma_load_3d(base + kBwV, &tm_v, fb, 0, bh, t0);
        tma_load_3d(base + kBwG, &tm_g, fb, 0, bh, t0);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idQK = umma_idesc_f16(128, 128, false, false);   // Q K^T ; gs V^T (K=64)
      constexpr uint32_t idPV = umma_idesc_f16(128, 64, false, true);     // P V ; Q S        (B MN-major)
      constexpr uint32_t idDAK = umma_idesc_f16(128, 128, false, true);   // dA K             (B MN-major)
      constexpr uint32_t idKtV = umma_idesc_f16(128, 64, true, true);     // K^T V ; Q^T gs   (A, B MN-major)
      // operand descriptors per stage (the shared-memory layout is static); a k-step is an add
      uint64_t dQk[2], dQm[2], dKk[2], dKm[2], dVk[2], dVm[2], dGk[2], dGm[2];
#pragma unroll
      for (int s2 = 0; s2 < 2; ++s2) {
        const uint32_t sb = sbase + s2 * kBwStage;
        dQk[s2] = umma_smem_desc(sb + kBwQ, 0, 1024, kSwizzle128B);       // Q  K-major
        dQm[s2] = umma_smem_desc(sb + kBwQ, kBox, 1024, kSwizzle128B);    // Q  MN-major (rows = contraction t)
        dKk[s2] = umma_smem_desc(sb + kBwK, 0, 1024, kSwizzle128B);       // K  K-major
        dKm[s2] = umma_smem_desc(sb + kBwK, kBox, 1024, kSwizzle128B);    // K  MN-major (rows = contraction s)
        dVk[s2] = umma_smem_desc(sb + kBwV, 0, 1024, kSwizzle128B);       // V  K-major
        dVm[s2] = umma_smem_desc(sb + kBwV, kBox, 1024, kSwizzle128B);    // V  MN-major
        dGk[s2] = umma_smem_desc(sb + kBwG, 0, 1024, kSwizzle128B);       // gs K-major
        dGm[s2] = umma_smem_desc(sb + kBwG, kBox, 1024, kSwizzle128B);    // gs MN-major
      }
      const uint64_t dSk = umma_smem_desc(sbase + kBwS, 0, 1024, kSwizzle128B);      // S as [N = k rows][K = n]
      const uint64_t dSm = umma_smem_desc(sbase + kBwS, kBox, 1024, kSwizzle128B);   // S as [K = k rows][N = n]
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        const uint32_t ph = c & 1;
        if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(2); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j)              // A = Q K^T
          umma_ss(tmem + q1ColA, dQk[st] + kstep_kmajor(j, kBox), dKk[st] + kstep_kmajor(j, kBox), idQK, j > 0);
        umma_commit(&bars[bA]);
        if (!mbar_wait(&bars[bP], ph)) { tc_fail(3); break; }
        if (!mbar_wait(&bars[bSt], ph)) { tc_fail(4); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j)              // N = P V
          umma_ts(tmem + q1ColN, tmem + q1ColA + j * 8, dVm[st] + kstep_mnmajor(j), idPV, j > 0);
#pragma unroll
        for (int j = 0; j < 8; ++j)              // N += Q S_prev   (S tile [k rows][n]: B MN-major over k)
          umma_ss(tmem + q1ColN, dQk[st] + kstep_kmajor(j, kBox), dSm + kstep_mnmajor(j), idPV, 1);
        umma_commit(&bars[bN]);
        if (!mbar_wait(&bars[bG], ph)) { tc_fail(5); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j)              // dA = gs V^T   (contraction over d = 64)
          umma_ss(tmem + q1ColA, dGk[st] + kstep_kmajor(j, kBox), dVk[st] + kstep_kmajor(j, kBox), idQK, j > 0);
        umma_commit(&bars[bDA]);
        if (want_dseg)
#pragma unroll
          for (int j = 0; j < 8; ++j)            // dSseg += Q^T gs
            umma_ss(tmem + q1ColDS, dQm[st] + kstep_mnmajor(j), dGm[st] + kstep_mnmajor(j), idKtV, (c > 0 || j > 0) ? 1 : 0);
        if (!mbar_wait(&bars[bDA16], ph)) { tc_fail(6); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 8; ++j)              // dQ = dA K
          umma_ts(tmem + q1ColDQ, tmem + q1ColA + j * 8, dKm[st] + kstep_mnmajor(j), idDAK, j > 0);
#pragma unroll
        for (int j = 0; j < 4; ++j)              // dQ += gs S_prev^T   (S tile as [N = k rows][K = n])
          umma_ss(tmem + q1ColDQ, dGk[st] + kstep_kmajor(j, kBox), dSk + kstep_kmajor(j, kBox), idQK, 1);
        umma_commit(&bars[bDQ]);
        const bool fresh = (c == 0 && s_in == nullptr);
#pragma unroll
        for (int j = 0; j < 8; ++j)              // S += K^T V
          umma_ss(tmem + q1ColS, dKm[st] + kstep_mnmajor(j), dVm[st] + kstep_mnmajor(j), idKtV, (fresh && j == 0) ? 0 : 1);
        umma_commit(&bars[bS]);
        umma_commit(&bars[bEmpty + st]);
      }
    }
  } else {
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int etid = tid - 64;
    unsigned char* s_tile = sm + kBwS;
    // state entering this run of tokens
    {
      uint32_t r[64];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
      store_state_row(s_tile, row, r);
      if (s_in) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) tmem_st16(tmem + lane_addr + q1ColS + c0, r + c0);
        tmem_st_wait();
      }
      zs[row] = z_in ? z_in[row] : 0.f;
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[bSt]);
    }
    bool ok = true;
    uint32_t epi_phase = 0;
    float dz_acc = 0.f;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t ph = c & 1;
      unsigned char* stage = sm + st * kBwStage;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      if (!mbar_wait(&bars[bFull + st], (c >> 1) & 1)) { tc_fail(7); ok = false; break; }
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(8); ok = false; break; }     // zs of the previous chunk is final
      // q . z_prev in fp32 from this thread's own Q row
      float qz = 0.f;
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const uint4 u = *reinterpret_cast<const uint4*>(stage + kBwQ + row_chunk2(row, ch));
        const float4 z0 = *reinterpret_cast<const float4*>(zs + ch * 8), z1 = *reinterpret_cast<const float4*>(zs + ch * 8 + 4);
        float2 f;
        f = unpack_half2(u.x); qz = fmaf(f.x, z0.x, qz); qz = fmaf(f.y, z0.y, qz);
        f = unpack_half2(u.y); qz = fmaf(f.x, z0.z, qz); qz = fmaf(f.y, z0.w, qz);
        f = unpack_half2(u.z); qz = fmaf(f.x, z1.x, qz); qz = fmaf(f.y, z1.y, qz);
        f = unpack_half2(u.w); qz = fmaf(f.x, z1.z, qz); qz = fmaf(f.y, z1.w, qz);
      }
      // ---- P = mask(A), row sums
      if (!mbar_wait(&bars[bA], ph)) { tc_fail(9); ok = false; break; }
      tc_fence_after_sync();
      float rowsum = 0.f;
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t p[16];
        if (piece <= quarter) {
          uint32_t a[32];
          tmem_ld32(tmem + lane_addr + q1ColA + piece * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0 = __uint_as_float(a[i]), x1 = __uint_as_float(a[i + 1]);
            if (piece == quarter) {
              if (i > lane) x0 = 0.f;
              if (i + 1 > lane) x1 = 0.f;
            }
            rowsum += x0 + x1;
            p[i >> 1] = pack_half2(x0, x1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) p[i] = 0u;
        }
        tmem_st16(tmem + lane_addr + q1ColA + piece * 16, p);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bP]);
      // ---- den, gz, gs
      if (!mbar_wait(&bars[bN], ph)) { tc_fail(10); ok = false; break; }
      tc_fence_after_sync();
      float gz;
      {
        uint32_t nn[64];
        tmem_ld32(tmem + lane_addr + q1ColN, nn);
        tmem_ld32(tmem + lane_addr + q1ColN + 32, nn + 32);
        tmem_ld_wait();
        const float raw = rowsum + qz;
        const float dn = fmaxf(raw, kEps), inv = 1.f / dn;
        float go = 0.f;
        unsigned char* grow = stage + kBwG;
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
        go *= inv;                                   // g . out
        gz = raw > kEps ? -go * inv : 0.f;           // strict >, upstream rfa.py:91
        if (t0 + row < t_end) {
          ws_den[(size_t)bh * T + t0 + row] = dn;
          ws_gz[(size_t)bh * T + t0 + row] = gz;
        }
        gzs[row] = gz;
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[bG]);
      if (want_dseg) {                               // dzseg += Q^T gz, while Q is still intact
        if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(11); ok = false; break; }
        dz_acc += column_sum2(stage + kBwQ, quarter, lane, gzs);
      }
      // ---- dA = mask(gs V^T + gz) -> fp16 over the P columns
      if (!mbar_wait(&bars[bDA], ph)) { tc_fail(12); ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t p[16];
        if (piece <= quarter) {
          uint32_t a[32];
          tmem_ld32(tmem + lane_addr + q1ColA + piece * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float x0 = __uint_as_float(a[i]) + gz, x1 = __uint_as_float(a[i + 1]) + gz;
            if (piece == quarter) {
              if (i > lane) x0 = 0.f;
              if (i + 1 > lane) x1 = 0.f;
            }
            p[i >> 1] = pack_half2(x0, x1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) p[i] = 0u;
        }
        tmem_st16(tmem + lane_addr + q1ColA + piece * 16, p);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bDA16]);
      // ---- grad_q = dQ + gz z_prev^T -> fp16 over this thread's row of the Q tile -> TMA store
      if (!mbar_wait(&bars[bDQ], ph)) { tc_fail(13); ok = false; break; }
      tc_fence_after_sync();
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        tmem_ld32(tmem + lane_addr + q1ColDQ + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k0 = piece * 32 + j * 8;
          const float4 z0 = *reinterpret_cast<const float4*>(zs + k0), z1 = *reinterpret_cast<const float4*>(zs + k0 + 4);
          uint4 u;
          u.x = pack_half2(fmaf(gz, z0.x, __uint_as_float(a[j * 8 + 0])), fmaf(gz, z0.y, __uint_as_float(a[j * 8 + 1])));
          u.y = pack_half2(fmaf(gz, z0.z, __uint_as_float(a[j * 8 + 2])), fmaf(gz, z0.w, __uint_as_float(a[j * 8 + 3])));
          u.z = pack_half2(fmaf(gz, z1.x, __uint_as_float(a[j * 8 + 4])), fmaf(gz, z1.y, __uint_as_float(a[j * 8 + 5])));
          u.w = pack_half2(fmaf(gz, z1.z, __uint_as_float(a[j * 8 + 6])), fmaf(gz, z1.w, __uint_as_float(a[j * 8 + 7])));
          *reinterpret_cast<uint4*>(stage + kBwQ + row_chunk2(row, piece * 4 + j)) = u;
        }
      }
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(14); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(&tm_gq, stage + kBwQ, 0, bh, (int)t0);
        tma_store_3d(&tm_gq, stage + kBwQ + kBox, 64, bh, (int)t0);
        tma_store_commit();
      }
      // ---- z += colsum(K)   (every thread is past its reads of zs for this chunk)
      zs[row] += column_sum2(stage + kBwK, quarter, lane, nullptr);
      // ---- state after this chunk -> fp16 operand tile
      if (!mbar_wait(&bars[bS], ph)) { tc_fail(15); ok = false; break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        uint32_t r[64];
        tmem_ld32(tmem + lane_addr + q1ColS, r);
        tmem_ld32(tmem + lane_addr + q1ColS + 32, r + 32);
        tmem_ld_wait();
        store_state_row(s_tile, row, r);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[bSt]);
      }
      // release the stage: every epilogue thread is past its last read of it, and the store has drained it
      if (etid == 0) tma_store_wait_read<0>();
      mbar_arrive(&bars[bEmpty + st]);
    }
    if (ok && want_dseg) {
      uint32_t r[64];
      if (nchunk > 0) {
        tmem_ld32(tmem + lane_addr + q1ColDS, r);
        tmem_ld32(tmem + lane_addr + q1ColDS + 32, r + 32);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int n = 0; n < 64; ++n) r[n] = 0u;
      }
      float4* dst = reinterpret_cast<float4*>(ds_seg + (slot * kK + row) * kD);
#pragma unroll
      for (int n = 0; n < 16; ++n)
        dst[n] = make_float4(__uint_as_float(r[4 * n]), __uint_as_float(r[4 * n + 1]), __uint_as_float(r[4 * n + 2]),
                             __uint_as_float(r[4 * n + 3]));
      dz_seg[slot * kK + row] = dz_acc;
    }
    if (etid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
int launch_causal_bwd_q_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq,
                           const float* s_seg, const float* z_seg, float* ws_den, float* ws_gz, float* ds_seg,
                           float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tg, tgq;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&tg, g, T, BH, kD, kTC) ||
      make_tmap_rows(&tgq, gq, T, BH, kK, kTC))
    return fail(RFA_EDEVICE, "causal_bwd_q: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_bwd_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBwSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_bwd_q: cannot reserve %u bytes of shared memory: %s", kBwSmem, cudaGetErrorString(e));
  causal_bwd_q_tc_kernel<<<dim3(BH, nseg), kBwThreads, kBwSmem, st>>>(tq, tk, tv, tg, tgq, s_seg, z_seg, ws_den, ws_gz, ds_seg,
                                                                     dz_seg, T, BH, nseg, tseg);
  return check_launch("rfa_causal_bwd_q");
}


int tc_status_causal_bwd() { return tc_status_read_clear(); }

}  // namespace rfa
