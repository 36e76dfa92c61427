// Causal RFA forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One CTA walks one (batch, head[, segment]) in chunks of C = 128 tokens.  Per chunk
// (Q, K: [C][128] fp16; V: [C][64] fp16; S: running [128][64] state; z: running [128]):
//     A   = Q K^T                      tcgen05.mma  M128 N128 K128   (smem x smem -> TMEM)
//     N   = Q [S|z]_prev^T             tcgen05.mma  M128 N80  K128   (smem x smem)
//     P   = mask(A) as fp16, row sums  epilogue warps, TMEM -> registers -> TMEM (aliases A)
//     N  += P V                        tcgen05.mma  M128 N64  K128   (TMEM x smem)
//     [S|z] += K^T [V|1]               tcgen05.mma  M128 N128 K128   (smem x smem, fp32 in TMEM)
//     out = N[:, :64] / max(rowsum + N[:, 64], 1)
// The fp32 state never leaves TMEM; its fp16 transposed copy ([80][128], K-major) is
// re-exported to shared memory once per chunk as the B operand of the next chunk.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = MMA issuer, warps 2..5 =
// epilogue (thread <-> TMEM lane <-> token row / state row).  Two shared-memory stages
// of Q, K, V; two TMEM buffers for A/P.  All waits are bounded.
#include "tc_common.cuh"

namespace rfa {

constexpr int kTcThreads = 192;

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kBoxQK = 128 * 128;         // one [128 rows][64 halves] box
constexpr uint32_t kOffQ = 0, kOffK = 2 * kBoxQK, kOffV = 4 * kBoxQK, kStage = 5 * kBoxQK;   // 81920 per stage
constexpr uint32_t kOffOnes = 2 * kStage;                       // [128][64] box: column 0 = 1, rest 0
constexpr uint32_t kOffSt = kOffOnes + kBoxQK;                  // [80][128] fp16, two [80][64] boxes
constexpr uint32_t kBoxSt = 80 * 128;
constexpr uint32_t kOffOut = kOffSt + 2 * kBoxSt;               // [128][64] output staging
constexpr uint32_t kOffBar = kOffOut + kBoxQK;
constexpr uint32_t kTcSmem = kOffBar + 256 + 1024;              // + alignment slack

// TMEM columns
constexpr uint32_t kColA = 0;        // two buffers of 128
constexpr uint32_t kColN = 256;      // 80
constexpr uint32_t kColS = 384;      // 128 (64 S + z + zeros)

enum { kBarFull = 0, kBarEmpty = 2, kBarA = 4, kBarP = 6, kBarN = 8, kBarNFree = 9, kBarS = 10, kBarSt = 11, kBarEpi = 12, kNumBars = 13 };


__global__ void __launch_bounds__(kTcThreads, 1)
causal_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                     const float* __restrict__ s_seg, const float* __restrict__ z_seg,
                     float* __restrict__ s_out, float* __restrict__ z_out,
                     int64_t T, int BH, int nseg, int64_t tseg) {
  extern __shared__ unsigned char tc_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kOffBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + kNumBars);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  const int nchunk = (int)((t_end - t_begin + kTC - 1) / kTC);
  const size_t slot = (size_t)bh * nseg + seg;
  const float* s_in = s_seg ? s_seg + slot * kK * kD : nullptr;
  const float* z_in = z_seg ? z_seg + slot * kK : nullptr;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[kBarFull + i], 1);
      mbar_init(&bars[kBarEmpty + i], 1);
      mbar_init(&bars[kBarA + i], 1);
      mbar_init(&bars[kBarP + i], 128);
    }
    mbar_init(&bars[kBarN], 1);
    mbar_init(&bars[kBarNFree], 128);
    mbar_init(&bars[kBarS], 1);
    mbar_init(&bars[kBarSt], 128);
    mbar_init(&bars[kBarEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // the ones box: row r is 128 bytes; logical column 0 lives in 16-byte chunk (r & 7)
  for (int i = tid; i < (int)(kBoxQK / 16); i += kTcThreads) {
    const int r = i >> 3, c = i & 7;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (c == (r & 7)) val.x = 0x00003C00u;     // fp16 1.0 in the low half
    *reinterpret_cast<uint4*>(sm + kOffOnes + i * 16) = val;
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[kBarEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * kStage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        mbar_arrive_expect_tx(&bars[kBarFull + st], kStage);
        tma_load_3d(base + kOffQ, &tm_q, &bars[kBarFull + st], 0, bh, t0);
        tma_load_3d(base + kOffQ + kBoxQK, &tm_q, &bars[kBarFull + st], 64, bh, t0);
        tma_load_3d(base + kOffK, &tm_k, &bars[kBarFull + st], 0, bh, t0);
        tma_load_3d(base + kOffK + kBoxQK, &tm_k, &bars[kBarFull + st], 64, bh, t0);
        tma_load_3d(base + kOffV, &tm_v, &bars[kBarFull + st], 0, bh, t0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idA = umma_idesc_f16(128, 128, false, false);   // Q K^T
      constexpr uint32_t idN = umma_idesc_f16(128, 80, false, false);    // Q St^T
      constexpr uint32_t idPV = umma_idesc_f16(128, 64, false, true);    // P V      (B MN-major)
      constexpr uint32_t idS = umma_idesc_f16(128, 128, true, true);     // K^T [V|1] (A, B MN-major)
      auto issue_A = [&](int c) {
        const uint32_t sb = sbase + (c & 1) * kStage;
        for (int j = 0; j < 8; ++j) {
          const uint32_t kk = (j >> 2) * kBoxQK + (j & 3) * 32;
          umma_ss(tmem + kColA + (c & 1) * 128, umma_smem_desc(sb + kOffQ + kk, 0, 1024, kSwizzle128B),
                  umma_smem_desc(sb + kOffK + kk, 0, 1024, kSwizzle128B), idA, j > 0);
        }
        umma_commit(&bars[kBarA + (c & 1)]);
      };
      bool ok = true;
      if (nchunk > 0) {
        ok = mbar_wait(&bars[kBarFull + 0], 0);
        if (ok) { tc_fence_after_sync(); issue_A(0); } else tc_fail(2);
      }
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        const uint32_t sb = sbase + st * kStage;
        if (c + 1 < nchunk) {
          if (!mbar_wait(&bars[kBarFull + ((c + 1) & 1)], ((c + 1) >> 1) & 1)) { tc_fail(3); break; }
          tc_fence_after_sync();
          issue_A(c + 1);
        }
        // N = Q St^T: needs the exported state of all earlier chunks, and N read out by the epilogue
        if (!mbar_wait(&bars[kBarSt], c & 1)) { tc_fail(4); break; }
        if (c > 0 && !mbar_wait(&bars[kBarNFree], (c - 1) & 1)) { tc_fail(5); break; }
        tc_fence_after_sync();
        for (int j = 0; j < 8; ++j) {
          const uint32_t kk = (j >> 2) * kBoxQK + (j & 3) * 32;
          umma_ss(tmem + kColN, umma_smem_desc(sb + kOffQ + kk, 0, 1024, kSwizzle128B),
                  umma_smem_desc(sbase + kOffSt + (j >> 2) * kBoxSt + (j & 3) * 32, 0, 1024, kSwizzle128B), idN, j > 0);
        }
        // N += P V
        if (!mbar_wait(&bars[kBarP + st], (c >> 1) & 1)) { tc_fail(6); break; }
        tc_fence_after_sync();
        for (int j = 0; j < 8; ++j)
          umma_ts(tmem + kColN, tmem + kColA + st * 128 + j * 8,
                  umma_smem_desc(sb + kOffV + j * 2048, kBoxQK, 1024, kSwizzle128B), idPV, 1);
        umma_commit(&bars[kBarN]);
        // [S|z] += K^T [V|1]
        const bool fresh = (c == 0 && s_in == nullptr);
        for (int j = 0; j < 8; ++j)
          umma_ss(tmem + kColS, umma_smem_desc(sb + kOffK + j * 2048, kBoxQK, 1024, kSwizzle128B),
                  umma_smem_desc(sb + kOffV + j * 2048, (kOffOnes - (st * kStage + kOffV)), 1024, kSwizzle128B), idS,
                  (fresh && j == 0) ? 0 : 1);
        umma_commit(&bars[kBarS]);
        umma_commit(&bars[kBarEmpty + st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue warps
    const int quarter = warp & 3;                 // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;          // token row in the chunk / state row k
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int etid = tid - 64;                    // 0..127
    // state entering this run of tokens -> TMEM (fp32) and its fp16 transpose -> shared memory
    {
      unsigned char* st_tile = sm + kOffSt;
      if (s_in) {
        for (int c0 = 0; c0 < 128; c0 += 16) {
          uint32_t r[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int n = c0 + i;
            float val = n < kD ? s_in[(size_t)row * kD + n] : (n == kD ? z_in[row] : 0.f);
            r[i] = __float_as_uint(val);
            if (n < 80) {
              const __half hv = __float2half_rn(val);
              *reinterpret_cast<__half*>(st_tile + (row >> 6) * kBoxSt + sw128_offset(n, row & 63)) = hv;
            }
          }
          tmem_st16(tmem + lane_addr + kColS + c0, r);
        }
        tmem_st_wait();
      } else {
        for (int i = etid; i < (int)(2 * kBoxSt / 16); i += 128) *reinterpret_cast<uint4*>(st_tile + i * 16) = make_uint4(0, 0, 0, 0);
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[kBarSt]);
    }
    bool ok = true;
    uint32_t epi_phase = 0;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t colA = kColA + st * 128;
      // ---- P = mask(A) (fp16, packed, over the first 64 columns of the A buffer) and row sums
      if (!mbar_wait(&bars[kBarA + st], (c >> 1) & 1)) { tc_fail(7); ok = false; break; }
      tc_fence_after_sync();
      float rowsum = 0.f;
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t p[16];
        if (piece <= quarter) {
          uint32_t a[32];
          tmem_ld32(tmem + lane_addr + colA + piece * 32, a);
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
        tmem_st16(tmem + lane_addr + colA + piece * 16, p);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[kBarP + st]);
      // ---- N: numerator (64 columns) and q.z_prev (column 64)
      if (!mbar_wait(&bars[kBarN], c & 1)) { tc_fail(8); ok = false; break; }
      tc_fence_after_sync();
      uint32_t nn[64], nz[16];
      tmem_ld32(tmem + lane_addr + kColN, nn);
      tmem_ld32(tmem + lane_addr + kColN + 32, nn + 32);
      tmem_ld16(tmem + lane_addr + kColN + 64, nz);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[kBarNFree]);
      // ---- export the updated state for the next chunk (critical path of the scan)
      if (!mbar_wait(&bars[kBarS], c & 1)) { tc_fail(9); ok = false; break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        unsigned char* st_col = sm + kOffSt + (row >> 6) * kBoxSt;
#pragma unroll
        for (int c0 = 0; c0 < 80; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(tmem + lane_addr + kColS + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int n = c0 + i;
            if (n <= kD)
              *reinterpret_cast<__half*>(st_col + sw128_offset(n, row & 63)) = __float2half_rn(__uint_as_float(r[i]));
          }
        }
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[kBarSt]);
      }
      // ---- out = N / max(rowsum + q.z_prev, 1) -> staging tile -> TMA store
      const float inv = 1.f / fmaxf(rowsum + __uint_as_float(nz[0]), kEps);
      if (c > 0) {
        if (etid == 0) tma_store_wait_read<0>();
        if (!epi_sync(&bars[kBarEpi], epi_phase)) { tc_fail(10); ok = false; break; }
      }
      unsigned char* orow = sm + kOffOut + row * 128;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        uint4 val;
        val.x = pack_half2(__uint_as_float(nn[ch * 8 + 0]) * inv, __uint_as_float(nn[ch * 8 + 1]) * inv);
        val.y = pack_half2(__uint_as_float(nn[ch * 8 + 2]) * inv, __uint_as_float(nn[ch * 8 + 3]) * inv);
        val.z = pack_half2(__uint_as_float(nn[ch * 8 + 4]) * inv, __uint_as_float(nn[ch * 8 + 5]) * inv);
        val.w = pack_half2(__uint_as_float(nn[ch * 8 + 6]) * inv, __uint_as_float(nn[ch * 8 + 7]) * inv);
        *reinterpret_cast<uint4*>(orow + ((ch ^ (row & 7)) << 4)) = val;
      }
      fence_async_smem();
      if (!epi_sync(&bars[kBarEpi], epi_phase)) { tc_fail(11); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(&tm_o, sm + kOffOut, 0, bh, (int)(t_begin + (int64_t)c * kTC));
        tma_store_commit();
      }
    }
    // ---- final state out (prefill -> decode hand-off, segment carry)
    if (ok && s_out && seg == nseg - 1) {
      if (nchunk == 0) {
        for (int n = 0; n < kD; ++n) s_out[((size_t)bh * kK + row) * kD + n] = s_in ? s_in[(size_t)row * kD + n] : 0.f;
        z_out[(size_t)bh * kK + row] = z_in ? z_in[row] : 0.f;
      } else {
        // the last chunk's kBarS wait above already ordered the final state
        for (int c0 = 0; c0 < 80; c0 += 16) {
          uint32_t r[16];
          tmem_ld16(tmem + lane_addr + kColS + c0, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int n = c0 + i;
            if (n < kD) s_out[((size_t)bh * kK + row) * kD + n] = __uint_as_float(r[i]);
            else if (n == kD) z_out[(size_t)bh * kK + row] = __uint_as_float(r[i]);
          }
        }
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
int launch_causal_fwd_tc(const __half* q, const __half* k, const __half* v, __half* out, const float* s_seg,
                         const float* z_seg, float* s_out, float* z_out, int64_t T, int BH, int nseg, int64_t tseg,
                         cudaStream_t st) {
  CUtensorMap tq, tk, tv, to;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&to, out, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "causal_fwd: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_fwd: cannot reserve %u bytes of shared memory: %s", kTcSmem, cudaGetErrorString(e));
  causal_fwd_tc_kernel<<<dim3(BH, nseg), kTcThreads, kTcSmem, st>>>(tq, tk, tv, to, s_seg, z_seg, s_out, z_out, T, BH, nseg, tseg);
  return check_launch("rfa_causal_fwd");
}

int tc_status_causal_fwd() { return tc_status_read_clear(); }

}  // namespace rfa
