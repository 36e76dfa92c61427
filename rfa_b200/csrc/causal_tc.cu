// Causal RFA forward on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// One CTA walks one (batch, head[, segment]) in chunks of C = 128 tokens.  Per chunk
// (Q, K: [C][128] fp16; V: [C][64] fp16; [S|z]: running [128][64+1] state, fp32 in TMEM):
//     A   = Q K^T                      tcgen05.mma  M128 N128 K128   (smem x smem -> TMEM)
//     N   = Q [S|z]_prev               tcgen05.mma  M128 N80  K128   (smem x smem; state tile MN-major)
//     P   = mask(A) as fp16, row sums  score warps: TMEM -> registers -> TMEM (over A)
//     N  += P V                        tcgen05.mma  M128 N64  K128   (TMEM x smem)
//     [S|z] += K^T [V|1]               tcgen05.mma  M128 N80  K128   (smem x smem)
//     out = N[:, :64] / max(rowsum + N[:, 64], 1)
// The fp32 state never leaves TMEM; its fp16 copy ([128 k][64 + 16] in two swizzled boxes)
// is re-exported to shared memory once per chunk as the B operand of the next chunk.
//
// Warp roles (352 threads): warp 0 = TMA producer, warps 1 and 10 = MMA issuers (A: scores and P V,
// B: Q [S|z] and the state update -- issuing one tcgen05.mma costs the issuing thread about as long as
// the tensor pipe needs to execute it, so a single issuer cannot keep the pipe fed), warps 2..5 = score
// group (A -> P), warps 6..9 = output/state group (N -> out, state export).  Within a group
// thread <-> TMEM lane <-> token row / state row.  Two shared-memory stages of Q, K, V; two
// TMEM buffers each for A/P and N, so the score group works one chunk ahead of the output
// group.  The only per-chunk serial chain is  state MMA -> state export -> next state MMA.
// All waits are bounded.
#include <type_traits>

#define RFA_TC_FAMILY 1
#include "tc_common.cuh"

namespace rfa {

constexpr int kFwThreads = 352;

// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kFwQ = 0, kFwK = 2 * kBox, kFwV = 4 * kBox, kFwStage = 5 * kBox;   // 81920 per stage
constexpr uint32_t kFwOnes = 2 * kFwStage;          // [128][64] box: logical column 0 = 1, rest 0
constexpr uint32_t kFwS = kFwOnes + kBox;           // state tile: box 0 = S [128 k][64 n], box 1 = [z | 0...]
constexpr uint32_t kFwOut = kFwS + 2 * kBox;        // [128][64] output staging for the TMA store
constexpr uint32_t kFwRs = kFwOut + kBox;           // fp32 [2][128] row sums handed from score to output group
constexpr uint32_t kFwBar = kFwRs + 1024;
constexpr uint32_t kFwSmem = kFwBar + 256 + 1024;   // + alignment slack

// TMEM columns
constexpr uint32_t fColA = 0;        // two buffers of 128
constexpr uint32_t fColN = 256;      // two buffers of 80
constexpr uint32_t fColS = 416;      // 80: S (64) | z | zeros

enum { fFull = 0, fEmpty = 2, fA = 4, fP = 6, fN = 8, fNFree = 10, fS = 12, fSt = 14, fY = 15, fFullV = 16, fEmptyV = 18, fNum = 20 };
// fS (per N buffer): issuer B's products of a chunk (Q [S|z] into the N buffer, the state update) are complete; waited
// on by issuer A (P V accumulates onto the N buffer) and by the output group (state export).
// fFull/fEmpty guard the Q and K tiles of a stage (free once the state MMA has read K), fFullV/fEmptyV its V tile
// (free once P V has run): the Q, K loads of chunk c+2 start while chunk c is still being finished.

__global__ void __launch_bounds__(kFwThreads, 1)
causal_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_o,
                     const float* __restrict__ s_seg, const float* __restrict__ z_seg,
                     float* __restrict__ s_out, float* __restrict__ z_out, float* __restrict__ den_out,
                     int64_t T, int BH, int nseg, int64_t tseg) {
  extern __shared__ unsigned char tc_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kFwBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + fNum);
  float* rs = reinterpret_cast<float*>(sm + kFwRs);
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
      mbar_init(&bars[fFull + i], 1);
      mbar_init(&bars[fEmpty + i], 2);        // one commit from each issuer
      mbar_init(&bars[fFullV + i], 1);
      mbar_init(&bars[fEmptyV + i], 2);
      mbar_init(&bars[fS + i], 1);
      mbar_init(&bars[fA + i], 1);
      mbar_init(&bars[fP + i], 128);
      mbar_init(&bars[fN + i], 1);
      mbar_init(&bars[fNFree + i], 128);
    }
    mbar_init(&bars[fSt], 128);
    mbar_init(&bars[fY], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_o);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // the ones box: row r is 128 bytes; logical column 0 lives in 16-byte chunk (r & 7)
  for (int i = tid; i < (int)(kBox / 16); i += kFwThreads) {
    const int r = i >> 3, c = i & 7;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (c == (r & 7)) val.x = 0x00003C00u;     // fp16 1.0 in the low half
    *reinterpret_cast<uint4*>(sm + kFwOnes + i * 16) = val;
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                   // everything above may overlap the tail of the previous kernel in the stream
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[fEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * kFwStage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        uint64_t* fb = &bars[fFull + st];
        mbar_arrive_expect_tx(fb, 4 * kBox);
        tma_load_3d(base + kFwQ, &tm_q, fb, 0, bh, t0);
        tma_load_3d(base + kFwQ + kBox, &tm_q, fb, 64, bh, t0);
        tma_load_3d(base + kFwK, &tm_k, fb, 0, bh, t0);
        tma_load_3d(base + kFwK + kBox, &tm_k, fb, 64, bh, t0);
        if (c >= 2 && !mbar_wait(&bars[fEmptyV + st], ((c >> 1) + 1) & 1)) { tc_fail(14); break; }
        mbar_arrive_expect_tx(&bars[fFullV + st], kBox);
        tma_load_3d(base + kFwV, &tm_v, &bars[fFullV + st], 0, bh, t0);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idA = umma_idesc_f16(128, 128, false, false);   // Q K^T
      constexpr uint32_t idQS = umma_idesc_f16(128, 80, false, true);    // Q [S|z]   (B MN-major)
      constexpr uint32_t idPV = umma_idesc_f16(128, 64, false, true);    // P V       (B MN-major)
      constexpr uint32_t idS = umma_idesc_f16(128, 80, true, true);      // K^T [V|1] (A, B MN-major)
      constexpr uint64_t kSt = kFwStage >> 4;
      const uint64_t dQ = umma_smem_desc(sbase + kFwQ, 0, 1024, kSwizzle128B);        // Q, K-major
      const uint64_t dK = umma_smem_desc(sbase + kFwK, 0, 1024, kSwizzle128B);        // K, K-major
      const uint64_t dKt = umma_smem_desc(sbase + kFwK, kBox, 1024, kSwizzle128B);    // K^T, MN-major
      const uint64_t dV = umma_smem_desc(sbase + kFwV, kBox, 1024, kSwizzle128B);     // V, MN-major (N = 64)
      // [V|1], MN-major (N = 80): the second 64-block is the ones box, at a different distance from each stage's V tile
      const uint64_t dW0 = umma_smem_desc(sbase + kFwV, kFwOnes - kFwV, 1024, kSwizzle128B);
      const uint64_t dW1 = umma_smem_desc(sbase + kFwStage + kFwV, kFwOnes - (kFwStage + kFwV), 1024, kSwizzle128B);
      const uint64_t dS = umma_smem_desc(sbase + kFwS, kBox, 1024, kSwizzle128B);     // state tile, MN-major (N = 80)
      if (warp == 1) {
        // ---- issuer A: scores of the next chunk as early as its Q, K are in; N += P V
        auto issue_A = [&](int c) {
          const int s2 = c & 1;
          umma_chain_ss<8, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + fColA + s2 * 128, dQ + s2 * kSt, dK + s2 * kSt, idA, 0);
          umma_commit(&bars[fA + s2]);
          umma_commit(&bars[fEmpty + s2]);       // this issuer's last read of the stage's Q and K
        };
        bool ok = true;
        if (nchunk > 0) {
          ok = mbar_wait(&bars[fFull + 0], 0);
          if (ok) { tc_fence_after_sync(); issue_A(0); } else tc_fail(2);
        }
#pragma unroll 1
        for (int c = 0; ok && c < nchunk; ++c) {
          const int st = c & 1;
          bool next_issued = (c + 1 >= nchunk);
          if (!next_issued && mbar_test(&bars[fFull + (st ^ 1)], ((c + 1) >> 1) & 1)) {
            tc_fence_after_sync();
            issue_A(c + 1);
            next_issued = true;
          }
          if (!mbar_wait(&bars[fP + st], (c >> 1) & 1)) { tc_fail(6); break; }
          if (!mbar_wait(&bars[fS + st], (c >> 1) & 1)) { tc_fail(16); break; }     // Q [S|z] has written the N buffer
          tc_fence_after_sync();
          umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + fColN + st * 80, tmem + fColA + st * 128, dV + st * kSt, idPV, 1);   // N += P V
          umma_commit(&bars[fN + st]);
          umma_commit(&bars[fEmptyV + st]);
          if (!next_issued) {
            if (!mbar_wait(&bars[fFull + (st ^ 1)], ((c + 1) >> 1) & 1)) { tc_fail(5); break; }
            tc_fence_after_sync();
            issue_A(c + 1);
          }
        }
      } else {
        // ---- issuer B: N = Q [S|z]_prev  and  [S|z] += K^T [V|1]
#pragma unroll 1
        for (int c = 0; c < nchunk; ++c) {
          const int st = c & 1;
          const uint64_t so = (uint64_t)st * kSt;
          const uint64_t w = st ? dW1 : dW0;
          // the state before this chunk is in the operand tile, and the output group has let go of S and of the N buffer
          if (!mbar_wait(&bars[fSt], c & 1)) { tc_fail(3); break; }
          if (c >= 2 && !mbar_wait(&bars[fNFree + st], ((c >> 1) + 1) & 1)) { tc_fail(4); break; }
          if (!mbar_wait(&bars[fFull + st], (c >> 1) & 1)) { tc_fail(17); break; }
          if (!mbar_wait(&bars[fFullV + st], (c >> 1) & 1)) { tc_fail(15); break; }
          tc_fence_after_sync();
          const uint32_t fresh_acc = (c == 0 && s_in == nullptr) ? 0u : 1u;
          umma_chain_ss<8, kStepK, kBlockK, kStepMN, kBlockMN>(lead, tmem + fColN + st * 80, dQ + so, dS, idQS, 0);
          umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + fColS, dKt + so, w, idS, fresh_acc);
          umma_commit(&bars[fS + st]);
          umma_commit(&bars[fEmpty + st]);       // this issuer's last read of the stage's Q and K ...
          umma_commit(&bars[fEmptyV + st]);      // ... and of its V
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ score group: P = mask(A), row sums
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t colA = fColA + st * 128;
      if (!mbar_wait(&bars[fA + st], (c >> 1) & 1)) { tc_fail(7); break; }
      // rs[st] of chunk c-2 must have been read by the output group
      if (c >= 2 && !mbar_wait(&bars[fNFree + st], ((c >> 1) + 1) & 1)) { tc_fail(8); break; }
      tc_fence_after_sync();
      float rowsum = 0.f, rowsum_b = 0.f;
      // 32-column pieces left of the diagonal one need no mask, the diagonal one keeps columns <= lane, the rest are zero
      auto pack_piece = [&](int piece, auto DIAG) {
        constexpr bool diag = decltype(DIAG)::value;
        uint32_t a[32], p[16];
        tmem_ld32(tmem + lane_addr + colA + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = __uint_as_float(a[i]), x1 = __uint_as_float(a[i + 1]);
          if (diag) {
            if (i > lane) x0 = 0.f;
            if (i + 1 > lane) x1 = 0.f;
          }
          if (i & 2) rowsum_b += x0 + x1; else rowsum += x0 + x1;
          p[i >> 1] = pack_half2(x0, x1);
        }
        tmem_st16(tmem + lane_addr + colA + piece * 16, p);
      };
#pragma unroll 1
      for (int piece = 0; piece < quarter; ++piece) pack_piece(piece, std::false_type{});
      pack_piece(quarter, std::true_type{});
      {
        uint32_t zero[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) zero[i] = 0u;
#pragma unroll 1
        for (int piece = quarter + 1; piece < 4; ++piece) tmem_st16(tmem + lane_addr + colA + piece * 16, zero);
      }
      rs[st * 128 + row] = rowsum + rowsum_b;
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[fP + st]);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ output / state group
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // token row in the chunk / state row k
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int ytid = tid - 192;                   // 0..127
    unsigned char* s_tile = sm + kFwS;
    // state entering this run of tokens -> TMEM (fp32) and the fp16 operand tile
    {
      uint32_t r[80];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
      r[64] = z_in ? __float_as_uint(z_in[row]) : 0u;
#pragma unroll
      for (int n = 65; n < 80; ++n) r[n] = 0u;
      store_state_row(s_tile, row, r);
#pragma unroll
      for (int ch = 1; ch < 8; ++ch) *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, ch)) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, 0)) = make_uint4(pack_half2(__uint_as_float(r[64]), 0.f), 0, 0, 0);
      if (s_in) {
#pragma unroll
        for (int c0 = 0; c0 < 80; c0 += 16) tmem_st16(tmem + lane_addr + fColS + c0, r + c0);
        tmem_st_wait();
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[fSt]);
    }
    bool ok = true;
    uint32_t y_phase = 0;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      // ---- the state after this chunk -> operand tile for the next chunk (the serial chain of the scan)
      if (!mbar_wait(&bars[fS + st], (c >> 1) & 1)) { tc_fail(9); ok = false; break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        uint32_t r[80];
        tmem_ld32(tmem + lane_addr + fColS, r);
        tmem_ld32(tmem + lane_addr + fColS + 32, r + 32);
        tmem_ld16(tmem + lane_addr + fColS + 64, r + 64);
        tmem_ld_wait();
        store_state_row(s_tile, row, r);
        *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, 0)) = make_uint4(pack_half2(__uint_as_float(r[64]), 0.f), 0, 0, 0);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[fSt]);
      }
      // ---- N: numerator (64 columns) and q.z_prev (column 64); row sum from the score group
      if (!mbar_wait(&bars[fP + st], (c >> 1) & 1)) { tc_fail(10); ok = false; break; }
      if (!mbar_wait(&bars[fN + st], (c >> 1) & 1)) { tc_fail(11); ok = false; break; }
      tc_fence_after_sync();
      uint32_t nn[64], nz[16];
      tmem_ld32(tmem + lane_addr + fColN + st * 80, nn);
      tmem_ld32(tmem + lane_addr + fColN + st * 80 + 32, nn + 32);
      tmem_ld16(tmem + lane_addr + fColN + st * 80 + 64, nz);
      const float rowsum = rs[st * 128 + row];
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[fNFree + st]);
      // ---- out = N / max(rowsum + q.z_prev, 1) -> staging tile -> TMA store
      const float raw = rowsum + __uint_as_float(nz[0]);
      const float inv = 1.f / fmaxf(raw, kEps);
      if (den_out) {                               // the raw denominators [BH][T], kept for a backward that does not recompute them
        const int64_t t = t_begin + (int64_t)c * kTC + row;
        if (t < t_end) den_out[(size_t)bh * T + t] = raw;
      }
      if (c > 0) {                                 // the previous chunk's store must have drained the staging tile
        if (ytid == 0) tma_store_wait_read<0>();
        if (!epi_sync(&bars[fY], y_phase)) { tc_fail(13); ok = false; break; }
      }
      unsigned char* orow = sm + kFwOut + row * 128;
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
      if (!epi_sync(&bars[fY], y_phase)) { tc_fail(12); ok = false; break; }
      if (ytid == 0) {
        tma_store_3d(&tm_o, sm + kFwOut, 0, bh, (int)(t_begin + (int64_t)c * kTC));
        tma_store_commit();
      }
    }
    // ---- final state out (prefill -> decode hand-off, segment carry); the last wait on fS ordered it
    if (ok && s_out && seg == nseg - 1) {
      uint32_t r[80];
      if (nchunk > 0) {
        tmem_ld32(tmem + lane_addr + fColS, r);
        tmem_ld32(tmem + lane_addr + fColS + 32, r + 32);
        tmem_ld16(tmem + lane_addr + fColS + 64, r + 64);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
        r[64] = z_in ? __float_as_uint(z_in[row]) : 0u;
      }
      float4* dst = reinterpret_cast<float4*>(s_out + ((size_t)bh * kK + row) * kD);
#pragma unroll
      for (int n = 0; n < 16; ++n)
        dst[n] = make_float4(__uint_as_float(r[4 * n]), __uint_as_float(r[4 * n + 1]), __uint_as_float(r[4 * n + 2]),
                             __uint_as_float(r[4 * n + 3]));
      z_out[(size_t)bh * kK + row] = __uint_as_float(r[64]);
    }
    if (ytid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
int launch_causal_fwd_tc(const __half* q, const __half* k, const __half* v, __half* out, const float* s_seg,
                         const float* z_seg, float* s_out, float* z_out, float* den_out, int64_t T, int BH, int nseg,
                         int64_t tseg, cudaStream_t st) {
  CUtensorMap tq, tk, tv, to;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&to, out, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "causal_fwd: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFwSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_fwd: cannot reserve %u bytes of shared memory: %s", kFwSmem, cudaGetErrorString(e));
  launch_pdl(causal_fwd_tc_kernel, dim3(BH, nseg), dim3(kFwThreads), kFwSmem, st, tq, tk, tv, to, s_seg, z_seg, s_out, z_out, den_out, T, BH, nseg, tseg);
  return check_launch("rfa_causal_fwd");
}

RFA_TC_UNIT(causal_fwd)

}  // namespace rfa
