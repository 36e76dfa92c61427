// Causal RFA backward, sweep 2 (reverse in time) on tcgen05 tensor cores: grad_k, grad_v
// (upstream cuda/backward.cu:373-451, kv_backward; math in rfa.py:96-101), chunks of 128 tokens.
//
// Per chunk, with gs = g/den and gz from sweep 1 (workspace), dS/dz the reverse running state:
//     At  = K Q^T        -> Pt  = At[s][t]  for t >= s            fp16, kept in TMEM
//     dAt = V gs^T       -> (dAt + gz_t)[s][t] for t >= s         fp16, kept in TMEM
//     dV  = Pt gs + K dS                                  -> grad_v
//     dK  = dAt Q + V dS^T + dz^T                         -> grad_k
//     dS += Q^T gs,   dz += Q^T gz
// The score matrices are computed TRANSPOSED (keys on the TMEM lanes) so that their fp16
// versions can stay in tensor memory as the A operands of the dK / dV products.
//
// Warp roles (480 threads): warp 0 TMA producer, warps 1 and 10 MMA issuers, warps 2..5 score/state group (packs Pt,
// then the scan's serial step: exports the reverse state, dz += Q^T gz), warps 11..14 score group 2 (scales g in
// place, packs dAt), warps 6..9 output group (grad_v, grad_k straight from registers).  Issuing one tcgen05.mma costs
// the issuing thread about as long as the tensor pipe needs to execute it (N <= 128), so the 48 MMAs of a chunk are
// split over two issuers: A (At, dAt, dK) and B (dV, dS).  The products that read the exported state tile are issued
// first in a chunk and the state update right after g is scaled, which keeps the serial chain of the scan (state MMA
// -> export -> next chunk's readers) short.  The gradients leave through plain 32-byte global stores: a stage is then
// free for its next load as soon as the chunk's products are complete, instead of serving as the staging area of a
// TMA store first (a load under full memory traffic takes about 3 us here, as long as a whole chunk, so what delays
// its issue delays the chunk).  All waits are bounded.
#include <type_traits>

#define RFA_TC_FAMILY 3
#include "tc_common.cuh"

namespace rfa {

constexpr int kKvThreads = 480;

constexpr uint32_t kvQ = 0, kvK = 2 * kBox, kvV = 4 * kBox, kvG = 5 * kBox, kvStage = 6 * kBox;   // 98304 per stage
constexpr uint32_t kvS = 2 * kvStage;            // dS as an operand: [128 k][64 n] fp16, swizzled
constexpr uint32_t kvDz = kvS + kBox;            // fp32 [3][128]: dz entering chunk i lives in buffer i % 3
constexpr uint32_t kvGz = kvDz + 1536;           // fp32 [2][128]: gz of the chunk's query rows
constexpr uint32_t kvBar = kvGz + 1024;
constexpr uint32_t kvSmem = kvBar + 256 + 1024;

constexpr uint32_t kvColAt = 0, kvColDAt = 128, kvColDK = 256, kvColDV = 384, kvColDS = 448;
enum { vFullKQ = 0, vFullVG = 2, vEmpty = 4, vAt = 6, vG = 7, vDAt = 9, vP = 10, vDA16 = 11, vDK = 12, vDV = 13, vDKFree = 14,
       vDVFree = 15, vS = 16, vSt = 17, vSR = 18, vDz = 19, vNum = 22 };
// vFullKQ / vFullVG: the K, Q tiles and the V, g tiles of a stage have landed (requested in the order g, V, K, Q).
// vSR: both issuers have finished reading the exported state tile (one commit each per chunk).
// vEmpty: a stage may be refilled: both issuers' last products of the chunk are complete and dz has been summed over Q.
// vG is one barrier per stage and vDz one per buffer (i % 3): their waiters may reach them late, when the producer
// could already have completed the same barrier's next phase; kept apart, a waiter is never two phases behind.

__global__ void __launch_bounds__(kKvThreads, 1)
causal_bwd_kv_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                        __half* __restrict__ gk_ptr, __half* __restrict__ gv_ptr,
                        const float* __restrict__ ws_den, const float* __restrict__ ws_gz,
                        const float* __restrict__ ds_seg, const float* __restrict__ dz_seg,
                        int64_t T, int BH, int nseg, int64_t tseg) {
  extern __shared__ unsigned char kv_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(kv_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kvBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + vNum);
  float* dzs = reinterpret_cast<float*>(sm + kvDz);
  float* gz_buf = reinterpret_cast<float*>(sm + kvGz);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  const int nchunk = (int)((t_end - t_begin + kTC - 1) / kTC);
  const size_t slot = (size_t)bh * nseg + seg;
  const float* ds_in = ds_seg ? ds_seg + slot * kK * kD : nullptr;
  const float* dz_in = dz_seg ? dz_seg + slot * kK : nullptr;

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[vFullKQ + i], 1); mbar_init(&bars[vFullVG + i], 1);
      mbar_init(&bars[vEmpty + i], 130);     // one commit from each issuer + the score/state group's column sums over Q
      mbar_init(&bars[vG + i], 128);
    }
    mbar_init(&bars[vAt], 1); mbar_init(&bars[vDAt], 1); mbar_init(&bars[vP], 128);
    mbar_init(&bars[vDA16], 128); mbar_init(&bars[vDK], 1); mbar_init(&bars[vDV], 1);
    mbar_init(&bars[vDKFree], 128); mbar_init(&bars[vDVFree], 128); mbar_init(&bars[vS], 1);
    mbar_init(&bars[vSt], 128); mbar_init(&bars[vSR], 2);
    for (int i = 0; i < 3; ++i) mbar_init(&bars[vDz + i], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_g);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;
  pdl_wait();                   // everything above may overlap the tail of the previous kernel in the stream
  pdl_launch_dependents();

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (chunks in reverse time order)
    if (lane == 0) {
      for (int i = 0; i < nchunk; ++i) {
        const int st = i & 1;
        unsigned char* base = sm + st * kvStage;
        const int t0 = (int)(t_begin + (int64_t)(nchunk - 1 - i) * kTC);
        if (i >= 2 && !mbar_wait(&bars[vEmpty + st], ((i >> 1) + 1) & 1)) { tc_fail(1); break; }
        uint64_t* fv = &bars[vFullVG + st];
        uint64_t* fk = &bars[vFullKQ + st];
        mbar_arrive_expect_tx(fv, 2 * kBox);           // g first: the longer of the chunk's two chains starts with its scaling
        tma_load_3d(base + kvG, &tm_g, fv, 0, bh, t0);
        tma_load_3d(base + kvV, &tm_v, fv, 0, bh, t0);
        mbar_arrive_expect_tx(fk, 4 * kBox);
        tma_load_3d(base + kvK, &tm_k, fk, 0, bh, t0);
        tma_load_3d(base + kvK + kBox, &tm_k, fk, 64, bh, t0);
        tma_load_3d(base + kvQ, &tm_q, fk, 0, bh, t0);
        tma_load_3d(base + kvQ + kBox, &tm_q, fk, 64, bh, t0);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idKK = umma_idesc_f16(128, 128, false, false);   // K Q^T ; V gs^T ; V dS^T
      constexpr uint32_t idKM128 = umma_idesc_f16(128, 128, false, true); // dAt Q            (B MN-major)
      constexpr uint32_t idKM64 = umma_idesc_f16(128, 64, false, true);   // Pt gs ; K dS     (B MN-major)
      constexpr uint32_t idMM64 = umma_idesc_f16(128, 64, true, true);    // Q^T gs           (A, B MN-major)
      // operand descriptors of stage 0; the other stage is a constant add on the start-address field
      const uint64_t dQk = umma_smem_desc(sbase + kvQ, 0, 1024, kSwizzle128B);       // Q  K-major  [t][k]
      const uint64_t dQm = umma_smem_desc(sbase + kvQ, kBox, 1024, kSwizzle128B);    // Q  MN-major (rows = contraction t)
      const uint64_t dKk = umma_smem_desc(sbase + kvK, 0, 1024, kSwizzle128B);       // K  K-major  [s][k]
      const uint64_t dVk = umma_smem_desc(sbase + kvV, 0, 1024, kSwizzle128B);       // V  K-major  [s][n]
      const uint64_t dGk = umma_smem_desc(sbase + kvG, 0, 1024, kSwizzle128B);       // gs K-major  [t][n]
      const uint64_t dGm = umma_smem_desc(sbase + kvG, kBox, 1024, kSwizzle128B);    // gs MN-major (rows = contraction t)
      constexpr uint64_t dStage = kvStage >> 4;
      const uint64_t dSk = umma_smem_desc(sbase + kvS, 0, 1024, kSwizzle128B);      // dS as [N = k rows][K = n]
      const uint64_t dSm = umma_smem_desc(sbase + kvS, kBox, 1024, kSwizzle128B);   // dS as [K = k rows][N = n]
      if (warp == 1) {
        // ---- issuer A: At (scores of the next chunk), dAt, dK
        auto issue_At = [&](int s2) {                                     // At = K Q^T
          umma_chain_ss<8, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + kvColAt, dKk + s2 * dStage, dQk + s2 * dStage, idKK, 0);
          umma_commit(&bars[vAt]);
        };
        bool ok = true;
        if (nchunk > 0) {
          ok = mbar_wait(&bars[vFullKQ], 0);
          if (ok) { tc_fence_after_sync(); issue_At(0); } else tc_fail(2);
        }
#pragma unroll 1
        for (int i = 0; ok && i < nchunk; ++i) {
          const int st = i & 1;
          const uint64_t so = (uint64_t)st * dStage;
          const uint32_t ph = i & 1;
          // dAt = V gs^T first: it heads the chunk's longest chain (dAt -> pack -> dK += dAt Q)
          if (!mbar_wait(&bars[vFullVG + st], (i >> 1) & 1)) { tc_fail(9); break; }
          if (!mbar_wait(&bars[vG + st], (i >> 1) & 1)) { tc_fail(5); break; }
          tc_fence_after_sync();
          umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + kvColDAt, dVk + so, dGk + so, idKK, 0);          // dAt = V gs^T
          umma_commit(&bars[vDAt]);
          // dK = V dS_next^T: it reads the state tile, which the score/state group overwrites once both issuers are done
          // with it, and it needs the output group to have drained the previous chunk's dK
          if (!mbar_wait(&bars[vSt], ph)) { tc_fail(3); break; }
          if (i > 0 && !mbar_wait(&bars[vDKFree], (i - 1) & 1)) { tc_fail(4); break; }
          tc_fence_after_sync();
          umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + kvColDK, dVk + so, dSk, idKK, 0);
          umma_commit(&bars[vSR]);
          // the next chunk's scores as soon as its tiles are in and Pt of this chunk has been consumed (dV complete)
          bool next_issued = (i + 1 >= nchunk);
          if (!next_issued && mbar_test(&bars[vFullKQ + (st ^ 1)], ((i + 1) >> 1) & 1) && mbar_test(&bars[vDV], ph)) {
            tc_fence_after_sync();
            issue_At(st ^ 1);
            next_issued = true;
          }
          if (!mbar_wait(&bars[vDA16], ph)) { tc_fail(6); break; }
          tc_fence_after_sync();
          umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + kvColDK, tmem + kvColDAt, dQm + so, idKM128, 1);                // dK += dAt Q
          umma_commit(&bars[vDK]);
          umma_commit(&bars[vEmpty + st]);           // this issuer's last product that reads the stage
          if (!next_issued) {
            if (!mbar_wait(&bars[vFullKQ + (st ^ 1)], ((i + 1) >> 1) & 1)) { tc_fail(7); break; }
            if (!mbar_wait(&bars[vDV], ph)) { tc_fail(8); break; }
            tc_fence_after_sync();
            issue_At(st ^ 1);
          }
        }
      } else {
        // ---- issuer B: dV and the state update
#pragma unroll 1
        for (int i = 0; i < nchunk; ++i) {
          const int st = i & 1;
          const uint64_t so = (uint64_t)st * dStage;
          const uint32_t ph = i & 1;
          if (!mbar_wait(&bars[vFullKQ + st], (i >> 1) & 1)) { tc_fail(20); break; }
          if (!mbar_wait(&bars[vSt], ph)) { tc_fail(21); break; }
          if (i > 0 && !mbar_wait(&bars[vDVFree], (i - 1) & 1)) { tc_fail(22); break; }
          tc_fence_after_sync();
          umma_chain_ss<8, kStepK, kBlockK, kStepMN, kBlockMN>(lead, tmem + kvColDV, dKk + so, dSm, idKM64, 0);           // dV = K dS_next
          umma_commit(&bars[vSR]);
          if (!mbar_wait(&bars[vG + st], (i >> 1) & 1)) { tc_fail(23); break; }
          tc_fence_after_sync();
          const bool fresh = (i == 0 && ds_in == nullptr);
          umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + kvColDS, dQm + so, dGm + so, idMM64, fresh ? 0u : 1u);   // dS += Q^T gs
          umma_commit(&bars[vS]);
          if (!mbar_wait(&bars[vP], ph)) { tc_fail(24); break; }
          tc_fence_after_sync();
          umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + kvColDV, tmem + kvColAt, dGm + so, idKM64, 1);                  // dV += Pt gs
          umma_commit(&bars[vDV]);
          umma_commit(&bars[vEmpty + st]);           // this issuer's last product that reads the stage
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ score/state group: Pt[s][t] = At[s][t] for t >= s;
    //                                                                     reverse state export; dz += Q^T gz
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // key row s of the chunk / state row k
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    unsigned char* s_tile = sm + kvS;
    {   // the reverse state entering this run of tokens -> TMEM (fp32) and the operand tile; dz version 0
      uint32_t r[64];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = ds_in ? __float_as_uint(ds_in[(size_t)row * kD + n]) : 0u;
      store_state_row(s_tile, row, r);
      if (ds_in) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) tmem_st16(tmem + lane_addr + kvColDS + c0, r + c0);
        tmem_st_wait();
      }
      dzs[row] = dz_in ? dz_in[row] : 0.f;
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[vSt]);
      mbar_arrive(&bars[vDz + 0]);
    }
    float dz_run = dz_in ? dz_in[row] : 0.f;       // dz[row] entering the current chunk
    for (int i = 0; i < nchunk; ++i) {
      const uint32_t ph = i & 1;
      if (!mbar_wait(&bars[vAt], ph)) { tc_fail(11); break; }
      tc_fence_after_sync();
      // 32-column pieces right of the diagonal one need no mask, the diagonal one keeps columns >= lane, the rest are zero
      auto pack_piece = [&](int piece, auto DIAG) {
        constexpr bool diag = decltype(DIAG)::value;
        uint32_t a[32], p[16];
        tmem_ld32(tmem + lane_addr + kvColAt + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
          float x0 = __uint_as_float(a[e]), x1 = __uint_as_float(a[e + 1]);
          if (diag) {
            if (e < lane) x0 = 0.f;
            if (e + 1 < lane) x1 = 0.f;
          }
          p[e >> 1] = pack_half2(x0, x1);
        }
        tmem_st16(tmem + lane_addr + kvColAt + piece * 16, p);
      };
      {
        uint32_t zero[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) zero[e] = 0u;
#pragma unroll 1
        for (int piece = 0; piece < quarter; ++piece) tmem_st16(tmem + lane_addr + kvColAt + piece * 16, zero);
      }
      pack_piece(quarter, std::true_type{});
#pragma unroll 1
      for (int piece = quarter + 1; piece < 4; ++piece) pack_piece(piece, std::false_type{});
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[vP]);
      // ---- the state update is complete and both issuers have finished reading the old state tile: reverse state
      //      after this chunk -> fp16 operand tile (the serial chain of the scan)
      const int st = i & 1;
      if (!mbar_wait(&bars[vS], ph)) { tc_fail(15); break; }
      if (!mbar_wait(&bars[vSR], ph)) { tc_fail(18); break; }
      tc_fence_after_sync();
      if (i + 1 < nchunk) {
        uint32_t r[64];
        tmem_ld32(tmem + lane_addr + kvColDS, r);
        tmem_ld32(tmem + lane_addr + kvColDS + 32, r + 32);
        tmem_ld_wait();
        store_state_row(s_tile, row, r);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[vSt]);
      }
      // ---- dz entering the next chunk = dz + Q^T gz (gz of every row is there once vG completed; the state update
      //      waited on it).  Buffer (i + 1) % 3 last held version i - 2, which the output group read in its iteration
      //      i - 2, before it released dV of chunk i - 1, which precedes this chunk's state update.
      if (!mbar_wait(&bars[vFullKQ + st], (i >> 1) & 1)) { tc_fail(16); break; }
      if (!mbar_wait(&bars[vG + st], (i >> 1) & 1)) { tc_fail(17); break; }
      dz_run += column_sum2(sm + st * kvStage + kvQ, quarter, lane, gz_buf + st * 128);
      mbar_arrive(&bars[vEmpty + st]);             // this group's last read of the stage's tiles
      dzs[((i + 1) % 3) * 128 + row] = dz_run;
      mbar_arrive(&bars[vDz + (i + 1) % 3]);
    }
  } else if (warp >= 11) {
    // ------------------------------------------------------------------ score group 2: gs = g / den, then dAt
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // query row t (scaling g) / key row s (packing)
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    // this thread's two per-token scalars from sweep 1, fetched one chunk ahead: a load from global memory takes about
    // as long as half a chunk under full traffic, and the scaling of g heads the chunk's longest chain
    float den_next = 1.f, gz_next = 0.f;
    auto fetch = [&](int i) {
      const int64_t t = t_begin + (int64_t)(nchunk - 1 - i) * kTC + row;
      if (i < nchunk && t < t_end) {
        den_next = __ldg(ws_den + (size_t)bh * T + t);
        gz_next = __ldg(ws_gz + (size_t)bh * T + t);
      } else {
        den_next = 1.f;
        gz_next = 0.f;
      }
    };
    fetch(0);
    for (int i = 0; i < nchunk; ++i) {
      const int st = i & 1;
      const uint32_t ph = i & 1;
      unsigned char* stage = sm + st * kvStage;
      float* gzs = gz_buf + (i & 1) * 128;
      // ---- gs = g / den over the staged g tile; gz of this thread's query row
      const float inv = 1.f / fmaxf(den_next, kEps);       // raw or already clamped denominators
      const float gz = gz_next;
      if (!mbar_wait(&bars[vFullVG + st], (i >> 1) & 1)) { tc_fail(10); break; }
      {
        unsigned char* grow = stage + kvG;
        // all eight loads of the row first (independent), then the scaling, then the stores
        uint4 gu[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) gu[ch] = *reinterpret_cast<const uint4*>(grow + row_chunk1(row, ch));
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 u = gu[ch];
          float2 f0 = unpack_half2(u.x), f1 = unpack_half2(u.y), f2 = unpack_half2(u.z), f3 = unpack_half2(u.w);
          gu[ch].x = pack_half2(f0.x * inv, f0.y * inv); gu[ch].y = pack_half2(f1.x * inv, f1.y * inv);
          gu[ch].z = pack_half2(f2.x * inv, f2.y * inv); gu[ch].w = pack_half2(f3.x * inv, f3.y * inv);
        }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(grow + row_chunk1(row, ch)) = gu[ch];
        gzs[row] = gz;
      }
      fence_async_smem();
      mbar_arrive(&bars[vG + st]);
      fetch(i + 1);
      // ---- dAt[s][t] = (v_s . gs_t + gz_t) for t >= s; gz of all rows is there once vG completed
      if (!mbar_wait(&bars[vG + st], (i >> 1) & 1)) { tc_fail(12); break; }
      if (!mbar_wait(&bars[vDAt], ph)) { tc_fail(13); break; }
      tc_fence_after_sync();
      auto pack_da = [&](int piece, auto DIAG) {
        constexpr bool diag = decltype(DIAG)::value;
        uint32_t a[32], p[16];
        tmem_ld32(tmem + lane_addr + kvColDAt + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 gz4 = *reinterpret_cast<const float4*>(gzs + piece * 32 + e);
          float x0 = __uint_as_float(a[e]) + gz4.x, x1 = __uint_as_float(a[e + 1]) + gz4.y;
          float x2 = __uint_as_float(a[e + 2]) + gz4.z, x3 = __uint_as_float(a[e + 3]) + gz4.w;
          if (diag) {
            if (e < lane) x0 = 0.f;
            if (e + 1 < lane) x1 = 0.f;
            if (e + 2 < lane) x2 = 0.f;
            if (e + 3 < lane) x3 = 0.f;
          }
          p[e >> 1] = pack_half2(x0, x1);
          p[(e >> 1) + 1] = pack_half2(x2, x3);
        }
        tmem_st16(tmem + lane_addr + kvColDAt + piece * 16, p);
      };
      {
        uint32_t zero[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) zero[e] = 0u;
#pragma unroll 1
        for (int piece = 0; piece < quarter; ++piece) tmem_st16(tmem + lane_addr + kvColDAt + piece * 16, zero);
      }
      pack_da(quarter, std::true_type{});
#pragma unroll 1
      for (int piece = quarter + 1; piece < 4; ++piece) pack_da(piece, std::false_type{});
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[vDA16]);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ output group: grad_v, grad_k
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // key row s of the chunk
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int i = 0; i < nchunk; ++i) {
      const uint32_t ph = i & 1;
      const int64_t t0 = t_begin + (int64_t)(nchunk - 1 - i) * kTC;
      const bool live = t0 + row < t_end;
      const float* dz_cur = dzs + (i % 3) * 128;
      // ---- grad_v: issuer B's last product of the chunk
      {
        uint32_t r[64];
        if (!mbar_wait(&bars[vDV], ph)) { tc_fail(13); break; }
        tc_fence_after_sync();
        tmem_ld32(tmem + lane_addr + kvColDV, r);
        tmem_ld32(tmem + lane_addr + kvColDV + 32, r + 32);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(&bars[vDVFree]);
        __half* vrow = gv_ptr + ((size_t)(t0 + row) * BH + bh) * kD;
#pragma unroll
        for (int j = 0; j < 4; ++j) {              // 32 bytes (one sector) per store
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o[e] = pack_half2(__uint_as_float(r[j * 16 + 2 * e]), __uint_as_float(r[j * 16 + 2 * e + 1]));
          if (live) st_global_v8(vrow + j * 16, o);
        }
      }
      // ---- grad_k = dK + dz (dz entering this chunk): issuer A's last product
      if (!mbar_wait(&bars[vDz + i % 3], (i / 3) & 1)) { tc_fail(14); break; }
      if (!mbar_wait(&bars[vDK], ph)) { tc_fail(19); break; }
      tc_fence_after_sync();
      __half* krow = gk_ptr + ((size_t)(t0 + row) * BH + bh) * kK;
#pragma unroll 1
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        float4 zv[8];
        tmem_ld32(tmem + lane_addr + kvColDK + piece * 32, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) zv[j] = *reinterpret_cast<const float4*>(dz_cur + piece * 32 + j * 4);
        tmem_ld_wait();
        // dK and this chunk's dz are in registers: the next chunk may overwrite dK (and, later, the dz buffer)
        if (piece == 3) { tc_fence_before_sync(); mbar_arrive(&bars[vDKFree]); }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int a0 = j * 16 + e * 8;
            const float4 z0 = zv[a0 / 4], z1 = zv[a0 / 4 + 1];
            o[e * 4 + 0] = pack_half2(__uint_as_float(a[a0 + 0]) + z0.x, __uint_as_float(a[a0 + 1]) + z0.y);
            o[e * 4 + 1] = pack_half2(__uint_as_float(a[a0 + 2]) + z0.z, __uint_as_float(a[a0 + 3]) + z0.w);
            o[e * 4 + 2] = pack_half2(__uint_as_float(a[a0 + 4]) + z1.x, __uint_as_float(a[a0 + 5]) + z1.y);
            o[e * 4 + 3] = pack_half2(__uint_as_float(a[a0 + 6]) + z1.z, __uint_as_float(a[a0 + 7]) + z1.w);
          }
          if (live) st_global_v8(krow + piece * 32 + j * 16, o);
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

int launch_causal_bwd_kv_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                            const float* ws_den, const float* ws_gz, const float* ds_seg, const float* dz_seg,
                            int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tg;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&tg, g, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "causal_bwd_kv: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_bwd_kv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kvSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_bwd_kv: cannot reserve %u bytes of shared memory: %s", kvSmem, cudaGetErrorString(e));
  launch_pdl(causal_bwd_kv_tc_kernel, dim3(BH, nseg), dim3(kKvThreads), kvSmem, st, tq, tk, tv, tg, gk, gv, ws_den, ws_gz, ds_seg, dz_seg,
                                                                     T, BH, nseg, tseg);
  return check_launch("rfa_causal_bwd_kv");
}

RFA_TC_UNIT(causal_bwd_kv)

}  // namespace rfa
