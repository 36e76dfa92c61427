// Causal RFA backward, sweep 1 (forward in time) on tcgen05 tensor cores: grad_q, plus the
// per-token scalars den and gz that sweep 2 needs (upstream cuda/backward.cu:303-371, q_backward;
// math in rfa.py:79-94), chunks of 128 tokens.
//
// Per chunk, with S/z the state of all earlier tokens:
//     A   = Q K^T              -> P = mask(A) fp16 (TMEM), rowsum
//     N   = P V + Q S          -> den = max(rowsum + q.z, 1), out = N/den
//     gs  = g/den (fp16, over the staged g tile),  gz = -(g.out)/den * [rowsum + q.z > 1]
//     dA  = gs V^T             -> mask(dA + gz) fp16 (TMEM, over P)
//     dQ  = gs S^T + dA K (+ gz z^T added in the epilogue)            -> grad_q
//     S  += K^T V,  z += colsum(K);   optionally  dSseg += Q^T gs, dzseg += Q^T gz
// S and dSseg are fp32 TMEM accumulators; z is fp32 in shared memory (CUDA-core update).
//
// Warp roles (480 threads): warp 0 TMA producer; warps 1 and 10 MMA issuers (A: scores and N, B: dA, dQ,
// state updates) -- issuing a tcgen05.mma costs the issuing thread about as long as the tensor pipe needs to
// execute it, so one issuer cannot keep the pipe fed; warps 2..5 score group 1 (P, row sums, q.z); warps
// 11..14 score group 2 (den/gz/gs, dA); warps 6..9 output/state group (grad_q, state export, z).  The score
// tile A/P/N/dA is double-buffered in TMEM, so score group 1 works on chunk c + 1 while score group 2 and the
// output group finish chunk c.  All waits are bounded.
#include <type_traits>

#define RFA_TC_FAMILY 2
#include "tc_common.cuh"

namespace rfa {

constexpr int kBqThreads = 480;

constexpr uint32_t bqQ = 0, bqK = 2 * kBox, bqV = 4 * kBox, bqG = 5 * kBox, bqStage = 6 * kBox;   // 98304 per stage
constexpr uint32_t bqS = 2 * bqStage;            // S as an operand: two tiles [128 k][64 n] fp16, swizzled; the state before
                                                 // chunk c is in tile c & 1, so the export after chunk c never waits for a reader
constexpr uint32_t bqZ = bqS + 2 * kBox;         // fp32 [3][128]: z before chunk c lives in buffer c % 3 (readers of version c,
                                                 // c + 1 and the writer of version c + 2 can be active at once)
constexpr uint32_t bqRg = bqZ + 1536;            // fp32 [2][128], buffer c & 1: row sum of P + q.z from score group 1, replaced
                                                 // in place by gz once score group 2 has consumed it
constexpr uint32_t bqBar = bqRg + 1024;
constexpr uint32_t bqSmem = bqBar + 256;         // every byte of the 227 KB is used: no slack to align the base, which the
                                                 // kernel therefore checks

// TMEM: two score buffers (A -> P in columns 0..63, N in columns 64..127, then dA -> fp16 dA in 0..63)
constexpr uint32_t bqColA = 0, bqColDQ = 256, bqColS = 384, bqColDS = 448;
enum { qFull = 0, qEmpty = 2, qA = 4, qP = 6, qN = 8, qG = 10, qDA = 12, qDA16 = 14, qZ = 16, qDQ = 18, qRS = 20, qSt = 22,
       qDQFree = 24, qS = 25, qFullV = 26, qNum = 28 };
// qFull guards the Q and K tiles of a stage, qFullV its V and g tiles, requested in that order: the scores start as soon
// as Q and K are in.
// Barriers that a waiter may reach late are kept per score buffer / stage (index c & 1), so that their producer
// cannot complete two phases before the waiter looks: qDQ has two waiters (the output group and issuer A, which
// reuses the score buffer), qRS hands (row sum, q.z) from score group 1 to score group 2.

__global__ void __launch_bounds__(kBqThreads, 1)
causal_bwd_q_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                       const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                       __half* __restrict__ gq_ptr,
                       const float* __restrict__ s_seg, const float* __restrict__ z_seg,
                       float* __restrict__ ws_den, float* __restrict__ ws_gz,
                       float* __restrict__ ds_seg, float* __restrict__ dz_seg,
                       int64_t T, int BH, int nseg, int64_t tseg) {
  extern __shared__ __align__(1024) unsigned char bq_raw[];
  unsigned char* sm = bq_raw;
  if (smem_u32(sm) & 1023u) {                    // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) tc_fail(99);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + bqBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + qNum);
  float* z_buf = reinterpret_cast<float*>(sm + bqZ);
  float* rg_buf = reinterpret_cast<float*>(sm + bqRg);
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
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[qFull + i], 1);
      mbar_init(&bars[qFullV + i], 1);
      mbar_init(&bars[qEmpty + i], 129);      // the MMA issuer's commit + the output group's last reads
      mbar_init(&bars[qA + i], 1);
      mbar_init(&bars[qP + i], 128);
      mbar_init(&bars[qN + i], 1);
      mbar_init(&bars[qG + i], 128);
      mbar_init(&bars[qDA + i], 1);
      mbar_init(&bars[qDA16 + i], 128);
      mbar_init(&bars[qZ + i], 128);
      mbar_init(&bars[qDQ + i], 1);
      mbar_init(&bars[qRS + i], 128);
      mbar_init(&bars[qSt + i], 128);         // S tile i holds the state before a chunk c with c & 1 == i
    }
    mbar_init(&bars[qDQFree], 128); mbar_init(&bars[qS], 1);
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
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (c >= 2 && !mbar_wait(&bars[qEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * bqStage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        uint64_t* fb = &bars[qFull + st];
        uint64_t* fv = &bars[qFullV + st];
        mbar_arrive_expect_tx(fb, 4 * kBox);
        tma_load_3d(base + bqQ, &tm_q, fb, 0, bh, t0);
        tma_load_3d(base + bqQ + kBox, &tm_q, fb, 64, bh, t0);
        tma_load_3d(base + bqK, &tm_k, fb, 0, bh, t0);
        tma_load_3d(base + bqK + kBox, &tm_k, fb, 64, bh, t0);
        mbar_arrive_expect_tx(fv, 2 * kBox);
        tma_load_3d(base + bqV, &tm_v, fv, 0, bh, t0);
        tma_load_3d(base + bqG, &tm_g, fv, 0, bh, t0);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ------------------------------------------------------------------ MMA issuers
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idKK = umma_idesc_f16(128, 128, false, false);   // Q K^T ; gs V^T ; gs S^T
      constexpr uint32_t idKM64 = umma_idesc_f16(128, 64, false, true);   // P V ; Q S        (B MN-major)
      constexpr uint32_t idKM128 = umma_idesc_f16(128, 128, false, true); // dA K             (B MN-major)
      constexpr uint32_t idMM64 = umma_idesc_f16(128, 64, true, true);    // K^T V ; Q^T gs   (A, B MN-major)
      constexpr uint64_t kSt = bqStage >> 4, kTile = kBox >> 4;
      const uint64_t dQk = umma_smem_desc(sbase + bqQ, 0, 1024, kSwizzle128B), dQm = umma_smem_desc(sbase + bqQ, kBox, 1024, kSwizzle128B);
      const uint64_t dKk = umma_smem_desc(sbase + bqK, 0, 1024, kSwizzle128B), dKm = umma_smem_desc(sbase + bqK, kBox, 1024, kSwizzle128B);
      const uint64_t dVk = umma_smem_desc(sbase + bqV, 0, 1024, kSwizzle128B), dVm = umma_smem_desc(sbase + bqV, kBox, 1024, kSwizzle128B);
      const uint64_t dGk = umma_smem_desc(sbase + bqG, 0, 1024, kSwizzle128B), dGm = umma_smem_desc(sbase + bqG, kBox, 1024, kSwizzle128B);
      const uint64_t dSk = umma_smem_desc(sbase + bqS, 0, 1024, kSwizzle128B);      // S as [N = k rows][K = n]
      const uint64_t dSm = umma_smem_desc(sbase + bqS, kBox, 1024, kSwizzle128B);   // S as [K = k rows][N = n]
      if (warp == 1) {
        // ---- issuer A: scores A = Q K^T of chunk c into score buffer c & 1, then N = P V + Q S into its columns 64..127
        auto issue_scores = [&](int c) -> bool {
          const int st = c & 1;
          const uint64_t so = (uint64_t)st * kSt;
          if (!mbar_wait(&bars[qFull + st], (c >> 1) & 1)) { tc_fail(7); return false; }
          // the buffer's previous user was chunk c - 2, whose last product (dQ += dA K, issuer B) read dA from it
          if (c >= 2 && !mbar_wait(&bars[qDQ + st], ((c - 2) >> 1) & 1)) { tc_fail(8); return false; }
          tc_fence_after_sync();
          umma_chain_ss<8, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + bqColA + st * 128, dQk + so, dKk + so, idKK, 0);
          umma_commit(&bars[qA + st]);
          return true;
        };
        auto issue_n = [&](int c) -> bool {
          const int st = c & 1;
          const uint64_t so = (uint64_t)st * kSt;
          if (!mbar_wait(&bars[qP + st], (c >> 1) & 1)) { tc_fail(2); return false; }
          if (!mbar_wait(&bars[qSt + (c & 1)], (c >> 1) & 1)) { tc_fail(3); return false; }
          if (!mbar_wait(&bars[qFullV + st], (c >> 1) & 1)) { tc_fail(23); return false; }
          tc_fence_after_sync();
          umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + bqColA + st * 128 + 64, tmem + bqColA + st * 128, dVm + so, idKM64, 0);
          umma_chain_ss<8, kStepK, kBlockK, kStepMN, kBlockMN>(lead, tmem + bqColA + st * 128 + 64, dQk + so, dSm + st * kTile, idKM64, 1);
          umma_commit(&bars[qN + st]);
          return true;
        };
        // in time order: N of chunk c needs P of chunk c (score group 1, about a microsecond after the scores); the
        // tiles of chunk c + 1 arrive one chunk period after those of chunk c
        bool ok = nchunk > 0;
        if (ok) ok = issue_scores(0);
#pragma unroll 1
        for (int c = 0; ok && c < nchunk; ++c) {
          ok = issue_n(c);
          if (ok && c + 1 < nchunk) ok = issue_scores(c + 1);
        }
      } else {
        // ---- issuer B: dA, dQ and the state updates
#pragma unroll 1
        for (int c = 0; c < nchunk; ++c) {
          const int st = c & 1;
          const uint64_t so = (uint64_t)st * kSt;
          // the state update needs only the chunk's K and V (and the output group's read of the previous state): it runs
          // ahead of everything else, so the export of the next S tile is never on the chunk's critical path
          if (!mbar_wait(&bars[qFull + st], (c >> 1) & 1)) { tc_fail(20); break; }
          if (!mbar_wait(&bars[qFullV + st], (c >> 1) & 1)) { tc_fail(24); break; }
          if (!mbar_wait(&bars[qSt + (c & 1)], (c >> 1) & 1)) { tc_fail(9); break; }
          tc_fence_after_sync();
          const uint32_t acc0 = (c == 0 && s_in == nullptr) ? 0u : 1u;
          umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + bqColS, dKm + so, dVm + so, idMM64, acc0);  // S += K^T V
          umma_commit(&bars[qS]);
          if (!mbar_wait(&bars[qG + st], (c >> 1) & 1)) { tc_fail(4); break; }
          tc_fence_after_sync();
          umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + bqColA + st * 128, dGk + so, dVk + so, idKK, 0);   // dA = gs V^T
          umma_commit(&bars[qDA + st]);
          if (c > 0 && !mbar_wait(&bars[qDQFree], (c - 1) & 1)) { tc_fail(5); break; }
          tc_fence_after_sync();
          umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + bqColDQ, dGk + so, dSk + st * kTile, idKK, 0);  // dQ = gs S_prev^T
          if (want_dseg)                                                                   // dSseg += Q^T gs
            umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + bqColDS, dQm + so, dGm + so, idMM64, c > 0 ? 1u : 0u);
          if (!mbar_wait(&bars[qDA16 + st], (c >> 1) & 1)) { tc_fail(6); break; }
          tc_fence_after_sync();
          umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + bqColDQ, tmem + bqColA + st * 128, dKm + so, idKM128, 1);       // dQ += dA K
          umma_commit(&bars[qDQ + st]);
          umma_commit(&bars[qEmpty + st]);       // every MMA that reads this stage is complete when this arrives
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ score group 1: P, row sums, q . z
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t colA = bqColA + st * 128;
      unsigned char* stage = sm + st * bqStage;
      const float* zs = z_buf + (c % 3) * 128;
      if (!mbar_wait(&bars[qFull + st], (c >> 1) & 1)) { tc_fail(15); break; }     // this group reads the Q tile itself
      if (!mbar_wait(&bars[qA + st], (c >> 1) & 1)) { tc_fail(12); break; }
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
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[qP + st]);
      // q . z_prev in fp32 from this thread's own Q row while the tensor pipe computes N from the P just handed over
      // (the scores completed, so the stage's tiles are in; z of this version comes from the output group)
      if (!mbar_wait(&bars[qZ + (c & 1)], (c >> 1) & 1)) { tc_fail(11); break; }
      float qz0 = 0.f, qz1 = 0.f, qz2 = 0.f, qz3 = 0.f;      // four partial sums: a single one is a 128-long dependent chain
#pragma unroll
      for (int ch = 0; ch < 16; ++ch) {
        const uint4 u = *reinterpret_cast<const uint4*>(stage + bqQ + row_chunk2(row, ch));
        const float4 z0 = *reinterpret_cast<const float4*>(zs + ch * 8), z1 = *reinterpret_cast<const float4*>(zs + ch * 8 + 4);
        float2 f;
        f = unpack_half2(u.x); qz0 = fmaf(f.x, z0.x, qz0); qz1 = fmaf(f.y, z0.y, qz1);
        f = unpack_half2(u.y); qz2 = fmaf(f.x, z0.z, qz2); qz3 = fmaf(f.y, z0.w, qz3);
        f = unpack_half2(u.z); qz0 = fmaf(f.x, z1.x, qz0); qz1 = fmaf(f.y, z1.y, qz1);
        f = unpack_half2(u.w); qz2 = fmaf(f.x, z1.z, qz2); qz3 = fmaf(f.y, z1.w, qz3);
      }
      const float qz = (qz0 + qz1) + (qz2 + qz3);
      rg_buf[(c & 1) * 128 + row] = (rowsum + rowsum_b) + qz;
      mbar_arrive(&bars[qRS + st]);
    }
  } else if (warp >= 11) {
    // ------------------------------------------------------------------ score group 2: den, gz, gs, then dA
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t colA = bqColA + st * 128;
      unsigned char* stage = sm + st * bqStage;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      if (!mbar_wait(&bars[qFullV + st], (c >> 1) & 1)) { tc_fail(15); break; }    // this group rewrites the g tile itself
      if (!mbar_wait(&bars[qN + st], (c >> 1) & 1)) { tc_fail(13); break; }
      if (!mbar_wait(&bars[qRS + st], (c >> 1) & 1)) { tc_fail(10); break; }
      tc_fence_after_sync();
      float gz;
      {
        uint32_t nn[64];
        tmem_ld32(tmem + lane_addr + colA + 64, nn);
        tmem_ld32(tmem + lane_addr + colA + 96, nn + 32);
        tmem_ld_wait();
        const float raw = rg_buf[(c & 1) * 128 + row];
        const float dn = fmaxf(raw, kEps), inv = 1.f / dn;
        float go = 0.f, go1 = 0.f, go2 = 0.f, go3 = 0.f;
        unsigned char* grow = stage + bqG;
        // all eight loads of the row first: they are independent, whereas a load behind an in-place store of the
        // same tile would have to wait for it (shared-memory accesses of this warp queue behind the tensor pipe's
        // operand reads, so every dependent round trip is expensive)
        uint4 gu[8];
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) gu[ch] = *reinterpret_cast<const uint4*>(grow + row_chunk1(row, ch));
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) {
          const uint4 u = gu[ch];
          float2 f0 = unpack_half2(u.x), f1 = unpack_half2(u.y), f2 = unpack_half2(u.z), f3 = unpack_half2(u.w);
          go = fmaf(f0.x, __uint_as_float(nn[ch * 8 + 0]), go); go1 = fmaf(f0.y, __uint_as_float(nn[ch * 8 + 1]), go1);
          go2 = fmaf(f1.x, __uint_as_float(nn[ch * 8 + 2]), go2); go3 = fmaf(f1.y, __uint_as_float(nn[ch * 8 + 3]), go3);
          go = fmaf(f2.x, __uint_as_float(nn[ch * 8 + 4]), go); go1 = fmaf(f2.y, __uint_as_float(nn[ch * 8 + 5]), go1);
          go2 = fmaf(f3.x, __uint_as_float(nn[ch * 8 + 6]), go2); go3 = fmaf(f3.y, __uint_as_float(nn[ch * 8 + 7]), go3);
          gu[ch].x = pack_half2(f0.x * inv, f0.y * inv); gu[ch].y = pack_half2(f1.x * inv, f1.y * inv);
          gu[ch].z = pack_half2(f2.x * inv, f2.y * inv); gu[ch].w = pack_half2(f3.x * inv, f3.y * inv);
        }
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(grow + row_chunk1(row, ch)) = gu[ch];
        go = ((go + go1) + (go2 + go3)) * inv;       // g . out
        gz = raw > kEps ? -go * inv : 0.f;           // strict >, upstream rfa.py:91
        if (t0 + row < t_end) {
          ws_den[(size_t)bh * T + t0 + row] = dn;
          ws_gz[(size_t)bh * T + t0 + row] = gz;
        }
        rg_buf[(c & 1) * 128 + row] = gz;            // over the value just consumed
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[qG + st]);
      // ---- dA = mask(gs V^T + gz) -> fp16 over the P columns
      if (!mbar_wait(&bars[qDA + st], (c >> 1) & 1)) { tc_fail(14); break; }
      tc_fence_after_sync();
      auto pack_da = [&](int piece, auto DIAG) {
        constexpr bool diag = decltype(DIAG)::value;
        uint32_t a[32], p[16];
        tmem_ld32(tmem + lane_addr + colA + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0 = __uint_as_float(a[i]) + gz, x1 = __uint_as_float(a[i + 1]) + gz;
          if (diag) {
            if (i > lane) x0 = 0.f;
            if (i + 1 > lane) x1 = 0.f;
          }
          p[i >> 1] = pack_half2(x0, x1);
        }
        tmem_st16(tmem + lane_addr + colA + piece * 16, p);
      };
#pragma unroll 1
      for (int piece = 0; piece < quarter; ++piece) pack_da(piece, std::false_type{});
      pack_da(quarter, std::true_type{});
      {
        uint32_t zero[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) zero[i] = 0u;
#pragma unroll 1
        for (int piece = quarter + 1; piece < 4; ++piece) tmem_st16(tmem + lane_addr + colA + piece * 16, zero);
      }
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[qDA16 + st]);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ output / state group
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk / state row k
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int ytid = tid - 192;
    unsigned char* s_tile = sm + bqS;
    {
      uint32_t r[64];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
      store_state_row(s_tile, row, r);
      if (s_in) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) tmem_st16(tmem + lane_addr + bqColS + c0, r + c0);
        tmem_st_wait();
      }
      z_buf[row] = z_in ? z_in[row] : 0.f;
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[qSt + 0]);
      mbar_arrive(&bars[qZ + 0]);
    }
    bool ok = true;
    float dz_acc = 0.f;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t ph = c & 1;
      unsigned char* stage = sm + st * bqStage;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      const float* zs = z_buf + (c % 3) * 128;
      const float* gzs = rg_buf + (c & 1) * 128;
      // ---- z before the next chunk = z + colsum(K): needs only the staged K tile
      if (!mbar_wait(&bars[qFull + st], (c >> 1) & 1)) { tc_fail(15); ok = false; break; }
      z_buf[((c + 1) % 3) * 128 + row] = zs[row] + column_sum2(stage + bqK, quarter, lane, nullptr);
      mbar_arrive(&bars[qZ + ((c + 1) & 1)]);
      // ---- the state after this chunk -> the other fp16 operand tile.  Its previous readers (the products of chunk
      //      c - 1 that read the state before chunk c - 1) were issued before this chunk's state update by the same
      //      issuer, or consumed before them, so qS alone orders the overwrite.
      if (!mbar_wait(&bars[qS], ph)) { tc_fail(16); ok = false; break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        uint32_t r[64];
        tmem_ld32(tmem + lane_addr + bqColS, r);
        tmem_ld32(tmem + lane_addr + bqColS + 32, r + 32);
        tmem_ld_wait();
        store_state_row(s_tile + ((c + 1) & 1) * kBox, row, r);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[qSt + ((c + 1) & 1)]);
      }
      // gz of every row of this chunk is in shared memory once qG completed (it did: the state MMA waited on it)
      if (!mbar_wait(&bars[qG + st], (c >> 1) & 1)) { tc_fail(17); ok = false; break; }
      if (want_dseg) dz_acc += column_sum2(stage + bqQ, quarter, lane, gzs);      // dzseg += Q^T gz
      const float gz = gzs[row];
      mbar_arrive(&bars[qEmpty + st]);             // this group's last read of the stage's tiles
      // ---- grad_q = dQ + gz z_prev^T -> fp16, written straight from registers (one 256-byte row per thread)
      if (!mbar_wait(&bars[qDQ + st], (c >> 1) & 1)) { tc_fail(18); ok = false; break; }
      tc_fence_after_sync();
      const bool live = t0 + row < t_end;
      __half* grow = reinterpret_cast<__half*>(gq_ptr) + ((size_t)(t0 + row) * BH + bh) * kK;
#pragma unroll 1
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        tmem_ld32(tmem + lane_addr + bqColDQ + piece * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 2; ++j) {              // 32 bytes (one sector) per store: half as many passes of the load/store unit
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int k0 = piece * 32 + j * 16 + e * 8, a0 = j * 16 + e * 8;
            const float4 z0 = *reinterpret_cast<const float4*>(zs + k0), z1 = *reinterpret_cast<const float4*>(zs + k0 + 4);
            o[e * 4 + 0] = pack_half2(fmaf(gz, z0.x, __uint_as_float(a[a0 + 0])), fmaf(gz, z0.y, __uint_as_float(a[a0 + 1])));
            o[e * 4 + 1] = pack_half2(fmaf(gz, z0.z, __uint_as_float(a[a0 + 2])), fmaf(gz, z0.w, __uint_as_float(a[a0 + 3])));
            o[e * 4 + 2] = pack_half2(fmaf(gz, z1.x, __uint_as_float(a[a0 + 4])), fmaf(gz, z1.y, __uint_as_float(a[a0 + 5])));
            o[e * 4 + 3] = pack_half2(fmaf(gz, z1.z, __uint_as_float(a[a0 + 6])), fmaf(gz, z1.w, __uint_as_float(a[a0 + 7])));
          }
          if (live) st_global_v8(grow + piece * 32 + j * 16, o);
        }
      }
      tc_fence_before_sync();
      mbar_arrive(&bars[qDQFree]);                 // after the last read of dQ and of this chunk's z, gz
    }
    if (ok && want_dseg) {
      uint32_t r[64];
      if (nchunk > 0) {
        tmem_ld32(tmem + lane_addr + bqColDS, r);
        tmem_ld32(tmem + lane_addr + bqColDS + 32, r + 32);
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
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
int launch_causal_bwd_q_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq,
                           const float* s_seg, const float* z_seg, float* ws_den, float* ws_gz, float* ds_seg,
                           float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st) {
  CUtensorMap tq, tk, tv, tg;
  if (make_tmap_rows(&tq, q, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&tg, g, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "causal_bwd_q: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_bwd_q_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bqSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_bwd_q: cannot reserve %u bytes of shared memory: %s", bqSmem, cudaGetErrorString(e));
  launch_pdl(causal_bwd_q_tc_kernel, dim3(BH, nseg), dim3(kBqThreads), bqSmem, st, tq, tk, tv, tg, gq, s_seg, z_seg, ws_den, ws_gz, ds_seg,
                                                                    dz_seg, T, BH, nseg, tseg);
  return check_launch("rfa_causal_bwd_q");
}

RFA_TC_UNIT(causal_bwd)

}  // namespace rfa
