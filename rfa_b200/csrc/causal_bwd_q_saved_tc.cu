// Causal RFA backward, sweep 1 (forward in time), for callers that kept the forward's results: grad_q and the
// per-token scalar gz from the SAVED attention output and raw denominators instead of recomputing them
// (upstream cuda/backward.cu:303-371, q_backward, recomputes; math in rfa.py:79-94).  Chunks of 128 tokens.
//
// Per chunk, with S/z the state of all earlier tokens, out and den_raw from the forward pass:
//     den = max(den_raw, 1);  gs = g/den (fp16, over the staged g tile);  gz = -(g.out)/den * [den_raw > 1]
//     dA  = gs V^T             -> mask(dA + gz) fp16 (TMEM, over dA)
//     dQ  = gs S^T + dA K (+ gz z^T added in the epilogue)            -> grad_q
//     S  += K^T V,  z += colsum(K);   WANT_DSEG:  dSseg += Q^T gs, dzseg += Q^T gz
// Without the score / numerator recomputation the chunk's chain is half as long as the recomputing sweep's, q is not
// read at all unless the reverse-state total of the run is wanted (WANT_DSEG: segmented or sharded sequences), and the
// saved output rows are read straight from global memory into registers one chunk ahead (they feed CUDA cores only).
//
// Warp roles (448 threads): warp 0 TMA producer; warp 1 MMA issuer; warps 2..5 scale group (den, gz, gs; dzseg);
// warps 10..13 pack/state group (dA -> masked fp16, then the scan's serial step: z += colsum(K), S -> fp16 operand
// tile); warps 6..9 output group (grad_q only).  Keeping the state export out of the output group matters: the
// issuer's next state update waits for the export, the output group waits for the issuer's dQ, and with both in one
// group the two waits chain into one long cycle per chunk.  dA is double-buffered in TMEM.  grad_q leaves through a staged TMA store when the q tiles are not resident
// (!WANT_DSEG: their shared memory holds two staging tiles), else straight from registers.  All waits are bounded.
#include <type_traits>

#define RFA_TC_FAMILY 6
#include "tc_common.cuh"

namespace rfa {

constexpr int kBsThreads = 448;

template <bool WANT_DSEG> struct BsLayout {
  // stage: [Q (2 boxes) when WANT_DSEG] K (2 boxes) V G
  static constexpr uint32_t Q = 0, K = WANT_DSEG ? 2 * kBox : 0, V = K + 2 * kBox, G = V + kBox, Stage = G + kBox;
  static constexpr uint32_t S = 2 * Stage;                  // two state operand tiles [128 k][64 n] fp16: state before chunk c in tile c & 1
  static constexpr uint32_t Gq = S + 2 * kBox;              // !WANT_DSEG: two [128][128] staging tiles for grad_q
  static constexpr uint32_t Z = Gq + (WANT_DSEG ? 0 : 4 * kBox);   // fp32 [3][128]: z before chunk c in buffer c % 3
  static constexpr uint32_t Rg = Z + 1536;                  // fp32 [2][128]: gz of the chunk's rows
  static constexpr uint32_t Bar = Rg + 1024;
  static constexpr uint32_t Smem = Bar + 256;               // 14 boxes + 2816 bytes: the base must come 1024-aligned (checked)
};

// TMEM: two dA buffers (fp32 dA -> fp16 dA packed into their first 64 columns), dQ, S, dSseg
constexpr uint32_t bsColA = 0, bsColDQ = 256, bsColS = 384, bsColDS = 448;
enum { sFullK = 0, sFullV = 2, sEmpty = 4, sG = 6, sDA = 8, sDA16 = 10, sDQ = 12, sSt = 14, sDQFree = 16, sS = 17, sY = 18, sZ = 19, sNum = 22 };
// sFullK guards the K (and Q) tiles of a stage, sFullV its V and g tiles.  Barriers that a waiter may reach late are
// kept per stage / buffer (index c & 1) so that their producer cannot complete two phases before the waiter looks.

template <bool WANT_DSEG>
__global__ void __launch_bounds__(kBsThreads, 1)
causal_bwd_q_saved_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                             const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_g,
                             const __grid_constant__ CUtensorMap tm_gq,
                             const __half* __restrict__ out_ptr, const float* __restrict__ den_raw,
                             __half* __restrict__ gq_ptr,
                             const float* __restrict__ s_seg, const float* __restrict__ z_seg,
                             float* __restrict__ ws_gz, float* __restrict__ ds_seg, float* __restrict__ dz_seg,
                             int64_t T, int BH, int nseg, int64_t tseg) {
  using L = BsLayout<WANT_DSEG>;
  extern __shared__ __align__(1024) unsigned char bs_raw[];
  unsigned char* sm = bs_raw;
  if (smem_u32(sm) & 1023u) {                    // swizzled tiles need a 1024-byte aligned base
    if (threadIdx.x == 0) tc_fail(99);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + L::Bar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + sNum);
  float* z_buf = reinterpret_cast<float*>(sm + L::Z);
  float* rg_buf = reinterpret_cast<float*>(sm + L::Rg);
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
      mbar_init(&bars[sFullK + i], 1);
      mbar_init(&bars[sFullV + i], 1);
      // the issuer's commit + the last reads of the output group (gz), the pack/state group (K) and, with WANT_DSEG,
      // the scale group (Q)
      mbar_init(&bars[sEmpty + i], WANT_DSEG ? 385 : 257);
      mbar_init(&bars[sG + i], 128);
      mbar_init(&bars[sDA + i], 1);
      mbar_init(&bars[sDA16 + i], 128);
      mbar_init(&bars[sDQ + i], 1);
      mbar_init(&bars[sSt + i], 128);         // S tile i holds the state before a chunk c with c & 1 == i
    }
    mbar_init(&bars[sDQFree], 128); mbar_init(&bars[sS], 1); mbar_init(&bars[sY], 128);
    // z before chunk c is in buffer c % 3, announced on barrier c % 3: three, because the pack/state group can be two
    // versions ahead of the output group, and a barrier that completes two phases before its waiter looks strands it
    for (int i = 0; i < 3; ++i) mbar_init(&bars[sZ + i], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_g);
    if (WANT_DSEG) tma_prefetch_desc(&tm_q); else tma_prefetch_desc(&tm_gq);
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
        if (c >= 2 && !mbar_wait(&bars[sEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * L::Stage;
        const int t0 = (int)(t_begin + (int64_t)c * kTC);
        uint64_t* fv = &bars[sFullV + st];
        uint64_t* fk = &bars[sFullK + st];
        // g and V first: the chunk's chain starts with the scaling of g
        mbar_arrive_expect_tx(fv, 2 * kBox);
        tma_load_3d(base + L::G, &tm_g, fv, 0, bh, t0);
        tma_load_3d(base + L::V, &tm_v, fv, 0, bh, t0);
        mbar_arrive_expect_tx(fk, (WANT_DSEG ? 4 : 2) * kBox);
        tma_load_3d(base + L::K, &tm_k, fk, 0, bh, t0);
        tma_load_3d(base + L::K + kBox, &tm_k, fk, 64, bh, t0);
        if (WANT_DSEG) {
          tma_load_3d(base + L::Q, &tm_q, fk, 0, bh, t0);
          tma_load_3d(base + L::Q + kBox, &tm_q, fk, 64, bh, t0);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idKK = umma_idesc_f16(128, 128, false, false);   // gs V^T ; gs S^T
      constexpr uint32_t idKM128 = umma_idesc_f16(128, 128, false, true); // dA K             (B MN-major)
      constexpr uint32_t idMM64 = umma_idesc_f16(128, 64, true, true);    // K^T V ; Q^T gs   (A, B MN-major)
      constexpr uint64_t kSt = L::Stage >> 4, kTile = kBox >> 4;
      const uint64_t dQm = umma_smem_desc(sbase + L::Q, kBox, 1024, kSwizzle128B);
      const uint64_t dKm = umma_smem_desc(sbase + L::K, kBox, 1024, kSwizzle128B);
      const uint64_t dVk = umma_smem_desc(sbase + L::V, 0, 1024, kSwizzle128B), dVm = umma_smem_desc(sbase + L::V, kBox, 1024, kSwizzle128B);
      const uint64_t dGk = umma_smem_desc(sbase + L::G, 0, 1024, kSwizzle128B), dGm = umma_smem_desc(sbase + L::G, kBox, 1024, kSwizzle128B);
      const uint64_t dSk = umma_smem_desc(sbase + L::S, 0, 1024, kSwizzle128B);      // S as [N = k rows][K = n]
      // state update of chunk c: needs the chunk's K and V and the output group's export of the previous state
      auto issue_state = [&](int c) -> bool {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * kSt;
        if (!mbar_wait(&bars[sFullK + st], (c >> 1) & 1)) { tc_fail(20); return false; }
        if (!mbar_wait(&bars[sFullV + st], (c >> 1) & 1)) { tc_fail(24); return false; }
        if (!mbar_wait(&bars[sSt + st], (c >> 1) & 1)) { tc_fail(9); return false; }
        tc_fence_after_sync();
        const uint32_t acc0 = (c == 0 && s_in == nullptr) ? 0u : 1u;
        umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + bsColS, dKm + so, dVm + so, idMM64, acc0);  // S += K^T V
        umma_commit(&bars[sS]);
        return true;
      };
      auto issue_da = [&](int c) -> bool {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * kSt;
        if (!mbar_wait(&bars[sG + st], (c >> 1) & 1)) { tc_fail(4); return false; }
        tc_fence_after_sync();
        umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + bsColA + st * 128, dGk + so, dVk + so, idKK, 0);   // dA = gs V^T
        umma_commit(&bars[sDA + st]);
        return true;
      };
      bool ok = nchunk > 0;
      // dQ(c) = gs S^T reads the state tile c & 1, which is next overwritten by the export that follows the state update
      // of chunk c + 1: this thread issues that update after dQ(c), the tensor pipe runs one thread's products in order,
      // and the export waits for the update's commit, so the read stays ahead of the write.
      if (ok) ok = issue_state(0);
      if (ok) ok = issue_da(0);
#pragma unroll 1
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * kSt;
        if (c > 0 && !mbar_wait(&bars[sDQFree], (c - 1) & 1)) { tc_fail(5); break; }
        tc_fence_after_sync();
        umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + bsColDQ, dGk + so, dSk + st * kTile, idKK, 0);     // dQ = gs S_prev^T
        if (WANT_DSEG)                                                                      // dSseg += Q^T gs
          umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + bsColDS, dQm + so, dGm + so, idMM64, c > 0 ? 1u : 0u);
        if (!mbar_wait(&bars[sDA16 + st], (c >> 1) & 1)) { tc_fail(6); break; }
        tc_fence_after_sync();
        umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + bsColDQ, tmem + bsColA + st * 128, dKm + so, idKM128, 1);         // dQ += dA K
        umma_commit(&bars[sDQ + st]);
        umma_commit(&bars[sEmpty + st]);       // every product that reads this stage is complete when this arrives
        // the next chunk's state update and dA: the pack/state group works on them while the output group drains dQ
        if (c + 1 < nchunk) {
          ok = issue_state(c + 1);
          if (ok) ok = issue_da(c + 1);
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------ scale group: den, gz, gs = g / den
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk
    // this thread's row of the saved output and its raw denominator, fetched one chunk ahead
    uint4 ou[8];
    float raw = 1.f, dz_acc = 0.f;
    // (the rows are asked into L2 a chunk earlier still: a load from DRAM takes about as long as a whole chunk)
    auto ask = [&](int c) {
      const int64_t t = t_begin + (int64_t)c * kTC + row;
      if (c < nchunk && t < t_end) {
        asm volatile("prefetch.global.L2 [%0];" ::"l"(out_ptr + ((size_t)t * BH + bh) * kD));
        if ((lane & 7) == 0) asm volatile("prefetch.global.L2 [%0];" ::"l"(den_raw + (size_t)bh * T + t));
      }
    };
    auto fetch = [&](int c) {
      const int64_t t = t_begin + (int64_t)c * kTC + row;
      if (c < nchunk && t < t_end) {
        const uint4* src = reinterpret_cast<const uint4*>(out_ptr + ((size_t)t * BH + bh) * kD);
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) ou[ch] = __ldg(src + ch);
        raw = __ldg(den_raw + (size_t)bh * T + t);
      } else {
#pragma unroll
        for (int ch = 0; ch < 8; ++ch) ou[ch] = make_uint4(0, 0, 0, 0);
        raw = 1.f;
      }
    };
    fetch(0);
    ask(1);
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      unsigned char* grow = sm + st * L::Stage + L::G;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      if (!mbar_wait(&bars[sFullV + st], (c >> 1) & 1)) { tc_fail(15); break; }
      const float dn = fmaxf(raw, kEps), inv = 1.f / dn;
      float go = 0.f, go1 = 0.f, go2 = 0.f, go3 = 0.f;
      // all eight loads of the row first (independent), then the arithmetic, then the stores
      uint4 gu[8];
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) gu[ch] = *reinterpret_cast<const uint4*>(grow + row_chunk1(row, ch));
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 u = gu[ch], o = ou[ch];
        const float2 f0 = unpack_half2(u.x), f1 = unpack_half2(u.y), f2 = unpack_half2(u.z), f3 = unpack_half2(u.w);
        const float2 o0 = unpack_half2(o.x), o1 = unpack_half2(o.y), o2 = unpack_half2(o.z), o3 = unpack_half2(o.w);
        go = fmaf(f0.x, o0.x, go); go1 = fmaf(f0.y, o0.y, go1); go2 = fmaf(f1.x, o1.x, go2); go3 = fmaf(f1.y, o1.y, go3);
        go = fmaf(f2.x, o2.x, go); go1 = fmaf(f2.y, o2.y, go1); go2 = fmaf(f3.x, o3.x, go2); go3 = fmaf(f3.y, o3.y, go3);
        gu[ch].x = pack_half2(f0.x * inv, f0.y * inv); gu[ch].y = pack_half2(f1.x * inv, f1.y * inv);
        gu[ch].z = pack_half2(f2.x * inv, f2.y * inv); gu[ch].w = pack_half2(f3.x * inv, f3.y * inv);
      }
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) *reinterpret_cast<uint4*>(grow + row_chunk1(row, ch)) = gu[ch];
      go = (go + go1) + (go2 + go3);                       // g . out
      const float gz = raw > kEps ? -go * inv : 0.f;       // strict >, upstream rfa.py:91
      if (t0 + row < t_end) ws_gz[(size_t)bh * T + t0 + row] = gz;
      rg_buf[st * 128 + row] = gz;
      fence_async_smem();
      mbar_arrive(&bars[sG + st]);
      fetch(c + 1);
      ask(c + 2);
      if (WANT_DSEG) {                             // dzseg += Q^T gz: needs every row's gz and the staged Q tile
        if (!mbar_wait(&bars[sG + st], (c >> 1) & 1)) { tc_fail(11); break; }
        if (!mbar_wait(&bars[sFullK + st], (c >> 1) & 1)) { tc_fail(12); break; }
        dz_acc += column_sum2(sm + st * L::Stage + L::Q, quarter, lane, rg_buf + st * 128);
        mbar_arrive(&bars[sEmpty + st]);
      }
    }
    if (WANT_DSEG) dz_seg[slot * kK + row] = dz_acc;       // (zero when the run has no tokens)
  } else if (warp >= 10) {
    // ------------------------------------------------------------------ pack/state group: dA -> masked fp16; z, S export
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk (dA) / state row k (S, z)
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    unsigned char* s_tile = sm + L::S;
    {   // the state entering this run of tokens -> TMEM (fp32) and operand tile 0; z version 0
      uint32_t r[64];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
      store_state_row(s_tile, row, r);
      if (s_in) {
#pragma unroll
        for (int c0 = 0; c0 < 64; c0 += 16) tmem_st16(tmem + lane_addr + bsColS + c0, r + c0);
        tmem_st_wait();
      }
      z_buf[row] = z_in ? z_in[row] : 0.f;
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[sSt + 0]);
      mbar_arrive(&bars[sZ + 0]);
    }
    float zrun = z_in ? z_in[row] : 0.f;           // z[row] before the current chunk
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      const uint32_t colA = bsColA + st * 128;
      unsigned char* stage = sm + st * L::Stage;
      // ---- first the scan's serial step (the issuer's next state update waits for it): the state after this chunk ->
      //      the other fp16 operand tile.  Its previous reader (dQ = gs S^T of chunk c - 1) was issued before this
      //      chunk's state update by the same thread, so sS alone orders the overwrite.
      if (!mbar_wait(&bars[sS], c & 1)) { tc_fail(16); break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        uint32_t r[64];
        tmem_ld32(tmem + lane_addr + bsColS, r);
        tmem_ld32(tmem + lane_addr + bsColS + 32, r + 32);
        tmem_ld_wait();
        store_state_row(s_tile + ((c + 1) & 1) * kBox, row, r);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[sSt + ((c + 1) & 1)]);
      }
      // ---- dA of this chunk
      if (!mbar_wait(&bars[sG + st], (c >> 1) & 1)) { tc_fail(10); break; }      // gz of this row is in shared memory
      const float gz = rg_buf[st * 128 + row];
      if (!mbar_wait(&bars[sDA + st], (c >> 1) & 1)) { tc_fail(14); break; }
      tc_fence_after_sync();
      // 32-column pieces left of the diagonal one need no mask, the diagonal one keeps columns <= lane, the rest are zero
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
      mbar_arrive(&bars[sDA16 + st]);
      // ---- z before the next chunk = z + colsum(K).  Buffer (c + 1) % 3 last held version c - 2, whose reader (the output
      //      group's epilogue of chunk c - 2) read it before it released dQ for chunk c - 1, which precedes this chunk's dA.
      if (!mbar_wait(&bars[sFullK + st], (c >> 1) & 1)) { tc_fail(15); break; }
      zrun += column_sum2(stage + L::K, quarter, lane, nullptr);
      mbar_arrive(&bars[sEmpty + st]);             // this group's last read of the stage's tiles
      z_buf[((c + 1) % 3) * 128 + row] = zrun;
      mbar_arrive(&bars[sZ + (c + 1) % 3]);
    }
  } else {
    // ------------------------------------------------------------------ output group (warps 6..9): grad_q
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;           // token row of the chunk
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int ytid = tid - 192;
    bool ok = true;
    uint32_t y_phase = 0;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      const int64_t t0 = t_begin + (int64_t)c * kTC;
      const float* zs = z_buf + (c % 3) * 128;
      // ---- gz of this row (shared memory, complete once sG completed); the buffer is rewritten two chunks on, after
      //      the stage has been released
      if (!mbar_wait(&bars[sG + st], (c >> 1) & 1)) { tc_fail(17); ok = false; break; }
      const float gz = rg_buf[st * 128 + row];
      mbar_arrive(&bars[sEmpty + st]);
      if (!mbar_wait(&bars[sZ + c % 3], (c / 3) & 1)) { tc_fail(19); ok = false; break; }
      // ---- !WANT_DSEG: the staging tile of chunk c - 2 has been read out by its store
      if (!WANT_DSEG) {
        if (ytid == 0 && c >= 2) tma_store_wait_read<1>();
        if (!epi_sync(&bars[sY], y_phase)) { tc_fail(12); ok = false; break; }
      }
      // ---- grad_q = dQ + gz z_prev^T -> fp16
      if (!mbar_wait(&bars[sDQ + st], (c >> 1) & 1)) { tc_fail(18); ok = false; break; }
      tc_fence_after_sync();
      const bool live = t0 + row < t_end;
      __half* grow = gq_ptr + ((size_t)(t0 + row) * BH + bh) * kK;
      unsigned char* gstage = sm + L::Gq + (uint32_t)st * 2 * kBox;
#pragma unroll 1
      for (int piece = 0; piece < 4; ++piece) {
        uint32_t a[32];
        float4 zv[8];
        tmem_ld32(tmem + lane_addr + bsColDQ + piece * 32, a);
#pragma unroll
        for (int j = 0; j < 8; ++j) zv[j] = *reinterpret_cast<const float4*>(zs + piece * 32 + j * 4);
        tmem_ld_wait();
        // dQ and this chunk's z are in registers: the next chunk may overwrite dQ (and, later, the z buffer)
        if (piece == 3) { tc_fence_before_sync(); mbar_arrive(&bars[sDQFree]); }
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int a0 = j * 16 + e * 8;
            const float4 z0 = zv[a0 / 4], z1 = zv[a0 / 4 + 1];
            o[e * 4 + 0] = pack_half2(fmaf(gz, z0.x, __uint_as_float(a[a0 + 0])), fmaf(gz, z0.y, __uint_as_float(a[a0 + 1])));
            o[e * 4 + 1] = pack_half2(fmaf(gz, z0.z, __uint_as_float(a[a0 + 2])), fmaf(gz, z0.w, __uint_as_float(a[a0 + 3])));
            o[e * 4 + 2] = pack_half2(fmaf(gz, z1.x, __uint_as_float(a[a0 + 4])), fmaf(gz, z1.y, __uint_as_float(a[a0 + 5])));
            o[e * 4 + 3] = pack_half2(fmaf(gz, z1.z, __uint_as_float(a[a0 + 6])), fmaf(gz, z1.w, __uint_as_float(a[a0 + 7])));
          }
          if (WANT_DSEG) {
            if (live) st_global_v8(grow + piece * 32 + j * 16, o);      // 32 bytes (one sector) per store
          } else {
            const int ch = piece * 4 + j * 2;                           // 16-byte chunks ch, ch + 1 of the row
            *reinterpret_cast<uint4*>(gstage + row_chunk2(row, ch)) = make_uint4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<uint4*>(gstage + row_chunk2(row, ch + 1)) = make_uint4(o[4], o[5], o[6], o[7]);
          }
        }
      }
      if (!WANT_DSEG) {
        fence_async_smem();
        if (!epi_sync(&bars[sY], y_phase)) { tc_fail(13); ok = false; break; }
        if (ytid == 0) {                          // rows past the end of the sequence are clipped by the store
          tma_store_3d(&tm_gq, gstage, 0, bh, (int)t0);
          tma_store_3d(&tm_gq, gstage + kBox, 64, bh, (int)t0);
          tma_store_commit();
        }
      }
    }
    if (ok && WANT_DSEG) {
      uint32_t r[64];
      if (nchunk > 0) {
        tmem_ld32(tmem + lane_addr + bsColDS, r);      // the wait on sDQ of the last chunk ordered the last dSseg product
        tmem_ld32(tmem + lane_addr + bsColDS + 32, r + 32);
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
    }
    if (!WANT_DSEG && ytid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// ---------------------------------------------------------------------------
// out [T][BH][d] and den_raw [BH][T] are the forward's saved results; ds_seg / dz_seg non-null = also write each segment's
// reverse-state total (then q is read).
int launch_causal_bwd_q_saved_tc(const __half* q, const __half* k, const __half* v, const __half* g, const __half* out,
                                 const float* den_raw, __half* gq, const float* s_seg, const float* z_seg, float* ws_gz,
                                 float* ds_seg, float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st) {
  const bool want = ds_seg != nullptr;
  CUtensorMap tq, tk, tv, tg, tgq;
  if (make_tmap_rows(&tq, want ? q : k, T, BH, kK, kTC) || make_tmap_rows(&tk, k, T, BH, kK, kTC) ||
      make_tmap_rows(&tv, v, T, BH, kD, kTC) || make_tmap_rows(&tg, g, T, BH, kD, kTC) ||
      make_tmap_rows(&tgq, gq, T, BH, kK, kTC))
    return fail(RFA_EDEVICE, "causal_bwd_q_saved: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e;
  if (want) {
    constexpr uint32_t smem = BsLayout<true>::Smem;
    e = cudaFuncSetAttribute(causal_bwd_q_saved_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail((int)e, "causal_bwd_q_saved: cannot reserve %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
    launch_pdl(causal_bwd_q_saved_tc_kernel<true>, dim3(BH, nseg), dim3(kBsThreads), smem, st, tq, tk, tv, tg, tgq, out, den_raw, gq, s_seg, z_seg,
               ws_gz, ds_seg, dz_seg, T, BH, nseg, tseg);
  } else {
    constexpr uint32_t smem = BsLayout<false>::Smem;
    e = cudaFuncSetAttribute(causal_bwd_q_saved_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return fail((int)e, "causal_bwd_q_saved: cannot reserve %u bytes of shared memory: %s", smem, cudaGetErrorString(e));
    launch_pdl(causal_bwd_q_saved_tc_kernel<false>, dim3(BH, nseg), dim3(kBsThreads), smem, st, tq, tk, tv, tg, tgq, out, den_raw, gq, s_seg, z_seg,
               ws_gz, ds_seg, dz_seg, T, BH, nseg, tseg);
  }
  return check_launch("rfa_causal_bwd_q_saved");
}

RFA_TC_UNIT(causal_bwd_saved)

}  // namespace rfa
