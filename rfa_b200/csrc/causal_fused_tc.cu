// Causal RFA forward with the feature map computed inside the kernel (tcgen05 + TMEM + TMA).
//
// Upstream forms phi(q), phi(k) with a chain of PyTorch kernels (utils.py:100-120, called at
// causal_attention.py:241-248) and hands [T][BH][128] features to its attention kernel (cuda/forward.cu:16-169).
// Here the RAW per-head vectors x_q, x_k [T][BH][64] are loaded (half the bytes of the features) and
//     u    = (W_h x) / (|x| + 1e-3)           tcgen05.mma  M128 N64 K64 on the raw tile, scaled in the epilogue
//     phi  = scale [sin u | cos u]            feature warps: TMEM -> registers -> the swizzled fp16 operand tile
// after which a chunk of 128 tokens proceeds as in the kernel that takes ready-made features:
//     A = phi_q phi_k^T,  N = phi_q [S|z]_prev,  P = mask(A),  N += P V,  [S|z] += phi_k^T [V|1],
//     out = N[:, :64] / max(rowsum(P) + N[:, 64], 1).
// phi never touches global memory.  A padded key (row_mask) and a row past the end get all-zero key features.
//
// Shared memory holds ONE pair of feature tiles (64 KB; two would not fit beside the raw rings), so the products that
// read them (A, N, the state update) of chunk c must finish before the features of chunk c + 1 are stored: the feature
// warps compute a chunk ahead into registers and only the 8 stores per thread sit on that chain.  Tensor memory is
// full (A/P 128, N 2 x 80, [S|z] 80, U_q 64, U_k 64 columns), hence a single A/P buffer: scores of chunk c + 1 follow
// P V of chunk c in the issuing thread's order.
//
// Warp roles (896 threads, seven warpgroups): 0 = TMA producer; 1 = issuer A (scores, P V); 2 = issuer B (phi_q [S|z],
// state update); 3 = issuer U (the projections: issuing a product costs its thread about as long as the tensor pipe takes
// to run it, so the three chains are issued by three threads); 4..7 = score group; 8..11 = output/state group; 12..19 =
// query features, 20..27 = key features (two warpgroups each: thread <-> row, and half of the 64 projected columns per
// warpgroup -- the sines and cosines are the longest step of a chunk and bound by the special-function unit, which
// sixteen warps keep busier than eight).  Register budgets differ by role (setmaxnreg): issuers 64, score group 96,
// output/state group 104, feature warps 56.  Within a group thread <-> TMEM lane <-> token row / state row.  All waits
// are bounded.
#include <type_traits>

#define RFA_TC_FAMILY 8
#include "tc_common.cuh"

namespace rfa {
namespace fz {
constexpr int kThreads_ = 896;
// Register budgets per thread by role.  setmaxnreg.inc blocks until the SM's pool holds the registers it asks for, with no
// time limit: the budgets must leave slack.  (A set that summed to exactly 64 K registers never got its increase and
// hung the kernel.)  The kernel starts with 72 registers x 896 threads = 63 K; after the changes 61 K.
constexpr int kRegIssue = 64, kRegScore = 96, kRegOut = 104, kRegFeat = 56;
static_assert(128 * (kRegIssue + kRegScore + kRegOut + 4 * kRegFeat) + 3072 <= 65536, "causal_fwd_fused: register budgets need slack");
static_assert(72 * kThreads_ <= 65536, "causal_fwd_fused: launch register count");
// shared memory map (bytes from a 1024-aligned base)
constexpr uint32_t kXq = 0, kXk = kBox, kRaw = 2 * kBox;          // raw ring: two stages of (x_q, x_k)
constexpr uint32_t kV = 2 * kRaw;                                  // V ring: two stages of one box
constexpr uint32_t kOnes = kV + 2 * kBox;                          // [128][64] box: logical column 0 = 1, rest 0
constexpr uint32_t kPhiQ = kOnes + kBox, kPhiK = kPhiQ + 2 * kBox; // feature tiles [128][128] (two boxes each)
constexpr uint32_t kS = kPhiK + 2 * kBox;                          // state tile: box 0 = S [128 k][64 n], box 1 = [z | 0...]
constexpr uint32_t kW = kS + 2 * kBox;                             // W_h as an fp16 K-major operand [64 j][64 i]
constexpr uint32_t kRs = kW + 8192;                                // fp32 [2][128] row sums, score -> output group
constexpr uint32_t kBar = kRs + 1024;
constexpr uint32_t kSmem = kBar + 256 + 1024;                      // + alignment slack
static_assert(kSmem <= 227 * 1024, "causal_fwd_fused: shared memory map");
// TMEM columns
constexpr uint32_t cA = 0, cN = 128, cS = 288, cUq = 368, cUk = 432;
enum { xFull = 0, xEmpty = 2, vFull = 4, vEmpty = 6, uFull = 8, uFree = 9, phiFull = 10, phiFree = 11, aFull = 12, pFull = 13,
       sDone = 14, nFull = 16, nFree = 18, bSt = 20, bCarry = 21, bNum = 22 };
// xFull/xEmpty: a raw stage (free once U has been formed from it and both feature groups have taken their rows' norms);
// vFull/vEmpty: a V tile (free once P V and the state update have read it); uFull/uFree: the U accumulators;
// phiFull/phiFree: the feature tiles (free = both issuers' products of the chunk are complete); aFull/pFull: scores
// written / packed; sDone (per N buffer): issuer B's products complete; nFull/nFree: an N buffer; bSt: state tile exported;
// bCarry: the state entering the sequence has been loaded (the producer starts after it).
}  // namespace fz

__global__ void __launch_bounds__(fz::kThreads_, 1)
causal_fwd_fused_tc_kernel(const __grid_constant__ CUtensorMap tm_xq, const __grid_constant__ CUtensorMap tm_xk,
                           const __grid_constant__ CUtensorMap tm_v, const float* __restrict__ w,
                           const uint8_t* __restrict__ row_mask, __half* __restrict__ out,
                           const float* __restrict__ s_in, const float* __restrict__ z_in,
                           float* __restrict__ s_out, float* __restrict__ z_out, float* __restrict__ den_out,
                           int64_t T, int BH, int H, float scale) {
  using namespace fz;
  extern __shared__ unsigned char fz_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fz_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBar);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bNum);
  float* rs = reinterpret_cast<float*>(sm + kRs);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bh = blockIdx.x, h = bh % H;
  const int nchunk = (int)((T + kTC - 1) / kTC);
  if (s_in) { s_in += (size_t)bh * kK * kD; z_in += (size_t)bh * kK; }

  if (tid == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[xFull + i], 1);
      mbar_init(&bars[xEmpty + i], 513);      // issuer U's commit + the four feature warpgroups
      mbar_init(&bars[vFull + i], 1);
      mbar_init(&bars[vEmpty + i], 2);        // one commit from each issuer
      mbar_init(&bars[sDone + i], 1);
      mbar_init(&bars[nFull + i], 1);
      mbar_init(&bars[nFree + i], 128);
    }
    mbar_init(&bars[uFull], 1);
    mbar_init(&bars[uFree], 512);
    mbar_init(&bars[phiFull], 512);
    mbar_init(&bars[phiFree], 2);             // one commit from each issuer
    mbar_init(&bars[aFull], 1);
    mbar_init(&bars[pFull], 128);
    mbar_init(&bars[bSt], 128);
    mbar_init(&bars[bCarry], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_xq); tma_prefetch_desc(&tm_xk); tma_prefetch_desc(&tm_v);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, 512);
    tmem_relinquish();
  }
  // the ones box: row r is 128 bytes; logical column 0 lives in 16-byte chunk (r & 7)
  for (int i = tid; i < (int)(kBox / 16); i += kThreads_) {
    const int r = i >> 3, c = i & 7;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (c == (r & 7)) val.x = 0x00003C00u;     // fp16 1.0 in the low half
    *reinterpret_cast<uint4*>(sm + kOnes + i * 16) = val;
  }
  pdl_wait();                   // everything above may overlap the tail of the previous kernel in the stream
  pdl_launch_dependents();
  // W_h -> fp16 K-major operand tile [64 rows j][64 i]
  for (int i = tid; i < 64 * 8; i += kThreads_) {
    const int j = i >> 3, ch = i & 7;
    const float4 a = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8);
    const float4 b = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8 + 4);
    uint4 u;
    u.x = pack_half2(a.x, a.y); u.y = pack_half2(a.z, a.w); u.z = pack_half2(b.x, b.y); u.w = pack_half2(b.z, b.w);
    *reinterpret_cast<uint4*>(sm + kW + row_chunk1(j, ch)) = u;
  }
  fence_async_smem();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  // Register budgets by role (the kernel starts with 72 per thread): the issuers and the feature warps give some back,
  // the score and output/state groups take more.  Each branch below is one or more whole warpgroups.
  if (warp < 4) {
  setmaxnreg_dec<kRegIssue>();
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      // The state entering the sequence is fetched by the output/state group before the first TMA load is issued: with
      // those global loads in flight while the first raw tiles landed, the feature warps' first reads of the tiles
      // returned stale data in an earlier version of this kernel.
      if (s_in && !mbar_wait(&bars[bCarry], 0)) tc_fail(20);
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        const int t0 = c * kTC;
        if (c >= 2 && !mbar_wait(&bars[xEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(1); break; }
        unsigned char* base = sm + st * kRaw;
        mbar_arrive_expect_tx(&bars[xFull + st], 2 * kBox);
        tma_load_3d(base + kXq, &tm_xq, &bars[xFull + st], 0, bh, t0);
        tma_load_3d(base + kXk, &tm_xk, &bars[xFull + st], 0, bh, t0);
        if (c >= 2 && !mbar_wait(&bars[vEmpty + st], ((c >> 1) + 1) & 1)) { tc_fail(2); break; }
        mbar_arrive_expect_tx(&bars[vFull + st], kBox);
        tma_load_3d(sm + kV + st * kBox, &tm_v, &bars[vFull + st], 0, bh, t0);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ issuer A: scores, P V
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idA = umma_idesc_f16(128, 128, false, false);   // phi_q phi_k^T
      constexpr uint32_t idPV = umma_idesc_f16(128, 64, false, true);    // P V (B MN-major)
      const uint64_t dQ = umma_smem_desc(sbase + kPhiQ, 0, 1024, kSwizzle128B), dK = umma_smem_desc(sbase + kPhiK, 0, 1024, kSwizzle128B);
      const uint64_t dV = umma_smem_desc(sbase + kV, kBox, 1024, kSwizzle128B);
      bool ok = true;
#pragma unroll 1
      for (int c = 0; ok && c < nchunk; ++c) {
        const int st = c & 1;
        if (!mbar_wait(&bars[phiFull], c & 1)) { tc_fail(5); break; }
        tc_fence_after_sync();
        // the A/P buffer is free: P V of the previous chunk precedes these in this thread's order
        umma_chain_ss<8, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + cA, dQ, dK, idA, 0);
        umma_commit(&bars[aFull]);
        umma_commit(&bars[phiFree]);
        if (!mbar_wait(&bars[pFull], c & 1)) { tc_fail(6); break; }
        if (!mbar_wait(&bars[sDone + st], (c >> 1) & 1)) { tc_fail(7); break; }      // phi_q [S|z] has written the N buffer
        if (!mbar_wait(&bars[vFull + st], (c >> 1) & 1)) { tc_fail(8); break; }
        tc_fence_after_sync();
        umma_chain_ts<8, kStepMN, kBlockMN>(lead, tmem + cN + st * 80, tmem + cA, dV + (uint64_t)st * (kBox >> 4), idPV, 1);   // N += P V
        umma_commit(&bars[nFull + st]);
        umma_commit(&bars[vEmpty + st]);
      }
    }
  } else if (warp == 2) {
    // ------------------------------------------------------------------ issuer B: N = phi_q [S|z]_prev, [S|z] += phi_k^T [V|1]
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idQS = umma_idesc_f16(128, 80, false, true);    // phi_q [S|z]   (B MN-major)
      constexpr uint32_t idS = umma_idesc_f16(128, 80, true, true);      // phi_k^T [V|1] (A, B MN-major)
      const uint64_t dQ = umma_smem_desc(sbase + kPhiQ, 0, 1024, kSwizzle128B);
      const uint64_t dKt = umma_smem_desc(sbase + kPhiK, kBox, 1024, kSwizzle128B);
      // [V|1], MN-major (N = 80): the second 64-block is the ones box, at a different distance from each V tile
      const uint64_t dW0 = umma_smem_desc(sbase + kV, kOnes - kV, 1024, kSwizzle128B);
      const uint64_t dW1 = umma_smem_desc(sbase + kV + kBox, kOnes - (kV + kBox), 1024, kSwizzle128B);
      const uint64_t dS = umma_smem_desc(sbase + kS, kBox, 1024, kSwizzle128B);
#pragma unroll 1
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        if (!mbar_wait(&bars[bSt], c & 1)) { tc_fail(9); break; }                    // the state before this chunk is in the operand tile
        if (c >= 2 && !mbar_wait(&bars[nFree + st], ((c >> 1) + 1) & 1)) { tc_fail(10); break; }
        if (!mbar_wait(&bars[phiFull], c & 1)) { tc_fail(11); break; }
        if (!mbar_wait(&bars[vFull + st], (c >> 1) & 1)) { tc_fail(12); break; }
        tc_fence_after_sync();
        const uint32_t fresh_acc = (c == 0 && s_in == nullptr) ? 0u : 1u;
        umma_chain_ss<8, kStepK, kBlockK, kStepMN, kBlockMN>(lead, tmem + cN + st * 80, dQ, dS, idQS, 0);
        umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + cS, dKt, st ? dW1 : dW0, idS, fresh_acc);
        umma_commit(&bars[sDone + st]);
        umma_commit(&bars[phiFree]);
        umma_commit(&bars[vEmpty + st]);
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ issuer U: the projections of chunk c as soon as its
    // raw tiles are in and the feature warps have taken the previous chunk's U out of tensor memory
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idU = umma_idesc_f16(128, 64, false, false);    // X W^T
      const uint64_t dXq = umma_smem_desc(sbase + kXq, 0, 1024, kSwizzle128B), dXk = umma_smem_desc(sbase + kXk, 0, 1024, kSwizzle128B);
      const uint64_t dW = umma_smem_desc(sbase + kW, 0, 1024, kSwizzle128B);
#pragma unroll 1
      for (int c = 0; c < nchunk; ++c) {
        const int st = c & 1;
        const uint64_t so = (uint64_t)st * (kRaw >> 4);
        if (!mbar_wait(&bars[xFull + st], (c >> 1) & 1)) { tc_fail(3); break; }
        if (c >= 1 && !mbar_wait(&bars[uFree], (c - 1) & 1)) { tc_fail(4); break; }
        tc_fence_after_sync();
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_ss_w(lead, tmem + cUq, dXq + so + (uint64_t)(j * 2), dW + (uint64_t)(j * 2), idU, j > 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_ss_w(lead, tmem + cUk, dXk + so + (uint64_t)(j * 2), dW + (uint64_t)(j * 2), idU, j > 0);
        umma_commit(&bars[uFull]);
        umma_commit(&bars[xEmpty + st]);
      }
    }
  }
  } else if (warp < 8) {
    setmaxnreg_inc<kRegScore>();
    // ------------------------------------------------------------------ score group: P = mask(A), row sums
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      if (!mbar_wait(&bars[aFull], c & 1)) { tc_fail(13); break; }
      // rs[st] of chunk c-2 must have been read by the output group
      if (c >= 2 && !mbar_wait(&bars[nFree + st], ((c >> 1) + 1) & 1)) { tc_fail(14); break; }
      tc_fence_after_sync();
      float rowsum = 0.f, rowsum_b = 0.f;
      // 32-column pieces left of the diagonal one need no mask, the diagonal one keeps columns <= lane, the rest are zero
      auto pack_piece = [&](int piece, auto DIAG) {
        constexpr bool diag = decltype(DIAG)::value;
        uint32_t a[32], p[16];
        tmem_ld32(tmem + lane_addr + cA + piece * 32, a);
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
        tmem_st16(tmem + lane_addr + cA + piece * 16, p);
      };
#pragma unroll 1
      for (int piece = 0; piece < quarter; ++piece) pack_piece(piece, std::false_type{});
      pack_piece(quarter, std::true_type{});
      {
        uint32_t zero[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) zero[i] = 0u;
#pragma unroll 1
        for (int piece = quarter + 1; piece < 4; ++piece) tmem_st16(tmem + lane_addr + cA + piece * 16, zero);
      }
      rs[st * 128 + row] = rowsum + rowsum_b;
      tmem_st_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[pFull]);
    }
  } else if (warp < 12) {
    setmaxnreg_inc<kRegOut>();
    // ------------------------------------------------------------------ output / state group
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;          // token row in the chunk / state row k
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    unsigned char* s_tile = sm + kS;
    // state entering the sequence -> TMEM (fp32) and the fp16 operand tile
    {
      uint32_t r[80];
#pragma unroll
      for (int n = 0; n < 64; ++n) r[n] = s_in ? __float_as_uint(s_in[(size_t)row * kD + n]) : 0u;
      r[64] = z_in ? __float_as_uint(z_in[row]) : 0u;
#pragma unroll
      for (int n = 65; n < 80; ++n) r[n] = 0u;
      if (s_in) {                       // every value has arrived (they are used below): the producer may start
        uint32_t any = 0;
#pragma unroll
        for (int n = 0; n < 65; ++n) any |= r[n];
        asm volatile("" ::"r"(any) : "memory");
        mbar_arrive(&bars[bCarry]);
      }
      store_state_row(s_tile, row, r);
#pragma unroll
      for (int ch = 1; ch < 8; ++ch) *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, ch)) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, 0)) = make_uint4(pack_half2(__uint_as_float(r[64]), 0.f), 0, 0, 0);
      if (s_in) {
#pragma unroll
        for (int c0 = 0; c0 < 80; c0 += 16) tmem_st16(tmem + lane_addr + cS + c0, r + c0);
        tmem_st_wait();
      }
      fence_async_smem();
      tc_fence_before_sync();
      mbar_arrive(&bars[bSt]);
    }
    bool ok = true;
    for (int c = 0; ok && c < nchunk; ++c) {
      const int st = c & 1;
      // ---- the state after this chunk -> operand tile for the next chunk (the serial chain of the scan)
      if (!mbar_wait(&bars[sDone + st], (c >> 1) & 1)) { tc_fail(15); ok = false; break; }
      tc_fence_after_sync();
      if (c + 1 < nchunk) {
        uint32_t r[80];
        tmem_ld32(tmem + lane_addr + cS, r);
        tmem_ld32(tmem + lane_addr + cS + 32, r + 32);
        tmem_ld16(tmem + lane_addr + cS + 64, r + 64);
        tmem_ld_wait();
        store_state_row(s_tile, row, r);
        *reinterpret_cast<uint4*>(s_tile + kBox + row_chunk1(row, 0)) = make_uint4(pack_half2(__uint_as_float(r[64]), 0.f), 0, 0, 0);
        fence_async_smem();
        tc_fence_before_sync();
        mbar_arrive(&bars[bSt]);
      }
      // ---- N: numerator (64 columns) and q.z_prev (column 64); the row sum from the score group (its write precedes
      // its arrival on pFull, which issuer A saw before it issued the P V whose completion nFull reports)
      if (!mbar_wait(&bars[nFull + st], (c >> 1) & 1)) { tc_fail(16); ok = false; break; }
      tc_fence_after_sync();
      uint32_t nn[64], nz[16];
      tmem_ld32(tmem + lane_addr + cN + st * 80, nn);
      tmem_ld32(tmem + lane_addr + cN + st * 80 + 32, nn + 32);
      tmem_ld16(tmem + lane_addr + cN + st * 80 + 64, nz);
      const float rowsum = rs[st * 128 + row];
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[nFree + st]);
      // ---- out = N / max(rowsum + q.z_prev, 1), stored from registers (a row is one 128-byte line)
      const float raw = rowsum + __uint_as_float(nz[0]);
      const float inv = 1.f / fmaxf(raw, kEps);
      const int64_t t = (int64_t)c * kTC + row;
      if (t < T) {
        if (den_out) den_out[(size_t)bh * T + t] = raw;      // raw denominators [BH][T] for a backward that does not recompute them
        __half* orow = out + ((size_t)t * BH + bh) * kD;
#pragma unroll
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t o[8];
#pragma unroll
          for (int e = 0; e < 8; ++e)
            o[e] = pack_half2(__uint_as_float(nn[ch * 16 + 2 * e]) * inv, __uint_as_float(nn[ch * 16 + 2 * e + 1]) * inv);
          st_global_v8(orow + ch * 16, o);
        }
      }
    }
    // ---- final state out (prefill -> decode hand-off); the last wait on sDone ordered it
    if (ok && s_out) {
      uint32_t r[80];
      if (nchunk > 0) {
        tmem_ld32(tmem + lane_addr + cS, r);
        tmem_ld32(tmem + lane_addr + cS + 32, r + 32);
        tmem_ld16(tmem + lane_addr + cS + 64, r + 64);
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
  } else {
    setmaxnreg_dec<kRegFeat>();
    // ------------------------------------------------------------------ feature groups: query (warps 12..19), key (20..27)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const bool is_key = warp >= 20;
    const int half = ((warp - 12) >> 2) & 1;       // which 32 of the 64 projected columns
    const uint32_t colU = is_key ? cUk : cUq;
    unsigned char* tile = sm + (is_key ? kPhiK : kPhiQ);
    const int nb = BH / H;                           // batch size: row_mask is [T][batch]
    for (int c = 0; c < nchunk; ++c) {
      const int st = c & 1;
      const unsigned char* raw = sm + st * kRaw + (is_key ? kXk : kXq);
      const int64_t t = (int64_t)c * kTC + row;
      if (!mbar_wait(&bars[xFull + st], (c >> 1) & 1)) { tc_fail(17); break; }
      // the row's norm is taken only once U has been formed from the tile (see below): by then the tensor pipe has read
      // every byte of it
      if (!mbar_wait(&bars[uFull], c & 1)) { tc_fail(18); break; }
      tc_fence_after_sync();
      uint32_t u[32];
      tmem_ld32(tmem + lane_addr + colU + 32 * half, u);
      float ss = 0.f, ss_b = 0.f;                    // |x|^2 of this thread's row
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 xr = *reinterpret_cast<const uint4*>(raw + row_chunk1(row, ch));
        float2 f;
        f = unpack_half2(xr.x); ss = fmaf(f.x, f.x, ss); ss_b = fmaf(f.y, f.y, ss_b);
        f = unpack_half2(xr.y); ss = fmaf(f.x, f.x, ss); ss_b = fmaf(f.y, f.y, ss_b);
        f = unpack_half2(xr.z); ss = fmaf(f.x, f.x, ss); ss_b = fmaf(f.y, f.y, ss_b);
        f = unpack_half2(xr.w); ss = fmaf(f.x, f.x, ss); ss_b = fmaf(f.y, f.y, ss_b);
      }
      mbar_arrive(&bars[xEmpty + st]);
      const float inv = 1.f / (sqrtf(ss + ss_b) + kNormEps);
      // a key past the end of the sequence or masked as padding contributes nothing: all-zero features
      float sc = scale;
      if (is_key && (t >= T || (row_mask && row_mask[t * nb + bh / H]))) sc = 0.f;
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[uFree]);
      // features into registers, packed fp16 in place: u[2i] <- the sines, u[2i + 1] <- the cosines of columns 2i, 2i + 1 ...
#pragma unroll
      for (int i = 0; i < 16; i += 1) {
        float s0, c0, s1, c1;
        __sincosf(__uint_as_float(u[2 * i]) * inv, &s0, &c0);
        __sincosf(__uint_as_float(u[2 * i + 1]) * inv, &s1, &c1);
        const uint32_t ps = pack_half2(s0 * sc, s1 * sc), pc = pack_half2(c0 * sc, c1 * sc);
        u[2 * i] = ps;
        u[2 * i + 1] = pc;
      }
      // ... and into the operand tile once the products of the previous chunk have let go of it
      if (c >= 1 && !mbar_wait(&bars[phiFree], (c - 1) & 1)) { tc_fail(19); break; }
#pragma unroll
      for (int ch = 0; ch < 4; ++ch) {
        *reinterpret_cast<uint4*>(tile + row_chunk2(row, 4 * half + ch)) = make_uint4(u[8 * ch], u[8 * ch + 2], u[8 * ch + 4], u[8 * ch + 6]);           // sin block
        *reinterpret_cast<uint4*>(tile + row_chunk2(row, 8 + 4 * half + ch)) = make_uint4(u[8 * ch + 1], u[8 * ch + 3], u[8 * ch + 5], u[8 * ch + 7]);   // cos block
      }
      fence_async_smem();
      mbar_arrive(&bars[phiFull]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// x_q, x_k, v, out [T][BH][64] fp16 (BH = batch * H, head index fastest); w [H][64][64] fp32; row_mask [T][batch] or null
int launch_causal_fwd_fused_tc(const __half* xq, const __half* xk, const __half* v, const float* w, const uint8_t* row_mask,
                               __half* out, const float* s_in, const float* z_in, float* s_out, float* z_out, float* den_out,
                               int64_t T, int BH, int H, float scale, cudaStream_t st) {
  CUtensorMap tq, tk, tv;
  if (make_tmap_rows(&tq, xq, T, BH, kD, kTC) || make_tmap_rows(&tk, xk, T, BH, kD, kTC) || make_tmap_rows(&tv, v, T, BH, kD, kTC))
    return fail(RFA_EDEVICE, "causal_fwd_fused: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(causal_fwd_fused_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fz::kSmem);
  if (e != cudaSuccess) return fail((int)e, "causal_fwd_fused: cannot reserve %u bytes of shared memory: %s", fz::kSmem, cudaGetErrorString(e));
  launch_pdl(causal_fwd_fused_tc_kernel, dim3(BH), dim3(fz::kThreads_), fz::kSmem, st, tq, tk, tv, w, row_mask, out, s_in, z_in, s_out,
             z_out, den_out, T, BH, H, scale);
  return check_launch("rfa_causal_fwd_fused");
}

RFA_TC_UNIT(causal_fwd_fused)

}  // namespace rfa
