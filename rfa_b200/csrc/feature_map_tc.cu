// Feature map forward on tcgen05 for the fp16, head_dim = proj_dim = 64 case:
//   phi = scale * [sin(u) | cos(u)],  u = (W_h x) / (|x| + 1e-3)        (upstream utils.py:100-120)
// The projection of a tile of 128 rows of one head is one small MMA chain (M128 N64 K64) on the RAW
// rows; the normalisation commutes with the projection and is applied to the fp32 result, so the
// staged x tile is never rewritten.  One CTA owns one head (W_h resident as an fp16 operand tile)
// and walks row tiles with a two-stage TMA ring; phi leaves through a staging tile and a TMA store.
// HBM-bound: 128 bytes in, 256 bytes out per (row, head).
#define RFA_TC_FAMILY 5
#include "tc_common.cuh"

namespace rfa {
namespace fm {
constexpr int kThreads_ = 192;
constexpr uint32_t kX = 0, kStage = kBox, kW = 2 * kStage, kOut = kW + 8192, kBarOff = kOut + 2 * kBox, kSmem = kBarOff + 128 + 1024;
enum { bFull = 0, bEmpty = 2, bU = 4, bUFree = 6, bEpi = 8, bNum = 9 };
}

__global__ void __launch_bounds__(fm::kThreads_, 2)
feature_map_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_phi,
                          const __grid_constant__ CUtensorMap tm_x2, const __grid_constant__ CUtensorMap tm_phi2,
                          const float* __restrict__ w, const uint8_t* __restrict__ row_mask, const uint8_t* __restrict__ row_mask2,
                          int64_t rows, int H, float scale, int pair) {
  using namespace fm;
  extern __shared__ unsigned char fm_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fm_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBarOff);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bNum);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  // pair != 0: two arrays of the same shape share the launch and W_h (phi of q and of k): virtual tile v is row tile
  // v / 2 of array v % 2
  const int ntile_all = (int)((rows + kTC - 1) / kTC) * (pair ? 2 : 1);
  const int ntile = blockIdx.x < ntile_all ? (ntile_all - 1 - blockIdx.x) / gridDim.x + 1 : 0;   // tiles blockIdx.x, +gridDim.x, ...
  auto tile_row0 = [&](int i, int& which) -> int {
    const int v = blockIdx.x + i * gridDim.x;
    which = pair ? (v & 1) : 0;
    return (pair ? (v >> 1) : v) * kTC;
  };
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 129); mbar_init(&bars[bU + i], 1); mbar_init(&bars[bUFree + i], 128); }
    mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    // the first tiles are requested before the rest of the prologue (W_h, tensor memory), which their flight then hides
    for (int i = 0; i < 2 && i < ntile; ++i) {
      int which;
      const int row0 = tile_row0(i, which);
      mbar_arrive_expect_tx(&bars[bFull + i], kBox);
      tma_load_3d(sm + kX + i * kStage, which ? &tm_x2 : &tm_x, &bars[bFull + i], 0, h, row0);
    }
    tma_prefetch_desc(&tm_phi);
  }
  // W_h as an fp16 K-major operand tile [64 rows j][64 i]
  for (int i = tid; i < 64 * 8; i += kThreads_) {
    const int j = i >> 3, ch = i & 7;
    const float4 a = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8);
    const float4 b = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8 + 4);
    uint4 u;
    u.x = pack_half2(a.x, a.y); u.y = pack_half2(a.z, a.w); u.z = pack_half2(b.x, b.y); u.w = pack_half2(b.z, b.w);
    *reinterpret_cast<uint4*>(sm + kW + row_chunk1(j, ch)) = u;
  }
  fence_async_smem();
  if (warp == 1) { tmem_alloc(tmem_slot, 128); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0)
      for (int i = 2; i < ntile; ++i) {
        const int st = i & 1;
        if (!mbar_wait(&bars[bEmpty + st], ((i >> 1) + 1) & 1)) { tc_fail(1); break; }
        int which;
        const int row0 = tile_row0(i, which);
        mbar_arrive_expect_tx(&bars[bFull + st], kBox);
        tma_load_3d(sm + kX + st * kStage, which ? &tm_x2 : &tm_x, &bars[bFull + st], 0, h, row0);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t id = umma_idesc_f16(128, 64, false, false);
      const uint64_t dX = umma_smem_desc(sbase + kX, 0, 1024, kSwizzle128B), dW = umma_smem_desc(sbase + kW, 0, 1024, kSwizzle128B);
      for (int i = 0; i < ntile; ++i) {
        const int st = i & 1;
        if (!mbar_wait(&bars[bFull + st], (i >> 1) & 1)) { tc_fail(2); break; }
        if (i >= 2 && !mbar_wait(&bars[bUFree + st], ((i >> 1) + 1) & 1)) { tc_fail(3); break; }
        tc_fence_after_sync();
        const uint64_t so = (uint64_t)st * (kStage >> 4);
#pragma unroll
        for (int j = 0; j < 4; ++j) umma_ss(tmem + st * 64, dX + so + (uint64_t)(j * 2), dW + (uint64_t)(j * 2), id, j > 0);
        umma_commit(&bars[bU + st]);
        umma_commit(&bars[bEmpty + st]);
      }
    }
  } else {
    const int quarter = warp & 3, row = quarter * 32 + lane, etid = tid - 64;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int i = 0; ok && i < ntile; ++i) {
      const int st = i & 1;
      int which;
      const int row0 = tile_row0(i, which);
      const uint8_t* mask = which ? row_mask2 : row_mask;
      if (!mbar_wait(&bars[bFull + st], (i >> 1) & 1)) { tc_fail(4); ok = false; break; }
      float ss = 0.f;                                  // |x|^2 of this thread's row
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 u = *reinterpret_cast<const uint4*>(sm + kX + st * kStage + row_chunk1(row, ch));
        float2 f;
        f = unpack_half2(u.x); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.y); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.z); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.w); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
      }
      mbar_arrive(&bars[bEmpty + st]);
      const float inv = 1.f / (sqrtf(ss) + kNormEps);
      if (!mbar_wait(&bars[bU + st], (i >> 1) & 1)) { tc_fail(5); ok = false; break; }
      tc_fence_after_sync();
      uint32_t u[64];
      tmem_ld32(tmem + lane_addr + st * 64, u);
      tmem_ld32(tmem + lane_addr + st * 64 + 32, u + 32);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bUFree + st]);
      if (i > 0) {                                     // the previous tile's store must have drained the staging tile
        if (etid == 0) tma_store_wait_read<0>();
        if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(6); ok = false; break; }
      }
      // a masked row (a padded key) gets all-zero features
      const float sc_row = (mask && (int64_t)row0 + row < rows && mask[(int64_t)row0 + row]) ? 0.f : scale;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float sn[8], cs[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          __sincosf(__uint_as_float(u[ch * 8 + e]) * inv, &sn[e], &cs[e]);
          sn[e] *= sc_row;
          cs[e] *= sc_row;
        }
        uint4 a, b;
        a.x = pack_half2(sn[0], sn[1]); a.y = pack_half2(sn[2], sn[3]); a.z = pack_half2(sn[4], sn[5]); a.w = pack_half2(sn[6], sn[7]);
        b.x = pack_half2(cs[0], cs[1]); b.y = pack_half2(cs[2], cs[3]); b.z = pack_half2(cs[4], cs[5]); b.w = pack_half2(cs[6], cs[7]);
        *reinterpret_cast<uint4*>(sm + kOut + row_chunk1(row, ch)) = a;            // sin block
        *reinterpret_cast<uint4*>(sm + kOut + kBox + row_chunk1(row, ch)) = b;     // cos block
      }
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(7); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(which ? &tm_phi2 : &tm_phi, sm + kOut, 0, h, row0);
        tma_store_3d(which ? &tm_phi2 : &tm_phi, sm + kOut + kBox, 64, h, row0);
        tma_store_commit();
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}

// x [rows][H][64] fp16, w [H][64][64] fp32, phi [rows][H][128] fp16; x2 / phi2 / row_mask2: a second array of the same
// shape sharing the launch (null: none)
int launch_feature_map_fwd_tc(const __half* x, const float* w, const uint8_t* row_mask, __half* phi, const __half* x2,
                              const uint8_t* row_mask2, __half* phi2, int64_t rows, int H, float scale, int sms, cudaStream_t st) {
  const int pair = x2 != nullptr;
  CUtensorMap tx, tp, tx2, tp2;
  if (make_tmap_rows(&tx, x, rows, H, 64, kTC) || make_tmap_rows(&tp, phi, rows, H, 128, kTC) ||
      make_tmap_rows(&tx2, pair ? x2 : x, rows, H, 64, kTC) || make_tmap_rows(&tp2, pair ? phi2 : phi, rows, H, 128, kTC))
    return fail(RFA_EDEVICE, "feature_map_fwd: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(feature_map_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fm::kSmem);
  if (e != cudaSuccess) return fail((int)e, "feature_map_fwd: cannot reserve %u bytes of shared memory: %s", fm::kSmem, cudaGetErrorString(e));
  const int64_t ntile = (rows + kTC - 1) / kTC * (pair ? 2 : 1);
  int64_t gx = 2LL * sms / H;                    // two CTAs per SM, and never more CTAs than fit at once
  if (gx > ntile) gx = ntile;
  if (gx < 1) gx = 1;
  feature_map_fwd_tc_kernel<<<dim3((unsigned)gx, H), fm::kThreads_, fm::kSmem, st>>>(tx, tp, tx2, tp2, w, row_mask, row_mask2, rows, H,
                                                                                     scale, pair);
  return check_launch("rfa_feature_map_fwd");
}


// ---------------------------------------------------------------------------------------------
// Feature map backward on tcgen05 for the same case (fp16, head_dim = proj_dim = 64).
// With inv = 1 / (|x| + 1e-3), u = (W x) inv and g_u = scale (g_sin cos u - g_cos sin u)   (upstream utils.py:100-120):
//     gh   = g_u inv                         fp16 tile [128 rows][64 j], written by epilogue group 1
//     gx'  = gh W                            (= (W^T g_u) inv)
//     g_x  = gx' - x (x . gx') inv / |x|
//     g_W += gh^T x                          accumulated over all row tiles of the CTA in tensor memory
// Three small MMA chains per tile of 128 rows: U = X W^T, gx' = gh W, g_W += gh^T X.  The last one has M = 64
// (rows j): it is issued with M = 128, the second 64-row block of its MN-major A operand being whatever tile
// follows gh in shared memory -- accumulator rows 64..127 are never read.
// HBM-bound: 384 bytes in, 128 bytes out per (row, head).
namespace fmb {
// warp 0 TMA, warp 1 MMA issuer, warps 2..5 and 6..9 group 1 (g_u: columns 0..31 and 32..63 of every row -- the sin/cos
// chain of a whole row in one thread was the slowest stage of the tile pipeline), warps 10..13 group 2 (g_x)
constexpr int kThreads_ = 448;
constexpr uint32_t kX = 0, kGP = kBox, kStage = 3 * kBox;          // per stage: x tile, g_phi tile (two boxes)
constexpr int kRing = 3;                       // staged tiles in flight: a stage lives through the tile's whole dependent chain
constexpr uint32_t kGH = kRing * kStage;       // two gh tiles; the output staging tile follows them
constexpr uint32_t kOut = kGH + 2 * kBox;
constexpr uint32_t kW = kOut + kBox;           // W  as [j][i] (K-major, contraction over i)
constexpr uint32_t kWt = kW + 8192;            // W^T as [i][j] (K-major, contraction over j)
constexpr uint32_t kRn = kWt + 8192;           // float2 [kRing][128]: (inv, inv / |x|) of the tile's rows, one set per stage
constexpr uint32_t kBarOff = kRn + kRing * 1024;
constexpr uint32_t kSmem = kBarOff + 256 + 1024;
constexpr uint32_t cU = 0, cGX = 128, cGW = 256;
enum { bFull = 0, bEmpty = 3, bU = 6, bUFree = 8, bGH = 10, bGHFree = 12, bGX = 14, bGXFree = 16, bEpi = 18, bDone = 19, bNum = 20 };
static_assert(kRing == 3 && bNum * 8 + 4 <= 256, "feature_map_bwd: barrier block");
}

__global__ void __launch_bounds__(fmb::kThreads_, 1)
feature_map_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_gp,
                          const __grid_constant__ CUtensorMap tm_gx, const __grid_constant__ CUtensorMap tm_x2,
                          const __grid_constant__ CUtensorMap tm_gp2, const __grid_constant__ CUtensorMap tm_gx2,
                          const float* __restrict__ w, float* __restrict__ g_w, const uint8_t* __restrict__ row_mask,
                          const uint8_t* __restrict__ row_mask2, int64_t rows, int H, float scale, int pair) {
  using namespace fmb;
  extern __shared__ unsigned char fmb_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fmb_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBarOff);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bNum);
  float2* rn = reinterpret_cast<float2*>(sm + kRn);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const bool want_gw = g_w != nullptr;
  // pair != 0: two arrays of the same shape share the launch, W_h and the g_W accumulator (q and k of one layer):
  // virtual tile v is row tile v / 2 of array v % 2
  const int ntile_all = (int)((rows + kTC - 1) / kTC) * (pair ? 2 : 1);
  const int ntile = blockIdx.x < ntile_all ? (ntile_all - 1 - blockIdx.x) / gridDim.x + 1 : 0;   // tiles blockIdx.x, +gridDim.x, ...
  auto tile_row0 = [&](int i, int& which) -> int {
    const int v = blockIdx.x + i * gridDim.x;
    which = pair ? (v & 1) : 0;
    return (pair ? (v >> 1) : v) * kTC;
  };
  if (tid == 0) {
    for (int i = 0; i < kRing; ++i) {
      mbar_init(&bars[bFull + i], 1);
      mbar_init(&bars[bEmpty + i], 385);       // the issuer's commit + the three epilogue groups
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&bars[bU + i], 1); mbar_init(&bars[bUFree + i], 256);
      mbar_init(&bars[bGH + i], 256); mbar_init(&bars[bGHFree + i], 1);
      mbar_init(&bars[bGX + i], 1); mbar_init(&bars[bGXFree + i], 128);
    }
    mbar_init(&bars[bEpi], 128); mbar_init(&bars[bDone], 1);
    mbar_fence_init();
    // the first tiles are requested before the rest of the prologue (W_h, tensor memory), which their flight then hides
    for (int i = 0; i < kRing && i < ntile; ++i) {
      int which;
      const int row0 = tile_row0(i, which);
      unsigned char* base = sm + i * kStage;
      mbar_arrive_expect_tx(&bars[bFull + i], kStage);
      tma_load_3d(base + kX, which ? &tm_x2 : &tm_x, &bars[bFull + i], 0, h, row0);
      tma_load_3d(base + kGP, which ? &tm_gp2 : &tm_gp, &bars[bFull + i], 0, h, row0);
      tma_load_3d(base + kGP + kBox, which ? &tm_gp2 : &tm_gp, &bars[bFull + i], 64, h, row0);
    }
    tma_prefetch_desc(&tm_gx);
  }
  // W_h as two fp16 K-major operand tiles: [j][i] and its transpose [i][j]
  for (int idx = tid; idx < 64 * 8; idx += kThreads_) {
    const int j = idx >> 3, ch = idx & 7;
    const float4 a = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8);
    const float4 b = *reinterpret_cast<const float4*>(w + ((size_t)h * 64 + j) * 64 + ch * 8 + 4);
    uint4 u;
    u.x = pack_half2(a.x, a.y); u.y = pack_half2(a.z, a.w); u.z = pack_half2(b.x, b.y); u.w = pack_half2(b.z, b.w);
    *reinterpret_cast<uint4*>(sm + kW + row_chunk1(j, ch)) = u;
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
    for (int e = 0; e < 8; ++e)                // element (i = ch * 8 + e, j) of the transposed tile
      *reinterpret_cast<__half*>(sm + kWt + sw128_offset(ch * 8 + e, j)) = __float2half_rn(v[e]);
  }
  fence_async_smem();
  if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0)
      for (int i = kRing; i < ntile; ++i) {
        const int sg = i % kRing;
        if (!mbar_wait(&bars[bEmpty + sg], ((i / kRing) + 1) & 1)) { tc_fail(11); break; }
        int which;
        const int row0 = tile_row0(i, which);
        unsigned char* base = sm + sg * kStage;
        mbar_arrive_expect_tx(&bars[bFull + sg], kStage);
        tma_load_3d(base + kX, which ? &tm_x2 : &tm_x, &bars[bFull + sg], 0, h, row0);
        tma_load_3d(base + kGP, which ? &tm_gp2 : &tm_gp, &bars[bFull + sg], 0, h, row0);
        tma_load_3d(base + kGP + kBox, which ? &tm_gp2 : &tm_gp, &bars[bFull + sg], 64, h, row0);
      }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t lead = 1u;
      constexpr uint32_t idKK = umma_idesc_f16(128, 64, false, false);     // X W^T ; gh W
      constexpr uint32_t idMM = umma_idesc_f16(128, 64, true, true);       // gh^T X
      const uint64_t dX = umma_smem_desc(sbase + kX, 0, 1024, kSwizzle128B);            // x, K-major [r][i]
      const uint64_t dXm = umma_smem_desc(sbase + kX, kBox, 1024, kSwizzle128B);        // x, MN-major (rows = contraction r)
      const uint64_t dW = umma_smem_desc(sbase + kW, 0, 1024, kSwizzle128B);
      const uint64_t dWt = umma_smem_desc(sbase + kWt, 0, 1024, kSwizzle128B);
      const uint64_t dGH = umma_smem_desc(sbase + kGH, 0, 1024, kSwizzle128B);          // gh, K-major [r][j]
      const uint64_t dGHm = umma_smem_desc(sbase + kGH, kBox, 1024, kSwizzle128B);      // gh, MN-major; second M block = next tile
      constexpr uint64_t kSt = kStage >> 4, kTile = kBox >> 4;
      auto issue_u = [&](int i) -> bool {
        const int st = i & 1, sg = i % kRing;
        if (!mbar_wait(&bars[bFull + sg], (i / kRing) & 1)) { tc_fail(12); return false; }
        if (i >= 2 && !mbar_wait(&bars[bUFree + st], ((i >> 1) + 1) & 1)) { tc_fail(13); return false; }
        tc_fence_after_sync();
        umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + cU + st * 64, dX + sg * kSt, dW, idKK, 0);
        umma_commit(&bars[bU + st]);
        return true;
      };
      bool ok = ntile > 0 ? issue_u(0) : true;
#pragma unroll 1
      for (int i = 0; ok && i < ntile; ++i) {
        const int st = i & 1, sg = i % kRing;
        if (i + 1 < ntile && !issue_u(i + 1)) break;
        if (!mbar_wait(&bars[bGH + st], (i >> 1) & 1)) { tc_fail(14); break; }
        if (i >= 2 && !mbar_wait(&bars[bGXFree + st], ((i >> 1) + 1) & 1)) { tc_fail(15); break; }
        tc_fence_after_sync();
        umma_chain_ss<4, kStepK, kBlockK, kStepK, kBlockK>(lead, tmem + cGX + st * 64, dGH + st * kTile, dWt, idKK, 0);   // gx' = gh W
        umma_commit(&bars[bGX + st]);
        if (want_gw)                                                                                                  // g_W += gh^T X
          umma_chain_ss<8, kStepMN, kBlockMN, kStepMN, kBlockMN>(lead, tmem + cGW, dGHm + st * kTile, dXm + sg * kSt, idMM, i > 0 ? 1u : 0u);
        umma_commit(&bars[bGHFree + st]);
        umma_commit(&bars[bEmpty + sg]);
      }
      umma_commit(&bars[bDone]);
    }
  } else if (warp < 10) {
    // ------------------------------------------------------------------ group 1: inv, u, g_u -> gh (half of the columns each)
    const int quarter = warp & 3, row = quarter * 32 + lane, half = (warp - 2) >> 2;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    for (int i = 0; i < ntile; ++i) {
      const int st = i & 1, sg = i % kRing;
      unsigned char* base = sm + sg * kStage;
      int which;
      const int64_t grow = (int64_t)tile_row0(i, which) + row;
      const uint8_t* mask = which ? row_mask2 : row_mask;
      // a masked row's features are constant zeros: no gradient flows through it
      const float scale_row = (mask && grow < rows && mask[grow]) ? 0.f : scale;
      if (!mbar_wait(&bars[bFull + sg], (i / kRing) & 1)) { tc_fail(16); break; }
      float ss = 0.f;                                  // |x|^2 of this thread's row
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 u = *reinterpret_cast<const uint4*>(base + kX + row_chunk1(row, ch));
        float2 f;
        f = unpack_half2(u.x); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.y); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.z); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
        f = unpack_half2(u.w); ss = fmaf(f.x, f.x, ss); ss = fmaf(f.y, f.y, ss);
      }
      const float n = sqrtf(ss), inv = 1.f / (n + kNormEps);
      if (!mbar_wait(&bars[bU + st], (i >> 1) & 1)) { tc_fail(17); break; }
      tc_fence_after_sync();
      uint32_t u[32];
      tmem_ld32(tmem + lane_addr + cU + st * 64 + half * 32, u);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bUFree + st]);
      // the gh tile of this parity was last read by the products of tile i - 2
      if (i >= 2 && !mbar_wait(&bars[bGHFree + st], ((i >> 1) + 1) & 1)) { tc_fail(18); break; }
      if (half == 0) rn[sg * 128 + row] = make_float2(inv, n > 0.f ? inv / n : 0.f);      // read by group 2 before it releases the stage
      const float sc = scale_row * inv;
#pragma unroll
      for (int c4 = 0; c4 < 4; ++c4) {
        const int ch = half * 4 + c4;
        const uint4 gs = *reinterpret_cast<const uint4*>(base + kGP + row_chunk1(row, ch));          // g_sin, columns 8 ch ..
        const uint4 gc = *reinterpret_cast<const uint4*>(base + kGP + kBox + row_chunk1(row, ch));   // g_cos
        const uint32_t gsw[4] = {gs.x, gs.y, gs.z, gs.w}, gcw[4] = {gc.x, gc.y, gc.z, gc.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 a = unpack_half2(gsw[e]), b = unpack_half2(gcw[e]);
          float s0, c0, s1, c1;
          __sincosf(__uint_as_float(u[c4 * 8 + 2 * e]) * inv, &s0, &c0);
          __sincosf(__uint_as_float(u[c4 * 8 + 2 * e + 1]) * inv, &s1, &c1);
          o[e] = pack_half2(sc * (a.x * c0 - b.x * s0), sc * (a.y * c1 - b.y * s1));
        }
        *reinterpret_cast<uint4*>(sm + kGH + st * kBox + row_chunk1(row, ch)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      fence_async_smem();
      mbar_arrive(&bars[bGH + st]);
      mbar_arrive(&bars[bEmpty + sg]);                 // this group's reads of the stage are done
    }
  } else {
    // ------------------------------------------------------------------ group 2: g_x
    const int quarter = warp & 3, row = quarter * 32 + lane, etid = tid - 320;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    uint32_t epi_phase = 0;
    bool ok = true;
    for (int i = 0; ok && i < ntile; ++i) {
      const int st = i & 1, sg = i % kRing;
      unsigned char* base = sm + sg * kStage;
      int which;
      const int row0 = tile_row0(i, which);
      if (!mbar_wait(&bars[bFull + sg], (i / kRing) & 1)) { tc_fail(19); ok = false; break; }
      // gx' of this tile exists only after the issuer saw group 1's gh, which group 1 signalled after writing rn: waiting
      // for the product orders the read of rn too.  (Group 1 may run two tiles ahead of this group, so this group must
      // not wait on bGH: that barrier can complete twice before this group looks.)
      if (!mbar_wait(&bars[bGX + st], (i >> 1) & 1)) { tc_fail(21); ok = false; break; }
      tc_fence_after_sync();
      uint32_t gx[64];
      tmem_ld32(tmem + lane_addr + cGX + st * 64, gx);
      tmem_ld32(tmem + lane_addr + cGX + st * 64 + 32, gx + 32);
      tmem_ld_wait();
      tc_fence_before_sync();
      mbar_arrive(&bars[bGXFree + st]);
      const float2 r2 = rn[sg * 128 + row];
      float dot = 0.f;
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 xu = *reinterpret_cast<const uint4*>(base + kX + row_chunk1(row, ch));
        const uint32_t xw[4] = {xu.x, xu.y, xu.z, xu.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_half2(xw[e]);
          dot = fmaf(f.x, __uint_as_float(gx[ch * 8 + 2 * e]), dot);
          dot = fmaf(f.y, __uint_as_float(gx[ch * 8 + 2 * e + 1]), dot);
        }
      }
      const float c2 = dot * r2.y;                     // (x . gx') inv / |x|
      if (i > 0) {                                     // the previous tile's store must have drained the staging tile
        if (etid == 0) tma_store_wait_read<0>();
        if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(22); ok = false; break; }
      }
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        const uint4 xu = *reinterpret_cast<const uint4*>(base + kX + row_chunk1(row, ch));   // read again rather than held: registers
        const uint32_t xw[4] = {xu.x, xu.y, xu.z, xu.w};
        uint32_t o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = unpack_half2(xw[e]);
          o[e] = pack_half2(__uint_as_float(gx[ch * 8 + 2 * e]) - f.x * c2, __uint_as_float(gx[ch * 8 + 2 * e + 1]) - f.y * c2);
        }
        *reinterpret_cast<uint4*>(sm + kOut + row_chunk1(row, ch)) = make_uint4(o[0], o[1], o[2], o[3]);
      }
      mbar_arrive(&bars[bEmpty + sg]);                 // this group's reads of the stage are done
      fence_async_smem();
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(23); ok = false; break; }
      if (etid == 0) {
        tma_store_3d(which ? &tm_gx2 : &tm_gx, sm + kOut, 0, h, row0);
        tma_store_commit();
      }
    }
    // ---- g_W of this CTA's tiles: rows j = 0..63 of the accumulator, transposed through shared memory (the first stage:
    // every load has been consumed once bDone fires) so that a warp's atomics fall on consecutive addresses
    if (ok && want_gw && ntile > 0) {
      float* tr = reinterpret_cast<float*>(sm);            // [64][65] floats
      if (!mbar_wait(&bars[bDone], 0)) { tc_fail(24); ok = false; }
      if (ok && row < 64) {
        tc_fence_after_sync();
        uint32_t gw[64];
        tmem_ld32(tmem + lane_addr + cGW, gw);
        tmem_ld32(tmem + lane_addr + cGW + 32, gw + 32);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 64; ++e) tr[row * 65 + e] = __uint_as_float(gw[e]);
      }
      if (!epi_sync(&bars[bEpi], epi_phase)) { tc_fail(25); ok = false; }
      if (ok) {
        float* dst = g_w + (size_t)h * 64 * 64;
#pragma unroll 4
        for (int idx = etid; idx < 64 * 64; idx += 128) atomicAdd(dst + idx, tr[(idx >> 6) * 65 + (idx & 63)]);
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 512);
}

// x, g_x [rows][H][64] fp16, g_phi [rows][H][128] fp16, w [H][64][64] fp32, g_w [H][64][64] fp32 accumulated into (may be null);
// x2 / g_phi2 / g_x2 / row_mask2: a second set of arrays of the same shape sharing the launch and g_w (x2 null: none)
int launch_feature_map_bwd_tc(const __half* x, const float* w, const uint8_t* row_mask, const __half* g_phi, __half* g_x,
                              const __half* x2, const uint8_t* row_mask2, const __half* g_phi2, __half* g_x2, float* g_w,
                              int64_t rows, int H, float scale, int sms, cudaStream_t st) {
  const int pair = x2 != nullptr;
  CUtensorMap tx, tg, to, tx2, tg2, to2;
  if (make_tmap_rows(&tx, x, rows, H, 64, kTC) || make_tmap_rows(&tg, g_phi, rows, H, 128, kTC) || make_tmap_rows(&to, g_x, rows, H, 64, kTC) ||
      make_tmap_rows(&tx2, pair ? x2 : x, rows, H, 64, kTC) || make_tmap_rows(&tg2, pair ? g_phi2 : g_phi, rows, H, 128, kTC) ||
      make_tmap_rows(&to2, pair ? g_x2 : g_x, rows, H, 64, kTC))
    return fail(RFA_EDEVICE, "feature_map_bwd: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(feature_map_bwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fmb::kSmem);
  if (e != cudaSuccess) return fail((int)e, "feature_map_bwd: cannot reserve %u bytes of shared memory: %s", fmb::kSmem, cudaGetErrorString(e));
  const int64_t ntile = (rows + kTC - 1) / kTC * (pair ? 2 : 1);
  int64_t gx = sms / H;                          // one CTA per SM (shared memory): never more CTAs than SMs, or a second wave runs
  if (gx > ntile) gx = ntile;
  if (gx < 1) gx = 1;
  feature_map_bwd_tc_kernel<<<dim3((unsigned)gx, H), fmb::kThreads_, fmb::kSmem, st>>>(tx, tg, to, tx2, tg2, to2, w, g_w, row_mask,
                                                                                        row_mask2, rows, H, scale, pair);
  return check_launch("rfa_feature_map_bwd");
}

RFA_TC_UNIT(feature_map)

}  // namespace rfa
