// Feature map forward on tcgen05 for the fp16, head_dim = proj_dim = 64 case:
//   phi = scale * [sin(u) | cos(u)],  u = (W_h x) / (|x| + 1e-3)        (upstream utils.py:100-120)
// The projection of a tile of 128 rows of one head is one small MMA chain (M128 N64 K64) on the RAW
// rows; the normalisation commutes with the projection and is applied to the fp32 result, so the
// staged x tile is never rewritten.  One CTA owns one head (W_h resident as an fp16 operand tile)
// and walks row tiles with a two-stage TMA ring; phi leaves through a staging tile and a TMA store.
// HBM-bound: 128 bytes in, 256 bytes out per (row, head).
#include "tc_common.cuh"

namespace rfa {
namespace fm {
constexpr int kThreads_ = 192;
constexpr uint32_t kX = 0, kStage = kBox, kW = 2 * kStage, kOut = kW + 8192, kBarOff = kOut + 2 * kBox, kSmem = kBarOff + 128 + 1024;
enum { bFull = 0, bEmpty = 2, bU = 4, bUFree = 6, bEpi = 8, bNum = 9 };
}

__global__ void __launch_bounds__(fm::kThreads_, 2)
feature_map_fwd_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_phi,
                          const float* __restrict__ w, int64_t rows, int H, float scale) {
  using namespace fm;
  extern __shared__ unsigned char fm_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(fm_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kBarOff);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + bNum);
  const uint32_t sbase = smem_u32(sm);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int ntile_all = (int)((rows + kTC - 1) / kTC);
  const int ntile = blockIdx.x < ntile_all ? (ntile_all - 1 - blockIdx.x) / gridDim.x + 1 : 0;   // tiles blockIdx.x, +gridDim.x, ...
  if (tid == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&bars[bFull + i], 1); mbar_init(&bars[bEmpty + i], 129); mbar_init(&bars[bU + i], 1); mbar_init(&bars[bUFree + i], 128); }
    mbar_init(&bars[bEpi], 128);
    mbar_fence_init();
    tma_prefetch_desc(&tm_x); tma_prefetch_desc(&tm_phi);
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
      for (int i = 0; i < ntile; ++i) {
        const int st = i & 1;
        if (i >= 2 && !mbar_wait(&bars[bEmpty + st], ((i >> 1) + 1) & 1)) { tc_fail(1); break; }
        const int row0 = (blockIdx.x + i * gridDim.x) * kTC;
        mbar_arrive_expect_tx(&bars[bFull + st], kBox);
        tma_load_3d(sm + kX + st * kStage, &tm_x, &bars[bFull + st], 0, h, row0);
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
      const int row0 = (blockIdx.x + i * gridDim.x) * kTC;
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
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) {
        float sn[8], cs[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          __sincosf(__uint_as_float(u[ch * 8 + e]) * inv, &sn[e], &cs[e]);
          sn[e] *= scale;
          cs[e] *= scale;
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
        tma_store_3d(&tm_phi, sm + kOut, 0, h, row0);
        tma_store_3d(&tm_phi, sm + kOut + kBox, 64, h, row0);
        tma_store_commit();
      }
    }
    if (etid == 0) tma_store_wait<0>();
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem, 128);
}

// x [rows][H][64] fp16, w [H][64][64] fp32, phi [rows][H][128] fp16
int launch_feature_map_fwd_tc(const __half* x, const float* w, __half* phi, int64_t rows, int H, float scale, int sms, cudaStream_t st) {
  CUtensorMap tx, tp;
  if (make_tmap_rows(&tx, x, rows, H, 64, kTC) || make_tmap_rows(&tp, phi, rows, H, 128, kTC))
    return fail(RFA_EDEVICE, "feature_map_fwd: cuTensorMapEncodeTiled failed or is unavailable");
  cudaError_t e = cudaFuncSetAttribute(feature_map_fwd_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)fm::kSmem);
  if (e != cudaSuccess) return fail((int)e, "feature_map_fwd: cannot reserve %u bytes of shared memory: %s", fm::kSmem, cudaGetErrorString(e));
  const int64_t ntile = (rows + kTC - 1) / kTC;
  int64_t gx = (2LL * sms + H - 1) / H;
  if (gx > ntile) gx = ntile;
  if (gx < 1) gx = 1;
  feature_map_fwd_tc_kernel<<<dim3((unsigned)gx, H), fm::kThreads_, fm::kSmem, st>>>(tx, tp, w, rows, H, scale);
  return check_launch("rfa_feature_map_fwd");
}

int tc_status_feature_map() { return tc_status_read_clear(); }

}  // namespace rfa
