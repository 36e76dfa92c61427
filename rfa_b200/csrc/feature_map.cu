// Fused random feature map and its gradient.
//
//   n = |x|_2,  xh = x / (n + 1e-3),  u = W_h xh,  phi = scale * [sin u | cos u]
// (upstream utils.py:100-120, one pass instead of norm/div/einsum/sin/cos/cat/mul).
// x [rows,H,d], W [H,D,d] fp32, phi [rows,H,2D].  One CTA owns one head and walks
// tiles of R rows with that head's W resident in shared memory; each x element is
// read once and each phi element written once with 16-byte accesses.
#include "common.cuh"

namespace rfa {

constexpr int kFmThreads = 256;

struct FmSmem {
  float* W;    // [D][d+1]
  float* X;    // [R][d+1]   normalised rows
  float* U;    // [R][LU]    projections / reused for g_xh
  float* GU;   // [R][LU]    (backward)
  float* GW;   // [D][d+1]   (backward, optional)
  float* nrm;  // [R]
};

// row stride of the U / GU buffers: they hold [R][D] projections and later [R][d] g_xh
__host__ __device__ inline int fm_ldu(int D, int d) { return (D > d ? D : d) + 1; }

__host__ __device__ inline size_t fm_smem_floats(int R, int D, int d, bool bwd, bool gw) {
  const int LU = fm_ldu(D, d);
  size_t n = (size_t)D * (d + 1) + (size_t)R * (d + 1) + (size_t)R * LU + R;
  if (bwd) n += (size_t)R * LU;
  if (bwd && gw) n += (size_t)D * (d + 1);
  return n;
}

__device__ __forceinline__ FmSmem fm_carve(float* base, int R, int D, int d, bool bwd, bool gw) {
  const int LU = fm_ldu(D, d);
  FmSmem s;
  s.W = base;
  s.X = s.W + D * (d + 1);
  s.U = s.X + R * (d + 1);
  s.nrm = s.U + R * LU;
  s.GU = s.nrm + R;
  s.GW = s.GU + (bwd ? R * LU : 0);
  return s;
}

// Load + normalise R rows of this head into s.X (zero rows past the end).
template <typename TX>
__device__ __forceinline__ void fm_load_rows(const FmSmem& s, const TX* __restrict__ x, int64_t row0,
                                             int64_t rows, int R, int H, int h, int d) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int r = warp; r < R; r += kFmThreads / 32) {
    const int64_t row = row0 + r;
    float ss = 0.f;
    if (row < rows) {
      const TX* src = x + ((size_t)row * H + h) * d;
      for (int i = lane; i < d; i += 32) {
        float t = to_f(src[i]);
        s.X[r * (d + 1) + i] = t;
        ss = fmaf(t, t, ss);
      }
    } else {
      for (int i = lane; i < d; i += 32) s.X[r * (d + 1) + i] = 0.f;
    }
    ss = warp_sum(ss);
    const float n = sqrtf(ss);
    const float inv = 1.f / (n + kNormEps);
    for (int i = lane; i < d; i += 32) s.X[r * (d + 1) + i] *= inv;
    if (lane == 0) s.nrm[r] = n;
  }
}

template <typename TX, typename TP>
__global__ void __launch_bounds__(kFmThreads)
feature_map_fwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, const uint8_t* __restrict__ row_mask,
                       TP* __restrict__ phi, int64_t rows, int H, int d, int D, float scale, int R) {
  extern __shared__ __align__(16) float fm_smem[];
  const FmSmem s = fm_carve(fm_smem, R, D, d, false, false);
  const int LU = fm_ldu(D, d);
  const int h = blockIdx.y;
  const float* wh = w + (size_t)h * D * d;
  for (int i = threadIdx.x; i < D * d; i += kFmThreads) s.W[(i / d) * (d + 1) + (i % d)] = wh[i];
  const int64_t ntiles = (rows + R - 1) / R;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t row0 = tile * R;
    __syncthreads();
    fm_load_rows(s, x, row0, rows, R, H, h, d);
    __syncthreads();
    tile_gemm<4, 4>(R, D, d,
                    [&](int r, int l) { return s.X[r * (d + 1) + l]; },
                    [&](int l, int j) { return s.W[j * (d + 1) + l]; },
                    [&](int r, int j, float v) { s.U[r * LU + j] = v; });
    __syncthreads();
    const int groups = D / 8;
    for (int idx = threadIdx.x; idx < R * groups; idx += kFmThreads) {
      const int r = idx / groups, j0 = (idx % groups) * 8;
      const int64_t row = row0 + r;
      if (row >= rows) continue;
      float sn[8], cs[8];
      const float sc_row = (row_mask && row_mask[row]) ? 0.f : scale;     // a masked row gets all-zero features
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        sincosf(s.U[r * LU + j0 + e], &sn[e], &cs[e]);
        sn[e] *= sc_row;
        cs[e] *= sc_row;
      }
      TP* dst = phi + ((size_t)row * H + h) * 2 * D + j0;
      if constexpr (sizeof(TP) == 2) {
        store8(dst, sn);
        store8(dst + D, cs);
      } else {
        store4(dst, make_float4(sn[0], sn[1], sn[2], sn[3]));
        store4(dst + 4, make_float4(sn[4], sn[5], sn[6], sn[7]));
        store4(dst + D, make_float4(cs[0], cs[1], cs[2], cs[3]));
        store4(dst + D + 4, make_float4(cs[4], cs[5], cs[6], cs[7]));
      }
    }
  }
}

// Backward.  With g_u = scale * (g_sin * cos u - g_cos * sin u):
//   g_xh = W^T g_u;  g_x = g_xh / (n + eps) - xh * (xh . g_xh) / n;  g_W += g_u (x) xh
template <typename TX, typename TG, typename TO>
__global__ void __launch_bounds__(kFmThreads)
feature_map_bwd_kernel(const TX* __restrict__ x, const float* __restrict__ w, const uint8_t* __restrict__ row_mask,
                       const TG* __restrict__ g_phi, TO* __restrict__ g_x, float* __restrict__ g_w,
                       int64_t rows, int H, int d, int D, float scale, int R) {
  extern __shared__ __align__(16) float fm_smem[];
  const bool want_gw = g_w != nullptr;
  const FmSmem s = fm_carve(fm_smem, R, D, d, true, want_gw);
  const int LU = fm_ldu(D, d);
  const int h = blockIdx.y;
  const float* wh = w + (size_t)h * D * d;
  for (int i = threadIdx.x; i < D * d; i += kFmThreads) {
    s.W[(i / d) * (d + 1) + (i % d)] = wh[i];
    if (want_gw) s.GW[(i / d) * (d + 1) + (i % d)] = 0.f;
  }
  const int64_t ntiles = (rows + R - 1) / R;
  for (int64_t tile = blockIdx.x; tile < ntiles; tile += gridDim.x) {
    const int64_t row0 = tile * R;
    __syncthreads();
    fm_load_rows(s, x, row0, rows, R, H, h, d);
    __syncthreads();
    tile_gemm<4, 4>(R, D, d,
                    [&](int r, int l) { return s.X[r * (d + 1) + l]; },
                    [&](int l, int j) { return s.W[j * (d + 1) + l]; },
                    [&](int r, int j, float v) { s.U[r * LU + j] = v; });
    __syncthreads();
    for (int idx = threadIdx.x; idx < R * D; idx += kFmThreads) {
      const int r = idx / D, j = idx % D;
      const int64_t row = row0 + r;
      float gu = 0.f;
      if (row < rows && !(row_mask && row_mask[row])) {     // a masked row's features are constants: no gradient
        float sn, cs;
        sincosf(s.U[r * LU + j], &sn, &cs);
        const TG* gp = g_phi + ((size_t)row * H + h) * 2 * D;
        gu = scale * (to_f(gp[j]) * cs - to_f(gp[D + j]) * sn);
      }
      s.GU[r * LU + j] = gu;
    }
    __syncthreads();
    // g_xh -> s.U (projections no longer needed)
    tile_gemm<4, 4>(R, d, D,
                    [&](int r, int l) { return s.GU[r * LU + l]; },
                    [&](int l, int i) { return s.W[l * (d + 1) + i]; },
                    [&](int r, int i, float v) { s.U[r * LU + i] = v; });
    if (want_gw)
      tile_gemm<4, 4>(D, d, R,
                      [&](int j, int l) { return s.GU[l * LU + j]; },
                      [&](int l, int i) { return s.X[l * (d + 1) + i]; },
                      [&](int j, int i, float v) { s.GW[j * (d + 1) + i] += v; });
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int r = warp; r < R; r += kFmThreads / 32) {
      const int64_t row = row0 + r;
      if (row >= rows) continue;
      float dot = 0.f;
      for (int i = lane; i < d; i += 32) dot = fmaf(s.X[r * (d + 1) + i], s.U[r * LU + i], dot);
      dot = warp_sum(dot);
      const float n = s.nrm[r];
      const float inv = 1.f / (n + kNormEps);
      const float c2 = n > 0.f ? dot / n : 0.f;
      TO* dst = g_x + ((size_t)row * H + h) * d;
      for (int i = lane; i < d; i += 32)
        dst[i] = from_f<TO>(s.U[r * LU + i] * inv - s.X[r * (d + 1) + i] * c2);
    }
  }
  if (want_gw) {
    __syncthreads();
    float* gwh = g_w + (size_t)h * D * d;
    for (int i = threadIdx.x; i < D * d; i += kFmThreads) atomicAdd(gwh + i, s.GW[(i / d) * (d + 1) + (i % d)]);
  }
}

// tensor-core forward for fp16 rows with head_dim = proj_dim = 64 (feature_map_tc.cu)
int launch_feature_map_fwd_tc(const __half* x, const float* w, const uint8_t* row_mask, __half* phi, const __half* x2,
                              const uint8_t* row_mask2, __half* phi2, int64_t rows, int H, float scale, int sms, cudaStream_t st);
int launch_feature_map_bwd_tc(const __half* x, const float* w, const uint8_t* row_mask, const __half* g_phi, __half* g_x,
                              const __half* x2, const uint8_t* row_mask2, const __half* g_phi2, __half* g_x2, float* g_w,
                              int64_t rows, int H, float scale, int sms, cudaStream_t st);

static int fm_check(const void* x, const float* w, int64_t rows, int H, int d, int D) {
  RFA_REQUIRE(x && w, RFA_EINVAL, "feature_map: null pointer");
  RFA_REQUIRE(rows >= 0 && H > 0 && d > 0 && D > 0, RFA_EINVAL, "feature_map: rows=%lld H=%d d=%d D=%d",
              (long long)rows, H, d, D);
  RFA_REQUIRE(d % 8 == 0 && D % 8 == 0 && d <= 128 && D <= 128, RFA_EUNSUPPORTED,
              "feature_map: need d%%8==0, D%%8==0, d<=128, D<=128 (got d=%d D=%d)", d, D);
  RFA_REQUIRE(H <= 65535, RFA_EUNSUPPORTED, "feature_map: H=%d exceeds 65535", H);
  return 0;
}

static int fm_pick_rows(int D, int d, bool bwd, bool gw, size_t* bytes) {
  for (int R = 64; R >= 16; R >>= 1) {
    size_t b = fm_smem_floats(R, D, d, bwd, gw) * sizeof(float);
    if (b <= 200 * 1024) { *bytes = b; return R; }
  }
  return 0;
}

static int fm_grid_x(int64_t ntiles, int H) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int64_t want = (2LL * sms + H - 1) / H;   // about two CTAs per SM over all heads
  if (want < 1) want = 1;
  return (int)(ntiles < want ? ntiles : want);
}

}  // namespace rfa

using namespace rfa;

extern "C" int rfa_feature_map_fwd_masked(const void* x, int x_dtype, const float* w, const uint8_t* row_mask, void* phi,
                                          int phi_dtype, int64_t rows, int H, int d, int D, float scale, rfa_stream_t stream) {
  if (int e = fm_check(x, w, rows, H, d, D)) return e;
  RFA_REQUIRE(phi, RFA_EINVAL, "feature_map_fwd: null output");
  RFA_REQUIRE(aligned16(x) && aligned16(w) && aligned16(phi), RFA_EALIGN, "feature_map_fwd: 16-byte alignment required");
  if (rows == 0) return 0;
  if (x_dtype == RFA_F16 && phi_dtype == RFA_F16 && d == 64 && D == 64) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return launch_feature_map_fwd_tc((const __half*)x, w, row_mask, (__half*)phi, nullptr, nullptr, nullptr, rows, H, scale, sms,
                                     as_stream(stream));
  }
  size_t smem = 0;
  const int R = fm_pick_rows(D, d, false, false, &smem);
  RFA_REQUIRE(R > 0, RFA_EUNSUPPORTED, "feature_map_fwd: shared memory budget exceeded");
  dim3 grid(fm_grid_x((rows + R - 1) / R, H), H);
  cudaStream_t st = as_stream(stream);
#define RFA_LAUNCH(TX, TP)                                                                         \
  do {                                                                                             \
    cudaFuncSetAttribute(feature_map_fwd_kernel<TX, TP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    feature_map_fwd_kernel<TX, TP><<<grid, kFmThreads, smem, st>>>((const TX*)x, w, row_mask, (TP*)phi, rows, H, d, D, scale, R); \
  } while (0)
  if (x_dtype == RFA_F16 && phi_dtype == RFA_F16) RFA_LAUNCH(__half, __half);
  else if (x_dtype == RFA_F32 && phi_dtype == RFA_F32) RFA_LAUNCH(float, float);
  else if (x_dtype == RFA_F16 && phi_dtype == RFA_F32) RFA_LAUNCH(__half, float);
  else if (x_dtype == RFA_F32 && phi_dtype == RFA_F16) RFA_LAUNCH(float, __half);
  else return fail(RFA_EUNSUPPORTED, "feature_map_fwd: bad dtype %d/%d", x_dtype, phi_dtype);
#undef RFA_LAUNCH
  return check_launch("rfa_feature_map_fwd");
}

extern "C" int rfa_feature_map_fwd(const void* x, int x_dtype, const float* w, void* phi, int phi_dtype,
                                   int64_t rows, int H, int d, int D, float scale, rfa_stream_t stream) {
  return rfa_feature_map_fwd_masked(x, x_dtype, w, nullptr, phi, phi_dtype, rows, H, d, D, scale, stream);
}

extern "C" int rfa_feature_map_bwd_masked(const void* x, int x_dtype, const float* w, const uint8_t* row_mask, const void* g_phi,
                                          int g_dtype, void* g_x, int gx_dtype, float* g_w, int64_t rows, int H, int d, int D,
                                          float scale, rfa_stream_t stream) {
  if (int e = fm_check(x, w, rows, H, d, D)) return e;
  RFA_REQUIRE(g_phi && g_x, RFA_EINVAL, "feature_map_bwd: null pointer");
  RFA_REQUIRE(aligned16(x) && aligned16(w) && aligned16(g_phi) && aligned16(g_x) && aligned16(g_w), RFA_EALIGN,
              "feature_map_bwd: 16-byte alignment required");
  RFA_REQUIRE(x_dtype == g_dtype && x_dtype == gx_dtype, RFA_EUNSUPPORTED,
              "feature_map_bwd: x, g_phi and g_x must share one dtype");
  if (rows == 0) return 0;
  if (x_dtype == RFA_F16 && d == 64 && D == 64) {
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    return launch_feature_map_bwd_tc((const __half*)x, w, row_mask, (const __half*)g_phi, (__half*)g_x, nullptr, nullptr, nullptr,
                                     nullptr, g_w, rows, H, scale, sms, as_stream(stream));
  }
  size_t smem = 0;
  const int R = fm_pick_rows(D, d, true, g_w != nullptr, &smem);
  RFA_REQUIRE(R > 0, RFA_EUNSUPPORTED, "feature_map_bwd: shared memory budget exceeded");
  dim3 grid(fm_grid_x((rows + R - 1) / R, H), H);
  cudaStream_t st = as_stream(stream);
#define RFA_LAUNCH(T)                                                                              \
  do {                                                                                             \
    cudaFuncSetAttribute(feature_map_bwd_kernel<T, T, T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    feature_map_bwd_kernel<T, T, T><<<grid, kFmThreads, smem, st>>>((const T*)x, w, row_mask, (const T*)g_phi, (T*)g_x, g_w, \
                                                                    rows, H, d, D, scale, R);      \
  } while (0)
  if (x_dtype == RFA_F16) RFA_LAUNCH(__half);
  else if (x_dtype == RFA_F32) RFA_LAUNCH(float);
  else return fail(RFA_EUNSUPPORTED, "feature_map_bwd: bad dtype %d", x_dtype);
#undef RFA_LAUNCH
  return check_launch("rfa_feature_map_bwd");
}

extern "C" int rfa_feature_map_bwd(const void* x, int x_dtype, const float* w, const void* g_phi, int g_dtype,
                                   void* g_x, int gx_dtype, float* g_w, int64_t rows, int H, int d, int D,
                                   float scale, rfa_stream_t stream) {
  return rfa_feature_map_bwd_masked(x, x_dtype, w, nullptr, g_phi, g_dtype, g_x, gx_dtype, g_w, rows, H, d, D, scale, stream);
}

// The feature maps of two arrays of one shape that share W (q and k of a self-attention layer) in one launch: one ramp
// and one W tile instead of two, and in the backward one g_W accumulator for both.  fp16, head_dim = proj_dim = 64 only
// (RFA_EUNSUPPORTED otherwise: call the single-array entry points twice).
extern "C" int rfa_feature_map_fwd_pair(const void* x_a, const void* x_b, const float* w, const uint8_t* row_mask_a,
                                        const uint8_t* row_mask_b, void* phi_a, void* phi_b, int64_t rows, int H, int d, int D,
                                        float scale, rfa_stream_t stream) {
  if (int e = fm_check(x_a, w, rows, H, d, D)) return e;
  RFA_REQUIRE(d == 64 && D == 64, RFA_EUNSUPPORTED, "feature_map_fwd_pair: built for head_dim = proj_dim = 64, fp16 (got %d, %d)", d, D);
  RFA_REQUIRE(rows == 0 || (x_b && phi_a && phi_b), RFA_EINVAL, "feature_map_fwd_pair: null pointer");
  RFA_REQUIRE(aligned16(x_a) && aligned16(x_b) && aligned16(w) && aligned16(phi_a) && aligned16(phi_b), RFA_EALIGN,
              "feature_map_fwd_pair: 16-byte alignment required");
  if (rows == 0) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return launch_feature_map_fwd_tc((const __half*)x_a, w, row_mask_a, (__half*)phi_a, (const __half*)x_b, row_mask_b, (__half*)phi_b,
                                   rows, H, scale, sms, as_stream(stream));
}

extern "C" int rfa_feature_map_bwd_pair(const void* x_a, const void* x_b, const float* w, const uint8_t* row_mask_a,
                                        const uint8_t* row_mask_b, const void* g_phi_a, const void* g_phi_b, void* g_x_a,
                                        void* g_x_b, float* g_w, int64_t rows, int H, int d, int D, float scale,
                                        rfa_stream_t stream) {
  if (int e = fm_check(x_a, w, rows, H, d, D)) return e;
  RFA_REQUIRE(d == 64 && D == 64, RFA_EUNSUPPORTED, "feature_map_bwd_pair: built for head_dim = proj_dim = 64, fp16 (got %d, %d)", d, D);
  RFA_REQUIRE(rows == 0 || (x_b && g_phi_a && g_phi_b && g_x_a && g_x_b), RFA_EINVAL, "feature_map_bwd_pair: null pointer");
  RFA_REQUIRE(aligned16(x_a) && aligned16(x_b) && aligned16(w) && aligned16(g_phi_a) && aligned16(g_phi_b) && aligned16(g_x_a) &&
                  aligned16(g_x_b) && aligned16(g_w), RFA_EALIGN, "feature_map_bwd_pair: 16-byte alignment required");
  if (rows == 0) return 0;
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  return launch_feature_map_bwd_tc((const __half*)x_a, w, row_mask_a, (const __half*)g_phi_a, (__half*)g_x_a, (const __half*)x_b,
                                   row_mask_b, (const __half*)g_phi_b, (__half*)g_x_b, g_w, rows, H, scale, sms, as_stream(stream));
}

// ---------------------------------------------------------------------------
// Effective random matrices of a whole step in one launch: out[i] = sigma[i] * bank[idx[i]] * inv_tau[i]
// (upstream gathers the sampled matrices on the host, utils.py:62-87, and applies sigma / tau per layer with separate
// PyTorch ops, utils.py:90-97).  bank [n_bank, D, d] fp16 or fp32 stays resident on the device.
// ---------------------------------------------------------------------------
namespace rfa {
template <typename TB>
__global__ void gather_matrices_kernel(const TB* __restrict__ bank, int64_t n_bank, const int64_t* __restrict__ idx,
                                       const float* __restrict__ sigma, const float* __restrict__ inv_tau,
                                       float* __restrict__ out, int64_t n_out, int D, int d, int* __restrict__ bad) {
  const int64_t per = (int64_t)D * d;
  const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n_out * per) return;
  const int64_t i = e / per, r = e % per;
  const int64_t src = idx[i];
  if (src < 0 || src >= n_bank) {          // a pick outside the bank: flag it and write zeros instead of reading out of bounds
    if (r == 0) atomicExch(bad, 1);
    out[e] = 0.f;
    return;
  }
  float w = to_f(bank[src * per + r]);
  if (sigma) w *= sigma[i * d + r % d];
  if (inv_tau) w *= inv_tau[i];
  out[e] = w;
}
}  // namespace rfa

extern "C" int rfa_gather_random_matrices(const void* bank, int bank_dtype, int64_t n_bank, const int64_t* idx, int64_t n_out,
                                          const float* sigma, const float* inv_tau, float* out, int D, int d, int* bad_index_flag,
                                          rfa_stream_t stream) {
  RFA_REQUIRE(bank && idx && out && bad_index_flag, RFA_EINVAL, "gather_random_matrices: null pointer");
  RFA_REQUIRE(n_bank > 0 && n_out >= 0 && D > 0 && d > 0, RFA_EINVAL, "gather_random_matrices: n_bank=%lld n_out=%lld D=%d d=%d",
              (long long)n_bank, (long long)n_out, D, d);
  RFA_REQUIRE(bank_dtype == RFA_F16 || bank_dtype == RFA_F32, RFA_EUNSUPPORTED, "gather_random_matrices: bank dtype %d", bank_dtype);
  if (n_out == 0) return 0;
  const int64_t total = n_out * D * d;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (bank_dtype == RFA_F16)
    gather_matrices_kernel<__half><<<blocks, 256, 0, as_stream(stream)>>>((const __half*)bank, n_bank, idx, sigma, inv_tau, out, n_out, D, d, bad_index_flag);
  else
    gather_matrices_kernel<float><<<blocks, 256, 0, as_stream(stream)>>>((const float*)bank, n_bank, idx, sigma, inv_tau, out, n_out, D, d, bad_index_flag);
  return check_launch("rfa_gather_random_matrices");
}
