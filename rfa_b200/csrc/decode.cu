// Single-token incremental decoding step: streams the per-head state once.
//
// Per (batch, head):  s += phi_k (x) v;  z += phi_k;  out = phi_q.s / max(phi_q.z, 1)
// (upstream causal_attention.py:42-50).  The state s [K,d] is read and written
// exactly once with 16-byte (fp32) / 8-byte (fp16) accesses; a warp covers whole
// 128-byte lines.  One CTA per (batch, head); HBM-bound: 2*K*d*sizeof(state)
// bytes per head per token.
#include "common.cuh"

namespace rfa {

constexpr int kDecodeThreads = 256;

// Shared tail of both decode kernels.  pq/pk hold phi_q/phi_k (K floats each) in
// shared memory, vs holds v (d floats).
template <typename TIn, typename TState>
__device__ __forceinline__ void decode_body(const float* pq, const float* pk, const float* vs,
                                            TState* __restrict__ S, TState* __restrict__ z,
                                            TIn* __restrict__ out, float4* red, float* den_s,
                                            int K, int d) {
  const int tid = threadIdx.x;
  const int d4 = d >> 2;                       // float4 columns per state row
  const int rows = kDecodeThreads / d4;        // state rows covered per pass
  const int c = tid % d4, r0 = tid / d4;

  // denominator and z update: warp 0
  if (tid < 32) {
    float part = 0.f;
    for (int k = tid; k < K; k += 32) {
      float zn = to_f(z[k]) + pk[k];
      z[k] = from_f<TState>(zn);
      part = fmaf(pq[k], zn, part);
    }
    part = warp_sum(part);
    if (tid == 0) *den_s = fmaxf(part, kEps);
  }

  const float4 v4 = *reinterpret_cast<const float4*>(vs + 4 * c);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  TState* Sc = S + 4 * c;
  int k = r0;
  // four independent 16-byte loads in flight per thread
  for (; k + 3 * rows < K; k += 4 * rows) {
    float4 s[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = load4(Sc + (size_t)(k + u * rows) * d);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float a = pk[k + u * rows], b = pq[k + u * rows];
      s[u].x = fmaf(a, v4.x, s[u].x); s[u].y = fmaf(a, v4.y, s[u].y);
      s[u].z = fmaf(a, v4.z, s[u].z); s[u].w = fmaf(a, v4.w, s[u].w);
      store4(Sc + (size_t)(k + u * rows) * d, s[u]);
      acc.x = fmaf(b, s[u].x, acc.x); acc.y = fmaf(b, s[u].y, acc.y);
      acc.z = fmaf(b, s[u].z, acc.z); acc.w = fmaf(b, s[u].w, acc.w);
    }
  }
  for (; k < K; k += rows) {
    float4 s = load4(Sc + (size_t)k * d);
    const float a = pk[k], b = pq[k];
    s.x = fmaf(a, v4.x, s.x); s.y = fmaf(a, v4.y, s.y);
    s.z = fmaf(a, v4.z, s.z); s.w = fmaf(a, v4.w, s.w);
    store4(Sc + (size_t)k * d, s);
    acc.x = fmaf(b, s.x, acc.x); acc.y = fmaf(b, s.y, acc.y);
    acc.z = fmaf(b, s.z, acc.z); acc.w = fmaf(b, s.w, acc.w);
  }
  red[tid] = acc;                              // red[r0 * d4 + c]
  __syncthreads();
  if (tid < d4) {
    float4 t = red[tid];
    for (int r = 1; r < rows; ++r) {
      float4 u = red[r * d4 + tid];
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    const float inv = 1.f / *den_s;
    t.x *= inv; t.y *= inv; t.z *= inv; t.w *= inv;
    store4(out + 4 * tid, t);
  }
}

template <typename TIn, typename TState>
__global__ void __launch_bounds__(kDecodeThreads)
decode_step_kernel(const TIn* __restrict__ phi_q, const TIn* __restrict__ phi_k,
                   const TIn* __restrict__ v, TState* __restrict__ S, TState* __restrict__ z,
                   TIn* __restrict__ out, int K, int d) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* red = reinterpret_cast<float4*>(smem_raw);                 // kDecodeThreads float4
  float* pq = reinterpret_cast<float*>(red + kDecodeThreads);        // K
  float* pk = pq + K;                                                // K
  float* vs = pk + K;                                                // d
  float* den_s = vs + d;
  const size_t bh = blockIdx.x;
  for (int i = threadIdx.x; i < K; i += kDecodeThreads) {
    pq[i] = to_f(phi_q[bh * K + i]);
    pk[i] = to_f(phi_k[bh * K + i]);
  }
  for (int i = threadIdx.x; i < d; i += kDecodeThreads) vs[i] = to_f(v[bh * d + i]);
  __syncthreads();
  decode_body<TIn, TState>(pq, pk, vs, S + bh * (size_t)K * d, z + bh * K, out + bh * d, red, den_s, K, d);
}

// Raw q,k in; the feature map (normalise, project with this head's W, sin|cos, scale)
// is applied in the prologue (upstream utils.py:100-120).
template <typename TIn, typename TState>
__global__ void __launch_bounds__(kDecodeThreads)
decode_step_fused_kernel(const TIn* __restrict__ q, const TIn* __restrict__ k,
                         const TIn* __restrict__ v, const float* __restrict__ w, float scale,
                         TState* __restrict__ S, TState* __restrict__ z, TIn* __restrict__ out,
                         int H, int D, int d) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int K = 2 * D;
  float4* red = reinterpret_cast<float4*>(smem_raw);
  float* pq = reinterpret_cast<float*>(red + kDecodeThreads);
  float* pk = pq + K;
  float* vs = pk + K;
  float* den_s = vs + d;
  float* xq = den_s + 4;     // d, normalised q
  float* xk = xq + d;        // d, normalised k
  const size_t bh = blockIdx.x;
  const int h = (int)(bh % H);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < d; i += kDecodeThreads) vs[i] = to_f(v[bh * d + i]);
  if (warp < 2) {            // warp 0 normalises q, warp 1 normalises k
    const TIn* src = (warp == 0 ? q : k) + bh * d;
    float* dst = warp == 0 ? xq : xk;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) { float t = to_f(src[i]); dst[i] = t; ss = fmaf(t, t, ss); }
    ss = warp_sum(ss);
    const float inv = 1.f / (sqrtf(ss) + kNormEps);
    for (int i = lane; i < d; i += 32) dst[i] *= inv;
  }
  __syncthreads();
  // one warp per projection row j: coalesced read of W[h][j][:], used for both vectors
  const float* wh = w + (size_t)h * D * d;
  for (int j = warp; j < D; j += kDecodeThreads / 32) {
    float uq = 0.f, uk = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float wv = wh[(size_t)j * d + i];
      uq = fmaf(wv, xq[i], uq);
      uk = fmaf(wv, xk[i], uk);
    }
    uq = warp_sum(uq);
    uk = warp_sum(uk);
    if (lane == 0) {
      float s_, c_;
      sincosf(uq, &s_, &c_); pq[j] = scale * s_; pq[D + j] = scale * c_;
      sincosf(uk, &s_, &c_); pk[j] = scale * s_; pk[D + j] = scale * c_;
    }
  }
  __syncthreads();
  if (sizeof(TIn) == 2) {    // features are handed over in the I/O precision, as the unfused path does
    for (int i = tid; i < K; i += kDecodeThreads) {
      pq[i] = to_f(from_f<TIn>(pq[i]));
      pk[i] = to_f(from_f<TIn>(pk[i]));
    }
    __syncthreads();
  }
  decode_body<TIn, TState>(pq, pk, vs, S + bh * (size_t)K * d, z + bh * K, out + bh * d, red, den_s, K, d);
}

static int check_decode_geometry(int BH, int K, int d) {
  RFA_REQUIRE(BH > 0 && K > 0 && d > 0, RFA_EINVAL, "decode: BH=%d K=%d d=%d must be positive", BH, K, d);
  const int d4 = d / 4;
  RFA_REQUIRE(d % 4 == 0 && d4 <= kDecodeThreads && kDecodeThreads % d4 == 0, RFA_EUNSUPPORTED,
              "decode: head_dim %d must be 4*2^m and <= %d", d, 4 * kDecodeThreads);
  RFA_REQUIRE(K <= 4096, RFA_EUNSUPPORTED, "decode: K=%d too large (max 4096)", K);
  return 0;
}

}  // namespace rfa

using namespace rfa;

extern "C" int rfa_decode_step(const void* phi_q, const void* phi_k, const void* v, int in_dtype,
                               void* s, void* z, int state_dtype, void* out,
                               int BH, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(phi_q && phi_k && v && s && z && out, RFA_EINVAL, "decode: null pointer");
  if (int e = check_decode_geometry(BH, K, d)) return e;
  RFA_REQUIRE(aligned16(phi_q) && aligned16(phi_k) && aligned16(v) && aligned16(s) && aligned16(z) && aligned16(out),
              RFA_EALIGN, "decode: pointers must be 16-byte aligned");
  const size_t smem = kDecodeThreads * sizeof(float4) + (2 * K + d + 4) * sizeof(float);
  cudaStream_t st = as_stream(stream);
#define RFA_LAUNCH(TI, TS)                                                                        \
  decode_step_kernel<TI, TS><<<BH, kDecodeThreads, smem, st>>>(                                   \
      (const TI*)phi_q, (const TI*)phi_k, (const TI*)v, (TS*)s, (TS*)z, (TI*)out, K, d)
  if (in_dtype == RFA_F16 && state_dtype == RFA_F32) RFA_LAUNCH(__half, float);
  else if (in_dtype == RFA_F16 && state_dtype == RFA_F16) RFA_LAUNCH(__half, __half);
  else if (in_dtype == RFA_F32 && state_dtype == RFA_F32) RFA_LAUNCH(float, float);
  else return fail(RFA_EUNSUPPORTED, "decode: unsupported dtype pair in=%d state=%d", in_dtype, state_dtype);
#undef RFA_LAUNCH
  return check_launch("rfa_decode_step");
}

extern "C" int rfa_decode_step_fused(const void* q, const void* k, const void* v, int in_dtype,
                                     const float* w, float scale, void* s, void* z, int state_dtype,
                                     void* out, int BH, int H, int D, int d, rfa_stream_t stream) {
  RFA_REQUIRE(q && k && v && w && s && z && out, RFA_EINVAL, "decode_fused: null pointer");
  RFA_REQUIRE(H > 0 && D > 0, RFA_EINVAL, "decode_fused: H=%d D=%d must be positive", H, D);
  if (int e = check_decode_geometry(BH, 2 * D, d)) return e;
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(s) && aligned16(z) && aligned16(out) && aligned16(w),
              RFA_EALIGN, "decode_fused: pointers must be 16-byte aligned");
  const int K = 2 * D;
  const size_t smem = kDecodeThreads * sizeof(float4) + (2 * K + 3 * d + 4) * sizeof(float);
  cudaStream_t st = as_stream(stream);
#define RFA_LAUNCH(TI, TS)                                                                        \
  decode_step_fused_kernel<TI, TS><<<BH, kDecodeThreads, smem, st>>>(                             \
      (const TI*)q, (const TI*)k, (const TI*)v, w, scale, (TS*)s, (TS*)z, (TI*)out, H, D, d)
  if (in_dtype == RFA_F16 && state_dtype == RFA_F32) RFA_LAUNCH(__half, float);
  else if (in_dtype == RFA_F16 && state_dtype == RFA_F16) RFA_LAUNCH(__half, __half);
  else if (in_dtype == RFA_F32 && state_dtype == RFA_F32) RFA_LAUNCH(float, float);
  else return fail(RFA_EUNSUPPORTED, "decode_fused: unsupported dtype pair in=%d state=%d", in_dtype, state_dtype);
#undef RFA_LAUNCH
  return check_launch("rfa_decode_step_fused");
}
