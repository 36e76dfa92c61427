// Single-token incremental decoding step: streams the per-head state once.
//
// Per (batch, head):  s += phi_k (x) v;  z += phi_k;  out = phi_q.s / max(phi_q.z, 1)
// (upstream causal_attention.py:42-50).  The state s [K,d] is read and written
// exactly once with 16-byte (fp32) / 8-byte (fp16) accesses; a warp covers whole
// 128-byte lines.  One CTA per (batch, head); HBM-bound: 2*K*d*sizeof(state)
// bytes per head per token.
#include "common.cuh"

namespace rfa {

constexpr int kDecodeThreads = 128;   // 7 CTAs per SM at <= 72 registers: 1024 (batch, head) pairs fit in one wave of 148 SMs

constexpr int kDecodePrefetch = 8;   // state rows per thread fetched before the prologue (all of them at K=128, d=64)

// Issue this thread's first state loads; they fly while the prologue (inputs, feature map) runs.
template <typename TState>
__device__ __forceinline__ void decode_prefetch(const TState* __restrict__ S, int K, int d, float4 (&buf)[kDecodePrefetch]) {
  const int d4 = d >> 2, rows = kDecodeThreads / d4;
  const int c = threadIdx.x % d4, r0 = threadIdx.x / d4;
#pragma unroll
  for (int u = 0; u < kDecodePrefetch; ++u) {
    const int k = r0 + u * rows;
    buf[u] = k < K ? load4(S + (size_t)k * d + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

// Shared tail of both decode kernels.  pq/pk hold phi_q/phi_k (K floats each) in
// shared memory, vs holds v (d floats); buf holds the prefetched state rows.
template <typename TIn, typename TState>
__device__ __forceinline__ void decode_body(const float* pq, const float* pk, const float* vs,
                                            TState* __restrict__ S, TState* __restrict__ z,
                                            TIn* __restrict__ out, float4* red, float* den_s,
                                            int K, int d, float4 (&buf)[kDecodePrefetch]) {
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
#pragma unroll
  for (int u = 0; u < kDecodePrefetch; ++u) {
    const int kk = r0 + u * rows;
    if (kk < K) {
      const float a = pk[kk], b = pq[kk];
      float4 t = buf[u];
      t.x = fmaf(a, v4.x, t.x); t.y = fmaf(a, v4.y, t.y); t.z = fmaf(a, v4.z, t.z); t.w = fmaf(a, v4.w, t.w);
      store4(Sc + (size_t)kk * d, t);
      acc.x = fmaf(b, t.x, acc.x); acc.y = fmaf(b, t.y, acc.y); acc.z = fmaf(b, t.z, acc.z); acc.w = fmaf(b, t.w, acc.w);
    }
  }
  int k = r0 + kDecodePrefetch * rows;
  // beyond the prefetched rows: four independent 16-byte loads in flight per thread
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
__global__ void __launch_bounds__(kDecodeThreads, 7)
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
  float4 buf[kDecodePrefetch];
  decode_prefetch(S + bh * (size_t)K * d, K, d, buf);
  for (int i = threadIdx.x; i < K; i += kDecodeThreads) {
    pq[i] = to_f(phi_q[bh * K + i]);
    pk[i] = to_f(phi_k[bh * K + i]);
  }
  for (int i = threadIdx.x; i < d; i += kDecodeThreads) vs[i] = to_f(v[bh * d + i]);
  __syncthreads();
  decode_body<TIn, TState>(pq, pk, vs, S + bh * (size_t)K * d, z + bh * K, out + bh * d, red, den_s, K, d, buf);
}

// Raw q,k in; the feature map (normalise, project with this head's W, sin|cos, scale)
// is applied in the prologue (upstream utils.py:100-120).
template <typename TIn, typename TState>
__global__ void __launch_bounds__(kDecodeThreads, 7)
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
  float4 buf[kDecodePrefetch];
  decode_prefetch(S + bh * (size_t)K * d, K, d, buf);
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
  // Projections u = W_h xhat for both vectors with the whole CTA: a group of 4 (8, 16) lanes owns one row j
  // and reads it as contiguous float4's; partial dot products are combined with shuffles; then one thread
  // per (vector, j) takes the sine and cosine.  us[] holds the 2*D projections in between.
  float* us = xk + d;
  const float* wh = w + (size_t)h * D * d;
  {
    const int per = kDecodeThreads / D >= 16 ? 16 : (kDecodeThreads / D >= 8 ? 8 : (kDecodeThreads / D >= 4 ? 4 : (kDecodeThreads / D >= 2 ? 2 : 1)));
    const int rows_per_pass = kDecodeThreads / per;
    const int sub = tid % per;
    for (int j = tid / per; j < D; j += rows_per_pass) {
      float uq = 0.f, uk = 0.f;
      for (int i = sub * 4; i < d; i += per * 4) {
        const float4 wv = *reinterpret_cast<const float4*>(wh + (size_t)j * d + i);
        uq = fmaf(wv.x, xq[i], uq); uq = fmaf(wv.y, xq[i + 1], uq); uq = fmaf(wv.z, xq[i + 2], uq); uq = fmaf(wv.w, xq[i + 3], uq);
        uk = fmaf(wv.x, xk[i], uk); uk = fmaf(wv.y, xk[i + 1], uk); uk = fmaf(wv.z, xk[i + 2], uk); uk = fmaf(wv.w, xk[i + 3], uk);
      }
      for (int o = per >> 1; o > 0; o >>= 1) {
        uq += __shfl_xor_sync(0xffffffffu, uq, o);
        uk += __shfl_xor_sync(0xffffffffu, uk, o);
      }
      if (sub == 0) { us[j] = uq; us[D + j] = uk; }
    }
  }
  __syncthreads();
  for (int t = tid; t < 2 * D; t += kDecodeThreads) {
    float s_, c_;
    sincosf(us[t], &s_, &c_);
    float* dst = t < D ? pq : pk;
    const int j = t < D ? t : t - D;
    dst[j] = scale * s_;
    dst[D + j] = scale * c_;
  }
  __syncthreads();
  if (sizeof(TIn) == 2) {    // features are handed over in the I/O precision, as the unfused path does
    for (int i = tid; i < K; i += kDecodeThreads) {
      pq[i] = to_f(from_f<TIn>(pq[i]));
      pk[i] = to_f(from_f<TIn>(pk[i]));
    }
    __syncthreads();
  }
  decode_body<TIn, TState>(pq, pk, vs, S + bh * (size_t)K * d, z + bh * K, out + bh * d, red, den_s, K, d, buf);
}

// One decoding step of cross attention for ALL layers in one launch: the states do not change while a sequence is
// decoded, so a step only streams them:  out[l] = phi_q[l] . s_l / max(|phi_q[l] . z_l|, 1)  (upstream
// cross_attention.py:266-269, called once per layer).  grid (BH, L); the layers' states are separate arrays, reached
// through device arrays of pointers.
template <typename TIn>
__global__ void __launch_bounds__(kDecodeThreads, 7)
cross_decode_kernel(const TIn* __restrict__ phi_q, const float* const* __restrict__ s_ptrs, const float* const* __restrict__ z_ptrs,
                    TIn* __restrict__ out, int BH, int K, int d) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float4* red = reinterpret_cast<float4*>(smem_raw);                 // kDecodeThreads float4
  float* pq = reinterpret_cast<float*>(red + kDecodeThreads);        // K
  float* den_s = pq + K;
  const size_t bh = blockIdx.x, l = blockIdx.y;
  const float* S = s_ptrs[l] + bh * (size_t)K * d;
  const float* z = z_ptrs[l] + bh * (size_t)K;
  const int tid = threadIdx.x;
  float4 buf[kDecodePrefetch];
  decode_prefetch(S, K, d, buf);
  for (int i = tid; i < K; i += kDecodeThreads) pq[i] = to_f(phi_q[(l * BH + bh) * K + i]);
  __syncthreads();
  if (tid < 32) {
    float part = 0.f;
    for (int k = tid; k < K; k += 32) part = fmaf(pq[k], z[k], part);
    part = warp_sum(part);
    if (tid == 0) *den_s = fmaxf(fabsf(part), kEps);
  }
  const int d4 = d >> 2, rows = kDecodeThreads / d4;
  const int c = tid % d4, r0 = tid / d4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int u = 0; u < kDecodePrefetch; ++u) {
    const int kk = r0 + u * rows;
    if (kk < K) {
      const float b = pq[kk];
      acc.x = fmaf(b, buf[u].x, acc.x); acc.y = fmaf(b, buf[u].y, acc.y); acc.z = fmaf(b, buf[u].z, acc.z); acc.w = fmaf(b, buf[u].w, acc.w);
    }
  }
  for (int k = r0 + kDecodePrefetch * rows; k < K; k += rows) {
    const float4 t = load4(S + (size_t)k * d + 4 * c);
    const float b = pq[k];
    acc.x = fmaf(b, t.x, acc.x); acc.y = fmaf(b, t.y, acc.y); acc.z = fmaf(b, t.z, acc.z); acc.w = fmaf(b, t.w, acc.w);
  }
  red[tid] = acc;
  __syncthreads();
  if (tid < d4) {
    float4 t = red[tid];
    for (int r = 1; r < rows; ++r) {
      const float4 u = red[r * d4 + tid];
      t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
    }
    const float inv = 1.f / *den_s;
    t.x *= inv; t.y *= inv; t.z *= inv; t.w *= inv;
    store4(out + (l * BH + bh) * d + 4 * tid, t);
  }
}

static int check_decode_dtypes(const char* what, int in_dtype, int state_dtype) {
  const bool ok = (in_dtype == RFA_F16 && (state_dtype == RFA_F32 || state_dtype == RFA_F16)) ||
                  (in_dtype == RFA_F32 && state_dtype == RFA_F32);
  RFA_REQUIRE(ok, RFA_EUNSUPPORTED, "%s: unsupported dtype pair in=%d state=%d", what, in_dtype, state_dtype);
  return 0;
}

static int check_decode_geometry(int BH, int K, int d) {
  RFA_REQUIRE(BH > 0 && K > 0 && d > 0, RFA_EINVAL, "decode: BH=%d K=%d d=%d must be positive", BH, K, d);
  const int d4 = d / 4;
  RFA_REQUIRE(d % 4 == 0 && d4 <= kDecodeThreads && kDecodeThreads % d4 == 0, RFA_EUNSUPPORTED,
              "decode: head_dim %d must be 4*2^m and <= %d", d, 4 * kDecodeThreads);
  RFA_REQUIRE(K <= 4096, RFA_EUNSUPPORTED, "decode: K=%d too large (max 4096)", K);
  // the kernel keeps v behind the two K-long feature vectors in shared memory and reads it 16 bytes at a time
  RFA_REQUIRE(K % 4 == 0, RFA_EUNSUPPORTED, "decode: K=%d must be a multiple of 4", K);
  return 0;
}

}  // namespace rfa

using namespace rfa;

extern "C" int rfa_decode_step(const void* phi_q, const void* phi_k, const void* v, int in_dtype,
                               void* s, void* z, int state_dtype, void* out,
                               int BH, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(phi_q && phi_k && v && s && z && out, RFA_EINVAL, "decode: null pointer");
  if (int e = check_decode_geometry(BH, K, d)) return e;
  if (int e = check_decode_dtypes("decode", in_dtype, state_dtype)) return e;
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
  RFA_REQUIRE(D % 8 == 0, RFA_EUNSUPPORTED, "decode_fused: proj_dim %d must be a multiple of 8", D);
  if (int e = check_decode_geometry(BH, 2 * D, d)) return e;
  if (int e = check_decode_dtypes("decode_fused", in_dtype, state_dtype)) return e;
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(s) && aligned16(z) && aligned16(out) && aligned16(w),
              RFA_EALIGN, "decode_fused: pointers must be 16-byte aligned");
  const int K = 2 * D;
  const size_t smem = kDecodeThreads * sizeof(float4) + (2 * K + 3 * d + 4 + 2 * D) * sizeof(float);
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

extern "C" int rfa_cross_decode_step(const void* phi_q, int in_dtype, const float* const* s_ptrs, const float* const* z_ptrs,
                                     void* out, int L, int BH, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(phi_q && s_ptrs && z_ptrs && out, RFA_EINVAL, "cross_decode: null pointer");
  RFA_REQUIRE(L > 0 && L <= 65535, RFA_EINVAL, "cross_decode: L=%d", L);
  if (int e = check_decode_geometry(BH, K, d)) return e;
  RFA_REQUIRE(in_dtype == RFA_F16 || in_dtype == RFA_F32, RFA_EUNSUPPORTED, "cross_decode: dtype %d", in_dtype);
  RFA_REQUIRE(aligned16(phi_q) && aligned16(out), RFA_EALIGN, "cross_decode: pointers must be 16-byte aligned");
  const size_t smem = kDecodeThreads * sizeof(float4) + (K + 4) * sizeof(float);
  const dim3 grid(BH, L);
  if (in_dtype == RFA_F16)
    cross_decode_kernel<__half><<<grid, kDecodeThreads, smem, as_stream(stream)>>>((const __half*)phi_q, s_ptrs, z_ptrs, (__half*)out, BH, K, d);
  else
    cross_decode_kernel<float><<<grid, kDecodeThreads, smem, as_stream(stream)>>>((const float*)phi_q, s_ptrs, z_ptrs, (float*)out, BH, K, d);
  return check_launch("rfa_cross_decode_step");
}
