// Causal and cross RFA for the geometries the tensor-core kernels are not built for (they are specialised for feature
// width K = 128 and head dim d = 64): any K % 8 == 0, d % 8 == 0 whose fp32 state [K][d + 1] fits in shared memory.
// Upstream's kernels accept any K % 16 == 0, d % 8 == 0 (cuda/forward.cu:150-153, cuda/backward.cu:560-562) and its
// cross attention is einsums of any size (cross_attention.py:97-104, 266-269); these kernels keep that reach.
//
// They are plain CUDA-core kernels that walk the tokens of one (batch, head) sequence one at a time, as upstream's
// do, with the state in shared memory in fp32 (upstream: fp16 registers): simple and exact rather than fast -- about
// 0.4 us per token and CTA.  Math per token (rfa.py:57-64, 79-101):
//     S += k (x) v, z += k;  num = q^T S, raw = q . z, den = max(raw, 1);  out = num / den
//     gs = g / den, gz = -(g . num) / den^2 * [raw > 1];  gq = S gs + gz z
//     reverse: dS += q (x) gs, dz += q gz;  gk = dS v + dz;  gv = dS^T k
// Cross attention is the same with a state that does not depend on the token and den = max(|raw|, 1).
#include "common.cuh"

namespace rfa {

constexpr int kGenThreads = 256;

struct GenSmem {          // carved from dynamic shared memory, all fp32
  float *S, *S2, *z, *z2, *a, *b, *c, *e, *red;
};

__host__ __device__ inline size_t gen_smem_floats(int K, int d, bool two_states) {
  return (size_t)K * (d + 1) * (two_states ? 2 : 1) + 2 * (size_t)K   // z, z2
         + 2 * (size_t)K + 2 * (size_t)d                             // a (K), b (K), c (d), e (d)
         + 64;                                                       // red
}

__device__ __forceinline__ GenSmem gen_carve(float* base, int K, int d, bool two_states) {
  GenSmem m;
  m.S = base; base += (size_t)K * (d + 1);
  m.S2 = two_states ? base : nullptr; if (two_states) base += (size_t)K * (d + 1);
  m.z = base; base += K;
  m.z2 = base; base += K;
  m.a = base; base += K;
  m.b = base; base += K;
  m.c = base; base += d;
  m.e = base; base += d;
  m.red = base;
  return m;
}

// ---- block-wide building blocks (every thread of the block calls them) --------------------------------------------------
__device__ __forceinline__ void gen_load(const __half* __restrict__ src, float* dst, int n) {
  for (int i = threadIdx.x; i < n; i += kGenThreads) dst[i] = __half2float(src[i]);
}
// S[kk][n] += a[kk] * b[n]
__device__ __forceinline__ void gen_rank1(float* S, const float* a, const float* b, int K, int d) {
  const int dp = d + 1;
  for (int e = threadIdx.x; e < K * d; e += kGenThreads) {
    const int kk = e / d, n = e - kk * d;
    S[kk * dp + n] = fmaf(a[kk], b[n], S[kk * dp + n]);
  }
}
// out[n] = sum_kk a[kk] * S[kk][n]   (threads over n: consecutive banks)
__device__ __forceinline__ void gen_cols(const float* S, const float* a, float* out, int K, int d) {
  const int dp = d + 1;
  for (int n = threadIdx.x; n < d; n += kGenThreads) {
    float acc = 0.f;
    for (int kk = 0; kk < K; ++kk) acc = fmaf(a[kk], S[kk * dp + n], acc);
    out[n] = acc;
  }
}
// out[kk] = sum_n S[kk][n] * b[n] + s * zz[kk]   (threads over kk: the row pitch d + 1 keeps the banks apart)
__device__ __forceinline__ void gen_rows(const float* S, const float* b, float s, const float* zz, float* out, int K, int d) {
  const int dp = d + 1;
  for (int kk = threadIdx.x; kk < K; kk += kGenThreads) {
    float acc = s * zz[kk];
    for (int n = 0; n < d; ++n) acc = fmaf(S[kk * dp + n], b[n], acc);
    out[kk] = acc;
  }
}
// sum_i a[i] * b[i] by warp 0 into red[slot]; the caller synchronises before reading it
__device__ __forceinline__ void gen_dot(const float* a, const float* b, int n, float* red, int slot) {
  if (threadIdx.x < 32) {
    float acc = 0.f;
    for (int i = threadIdx.x; i < n; i += 32) acc = fmaf(a[i], b[i], acc);
    acc = warp_sum(acc);
    if (threadIdx.x == 0) red[slot] = acc;
  }
}
__device__ __forceinline__ void gen_store_half(__half* dst, const float* src, int n, float scale) {
  for (int i = threadIdx.x; i < n; i += kGenThreads) dst[i] = __float2half_rn(src[i] * scale);
}
__device__ __forceinline__ void gen_state_in(float* S, float* z, const float* s_in, const float* z_in, int K, int d) {
  const int dp = d + 1;
  for (int e = threadIdx.x; e < K * d; e += kGenThreads) S[(e / d) * dp + e % d] = s_in ? s_in[e] : 0.f;
  for (int i = threadIdx.x; i < K; i += kGenThreads) z[i] = z_in ? z_in[i] : 0.f;
}
__device__ __forceinline__ void gen_state_out(const float* S, const float* z, float* s_out, float* z_out, int K, int d) {
  const int dp = d + 1;
  for (int e = threadIdx.x; e < K * d; e += kGenThreads) s_out[e] = S[(e / d) * dp + e % d];
  for (int i = threadIdx.x; i < K; i += kGenThreads) z_out[i] = z[i];
}

// ===========================================================================
// causal forward.  grid (BH)
// ===========================================================================
__global__ void __launch_bounds__(kGenThreads)
causal_generic_fwd_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                          __half* __restrict__ out, const float* __restrict__ s_in, const float* __restrict__ z_in,
                          float* __restrict__ s_out, float* __restrict__ z_out, float* __restrict__ den_out,
                          int64_t T, int BH, int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, false);
  const int bh = blockIdx.x;
  gen_state_in(m.S, m.z, s_in ? s_in + (size_t)bh * K * d : nullptr, z_in ? z_in + (size_t)bh * K : nullptr, K, d);
  __syncthreads();
  for (int64_t t = 0; t < T; ++t) {
    const size_t row = (size_t)t * BH + bh;
    gen_load(q + row * K, m.a, K);
    gen_load(k + row * K, m.b, K);
    gen_load(v + row * d, m.c, d);
    __syncthreads();
    gen_rank1(m.S, m.b, m.c, K, d);
    for (int i = threadIdx.x; i < K; i += kGenThreads) m.z[i] += m.b[i];
    __syncthreads();
    gen_cols(m.S, m.a, m.e, K, d);
    gen_dot(m.a, m.z, K, m.red, 0);
    __syncthreads();
    const float raw = m.red[0];
    gen_store_half(out + row * d, m.e, d, 1.f / fmaxf(raw, kEps));
    if (den_out && threadIdx.x == 0) den_out[(size_t)bh * T + t] = raw;
    __syncthreads();
  }
  if (s_out) gen_state_out(m.S, m.z, s_out + (size_t)bh * K * d, z_out + (size_t)bh * K, K, d);
}

// ===========================================================================
// causal backward, sweep 1 (forward in time): gq, den / gz per token, optionally the run's reverse-state total.  grid (BH)
// ===========================================================================
__global__ void __launch_bounds__(kGenThreads)
causal_generic_bwd_q_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                            const __half* __restrict__ g, __half* __restrict__ gq,
                            const float* __restrict__ s_in, const float* __restrict__ z_in,
                            float* __restrict__ ws_den, float* __restrict__ ws_gz,
                            float* __restrict__ ds_tot, float* __restrict__ dz_tot, int64_t T, int BH, int K, int d) {
  extern __shared__ float gen_raw[];
  const bool want_tot = ds_tot != nullptr;
  const GenSmem m = gen_carve(gen_raw, K, d, want_tot);
  const int bh = blockIdx.x;
  gen_state_in(m.S, m.z, s_in ? s_in + (size_t)bh * K * d : nullptr, z_in ? z_in + (size_t)bh * K : nullptr, K, d);
  if (want_tot) gen_state_in(m.S2, m.z2, nullptr, nullptr, K, d);
  __syncthreads();
  for (int64_t t = 0; t < T; ++t) {
    const size_t row = (size_t)t * BH + bh;
    gen_load(q + row * K, m.a, K);
    gen_load(k + row * K, m.b, K);
    gen_load(v + row * d, m.c, d);
    __syncthreads();
    gen_rank1(m.S, m.b, m.c, K, d);
    for (int i = threadIdx.x; i < K; i += kGenThreads) m.z[i] += m.b[i];
    __syncthreads();
    gen_cols(m.S, m.a, m.e, K, d);                    // e = num
    gen_dot(m.a, m.z, K, m.red, 0);                   // raw
    gen_load(g + row * d, m.c, d);                    // c = g  (v is no longer needed)
    __syncthreads();
    gen_dot(m.c, m.e, d, m.red, 1);                   // g . num
    __syncthreads();
    const float raw = m.red[0], dn = fmaxf(raw, kEps), inv = 1.f / dn;
    const float gz = raw > kEps ? -m.red[1] * inv * inv : 0.f;      // strict >, upstream rfa.py:91
    for (int i = threadIdx.x; i < d; i += kGenThreads) m.c[i] *= inv;   // c = gs
    if (threadIdx.x == 0) { ws_den[(size_t)bh * T + t] = raw; ws_gz[(size_t)bh * T + t] = gz; }
    __syncthreads();
    gen_rows(m.S, m.c, gz, m.z, m.b, K, d);           // b = gq  (k is no longer needed)
    if (want_tot) {
      gen_rank1(m.S2, m.a, m.c, K, d);
      for (int i = threadIdx.x; i < K; i += kGenThreads) m.z2[i] = fmaf(m.a[i], gz, m.z2[i]);
    }
    __syncthreads();
    gen_store_half(gq + row * K, m.b, K, 1.f);
    __syncthreads();
  }
  if (want_tot) gen_state_out(m.S2, m.z2, ds_tot + (size_t)bh * K * d, dz_tot + (size_t)bh * K, K, d);
}

// ===========================================================================
// causal backward, sweep 2 (reverse in time): gk, gv.  grid (BH)
// ===========================================================================
__global__ void __launch_bounds__(kGenThreads)
causal_generic_bwd_kv_kernel(const __half* __restrict__ q, const __half* __restrict__ k, const __half* __restrict__ v,
                             const __half* __restrict__ g, __half* __restrict__ gk, __half* __restrict__ gv,
                             const float* __restrict__ ws_den, const float* __restrict__ ws_gz,
                             const float* __restrict__ ds_in, const float* __restrict__ dz_in, int64_t T, int BH, int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, false);
  const int bh = blockIdx.x;
  gen_state_in(m.S, m.z, ds_in ? ds_in + (size_t)bh * K * d : nullptr, dz_in ? dz_in + (size_t)bh * K : nullptr, K, d);
  __syncthreads();
  for (int64_t t = T - 1; t >= 0; --t) {
    const size_t row = (size_t)t * BH + bh;
    gen_load(q + row * K, m.a, K);
    gen_load(g + row * d, m.c, d);
    gen_load(v + row * d, m.e, d);
    gen_load(k + row * K, m.b, K);
    const float inv = 1.f / fmaxf(ws_den[(size_t)bh * T + t], kEps), gz = ws_gz[(size_t)bh * T + t];
    __syncthreads();
    for (int i = threadIdx.x; i < d; i += kGenThreads) m.c[i] *= inv;   // c = gs
    __syncthreads();
    gen_rank1(m.S, m.a, m.c, K, d);                   // dS += q (x) gs   (inclusive of this token)
    for (int i = threadIdx.x; i < K; i += kGenThreads) m.z[i] = fmaf(m.a[i], gz, m.z[i]);
    __syncthreads();
    gen_rows(m.S, m.e, 1.f, m.z, m.a, K, d);          // a = gk = dS v + dz   (q is no longer needed)
    gen_cols(m.S, m.b, m.c, K, d);                    // c = gv = dS^T k      (gs is no longer needed)
    __syncthreads();
    gen_store_half(gk + row * K, m.a, K, 1.f);
    gen_store_half(gv + row * d, m.c, d, 1.f);
    __syncthreads();
  }
}

// ===========================================================================
// state reduction over runs of tokens (cross attention; shard totals).  grid (BH, nseg)
// ===========================================================================
__global__ void __launch_bounds__(kGenThreads)
state_generic_fwd_kernel(const __half* __restrict__ k, const __half* __restrict__ v, const uint8_t* __restrict__ pad_mask,
                         float* __restrict__ s_out, float* __restrict__ z_out, int64_t T, int BH, int H, int nseg, int64_t tseg,
                         int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, false);
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  const uint8_t* mrow = pad_mask ? pad_mask + (size_t)(bh / H) * T : nullptr;
  gen_state_in(m.S, m.z, nullptr, nullptr, K, d);
  __syncthreads();
  for (int64_t t = t_begin; t < t_end; ++t) {
    if (mrow && mrow[t]) continue;                    // padded keys contribute nothing (uniform across the block)
    const size_t row = (size_t)t * BH + bh;
    gen_load(k + row * K, m.b, K);
    gen_load(v + row * d, m.c, d);
    __syncthreads();
    gen_rank1(m.S, m.b, m.c, K, d);
    for (int i = threadIdx.x; i < K; i += kGenThreads) m.z[i] += m.b[i];
    __syncthreads();
  }
  const size_t slot = (size_t)bh * nseg + seg;
  gen_state_out(m.S, m.z, s_out + slot * K * d, z_out + slot * K, K, d);
}

// ===========================================================================
// cross attention, query side.  One CTA loads the state once and walks a run of query tokens.  grid (BH, nrun)
// ===========================================================================
constexpr int kGenRun = 64;      // query tokens per CTA

__global__ void __launch_bounds__(kGenThreads)
cross_generic_query_fwd_kernel(const __half* __restrict__ q, const float* __restrict__ s, const float* __restrict__ z,
                               __half* __restrict__ out, int64_t T, int BH, int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, false);
  const int bh = blockIdx.x;
  const int64_t t_begin = (int64_t)blockIdx.y * kGenRun, t_end = min(T, t_begin + kGenRun);
  gen_state_in(m.S, m.z, s + (size_t)bh * K * d, z + (size_t)bh * K, K, d);
  __syncthreads();
  for (int64_t t = t_begin; t < t_end; ++t) {
    const size_t row = (size_t)t * BH + bh;
    gen_load(q + row * K, m.a, K);
    __syncthreads();
    gen_cols(m.S, m.a, m.e, K, d);
    gen_dot(m.a, m.z, K, m.red, 0);
    __syncthreads();
    gen_store_half(out + row * d, m.e, d, 1.f / fmaxf(fabsf(m.red[0]), kEps));     // |q . z|, upstream cross_attention.py:267-268
    __syncthreads();
  }
}

// gq per token; d_s, d_z ACCUMULATED into with atomics (the host zeroes them first)
__global__ void __launch_bounds__(kGenThreads)
cross_generic_query_bwd_kernel(const __half* __restrict__ q, const float* __restrict__ s, const float* __restrict__ z,
                               const __half* __restrict__ g, __half* __restrict__ gq, float* __restrict__ d_s,
                               float* __restrict__ d_z, int64_t T, int BH, int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, true);
  const int bh = blockIdx.x;
  const int64_t t_begin = (int64_t)blockIdx.y * kGenRun, t_end = min(T, t_begin + kGenRun);
  gen_state_in(m.S, m.z, s + (size_t)bh * K * d, z + (size_t)bh * K, K, d);
  gen_state_in(m.S2, m.z2, nullptr, nullptr, K, d);
  __syncthreads();
  for (int64_t t = t_begin; t < t_end; ++t) {
    const size_t row = (size_t)t * BH + bh;
    gen_load(q + row * K, m.a, K);
    gen_load(g + row * d, m.c, d);
    __syncthreads();
    gen_cols(m.S, m.a, m.e, K, d);                    // e = num
    gen_dot(m.a, m.z, K, m.red, 0);                   // raw
    __syncthreads();
    gen_dot(m.c, m.e, d, m.red, 1);                   // g . num
    __syncthreads();
    const float raw = m.red[0], dn = fmaxf(fabsf(raw), kEps), inv = 1.f / dn;
    // d/d raw of 1 / max(|raw|, 1): zero inside the clamp, -sign(raw) / raw^2 outside
    const float gr = fabsf(raw) > kEps ? (raw > 0.f ? -m.red[1] * inv * inv : m.red[1] * inv * inv) : 0.f;
    for (int i = threadIdx.x; i < d; i += kGenThreads) m.c[i] *= inv;   // c = gs
    __syncthreads();
    gen_rows(m.S, m.c, gr, m.z, m.b, K, d);           // b = gq
    gen_rank1(m.S2, m.a, m.c, K, d);                  // dS += q (x) gs
    for (int i = threadIdx.x; i < K; i += kGenThreads) m.z2[i] = fmaf(m.a[i], gr, m.z2[i]);
    __syncthreads();
    gen_store_half(gq + row * K, m.b, K, 1.f);
    __syncthreads();
  }
  const int dp = d + 1;
  for (int e = threadIdx.x; e < K * d; e += kGenThreads) atomicAdd(d_s + (size_t)bh * K * d + e, m.S2[(e / d) * dp + e % d]);
  for (int i = threadIdx.x; i < K; i += kGenThreads) atomicAdd(d_z + (size_t)bh * K + i, m.z2[i]);
}

// gk = dS v + dz (zero at padded keys), gv = dS^T k (k counts as zero at padded keys).  grid (BH, nrun)
__global__ void __launch_bounds__(kGenThreads)
state_generic_bwd_kernel(const __half* __restrict__ k, const __half* __restrict__ v, const uint8_t* __restrict__ pad_mask,
                         const float* __restrict__ d_s, const float* __restrict__ d_z, __half* __restrict__ gk,
                         __half* __restrict__ gv, int64_t T, int BH, int H, int K, int d) {
  extern __shared__ float gen_raw[];
  const GenSmem m = gen_carve(gen_raw, K, d, false);
  const int bh = blockIdx.x;
  const int64_t t_begin = (int64_t)blockIdx.y * kGenRun, t_end = min(T, t_begin + kGenRun);
  const uint8_t* mrow = pad_mask ? pad_mask + (size_t)(bh / H) * T : nullptr;
  gen_state_in(m.S, m.z, d_s + (size_t)bh * K * d, d_z + (size_t)bh * K, K, d);
  __syncthreads();
  for (int64_t t = t_begin; t < t_end; ++t) {
    const size_t row = (size_t)t * BH + bh;
    if (mrow && mrow[t]) {                            // uniform across the block
      for (int i = threadIdx.x; i < K; i += kGenThreads) gk[row * K + i] = __float2half_rn(0.f);
      for (int i = threadIdx.x; i < d; i += kGenThreads) gv[row * d + i] = __float2half_rn(0.f);
      continue;
    }
    gen_load(k + row * K, m.b, K);
    gen_load(v + row * d, m.e, d);
    __syncthreads();
    gen_rows(m.S, m.e, 1.f, m.z, m.a, K, d);
    gen_cols(m.S, m.b, m.c, K, d);
    __syncthreads();
    gen_store_half(gk + row * K, m.a, K, 1.f);
    gen_store_half(gv + row * d, m.c, d, 1.f);
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
constexpr size_t kGenSmemMax = 227 * 1024;

// The geometry fits one state (two_states: two) in shared memory.
bool generic_geometry_ok(int K, int d, bool two_states) {
  return K > 0 && d > 0 && K % 8 == 0 && d % 8 == 0 && gen_smem_floats(K, d, two_states) * sizeof(float) <= kGenSmemMax;
}

template <class KERNEL>
static int gen_reserve(KERNEL kernel, size_t bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail((int)e, "%s: cannot reserve %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  return 0;
}

int launch_causal_generic_fwd(const __half* q, const __half* k, const __half* v, __half* out, const float* s_in, const float* z_in,
                              float* s_out, float* z_out, float* den_out, int64_t T, int BH, int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, false) * sizeof(float);
  if (int e = gen_reserve(causal_generic_fwd_kernel, smem, "causal_fwd")) return e;
  causal_generic_fwd_kernel<<<BH, kGenThreads, smem, st>>>(q, k, v, out, s_in, z_in, s_out, z_out, den_out, T, BH, K, d);
  return check_launch("rfa_causal_fwd (generic geometry)");
}

int launch_causal_generic_bwd_q(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq, const float* s_in,
                                const float* z_in, float* ws_den, float* ws_gz, float* ds_tot, float* dz_tot, int64_t T, int BH,
                                int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, ds_tot != nullptr) * sizeof(float);
  if (int e = gen_reserve(causal_generic_bwd_q_kernel, smem, "causal_bwd_q")) return e;
  causal_generic_bwd_q_kernel<<<BH, kGenThreads, smem, st>>>(q, k, v, g, gq, s_in, z_in, ws_den, ws_gz, ds_tot, dz_tot, T, BH, K, d);
  return check_launch("rfa_causal_bwd_q (generic geometry)");
}

int launch_causal_generic_bwd_kv(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                                 const float* ws_den, const float* ws_gz, const float* ds_in, const float* dz_in, int64_t T,
                                 int BH, int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, false) * sizeof(float);
  if (int e = gen_reserve(causal_generic_bwd_kv_kernel, smem, "causal_bwd_kv")) return e;
  causal_generic_bwd_kv_kernel<<<BH, kGenThreads, smem, st>>>(q, k, v, g, gk, gv, ws_den, ws_gz, ds_in, dz_in, T, BH, K, d);
  return check_launch("rfa_causal_bwd_kv (generic geometry)");
}

int launch_state_generic_fwd(const __half* k, const __half* v, const uint8_t* pad_mask, float* s, float* z, int64_t T, int BH, int H,
                             int nseg, int64_t tseg, int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, false) * sizeof(float);
  if (int e = gen_reserve(state_generic_fwd_kernel, smem, "state reduction")) return e;
  state_generic_fwd_kernel<<<dim3(BH, nseg), kGenThreads, smem, st>>>(k, v, pad_mask, s, z, T, BH, H, nseg, tseg, K, d);
  return check_launch("state reduction (generic geometry)");
}

int launch_cross_generic_query_fwd(const __half* q, const float* s, const float* z, __half* out, int64_t T, int BH, int K, int d,
                                   cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, false) * sizeof(float);
  if (int e = gen_reserve(cross_generic_query_fwd_kernel, smem, "cross_query_fwd")) return e;
  cross_generic_query_fwd_kernel<<<dim3(BH, (unsigned)((T + kGenRun - 1) / kGenRun)), kGenThreads, smem, st>>>(q, s, z, out, T, BH, K, d);
  return check_launch("rfa_cross_query_fwd (generic geometry)");
}

int launch_cross_generic_query_bwd(const __half* q, const float* s, const float* z, const __half* g, __half* gq, float* d_s,
                                   float* d_z, int64_t T, int BH, int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, true) * sizeof(float);
  if (int e = gen_reserve(cross_generic_query_bwd_kernel, smem, "cross_query_bwd")) return e;
  cudaMemsetAsync(d_s, 0, (size_t)BH * K * d * sizeof(float), st);
  cudaMemsetAsync(d_z, 0, (size_t)BH * K * sizeof(float), st);
  cross_generic_query_bwd_kernel<<<dim3(BH, (unsigned)((T + kGenRun - 1) / kGenRun)), kGenThreads, smem, st>>>(q, s, z, g, gq, d_s,
                                                                                                            d_z, T, BH, K, d);
  return check_launch("rfa_cross_query_bwd (generic geometry)");
}

int launch_state_generic_bwd(const __half* k, const __half* v, const uint8_t* pad_mask, const float* d_s, const float* d_z,
                             __half* gk, __half* gv, int64_t T, int BH, int H, int K, int d, cudaStream_t st) {
  const size_t smem = gen_smem_floats(K, d, false) * sizeof(float);
  if (int e = gen_reserve(state_generic_bwd_kernel, smem, "cross_state_bwd")) return e;
  state_generic_bwd_kernel<<<dim3(BH, (unsigned)((T + kGenRun - 1) / kGenRun)), kGenThreads, smem, st>>>(k, v, pad_mask, d_s, d_z, gk, gv,
                                                                                                      T, BH, H, K, d);
  return check_launch("rfa_cross_state_bwd (generic geometry)");
}

}  // namespace rfa
