// Host orchestration of causal RFA (segment planning, workspace, boundary-state scan; the
// chunk kernels themselves are the tcgen05 kernels in causal_tc.cu / causal_bwd_tc.cu), the
// state-reduction and scan kernels, and the cross-attention kernels (K = 128, d = 64, fp16
// I/O, fp32 arithmetic and fp32 state).
//
// Notation per (batch, head):  S = sum k v^T [K,d],  z = sum k [K]  (upstream rfa.py:57-64).
// With few (batch, head) pairs a sequence is cut into segments that run as separate CTAs;
// the states at their boundaries come from a reduction pre-pass plus an exclusive scan, the
// same primitive a multi-device split of the sequence uses.
#include "tiles.cuh"

namespace rfa {

// ---------------------------------------------------------------------------
// segment planning (host) -- depends on (T, BH) only, so that the workspace size
// query and every launch agree.
// ---------------------------------------------------------------------------
struct CausalPlan {
  int nseg;        // segments per (batch, head)
  int64_t tseg;    // tokens per segment (multiple of every kernel's chunk length)
};

constexpr int kSegAlign = 128;

// tensor-core forward (causal_tc.cu)
int launch_causal_fwd_tc(const __half* q, const __half* k, const __half* v, __half* out, const float* s_seg,
                         const float* z_seg, float* s_out, float* z_out, int64_t T, int BH, int nseg, int64_t tseg,
                         cudaStream_t st);
// tensor-core backward, forward-direction sweep (causal_bwd_tc.cu)
int launch_causal_bwd_q_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq,
                           const float* s_seg, const float* z_seg, float* ws_den, float* ws_gz, float* ds_seg,
                           float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);

int launch_causal_bwd_kv_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                            const float* ws_den, const float* ws_gz, const float* ds_seg, const float* dz_seg,
                            int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);

static CausalPlan plan_causal(int64_t T, int BH) {
  CausalPlan p{1, ((T + kSegAlign - 1) / kSegAlign) * kSegAlign};
  if (BH >= 120 || T < 1024) return p;
  int64_t want = (148 + BH - 1) / BH;           // CTAs to cover the SMs
  int64_t maxseg = T / 512;                     // keep segments >= 512 tokens
  int64_t n = want < maxseg ? want : maxseg;
  if (n < 1) n = 1;
  int64_t tseg = ((T + n - 1) / n + kSegAlign - 1) / kSegAlign * kSegAlign;
  p.nseg = (int)((T + tseg - 1) / tseg);
  p.tseg = tseg;
  return p;
}

struct CausalWs {
  float* den;      // [T][BH]   clamped denominators
  float* gz;       // [T][BH]   gradient w.r.t. the raw denominator
  float* s_seg;    // [BH][nseg][K*d]  forward state entering each segment
  float* z_seg;    // [BH][nseg][K]
  float* ds_seg;   // [BH][nseg][K*d]  reverse state entering each segment
  float* dz_seg;   // [BH][nseg][K]
  size_t bytes;
};

static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }

static CausalWs carve_ws(void* base, int64_t T, int BH, const CausalPlan& p) {
  CausalWs w;
  char* c = reinterpret_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) { float* r = reinterpret_cast<float*>(c + off); off += align256(n * sizeof(float)); return r; };
  w.den = take((size_t)T * BH);
  w.gz = take((size_t)T * BH);
  w.s_seg = take((size_t)BH * p.nseg * kK * kD);
  w.z_seg = take((size_t)BH * p.nseg * kK);
  w.ds_seg = take((size_t)BH * p.nseg * kK * kD);
  w.dz_seg = take((size_t)BH * p.nseg * kK);
  w.bytes = off;
  return w;
}

// ---------------------------------------------------------------------------
// state reduction over a run of tokens (cross-attention S,z and segment totals)
// grid (BH, nseg).  pad_mask [B][T] (non-zero = padding) zeroes k rows.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
segment_state_kernel(const __half* __restrict__ k, const __half* __restrict__ v,
                     const uint8_t* __restrict__ pad_mask, float* __restrict__ s_out,
                     float* __restrict__ z_out, int64_t T, int BH, int H, int nseg, int64_t tseg) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;
  float* Vs = Ks + kC * kLK;
  float* St = Vs + kC * kLD;
  float* zs = St + kK * kLD;
  const int bh = blockIdx.x, seg = blockIdx.y;
  const int64_t t_begin = seg * tseg, t_end = min(T, t_begin + tseg);
  load_state(St, zs, nullptr, nullptr);
  for (int64_t t0 = t_begin; t0 < t_end; t0 += kC) {
    const int valid = (int)min((int64_t)kC, t_end - t0);
    __syncthreads();
    stage_rows<kK>(Ks, kLK, k + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, valid);
    stage_rows<kD>(Vs, kLD, v + ((size_t)t0 * BH + bh) * kD, (size_t)BH * kD, valid);
    __syncthreads();
    if (pad_mask) {
      const uint8_t* m = pad_mask + (size_t)(bh / H) * T + t0;
      for (int idx = threadIdx.x; idx < valid * kK; idx += kThreads)
        if (m[idx / kK]) Ks[(idx / kK) * kLK + (idx % kK)] = 0.f;
      __syncthreads();
    }
    accumulate_state(St, zs, Ks, Vs, nullptr);
  }
  __syncthreads();
  const size_t slot = (size_t)bh * nseg + seg;
  store_state(s_out + slot * kK * kD, z_out + slot * kK, St, zs);
}

// In-place exclusive scan over the segment axis of seg [BH][nseg][n] (forward or
// reverse order), seeded with carry [BH][n] (may be null); optionally also the plain
// sum over segments into total [BH][n].
__global__ void scan_states_kernel(float* __restrict__ seg, const float* __restrict__ carry,
                                   float* __restrict__ total, int BH, int nseg, int n, int reverse,
                                   int do_scan) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)BH * n) return;
  const size_t bh = i / n, e = i % n;
  float run = carry ? carry[i] : 0.f, sum = 0.f;
  for (int j = 0; j < nseg; ++j) {
    const int sgi = reverse ? nseg - 1 - j : j;
    float* p = seg + (bh * nseg + sgi) * n + e;
    const float t = *p;
    if (do_scan) *p = run;
    run += t;
    sum += t;
  }
  if (total) total[i] = sum;
}

// ---------------------------------------------------------------------------
// cross attention, query side.  grid (chunks, BH)
//   out_t = phi_q_t . S / max(|phi_q_t . z|, 1)      (upstream cross_attention.py:266-269)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
cross_query_fwd_kernel(const __half* __restrict__ q, const float* __restrict__ s, const float* __restrict__ z,
                       __half* __restrict__ out, int64_t T, int BH) {
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;
  float* Ns = Qs + kC * kLK;
  float* St = Ns + kC * kLD;
  float* zs = St + kK * kLD;
  float* den = zs + kK;
  const int bh = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t t0 = (int64_t)blockIdx.x * kC;
  const int valid = (int)min((int64_t)kC, T - t0);
  load_state(St, zs, s + (size_t)bh * kK * kD, z + (size_t)bh * kK);
  stage_rows<kK>(Qs, kLK, q + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, valid);
  __syncthreads();
  tile_gemm<4, 4>(kC, kD, kK,
                  [&](int r, int l) { return Qs[r * kLK + l]; },
                  [&](int l, int j) { return St[l * kLD + j]; },
                  [&](int r, int j, float a) { Ns[r * kLD + j] = a; });
  for (int r = warp; r < kC; r += kThreads / 32) {
    float p = 0.f;
#pragma unroll
    for (int l = lane; l < kK; l += 32) p = fmaf(Qs[r * kLK + l], zs[l], p);
    p = warp_sum(p);
    if (lane == 0) den[r] = fmaxf(fabsf(p), kEps);
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < kC * (kD / 8); idx += kThreads) {
    const int r = idx / (kD / 8), c = (idx % (kD / 8)) * 8;
    if (r >= valid) continue;
    const float inv = 1.f / den[r];
    float f[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = Ns[r * kLD + c + e] * inv;
    store8(out + ((size_t)(t0 + r) * BH + bh) * kD + c, f);
  }
}

// Query-side backward: one CTA per (batch, head) walks all query chunks and keeps
// dS, dz on chip.  With raw = phi_q.z, den = max(|raw|,1):
//   gs = g/den,  gr = -(g.out)/den * sign(raw) * [|raw| > 1]
//   g_phi_q = gs S^T + gr z^T,   dS = sum_t phi_q_t (x) gs_t,   dz = sum_t gr_t phi_q_t
__global__ void __launch_bounds__(kThreads)
cross_query_bwd_kernel(const __half* __restrict__ q, const float* __restrict__ s, const float* __restrict__ z,
                       const __half* __restrict__ g, __half* __restrict__ gq, float* __restrict__ d_s,
                       float* __restrict__ d_z, int64_t T, int BH) {
  extern __shared__ __align__(16) float sm[];
  float* Qs = sm;
  float* Ds = Qs + kC * kLK;
  float* Gs = Ds + kC * kLK;
  float* Ns = Gs + kC * kLD;
  float* St = Ns + kC * kLD;
  float* dSt = St + kK * kLD;
  float* zs = dSt + kK * kLD;
  float* dzs = zs + kK;
  float* den = dzs + kK;
  float* grs = den + kC;
  const int bh = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  load_state(St, zs, s + (size_t)bh * kK * kD, z + (size_t)bh * kK);
  load_state(dSt, dzs, nullptr, nullptr);
  for (int64_t t0 = 0; t0 < T; t0 += kC) {
    const int valid = (int)min((int64_t)kC, T - t0);
    __syncthreads();
    stage_rows<kK>(Qs, kLK, q + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, valid);
    stage_rows<kD>(Gs, kLD, g + ((size_t)t0 * BH + bh) * kD, (size_t)BH * kD, valid);
    __syncthreads();
    tile_gemm<4, 4>(kC, kD, kK,
                    [&](int r, int l) { return Qs[r * kLK + l]; },
                    [&](int l, int j) { return St[l * kLD + j]; },
                    [&](int r, int j, float a) { Ns[r * kLD + j] = a; });
    for (int r = warp; r < kC; r += kThreads / 32) {
      float p = 0.f;
#pragma unroll
      for (int l = lane; l < kK; l += 32) p = fmaf(Qs[r * kLK + l], zs[l], p);
      p = warp_sum(p);
      if (lane == 0) den[r] = p;
    }
    __syncthreads();
    for (int r = warp; r < kC; r += kThreads / 32) {
      const float raw = den[r];
      const float dn = fmaxf(fabsf(raw), kEps), inv = 1.f / dn;
      const float g0 = Gs[r * kLD + lane], g1 = Gs[r * kLD + lane + 32];
      float go = g0 * Ns[r * kLD + lane] + g1 * Ns[r * kLD + lane + 32];
      go = warp_sum(go) * inv;
      const float grv = fabsf(raw) > kEps ? (raw > 0.f ? -go * inv : go * inv) : 0.f;
      Gs[r * kLD + lane] = g0 * inv;
      Gs[r * kLD + lane + 32] = g1 * inv;
      __syncwarp();
      if (lane == 0) grs[r] = grv;
    }
    __syncthreads();
    tile_gemm<4, 8>(kC, kK, kD,
                    [&](int r, int l) { return Gs[r * kLD + l]; },
                    [&](int l, int c) { return St[c * kLD + l]; },
                    [&](int r, int c, float a) { Ds[r * kLK + c] = fmaf(grs[r], zs[c], a); });
    __syncthreads();
    unstage_rows<kK>(gq + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, Ds, kLK, valid);
    accumulate_state(dSt, dzs, Qs, Gs, grs);
  }
  __syncthreads();
  store_state(d_s + (size_t)bh * kK * kD, d_z + (size_t)bh * kK, dSt, dzs);
}

// Key-side backward of the state reduction.  grid (chunks, BH)
//   g_phi_k[s] = dS v_s + dz  (zero at padded keys),   g_v[s] = dS^T phi_k[s] (masked phi_k)
__global__ void __launch_bounds__(kThreads)
cross_state_bwd_kernel(const __half* __restrict__ k, const __half* __restrict__ v,
                       const uint8_t* __restrict__ pad_mask, const float* __restrict__ d_s,
                       const float* __restrict__ d_z, __half* __restrict__ gk, __half* __restrict__ gv,
                       int64_t T, int BH, int H) {
  extern __shared__ __align__(16) float sm[];
  float* Ks = sm;
  float* Ds = Ks + kC * kLK;
  float* Vs = Ds + kC * kLK;
  float* Os = Vs + kC * kLD;
  float* dSt = Os + kC * kLD;
  float* dzs = dSt + kK * kLD;
  float* keep = dzs + kK;      // 1 = real key, 0 = padding
  const int bh = blockIdx.y;
  const int64_t t0 = (int64_t)blockIdx.x * kC;
  const int valid = (int)min((int64_t)kC, T - t0);
  load_state(dSt, dzs, d_s + (size_t)bh * kK * kD, d_z + (size_t)bh * kK);
  stage_rows<kK>(Ks, kLK, k + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, valid);
  stage_rows<kD>(Vs, kLD, v + ((size_t)t0 * BH + bh) * kD, (size_t)BH * kD, valid);
  if (threadIdx.x < kC) {
    const int r = threadIdx.x;
    keep[r] = (r < valid && !(pad_mask && pad_mask[(size_t)(bh / H) * T + t0 + r])) ? 1.f : 0.f;
  }
  __syncthreads();
  tile_gemm<4, 8>(kC, kK, kD,
                  [&](int r, int l) { return Vs[r * kLD + l]; },
                  [&](int l, int c) { return dSt[c * kLD + l]; },
                  [&](int r, int c, float a) { Ds[r * kLK + c] = keep[r] * (a + dzs[c]); });
  tile_gemm<4, 4>(kC, kD, kK,
                  [&](int r, int l) { return Ks[r * kLK + l]; },
                  [&](int l, int j) { return dSt[l * kLD + j]; },
                  [&](int r, int j, float a) { Os[r * kLD + j] = keep[r] * a; });
  __syncthreads();
  unstage_rows<kK>(gk + ((size_t)t0 * BH + bh) * kK, (size_t)BH * kK, Ds, kLK, valid);
  unstage_rows<kD>(gv + ((size_t)t0 * BH + bh) * kD, (size_t)BH * kD, Os, kLD, valid);
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
constexpr size_t kSmemState = (size_t)(kC * kLK + kC * kLD + kK * kLD + kK) * sizeof(float);
constexpr size_t kSmemXqFwd = (size_t)(kC * kLK + kC * kLD + kK * kLD + kK + kC) * sizeof(float);
constexpr size_t kSmemXqBwd = (size_t)(2 * kC * kLK + 2 * kC * kLD + 2 * kK * kLD + 2 * kK + 2 * kC) * sizeof(float);
constexpr size_t kSmemXsBwd = (size_t)(2 * kC * kLK + 2 * kC * kLD + kK * kLD + kK + kC) * sizeof(float);

template <class Kern>
static int opt_in_smem(Kern kern, size_t bytes, const char* what) {
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail((int)e, "%s: cannot reserve %zu bytes of shared memory: %s", what, bytes, cudaGetErrorString(e));
  return 0;
}

static int check_geometry(const char* what, int64_t T, int BH, int K, int d) {
  RFA_REQUIRE(T >= 0 && BH > 0, RFA_EINVAL, "%s: T=%lld BH=%d", what, (long long)T, BH);
  RFA_REQUIRE(K == kK && d == kD, RFA_EUNSUPPORTED, "%s: only K=%d, d=%d is built (got K=%d d=%d)", what, kK, kD, K, d);
  RFA_REQUIRE(BH <= 65535, RFA_EUNSUPPORTED, "%s: BH=%d exceeds 65535", what, BH);
  return 0;
}

static int scan_launch(float* seg, const float* carry, float* total, int BH, int nseg, int n, int reverse,
                       int do_scan, cudaStream_t st) {
  const size_t items = (size_t)BH * n;
  scan_states_kernel<<<(unsigned)((items + 255) / 256), 256, 0, st>>>(seg, carry, total, BH, nseg, n, reverse, do_scan);
  return check_launch("scan_states");
}

// Forward states entering every segment -> ws.s_seg / ws.z_seg (nseg > 1 only).
static int build_segment_states(const __half* k, const __half* v, const float* s_in, const float* z_in,
                                const CausalWs& ws, const CausalPlan& p, int64_t T, int BH, cudaStream_t st) {
  if (int e = opt_in_smem(segment_state_kernel, kSmemState, "segment_state")) return e;
  segment_state_kernel<<<dim3(BH, p.nseg), kThreads, kSmemState, st>>>(k, v, nullptr, ws.s_seg, ws.z_seg, T, BH, 1,
                                                                      p.nseg, p.tseg);
  if (int e = check_launch("segment_state")) return e;
  if (int e = scan_launch(ws.s_seg, s_in, nullptr, BH, p.nseg, kK * kD, 0, 1, st)) return e;
  return scan_launch(ws.z_seg, z_in, nullptr, BH, p.nseg, kK, 0, 1, st);
}

static int check_ws(const char* what, void* workspace, size_t bytes, int64_t T, int BH, const CausalPlan& p, CausalWs* out) {
  RFA_REQUIRE(workspace, RFA_EWORKSPACE, "%s: workspace is null", what);
  RFA_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, RFA_EALIGN, "%s: workspace must be 256-byte aligned", what);
  *out = carve_ws(workspace, T, BH, p);
  RFA_REQUIRE(bytes >= out->bytes, RFA_EWORKSPACE, "%s: workspace has %zu bytes, %zu needed", what, bytes, out->bytes);
  return 0;
}

}  // namespace rfa

using namespace rfa;

extern "C" size_t rfa_causal_workspace_bytes(int64_t T, int BH, int K, int d) {
  if (T < 0 || BH <= 0 || K != kK || d != kD) return 0;
  const CausalPlan p = plan_causal(T, BH);
  return carve_ws(nullptr, T, BH, p).bytes;
}

extern "C" int rfa_causal_fwd(const void* q, const void* k, const void* v, void* out,
                              const float* s_in, const float* z_in, float* s_out, float* z_out,
                              void* workspace, size_t workspace_bytes,
                              int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("causal_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE(q && k && v && out, RFA_EINVAL, "causal_fwd: null pointer");
  RFA_REQUIRE((s_in == nullptr) == (z_in == nullptr) && (s_out == nullptr) == (z_out == nullptr), RFA_EINVAL,
              "causal_fwd: s/z pointers must be given in pairs");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(s_in) && aligned16(z_in) &&
                  aligned16(s_out) && aligned16(z_out), RFA_EALIGN, "causal_fwd: 16-byte alignment required");
  const CausalPlan p = plan_causal(T, BH);
  cudaStream_t st = as_stream(stream);
  const float *s_seg = s_in, *z_seg = z_in;
  if (T == 0) {
    if (s_out) {
      if (s_in) {
        cudaMemcpyAsync(s_out, s_in, (size_t)BH * kK * kD * sizeof(float), cudaMemcpyDeviceToDevice, st);
        cudaMemcpyAsync(z_out, z_in, (size_t)BH * kK * sizeof(float), cudaMemcpyDeviceToDevice, st);
      } else {
        cudaMemsetAsync(s_out, 0, (size_t)BH * kK * kD * sizeof(float), st);
        cudaMemsetAsync(z_out, 0, (size_t)BH * kK * sizeof(float), st);
      }
    }
    return check_launch("causal_fwd(T=0)");
  }
  if (p.nseg > 1) {
    CausalWs ws;
    if (int e = check_ws("causal_fwd", workspace, workspace_bytes, T, BH, p, &ws)) return e;
    if (int e = build_segment_states((const __half*)k, (const __half*)v, s_in, z_in, ws, p, T, BH, st)) return e;
    s_seg = ws.s_seg;
    z_seg = ws.z_seg;
  }
  return launch_causal_fwd_tc((const __half*)q, (const __half*)k, (const __half*)v, (__half*)out, s_seg, z_seg, s_out,
                              z_out, T, BH, p.nseg, p.tseg, st);
}

extern "C" int rfa_causal_bwd_q(const void* q, const void* k, const void* v, const void* g, void* gq,
                                const float* s_in, const float* z_in, float* ds_seg, float* dz_seg,
                                void* workspace, size_t workspace_bytes,
                                int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("causal_bwd_q", T, BH, K, d)) return e;
  RFA_REQUIRE(q && k && v && g && gq, RFA_EINVAL, "causal_bwd_q: null pointer");
  RFA_REQUIRE((s_in == nullptr) == (z_in == nullptr) && (ds_seg == nullptr) == (dz_seg == nullptr), RFA_EINVAL,
              "causal_bwd_q: s/z pointers must be given in pairs");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) && aligned16(gq) && aligned16(s_in) &&
                  aligned16(z_in) && aligned16(ds_seg) && aligned16(dz_seg), RFA_EALIGN,
              "causal_bwd_q: 16-byte alignment required");
  const CausalPlan p = plan_causal(T, BH);
  cudaStream_t st = as_stream(stream);
  if (T == 0) {
    if (ds_seg) {
      cudaMemsetAsync(ds_seg, 0, (size_t)BH * kK * kD * sizeof(float), st);
      cudaMemsetAsync(dz_seg, 0, (size_t)BH * kK * sizeof(float), st);
    }
    return check_launch("causal_bwd_q(T=0)");
  }
  CausalWs ws;
  if (int e = check_ws("causal_bwd_q", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  const float *s_seg = s_in, *z_seg = z_in;
  if (p.nseg > 1) {
    if (int e = build_segment_states((const __half*)k, (const __half*)v, s_in, z_in, ws, p, T, BH, st)) return e;
    s_seg = ws.s_seg;
    z_seg = ws.z_seg;
  }
  const bool want_dseg = p.nseg > 1 || ds_seg != nullptr;
  if (int e = launch_causal_bwd_q_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g,
                                     (__half*)gq, s_seg, z_seg, ws.den, ws.gz, want_dseg ? ws.ds_seg : nullptr,
                                     want_dseg ? ws.dz_seg : nullptr, T, BH, p.nseg, p.tseg, st))
    return e;
  if (ds_seg) {   // this shard's own total, before any carry is known
    if (int e = scan_launch(ws.ds_seg, nullptr, ds_seg, BH, p.nseg, kK * kD, 1, 0, st)) return e;
    if (int e = scan_launch(ws.dz_seg, nullptr, dz_seg, BH, p.nseg, kK, 1, 0, st)) return e;
  }
  return 0;
}

extern "C" int rfa_causal_bwd_kv(const void* q, const void* k, const void* v, const void* g, void* gk, void* gv,
                                 const float* ds_in, const float* dz_in, void* workspace, size_t workspace_bytes,
                                 int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("causal_bwd_kv", T, BH, K, d)) return e;
  RFA_REQUIRE(q && k && v && g && gk && gv, RFA_EINVAL, "causal_bwd_kv: null pointer");
  RFA_REQUIRE((ds_in == nullptr) == (dz_in == nullptr), RFA_EINVAL, "causal_bwd_kv: ds/dz must be given in pairs");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) && aligned16(gk) && aligned16(gv) &&
                  aligned16(ds_in) && aligned16(dz_in), RFA_EALIGN, "causal_bwd_kv: 16-byte alignment required");
  if (T == 0) return 0;
  const CausalPlan p = plan_causal(T, BH);
  cudaStream_t st = as_stream(stream);
  CausalWs ws;
  if (int e = check_ws("causal_bwd_kv", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  const float *ds_seg = ds_in, *dz_seg = dz_in;
  if (p.nseg > 1) {   // segment totals left by _bwd_q -> reverse exclusive scan seeded with the carry
    if (int e = scan_launch(ws.ds_seg, ds_in, nullptr, BH, p.nseg, kK * kD, 1, 1, st)) return e;
    if (int e = scan_launch(ws.dz_seg, dz_in, nullptr, BH, p.nseg, kK, 1, 1, st)) return e;
    ds_seg = ws.ds_seg;
    dz_seg = ws.dz_seg;
  }
  return launch_causal_bwd_kv_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g, (__half*)gk,
                                 (__half*)gv, ws.den, ws.gz, ds_seg, dz_seg, T, BH, p.nseg, p.tseg, st);
}

extern "C" int rfa_causal_bwd(const void* q, const void* k, const void* v, const void* g,
                              void* gq, void* gk, void* gv, const float* s_in, const float* z_in,
                              const float* ds_in, const float* dz_in, void* workspace, size_t workspace_bytes,
                              int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = rfa_causal_bwd_q(q, k, v, g, gq, s_in, z_in, nullptr, nullptr, workspace, workspace_bytes, T, BH, K, d, stream))
    return e;
  return rfa_causal_bwd_kv(q, k, v, g, gk, gv, ds_in, dz_in, workspace, workspace_bytes, T, BH, K, d, stream);
}

extern "C" int rfa_cross_state_fwd(const void* phi_k, const void* v, const uint8_t* pad_mask, float* s, float* z,
                                   int64_t T, int B, int H, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(B > 0 && H > 0, RFA_EINVAL, "cross_state_fwd: B=%d H=%d", B, H);
  const int BH = B * H;
  if (int e = check_geometry("cross_state_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE(phi_k && v && s && z, RFA_EINVAL, "cross_state_fwd: null pointer");
  RFA_REQUIRE(aligned16(phi_k) && aligned16(v) && aligned16(s) && aligned16(z), RFA_EALIGN,
              "cross_state_fwd: 16-byte alignment required");
  cudaStream_t st = as_stream(stream);
  if (int e = opt_in_smem(segment_state_kernel, kSmemState, "cross_state_fwd")) return e;
  const int64_t tseg = ((T + kC - 1) / kC) * kC;
  segment_state_kernel<<<dim3(BH, 1), kThreads, kSmemState, st>>>((const __half*)phi_k, (const __half*)v, pad_mask, s, z, T,
                                                                  BH, H, 1, tseg > 0 ? tseg : kC);
  return check_launch("rfa_cross_state_fwd");
}

extern "C" int rfa_cross_state_bwd(const void* phi_k, const void* v, const uint8_t* pad_mask, const float* d_s,
                                   const float* d_z, void* g_phi_k, void* g_v,
                                   int64_t T, int B, int H, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(B > 0 && H > 0, RFA_EINVAL, "cross_state_bwd: B=%d H=%d", B, H);
  const int BH = B * H;
  if (int e = check_geometry("cross_state_bwd", T, BH, K, d)) return e;
  RFA_REQUIRE(phi_k && v && d_s && d_z && g_phi_k && g_v, RFA_EINVAL, "cross_state_bwd: null pointer");
  RFA_REQUIRE(aligned16(phi_k) && aligned16(v) && aligned16(d_s) && aligned16(d_z) && aligned16(g_phi_k) && aligned16(g_v),
              RFA_EALIGN, "cross_state_bwd: 16-byte alignment required");
  if (T == 0) return 0;
  if (int e = opt_in_smem(cross_state_bwd_kernel, kSmemXsBwd, "cross_state_bwd")) return e;
  const unsigned chunks = (unsigned)((T + kC - 1) / kC);
  cross_state_bwd_kernel<<<dim3(chunks, BH), kThreads, kSmemXsBwd, as_stream(stream)>>>(
      (const __half*)phi_k, (const __half*)v, pad_mask, d_s, d_z, (__half*)g_phi_k, (__half*)g_v, T, BH, H);
  return check_launch("rfa_cross_state_bwd");
}

extern "C" int rfa_cross_query_fwd(const void* phi_q, const float* s, const float* z, void* out,
                                   int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("cross_query_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE(phi_q && s && z && out, RFA_EINVAL, "cross_query_fwd: null pointer");
  RFA_REQUIRE(aligned16(phi_q) && aligned16(s) && aligned16(z) && aligned16(out), RFA_EALIGN,
              "cross_query_fwd: 16-byte alignment required");
  if (T == 0) return 0;
  if (int e = opt_in_smem(cross_query_fwd_kernel, kSmemXqFwd, "cross_query_fwd")) return e;
  const unsigned chunks = (unsigned)((T + kC - 1) / kC);
  cross_query_fwd_kernel<<<dim3(chunks, BH), kThreads, kSmemXqFwd, as_stream(stream)>>>((const __half*)phi_q, s, z,
                                                                                       (__half*)out, T, BH);
  return check_launch("rfa_cross_query_fwd");
}

extern "C" int rfa_cross_query_bwd(const void* phi_q, const float* s, const float* z, const void* g,
                                   void* g_phi_q, float* d_s, float* d_z,
                                   int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("cross_query_bwd", T, BH, K, d)) return e;
  RFA_REQUIRE(phi_q && s && z && g && g_phi_q && d_s && d_z, RFA_EINVAL, "cross_query_bwd: null pointer");
  RFA_REQUIRE(aligned16(phi_q) && aligned16(s) && aligned16(z) && aligned16(g) && aligned16(g_phi_q) && aligned16(d_s) &&
                  aligned16(d_z), RFA_EALIGN, "cross_query_bwd: 16-byte alignment required");
  if (int e = opt_in_smem(cross_query_bwd_kernel, kSmemXqBwd, "cross_query_bwd")) return e;
  cross_query_bwd_kernel<<<BH, kThreads, kSmemXqBwd, as_stream(stream)>>>((const __half*)phi_q, s, z, (const __half*)g,
                                                                        (__half*)g_phi_q, d_s, d_z, T, BH);
  return check_launch("rfa_cross_query_bwd");
}
