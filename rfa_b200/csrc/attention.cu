// Host side of the attention entry points: argument checks, segment planning, workspace, the
// boundary-state scan.  The kernels themselves are the tcgen05 kernels in causal_tc.cu,
// causal_bwd_q_tc.cu, causal_bwd_kv_tc.cu and cross_tc.cu (K = 128, d = 64, fp16 I/O, fp32
// accumulation and fp32 state).
//
// Notation per (batch, head):  S = sum k v^T [K,d],  z = sum k [K]  (upstream rfa.py:57-64).
// With few (batch, head) pairs a sequence is cut into segments that run as separate CTAs;
// the states at their boundaries come from a reduction pre-pass plus an exclusive scan, the
// same primitive a multi-device split of the sequence uses.
#include "common.cuh"
#include "sm100.cuh"

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
                         const float* z_seg, float* s_out, float* z_out, float* den_out, int64_t T, int BH, int nseg,
                         int64_t tseg, cudaStream_t st);
// forward with the feature map of q and k computed in the kernel (causal_fused_tc.cu)
int launch_causal_fwd_fused_tc(const __half* xq, const __half* xk, const __half* v, const float* w, const uint8_t* row_mask,
                               __half* out, const float* s_in, const float* z_in, float* s_out, float* z_out, float* den_out,
                               int64_t T, int BH, int H, float scale, cudaStream_t st);
// forward-direction sweep from the forward's saved output and raw denominators (causal_bwd_q_saved_tc.cu)
int launch_causal_bwd_q_saved_tc(const __half* q, const __half* k, const __half* v, const __half* g, const __half* out,
                                 const float* den_raw, __half* gq, const float* s_seg, const float* z_seg, float* ws_gz,
                                 float* ds_seg, float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);
// tensor-core backward, forward-direction sweep (causal_bwd_tc.cu)
int launch_causal_bwd_q_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq,
                           const float* s_seg, const float* z_seg, float* ws_den, float* ws_gz, float* ds_seg,
                           float* dz_seg, int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);

int launch_causal_bwd_kv_tc(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                            const float* ws_den, const float* ws_gz, const float* ds_seg, const float* dz_seg,
                            int64_t T, int BH, int nseg, int64_t tseg, cudaStream_t st);

// tensor-core state reduction and cross-attention kernels (cross_tc.cu)
int launch_cross_state_fwd_tc(const __half* k, const __half* v, const uint8_t* pad_mask, float* s, float* z, int64_t T, int BH,
                              int H, int nseg, int64_t tseg, cudaStream_t st);
int launch_cross_query_fwd_tc(const __half* q, const float* s, const float* z, __half* out, int64_t T, int BH, cudaStream_t st);
int launch_cross_query_bwd_tc(const __half* q, const float* s, const float* z, const __half* g, __half* gq, float* d_s, float* d_z,
                              int64_t T, int BH, cudaStream_t st);
int launch_cross_state_bwd_tc(const __half* k, const __half* v, const uint8_t* pad_mask, const float* d_s, const float* d_z,
                              __half* gk, __half* gv, int64_t T, int BH, int H, cudaStream_t st);

// CUDA-core kernels for every other geometry (generic.cu)
bool generic_geometry_ok(int K, int d, bool two_states);
int launch_causal_generic_fwd(const __half* q, const __half* k, const __half* v, __half* out, const float* s_in, const float* z_in,
                              float* s_out, float* z_out, float* den_out, int64_t T, int BH, int K, int d, cudaStream_t st);
int launch_causal_generic_bwd_q(const __half* q, const __half* k, const __half* v, const __half* g, __half* gq, const float* s_in,
                                const float* z_in, float* ws_den, float* ws_gz, float* ds_tot, float* dz_tot, int64_t T, int BH,
                                int K, int d, cudaStream_t st);
int launch_causal_generic_bwd_kv(const __half* q, const __half* k, const __half* v, const __half* g, __half* gk, __half* gv,
                                 const float* ws_den, const float* ws_gz, const float* ds_in, const float* dz_in, int64_t T,
                                 int BH, int K, int d, cudaStream_t st);
int launch_state_generic_fwd(const __half* k, const __half* v, const uint8_t* pad_mask, float* s, float* z, int64_t T, int BH, int H,
                             int nseg, int64_t tseg, int K, int d, cudaStream_t st);
int launch_cross_generic_query_fwd(const __half* q, const float* s, const float* z, __half* out, int64_t T, int BH, int K, int d,
                                   cudaStream_t st);
int launch_cross_generic_query_bwd(const __half* q, const float* s, const float* z, const __half* g, __half* gq, float* d_s,
                                   float* d_z, int64_t T, int BH, int K, int d, cudaStream_t st);
int launch_state_generic_bwd(const __half* k, const __half* v, const uint8_t* pad_mask, const float* d_s, const float* d_z,
                             __half* gk, __half* gv, int64_t T, int BH, int H, int K, int d, cudaStream_t st);

static CausalPlan plan_causal(int64_t T, int BH) {
  CausalPlan p{1, ((T + kSegAlign - 1) / kSegAlign) * kSegAlign};
  if (BH >= 120 || T < 1024) return p;
  int64_t want = 148 / BH;                      // segments per head that still fit one wave of 148 SMs
  int64_t maxseg = T / 512;                     // keep segments >= 512 tokens
  int64_t n = want < maxseg ? want : maxseg;
  if (n < 1) n = 1;
  int64_t tseg = ((T + n - 1) / n + kSegAlign - 1) / kSegAlign * kSegAlign;
  p.nseg = (int)((T + tseg - 1) / tseg);
  p.tseg = tseg;
  return p;
}

struct CausalWs {
  float* den;      // [BH][T]   clamped denominators
  float* gz;       // [BH][T]   gradient w.r.t. the raw denominator
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

constexpr int kStateN = kK * kD + kK;          // floats of one packed state [S (K*d) | z (K)]

// element e of the packed state of (bh, segment): S and z live in two arrays
__device__ __forceinline__ float* state_elem(float* s_seg, float* z_seg, size_t bh, int nseg, int sg, int e) {
  return e < kK * kD ? s_seg + (bh * nseg + sg) * (size_t)(kK * kD) + e : z_seg + (bh * nseg + sg) * (size_t)kK + (e - kK * kD);
}

// In-place exclusive scan over the segment axis of s_seg [BH][nseg][K*d] and z_seg [BH][nseg][K] (forward or reverse
// order), seeded with carry_s [BH][K*d] / carry_z [BH][K] (may be null).
__global__ void scan_states_kernel(float* __restrict__ s_seg, float* __restrict__ z_seg, const float* __restrict__ carry_s,
                                   const float* __restrict__ carry_z, int BH, int nseg, int reverse) {
  sm100::pdl_wait();
  sm100::pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)BH * kStateN) return;
  const size_t bh = i / kStateN;
  const int e = (int)(i % kStateN);
  float run = 0.f;
  if (carry_s) run = e < kK * kD ? carry_s[bh * (kK * kD) + e] : carry_z[bh * kK + (e - kK * kD)];
  for (int j = 0; j < nseg; ++j) {
    float* p = state_elem(s_seg, z_seg, bh, nseg, reverse ? nseg - 1 - j : j, e);
    const float t = *p;
    *p = run;
    run += t;
  }
}

// Sum over the segment axis -> packed [BH][K*d + K] and / or the two plain arrays tot_s [BH][K*d], tot_z [BH][K].
__global__ void total_states_kernel(const float* __restrict__ s_seg, const float* __restrict__ z_seg, float* __restrict__ packed,
                                    float* __restrict__ tot_s, float* __restrict__ tot_z, int BH, int nseg) {
  sm100::pdl_wait();
  sm100::pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)BH * kStateN) return;
  const size_t bh = i / kStateN;
  const int e = (int)(i % kStateN);
  float sum = 0.f;
  for (int j = 0; j < nseg; ++j)
    sum += *state_elem(const_cast<float*>(s_seg), const_cast<float*>(z_seg), bh, nseg, j, e);
  if (packed) packed[i] = sum;
  if (tot_s) {
    if (e < kK * kD) tot_s[bh * (kK * kD) + e] = sum; else tot_z[bh * kK + (e - kK * kD)] = sum;
  }
}

// gathered [world][BH][K*d + K]: the packed totals of all shards.  out = sum over the shards before (reverse: after)
// shard `rank`, written as the two plain arrays a kernel takes as its carry.
__global__ void scan_gathered_kernel(const float* __restrict__ gathered, int world, int rank, int reverse,
                                     float* __restrict__ out_s, float* __restrict__ out_z, int BH) {
  sm100::pdl_wait();
  sm100::pdl_launch_dependents();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const size_t n = (size_t)BH * kStateN;
  if (i >= n) return;
  float sum = 0.f;
  const int lo = reverse ? rank + 1 : 0, hi = reverse ? world : rank;
  for (int r = lo; r < hi; ++r) sum += gathered[(size_t)r * n + i];
  const size_t bh = i / kStateN;
  const int e = (int)(i % kStateN);
  if (e < kK * kD) out_s[bh * (kK * kD) + e] = sum; else out_z[bh * kK + (e - kK * kD)] = sum;
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// Which kernels serve a geometry: the tensor-core ones (K = 128, d = 64) or the generic CUDA-core ones.
static bool is_tc(int K, int d) { return K == kK && d == kD; }

static int check_geometry(const char* what, int64_t T, int BH, int K, int d, bool generic_allowed = true, bool two_states = false) {
  RFA_REQUIRE(T >= 0 && BH > 0, RFA_EINVAL, "%s: T=%lld BH=%d", what, (long long)T, BH);
  RFA_REQUIRE(BH <= 65535, RFA_EUNSUPPORTED, "%s: BH=%d exceeds 65535", what, BH);
  if (is_tc(K, d)) return 0;
  RFA_REQUIRE(generic_allowed, RFA_EUNSUPPORTED, "%s: this entry point is built for K=%d, d=%d only (got K=%d d=%d)", what, kK, kD, K, d);
  RFA_REQUIRE(generic_geometry_ok(K, d, two_states), RFA_EUNSUPPORTED,
              "%s: K=%d d=%d: K and d must be multiples of 8 and the fp32 state%s must fit in shared memory", what, K, d,
              two_states ? "s (two of them for this call)" : "");
  return 0;
}

static unsigned state_blocks(int BH) { return (unsigned)(((size_t)BH * kStateN + 255) / 256); }

static int scan_launch(float* s_seg, float* z_seg, const float* carry_s, const float* carry_z, int BH, int nseg, int reverse,
                       cudaStream_t st) {
  sm100::launch_pdl(scan_states_kernel, dim3(state_blocks(BH)), dim3(256), 0, st, s_seg, z_seg, carry_s, carry_z, BH, nseg, reverse);
  return check_launch("scan_states");
}

static int total_launch(const float* s_seg, const float* z_seg, float* packed, float* tot_s, float* tot_z, int BH, int nseg,
                        cudaStream_t st) {
  sm100::launch_pdl(total_states_kernel, dim3(state_blocks(BH)), dim3(256), 0, st, s_seg, z_seg, packed, tot_s, tot_z, BH, nseg);
  return check_launch("total_states");
}

// Per-segment sums of k (x) v and k -> ws.s_seg / ws.z_seg (one CTA per (batch, head, segment)).
static int segment_partials(const __half* k, const __half* v, const CausalWs& ws, const CausalPlan& p, int64_t T, int BH,
                            cudaStream_t st) {
  return launch_cross_state_fwd_tc(k, v, nullptr, ws.s_seg, ws.z_seg, T, BH, 1, p.nseg, p.tseg, st);
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
  if (T < 0 || BH <= 0) return 0;
  if (!is_tc(K, d)) {                     // generic geometry: one run per sequence, only the two per-token scalars
    if (!generic_geometry_ok(K, d, false)) return 0;
    return carve_ws(nullptr, T, BH, CausalPlan{1, T}).bytes;
  }
  const CausalPlan p = plan_causal(T, BH);
  return carve_ws(nullptr, T, BH, p).bytes;
}

// ---- forward ---------------------------------------------------------------------------------------------------
extern "C" int rfa_causal_fwd_staged(const void* q, const void* k, const void* v, void* out,
                                     const float* s_in, const float* z_in, float* s_out, float* z_out,
                                     void* workspace, size_t workspace_bytes,
                                     int64_t T, int BH, int K, int d, int ws_has, int save_den, rfa_stream_t stream) {
  if (int e = check_geometry("causal_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE((s_in == nullptr) == (z_in == nullptr) && (s_out == nullptr) == (z_out == nullptr), RFA_EINVAL,
              "causal_fwd: s/z pointers must be given in pairs");
  RFA_REQUIRE(T == 0 || (q && k && v && out), RFA_EINVAL, "causal_fwd: null pointer");   // empty arrays have no address
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out) && aligned16(s_in) && aligned16(z_in) &&
                  aligned16(s_out) && aligned16(z_out), RFA_EALIGN, "causal_fwd: 16-byte alignment required");
  RFA_REQUIRE((ws_has & ~RFA_WS_PARTIALS) == 0, RFA_EINVAL, "causal_fwd: ws_has may only name RFA_WS_PARTIALS (got %d)", ws_has);
  const CausalPlan p = is_tc(K, d) ? plan_causal(T, BH) : CausalPlan{1, T};
  cudaStream_t st = as_stream(stream);
  const float *s_seg = s_in, *z_seg = z_in;
  if (T == 0) {
    if (s_out) {
      if (s_in) {
        cudaMemcpyAsync(s_out, s_in, (size_t)BH * K * d * sizeof(float), cudaMemcpyDeviceToDevice, st);
        cudaMemcpyAsync(z_out, z_in, (size_t)BH * K * sizeof(float), cudaMemcpyDeviceToDevice, st);
      } else {
        cudaMemsetAsync(s_out, 0, (size_t)BH * K * d * sizeof(float), st);
        cudaMemsetAsync(z_out, 0, (size_t)BH * K * sizeof(float), st);
      }
    }
    return check_launch("causal_fwd(T=0)");
  }
  if (!is_tc(K, d)) {
    CausalWs gws{};
    if (save_den)
      if (int e = check_ws("causal_fwd", workspace, workspace_bytes, T, BH, p, &gws)) return e;
    return launch_causal_generic_fwd((const __half*)q, (const __half*)k, (const __half*)v, (__half*)out, s_in, z_in, s_out, z_out,
                                     save_den ? gws.den : nullptr, T, BH, K, d, st);
  }
  CausalWs ws{};
  if (p.nseg > 1 || save_den)
    if (int e = check_ws("causal_fwd", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  if (p.nseg > 1) {
    if (!(ws_has & RFA_WS_PARTIALS))
      if (int e = segment_partials((const __half*)k, (const __half*)v, ws, p, T, BH, st)) return e;
    if (int e = scan_launch(ws.s_seg, ws.z_seg, s_in, z_in, BH, p.nseg, 0, st)) return e;
    s_seg = ws.s_seg;
    z_seg = ws.z_seg;
  }
  return launch_causal_fwd_tc((const __half*)q, (const __half*)k, (const __half*)v, (__half*)out, s_seg, z_seg, s_out,
                              z_out, save_den ? ws.den : nullptr, T, BH, p.nseg, p.tseg, st);
}

extern "C" int rfa_causal_fwd_fused(const void* x_q, const void* x_k, const void* v, const float* w, const uint8_t* row_mask,
                                    float scale, void* out, const float* s_in, const float* z_in, float* s_out, float* z_out,
                                    void* workspace, size_t workspace_bytes, int64_t T, int B, int H, int d, int D,
                                    int save_den, rfa_stream_t stream) {
  RFA_REQUIRE(B > 0 && H > 0, RFA_EINVAL, "causal_fwd_fused: B=%d H=%d", B, H);
  RFA_REQUIRE(d == kD && D == kK / 2, RFA_EUNSUPPORTED,
              "causal_fwd_fused: built for head_dim = %d, proj_dim = %d (got %d, %d): use rfa_feature_map_fwd + rfa_causal_fwd", kD,
              kK / 2, d, D);
  const int BH = B * H;
  if (int e = check_geometry("causal_fwd_fused", T, BH, kK, kD, false)) return e;
  RFA_REQUIRE((s_in == nullptr) == (z_in == nullptr) && (s_out == nullptr) == (z_out == nullptr), RFA_EINVAL,
              "causal_fwd_fused: s/z pointers must be given in pairs");
  RFA_REQUIRE(T == 0 || (x_q && x_k && v && out && w), RFA_EINVAL, "causal_fwd_fused: null pointer");
  RFA_REQUIRE(aligned16(x_q) && aligned16(x_k) && aligned16(v) && aligned16(out) && aligned16(w) && aligned16(s_in) &&
                  aligned16(z_in) && aligned16(s_out) && aligned16(z_out), RFA_EALIGN, "causal_fwd_fused: 16-byte alignment required");
  RFA_REQUIRE(((uintptr_t)out & 31u) == 0, RFA_EALIGN, "causal_fwd_fused: out must be 32-byte aligned");
  cudaStream_t st = as_stream(stream);
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
    return check_launch("causal_fwd_fused(T=0)");
  }
  CausalWs ws{};
  if (save_den)      // the denominators go where a later backward on the same T, BH expects them
    if (int e = check_ws("causal_fwd_fused", workspace, workspace_bytes, T, BH, plan_causal(T, BH), &ws)) return e;
  return launch_causal_fwd_fused_tc((const __half*)x_q, (const __half*)x_k, (const __half*)v, w, row_mask, (__half*)out, s_in, z_in,
                                    s_out, z_out, save_den ? ws.den : nullptr, T, BH, H, scale, st);
}

extern "C" int rfa_causal_fwd(const void* q, const void* k, const void* v, void* out,
                              const float* s_in, const float* z_in, float* s_out, float* z_out,
                              void* workspace, size_t workspace_bytes,
                              int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  return rfa_causal_fwd_staged(q, k, v, out, s_in, z_in, s_out, z_out, workspace, workspace_bytes, T, BH, K, d, RFA_WS_EMPTY, 0,
                               stream);
}

// This shard's (or call's) own total of k (x) v and k, packed [BH][K*d + K]; leaves the per-segment partial sums in the
// workspace for rfa_causal_fwd_staged(..., RFA_WS_PARTIALS, ...).
extern "C" int rfa_causal_shard_total(const void* k, const void* v, float* total_packed, void* workspace, size_t workspace_bytes,
                                      int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("causal_shard_total", T, BH, K, d, false)) return e;
  RFA_REQUIRE(total_packed && (T == 0 || (k && v)), RFA_EINVAL, "causal_shard_total: null pointer");
  RFA_REQUIRE(aligned16(k) && aligned16(v) && aligned16(total_packed), RFA_EALIGN, "causal_shard_total: 16-byte alignment required");
  cudaStream_t st = as_stream(stream);
  if (T == 0) {
    cudaMemsetAsync(total_packed, 0, (size_t)BH * kStateN * sizeof(float), st);
    return check_launch("causal_shard_total(T=0)");
  }
  const CausalPlan p = plan_causal(T, BH);
  CausalWs ws;
  if (int e = check_ws("causal_shard_total", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  if (int e = segment_partials((const __half*)k, (const __half*)v, ws, p, T, BH, st)) return e;
  return total_launch(ws.s_seg, ws.z_seg, total_packed, nullptr, nullptr, BH, p.nseg, st);
}

extern "C" int rfa_exclusive_scan_gathered(const float* gathered, int world, int rank, int reverse, float* s_out, float* z_out,
                                           int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("exclusive_scan_gathered", 0, BH, K, d, false)) return e;
  RFA_REQUIRE(gathered && s_out && z_out, RFA_EINVAL, "exclusive_scan_gathered: null pointer");
  RFA_REQUIRE(world > 0 && rank >= 0 && rank < world, RFA_EINVAL, "exclusive_scan_gathered: rank %d of %d", rank, world);
  sm100::launch_pdl(scan_gathered_kernel, dim3(state_blocks(BH)), dim3(256), 0, as_stream(stream), gathered, world, rank, reverse ? 1 : 0, s_out, z_out, BH);
  return check_launch("rfa_exclusive_scan_gathered");
}

// ---- backward, forward-direction sweep ------------------------------------------------------------------------------
static int bwd_q_impl(const void* q, const void* k, const void* v, const void* g, const void* out, void* gq,
                      const float* s_in, const float* z_in, float* ds_tot, float* dz_tot, float* dtotal_packed,
                      void* workspace, size_t workspace_bytes, int64_t T, int BH, int K, int d, int ws_has,
                      rfa_stream_t stream) {
  if (int e = check_geometry("causal_bwd_q", T, BH, K, d, dtotal_packed == nullptr, ds_tot != nullptr)) return e;
  RFA_REQUIRE(T == 0 || (q && k && v && g && gq), RFA_EINVAL, "causal_bwd_q: null pointer");   // empty arrays have no address
  RFA_REQUIRE((s_in == nullptr) == (z_in == nullptr) && (ds_tot == nullptr) == (dz_tot == nullptr), RFA_EINVAL,
              "causal_bwd_q: s/z pointers must be given in pairs");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) && aligned16(gq) && aligned16(s_in) &&
                  aligned16(z_in) && aligned16(ds_tot) && aligned16(dz_tot) && aligned16(out) && aligned16(dtotal_packed),
              RFA_EALIGN, "causal_bwd_q: 16-byte alignment required");
  RFA_REQUIRE((ws_has & ~(RFA_WS_STATES | RFA_WS_DEN)) == 0, RFA_EINVAL,
              "causal_bwd_q: ws_has may only name RFA_WS_STATES and RFA_WS_DEN (got %d)", ws_has);
  RFA_REQUIRE(!(ws_has & RFA_WS_DEN) || out, RFA_EINVAL, "causal_bwd_q: RFA_WS_DEN needs the forward's output as well");
  const CausalPlan p = is_tc(K, d) ? plan_causal(T, BH) : CausalPlan{1, T};
  cudaStream_t st = as_stream(stream);
  const bool want_tot = ds_tot != nullptr || dtotal_packed != nullptr;
  if (T == 0) {
    if (ds_tot) {
      cudaMemsetAsync(ds_tot, 0, (size_t)BH * K * d * sizeof(float), st);
      cudaMemsetAsync(dz_tot, 0, (size_t)BH * K * sizeof(float), st);
    }
    if (dtotal_packed) cudaMemsetAsync(dtotal_packed, 0, (size_t)BH * kStateN * sizeof(float), st);
    return check_launch("causal_bwd_q(T=0)");
  }
  CausalWs ws;
  if (int e = check_ws("causal_bwd_q", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  if (!is_tc(K, d))      // the generic sweep recomputes (it does not use a saved output) and writes the totals itself
    return launch_causal_generic_bwd_q((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g, (__half*)gq, s_in,
                                       z_in, ws.den, ws.gz, ds_tot, dz_tot, T, BH, K, d, st);
  const float *s_seg = s_in, *z_seg = z_in;
  if (p.nseg > 1) {
    if (!(ws_has & RFA_WS_STATES)) {    // the states entering each segment: partial sums, then an exclusive scan
      if (int e = segment_partials((const __half*)k, (const __half*)v, ws, p, T, BH, st)) return e;
      if (int e = scan_launch(ws.s_seg, ws.z_seg, s_in, z_in, BH, p.nseg, 0, st)) return e;
    }
    s_seg = ws.s_seg;
    z_seg = ws.z_seg;
  }
  const bool want_dseg = p.nseg > 1 || want_tot;
  if (ws_has & RFA_WS_DEN) {
    if (int e = launch_causal_bwd_q_saved_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g,
                                             (const __half*)out, ws.den, (__half*)gq, s_seg, z_seg, ws.gz,
                                             want_dseg ? ws.ds_seg : nullptr, want_dseg ? ws.dz_seg : nullptr, T, BH, p.nseg,
                                             p.tseg, st))
      return e;
  } else {
    if (int e = launch_causal_bwd_q_tc((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g,
                                       (__half*)gq, s_seg, z_seg, ws.den, ws.gz, want_dseg ? ws.ds_seg : nullptr,
                                       want_dseg ? ws.dz_seg : nullptr, T, BH, p.nseg, p.tseg, st))
      return e;
  }
  if (want_tot)   // this shard's own total, before any carry is known
    return total_launch(ws.ds_seg, ws.dz_seg, dtotal_packed, ds_tot, dz_tot, BH, p.nseg, st);
  return 0;
}

extern "C" int rfa_causal_bwd_q(const void* q, const void* k, const void* v, const void* g, void* gq,
                                const float* s_in, const float* z_in, float* ds_seg, float* dz_seg,
                                void* workspace, size_t workspace_bytes,
                                int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  return bwd_q_impl(q, k, v, g, nullptr, gq, s_in, z_in, ds_seg, dz_seg, nullptr, workspace, workspace_bytes, T, BH, K, d,
                    RFA_WS_EMPTY, stream);
}

extern "C" int rfa_causal_bwd_q_staged(const void* q, const void* k, const void* v, const void* g, const void* out, void* gq,
                                       const float* s_in, const float* z_in, float* dtotal_packed,
                                       void* workspace, size_t workspace_bytes,
                                       int64_t T, int BH, int K, int d, int ws_has, rfa_stream_t stream) {
  return bwd_q_impl(q, k, v, g, out, gq, s_in, z_in, nullptr, nullptr, dtotal_packed, workspace, workspace_bytes, T, BH, K, d,
                    ws_has, stream);
}

// ---- backward, reverse sweep ----------------------------------------------------------------------------------------
extern "C" int rfa_causal_bwd_kv(const void* q, const void* k, const void* v, const void* g, void* gk, void* gv,
                                 const float* ds_in, const float* dz_in, void* workspace, size_t workspace_bytes,
                                 int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("causal_bwd_kv", T, BH, K, d)) return e;
  RFA_REQUIRE(T == 0 || (q && k && v && g && gk && gv), RFA_EINVAL, "causal_bwd_kv: null pointer");
  RFA_REQUIRE((ds_in == nullptr) == (dz_in == nullptr), RFA_EINVAL, "causal_bwd_kv: ds/dz must be given in pairs");
  RFA_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(g) && aligned16(gk) && aligned16(gv) &&
                  aligned16(ds_in) && aligned16(dz_in), RFA_EALIGN, "causal_bwd_kv: 16-byte alignment required");
  if (T == 0) return 0;
  const CausalPlan p = is_tc(K, d) ? plan_causal(T, BH) : CausalPlan{1, T};
  cudaStream_t st = as_stream(stream);
  CausalWs ws;
  if (int e = check_ws("causal_bwd_kv", workspace, workspace_bytes, T, BH, p, &ws)) return e;
  if (!is_tc(K, d))
    return launch_causal_generic_bwd_kv((const __half*)q, (const __half*)k, (const __half*)v, (const __half*)g, (__half*)gk,
                                        (__half*)gv, ws.den, ws.gz, ds_in, dz_in, T, BH, K, d, st);
  const float *ds_seg = ds_in, *dz_seg = dz_in;
  if (p.nseg > 1) {   // segment totals left by the forward-direction sweep -> reverse exclusive scan seeded with the carry
    if (int e = scan_launch(ws.ds_seg, ws.dz_seg, ds_in, dz_in, BH, p.nseg, 1, st)) return e;
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

// Backward from the forward's saved results: out and a workspace that rfa_causal_fwd_staged(..., save_den = 1) filled.
extern "C" int rfa_causal_bwd_saved(const void* q, const void* k, const void* v, const void* g, const void* out,
                                    void* gq, void* gk, void* gv, const float* s_in, const float* z_in,
                                    const float* ds_in, const float* dz_in, void* workspace, size_t workspace_bytes,
                                    int64_t T, int BH, int K, int d, int ws_has, rfa_stream_t stream) {
  if (int e = rfa_causal_bwd_q_staged(q, k, v, g, out, gq, s_in, z_in, nullptr, workspace, workspace_bytes, T, BH, K, d, ws_has, stream))
    return e;
  return rfa_causal_bwd_kv(q, k, v, g, gk, gv, ds_in, dz_in, workspace, workspace_bytes, T, BH, K, d, stream);
}

extern "C" int rfa_cross_state_fwd(const void* phi_k, const void* v, const uint8_t* pad_mask, float* s, float* z,
                                   int64_t T, int B, int H, int K, int d, rfa_stream_t stream) {
  RFA_REQUIRE(B > 0 && H > 0, RFA_EINVAL, "cross_state_fwd: B=%d H=%d", B, H);
  const int BH = B * H;
  if (int e = check_geometry("cross_state_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE(s && z && (T == 0 || (phi_k && v)), RFA_EINVAL, "cross_state_fwd: null pointer");
  RFA_REQUIRE(aligned16(phi_k) && aligned16(v) && aligned16(s) && aligned16(z), RFA_EALIGN,
              "cross_state_fwd: 16-byte alignment required");
  if (T == 0) {
    cudaMemsetAsync(s, 0, (size_t)BH * K * d * sizeof(float), as_stream(stream));
    cudaMemsetAsync(z, 0, (size_t)BH * K * sizeof(float), as_stream(stream));
    return check_launch("rfa_cross_state_fwd(T=0)");
  }
  if (!is_tc(K, d))
    return launch_state_generic_fwd((const __half*)phi_k, (const __half*)v, pad_mask, s, z, T, BH, H, 1, T, K, d, as_stream(stream));
  const int64_t tseg = ((T + kSegAlign - 1) / kSegAlign) * kSegAlign;
  return launch_cross_state_fwd_tc((const __half*)phi_k, (const __half*)v, pad_mask, s, z, T, BH, H, 1, tseg, as_stream(stream));
}

extern "C" int64_t rfa_state_partials_run_length(int64_t T, int nseg) {
  if (T <= 0 || nseg <= 0) return 0;
  const int64_t per = (T + nseg - 1) / nseg;
  return ((per + kSegAlign - 1) / kSegAlign) * kSegAlign;
}

extern "C" int rfa_state_partials(const void* phi_k, const void* v, float* s_part, float* z_part,
                                  int64_t T, int BH, int K, int d, int nseg, rfa_stream_t stream) {
  if (int e = check_geometry("state_partials", T, BH, K, d)) return e;
  RFA_REQUIRE(nseg > 0 && nseg <= 65535, RFA_EINVAL, "state_partials: nseg=%d", nseg);
  RFA_REQUIRE(s_part && z_part && (T == 0 || (phi_k && v)), RFA_EINVAL, "state_partials: null pointer");
  RFA_REQUIRE(aligned16(phi_k) && aligned16(v) && aligned16(s_part) && aligned16(z_part), RFA_EALIGN,
              "state_partials: 16-byte alignment required");
  if (T == 0) {
    cudaMemsetAsync(s_part, 0, (size_t)BH * nseg * K * d * sizeof(float), as_stream(stream));
    cudaMemsetAsync(z_part, 0, (size_t)BH * nseg * K * sizeof(float), as_stream(stream));
    return check_launch("rfa_state_partials(T=0)");
  }
  if (!is_tc(K, d))
    return launch_state_generic_fwd((const __half*)phi_k, (const __half*)v, nullptr, s_part, z_part, T, BH, 1, nseg,
                                    rfa_state_partials_run_length(T, nseg), K, d, as_stream(stream));
  return launch_cross_state_fwd_tc((const __half*)phi_k, (const __half*)v, nullptr, s_part, z_part, T, BH, 1, nseg,
                                   rfa_state_partials_run_length(T, nseg), as_stream(stream));
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
  if (!is_tc(K, d))
    return launch_state_generic_bwd((const __half*)phi_k, (const __half*)v, pad_mask, d_s, d_z, (__half*)g_phi_k, (__half*)g_v, T, BH,
                                    H, K, d, as_stream(stream));
  return launch_cross_state_bwd_tc((const __half*)phi_k, (const __half*)v, pad_mask, d_s, d_z, (__half*)g_phi_k, (__half*)g_v, T, BH,
                                   H, as_stream(stream));
}

extern "C" int rfa_cross_query_fwd(const void* phi_q, const float* s, const float* z, void* out,
                                   int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("cross_query_fwd", T, BH, K, d)) return e;
  RFA_REQUIRE(phi_q && s && z && out, RFA_EINVAL, "cross_query_fwd: null pointer");
  RFA_REQUIRE(aligned16(phi_q) && aligned16(s) && aligned16(z) && aligned16(out), RFA_EALIGN,
              "cross_query_fwd: 16-byte alignment required");
  if (T == 0) return 0;
  if (!is_tc(K, d))
    return launch_cross_generic_query_fwd((const __half*)phi_q, s, z, (__half*)out, T, BH, K, d, as_stream(stream));
  return launch_cross_query_fwd_tc((const __half*)phi_q, s, z, (__half*)out, T, BH, as_stream(stream));
}

extern "C" int rfa_cross_query_bwd(const void* phi_q, const float* s, const float* z, const void* g,
                                   void* g_phi_q, float* d_s, float* d_z,
                                   int64_t T, int BH, int K, int d, rfa_stream_t stream) {
  if (int e = check_geometry("cross_query_bwd", T, BH, K, d, true, true)) return e;
  RFA_REQUIRE(s && z && d_s && d_z && (T == 0 || (phi_q && g && g_phi_q)), RFA_EINVAL, "cross_query_bwd: null pointer");
  RFA_REQUIRE(aligned16(phi_q) && aligned16(s) && aligned16(z) && aligned16(g) && aligned16(g_phi_q) && aligned16(d_s) &&
                  aligned16(d_z), RFA_EALIGN, "cross_query_bwd: 16-byte alignment required");
  if (T == 0) {
    cudaMemsetAsync(d_s, 0, (size_t)BH * K * d * sizeof(float), as_stream(stream));
    cudaMemsetAsync(d_z, 0, (size_t)BH * K * sizeof(float), as_stream(stream));
    return check_launch("rfa_cross_query_bwd(T=0)");
  }
  if (!is_tc(K, d))
    return launch_cross_generic_query_bwd((const __half*)phi_q, s, z, (const __half*)g, (__half*)g_phi_q, d_s, d_z, T, BH, K, d,
                                          as_stream(stream));
  return launch_cross_query_bwd_tc((const __half*)phi_q, s, z, (const __half*)g, (__half*)g_phi_q, d_s, d_z, T, BH, as_stream(stream));
}
