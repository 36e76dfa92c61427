/*
 * rfa_b200 -- C ABI of the B200 (sm_100a) Random Feature Attention kernels.
 *
 * Plain pointers and sizes only; no framework types.  Every pointer is a DEVICE
 * pointer unless stated otherwise, every array is contiguous in the layout
 * given, and the caller owns all memory: the library never allocates or frees
 * (the one query function below tells the caller how much scratch to bring).
 * All launches are asynchronous on the stream handed in (a cudaStream_t passed
 * as void*; NULL = the legacy default stream) on the CURRENT device.
 *
 * Return value of every int function: 0 on success; a negative RFA_E* code for
 * a rejected argument (nothing was launched); a positive value is the
 * cudaError_t of a failed launch.  rfa_last_error() gives the text for the
 * calling thread's most recent failure.
 *
 * Upstream = Noahs-ARK/RFA, package random_feature_attention; "replaces" names
 * the upstream interface (file:line) each entry point stands in for.
 *
 * Shapes: T tokens (time-major), BH = batch*heads, K = 2*D = width of phi,
 * d = head_dim.  The tensor-core attention kernels are built for K == 128 and
 * d == 64 (the only geometry upstream's benchmarks and checks use).  Any other
 * K % 8 == 0, d % 8 == 0 whose fp32 state [K][d+1] fits in shared memory (e.g.
 * K <= 256 with d <= 128) runs on plain CUDA-core kernels that walk a sequence
 * token by token, as upstream's do (cuda/forward.cu:112-125): correct, not fast.
 * The packed-total / gathered-scan entry points of the sequence-sharded path and
 * rfa_causal_bwd_noalloc exist for K == 128, d == 64 only.  Unsupported
 * geometries are rejected with RFA_EUNSUPPORTED.  fp16 arrays are IEEE binary16.
 */
#ifndef RFA_B200_H_
#define RFA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RFA_B200_VERSION 100

enum {
  RFA_OK = 0,
  RFA_EINVAL = -1,       /* null pointer, negative size, bad enum              */
  RFA_EALIGN = -2,       /* pointer not 16-byte aligned                        */
  RFA_EUNSUPPORTED = -3, /* geometry or dtype this build has no kernel for     */
  RFA_EWORKSPACE = -4,   /* workspace missing or too small                     */
  RFA_EDEVICE = -5       /* not an sm_100 device / driver entry point missing  */
};

/* element types accepted where a signature has a *_dtype argument */
enum { RFA_F16 = 0, RFA_F32 = 1 };

typedef void* rfa_stream_t;

int rfa_version(void);
const char* rfa_last_error(void);

/* Device-side health of the tensor-core kernels on the current device.  Every wait
 * inside them is bounded (about four seconds of wall-clock time); a wait that runs out
 * records its site and the kernel leaves early (its outputs are then invalid).
 * rfa_debug_status(): 0 when no wait ever ran out, else 100 * kernel family + site code;
 * synchronises the device and clears the flag.
 * rfa_status_mirror_enable(): makes the kernels on the current device also write that
 * code to one word of mapped host memory (allocated once per process with cudaHostAlloc
 * by the first call; call it once per device, outside stream capture).
 * rfa_status_peek(): that word -- no synchronisation, no clearing -- so a host can look
 * after every call and learn of a failure in an EARLIER kernel without stalling.
 * No upstream counterpart (upstream never reads launch or device errors,
 * cuda/forward.cu:155). */
int rfa_debug_status(void);
int rfa_status_mirror_enable(void);
int rfa_status_peek(void);

/* ------------------------------------------------------------------------
 * Feature map  phi(x) = scale * [sin(W xhat) | cos(W xhat)], xhat = x/(|x|+1e-3)
 * replaces utils.py:100-120 (_normalize + random_project); W is the effective
 * matrix sigma*W/tau of utils.py:90-97, fp32 [H, D, d].
 * x [rows, H, d] (rows = T*B), phi [rows, H, 2D].  d <= 128, d % 8 == 0,
 * D % 8 == 0, D <= 128.
 * ---------------------------------------------------------------------- */
int rfa_feature_map_fwd(const void* x, int x_dtype, const float* w,
                        void* phi, int phi_dtype,
                        int64_t rows, int H, int d, int D, float scale,
                        rfa_stream_t stream);

/* Gradient of the above: g_x [rows,H,d] and g_w [H,D,d] fp32.  g_w is
 * ACCUMULATED into (atomic adds): the caller zeroes it.  g_w may be NULL. */
int rfa_feature_map_bwd(const void* x, int x_dtype, const float* w,
                        const void* g_phi, int g_dtype,
                        void* g_x, int gx_dtype, float* g_w,
                        int64_t rows, int H, int d, int D, float scale,
                        rfa_stream_t stream);

/* The same two with a row mask: row_mask [rows] bytes (may be NULL), non-zero =
 * the row's features are all zero and no gradient flows through it -- a padded
 * key.  replaces the separate masked_fill pass over phi_k in cuda_causal_rfa
 * (causal_attention.py:137-143) when the caller computes phi_k itself. */
int rfa_feature_map_fwd_masked(const void* x, int x_dtype, const float* w,
                               const uint8_t* row_mask, void* phi, int phi_dtype,
                               int64_t rows, int H, int d, int D, float scale,
                               rfa_stream_t stream);
int rfa_feature_map_bwd_masked(const void* x, int x_dtype, const float* w,
                               const uint8_t* row_mask, const void* g_phi, int g_dtype,
                               void* g_x, int gx_dtype, float* g_w,
                               int64_t rows, int H, int d, int D, float scale,
                               rfa_stream_t stream);

/* The same for two arrays of one shape that share w (q and k of a self-attention
 * layer: random_project is called on both, causal_attention.py:241-248) in ONE
 * launch: one ramp and one copy of W_h instead of two, and in the backward one g_w
 * accumulator for both (g_w receives the sum of the two contributions).  fp16
 * arrays with d = D = 64 only (RFA_EUNSUPPORTED otherwise); either mask may be
 * NULL. */
int rfa_feature_map_fwd_pair(const void* x_a, const void* x_b, const float* w,
                             const uint8_t* row_mask_a, const uint8_t* row_mask_b,
                             void* phi_a, void* phi_b,
                             int64_t rows, int H, int d, int D, float scale,
                             rfa_stream_t stream);
int rfa_feature_map_bwd_pair(const void* x_a, const void* x_b, const float* w,
                             const uint8_t* row_mask_a, const uint8_t* row_mask_b,
                             const void* g_phi_a, const void* g_phi_b,
                             void* g_x_a, void* g_x_b, float* g_w,
                             int64_t rows, int H, int d, int D, float scale,
                             rfa_stream_t stream);

/* Effective random matrices for a whole step in one launch:
 *   out[i] = sigma[i] * bank[idx[i]] * inv_tau[i],  i < n_out
 * bank [n_bank, D, d] (fp16 or fp32, resident on the device), idx [n_out] int64,
 * sigma [n_out, d] fp32 or NULL, inv_tau [n_out] fp32 or NULL, out [n_out, D, d]
 * fp32.  An index outside the bank sets *bad_index_flag (a device int the caller
 * zeroes) and yields zeros.  replaces the host-side gather of
 * sample_random_matrices (utils.py:62-87) plus build_random_matrices per layer
 * (utils.py:90-97). */
int rfa_gather_random_matrices(const void* bank, int bank_dtype, int64_t n_bank,
                               const int64_t* idx, int64_t n_out,
                               const float* sigma, const float* inv_tau, float* out,
                               int D, int d, int* bad_index_flag, rfa_stream_t stream);

/* ------------------------------------------------------------------------
 * Causal RFA.  q,k [T,BH,K] fp16, v/out/g [T,BH,d] fp16, time-major.
 *   out_t = q_t^T S_t / max(q_t . z_t, 1),  S_t = S_in + sum_{s<=t} k_s v_s^T,
 *   z_t = z_in + sum_{s<=t} k_s.
 * replaces rfa_cuda.forward  (cuda/rfa_cuda.cpp:22-27 -> cuda/forward.cu:128-169)
 *      and rfa_cuda.backward (cuda/rfa_cuda.cpp:29-36 -> cuda/backward.cu:530-585),
 * reached from RFA.forward/backward (rfa.py:113-145).
 *
 * s_in/z_in ([BH,K,d] / [BH,K] fp32, may both be NULL = zeros) is the state of
 * tokens before this call's first token; s_out/z_out (may be NULL) receives
 * the state after its last token (prefill -> decode hand-off; segment carry).
 * workspace: rfa_causal_workspace_bytes(T,BH,K,d) bytes, 256-byte aligned.
 * ---------------------------------------------------------------------- */
size_t rfa_causal_workspace_bytes(int64_t T, int BH, int K, int d);

int rfa_causal_fwd(const void* q, const void* k, const void* v, void* out,
                   const float* s_in, const float* z_in,
                   float* s_out, float* z_out,
                   void* workspace, size_t workspace_bytes,
                   int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* Full backward.  ds_in/dz_in (NULL = zeros) is the reverse carry: the sum over
 * tokens AFTER this call's last token of q (x) grad_qs and of q*grad_qz. */
int rfa_causal_bwd(const void* q, const void* k, const void* v, const void* g,
                   void* gq, void* gk, void* gv,
                   const float* s_in, const float* z_in,
                   const float* ds_in, const float* dz_in,
                   void* workspace, size_t workspace_bytes,
                   int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* Backward without any caller scratch and without any allocation: the same two
 * sweeps as rfa_causal_bwd from a zero state (no carries), with the per-token
 * scalars kept in a fixed 4 MiB array inside the library (present on every GPU
 * that loads it).  For hosts that may not call cudaMalloc once they are running
 * (a server that owns all device memory in its own pools; a C caller without a
 * device allocator).  It has no counterpart in upstream, whose extension
 * allocates its outputs itself (cuda/backward.cu:556-558).
 *   - T * BH must not exceed rfa_causal_bwd_noalloc_max_token_heads() (524288);
 *     larger problems are refused with RFA_EWORKSPACE.
 *   - The first call on each device looks up the array's device address
 *     (cudaGetSymbolAddress), and a host thread's first launch of any kernel of
 *     this library binds the device's primary context to that thread
 *     (cudaSetDevice on the current device); make the first call on each device
 *     and from each calling thread before starting any stream capture.
 *   - All calls on a device share the one array: two calls whose kernels can
 *     overlap on the GPU (different streams, no dependency) race on it.  Calls
 *     on one stream are safe.  Nothing in it needs clearing between calls: each
 *     call's first sweep rewrites every element its second sweep reads.
 *   - Allocates nothing: no cudaMalloc, cudaFree, cudaHostAlloc or allocating
 *     library routine is called, on the first call or later. */
int64_t rfa_causal_bwd_noalloc_max_token_heads(void);
int rfa_causal_bwd_noalloc(const void* q, const void* k, const void* v, const void* g,
                           void* gq, void* gk, void* gv,
                           int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* ------------------------------------------------------------------------
 * Staged forms of the causal path: the same kernels, for callers that keep the
 * workspace (and the forward's output) from one call to the next -- an autograd
 * function between forward and backward, the shards of a split sequence between
 * their local steps and the exchange.  No counterpart upstream, whose backward
 * recomputes everything from (q, k, v) (rfa.py:126-145, cuda/backward.cu:303-371)
 * and whose kernels walk a whole sequence in one CTA (cuda/forward.cu:112-125).
 *
 * ws_has says what the workspace already holds FOR THESE SAME ARGUMENTS:
 *   RFA_WS_PARTIALS  per-segment sums of k (x) v and k, left by
 *                    rfa_causal_shard_total (the forward then skips that pass);
 *   RFA_WS_STATES    the states entering each segment, left by any forward call
 *                    with the same s_in/z_in (the backward then skips both the
 *                    pass and the scan);
 *   RFA_WS_DEN       the raw denominators q_t . z_t, left by a forward call with
 *                    save_den != 0.  Together with the forward's output `out`
 *                    the forward-direction sweep then recomputes neither the
 *                    scores nor the numerators and reads q only when a
 *                    reverse-state total is asked for or the sequence is cut
 *                    into segments.
 * A call that names something the workspace does not hold computes garbage.
 *
 * rfa_causal_shard_total: total_packed [BH, K*d + K] = [sum k (x) v | sum k] over
 * this call's tokens.  rfa_exclusive_scan_gathered: from gathered
 * [world, BH, K*d + K] (every shard's packed total, e.g. after an all-gather) the
 * sum over the shards before (reverse != 0: after) shard `rank`, as s_out
 * [BH,K,d] and z_out [BH,K].  rfa_causal_bwd_q_staged: as rfa_causal_bwd_q, with
 * the reverse-state total written packed (dtotal_packed, may be NULL) and `out`
 * (may be NULL without RFA_WS_DEN).  rfa_causal_bwd_saved: both sweeps.
 * ---------------------------------------------------------------------- */
enum { RFA_WS_EMPTY = 0, RFA_WS_PARTIALS = 1, RFA_WS_STATES = 2, RFA_WS_DEN = 4 };

int rfa_causal_fwd_staged(const void* q, const void* k, const void* v, void* out,
                          const float* s_in, const float* z_in,
                          float* s_out, float* z_out,
                          void* workspace, size_t workspace_bytes,
                          int64_t T, int BH, int K, int d,
                          int ws_has, int save_den, rfa_stream_t stream);
int rfa_causal_shard_total(const void* k, const void* v, float* total_packed,
                           void* workspace, size_t workspace_bytes,
                           int64_t T, int BH, int K, int d, rfa_stream_t stream);
int rfa_exclusive_scan_gathered(const float* gathered, int world, int rank, int reverse,
                                float* s_out, float* z_out,
                                int BH, int K, int d, rfa_stream_t stream);
int rfa_causal_bwd_q_staged(const void* q, const void* k, const void* v, const void* g,
                            const void* out, void* gq,
                            const float* s_in, const float* z_in, float* dtotal_packed,
                            void* workspace, size_t workspace_bytes,
                            int64_t T, int BH, int K, int d, int ws_has, rfa_stream_t stream);
int rfa_causal_bwd_saved(const void* q, const void* k, const void* v, const void* g,
                         const void* out, void* gq, void* gk, void* gv,
                         const float* s_in, const float* z_in,
                         const float* ds_in, const float* dz_in,
                         void* workspace, size_t workspace_bytes,
                         int64_t T, int BH, int K, int d, int ws_has, rfa_stream_t stream);

/* The two halves of the backward, for a sequence sharded across devices:
 * _bwd_q runs the forward-direction sweep (gq; leaves per-token scalars in the
 * workspace) and writes this shard's own reverse-state total to ds_seg/dz_seg;
 * after the shards have exchanged those, _bwd_kv runs the reverse sweep with
 * the carry ds_in/dz_in.  The same workspace must be passed to both. */
int rfa_causal_bwd_q(const void* q, const void* k, const void* v, const void* g,
                     void* gq, const float* s_in, const float* z_in,
                     float* ds_seg, float* dz_seg,
                     void* workspace, size_t workspace_bytes,
                     int64_t T, int BH, int K, int d, rfa_stream_t stream);
int rfa_causal_bwd_kv(const void* q, const void* k, const void* v, const void* g,
                      void* gk, void* gv, const float* ds_in, const float* dz_in,
                      void* workspace, size_t workspace_bytes,
                      int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* ------------------------------------------------------------------------
 * State reduction  s = sum_t k_t v_t^T [BH,K,d], z = sum_t k_t [BH,K]  (fp32)
 * over unpadded positions; k [T,BH,K], v [T,BH,d] fp16; pad_mask [B,T] bytes
 * (non-zero = padding, may be NULL), BH = B*H with bh = b*H + h.
 * replaces cross_attention.py:97-104 (masked_fill + einsum + sum); also the
 * per-shard total of the sequence-sharded causal path.
 * ---------------------------------------------------------------------- */
int rfa_cross_state_fwd(const void* phi_k, const void* v, const uint8_t* pad_mask,
                        float* s, float* z,
                        int64_t T, int B, int H, int K, int d, rfa_stream_t stream);

/* The same reduction over nseg contiguous runs of tokens at once (nseg CTAs per
 * (batch, head) instead of one, for few long sequences): s_part [BH,nseg,K,d],
 * z_part [BH,nseg,K] fp32, run i covering tokens [i*L, min(T,(i+1)*L)) with
 * L = rfa_state_partials_run_length(T, nseg) (a multiple of 128); the caller
 * sums over nseg.  No padding mask.  No counterpart upstream (its kernels walk a
 * whole sequence in one CTA, cuda/forward.cu:112-125); used for the per-shard
 * totals of the sequence-sharded causal path. */
int64_t rfa_state_partials_run_length(int64_t T, int nseg);
int rfa_state_partials(const void* phi_k, const void* v, float* s_part, float* z_part,
                       int64_t T, int BH, int K, int d, int nseg, rfa_stream_t stream);

/* Gradient of the reduction: g_phi_k [T,BH,K] (zero at padded rows),
 * g_v [T,BH,d] from d_s [BH,K,d], d_z [BH,K] fp32. */
int rfa_cross_state_bwd(const void* phi_k, const void* v, const uint8_t* pad_mask,
                        const float* d_s, const float* d_z,
                        void* g_phi_k, void* g_v,
                        int64_t T, int B, int H, int K, int d, rfa_stream_t stream);

/* out_t = phi_q_t . s / max(|phi_q_t . z|, 1);  phi_q [T,BH,K], out [T,BH,d] fp16.
 * replaces CrossAttention.rfa, cross_attention.py:266-269. */
int rfa_cross_query_fwd(const void* phi_q, const float* s, const float* z, void* out,
                        int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* Gradient of the above for upstream g [T,BH,d]: g_phi_q [T,BH,K] fp16 and the
 * state gradients d_s [BH,K,d], d_z [BH,K] fp32 (overwritten, not accumulated). */
int rfa_cross_query_bwd(const void* phi_q, const float* s, const float* z, const void* g,
                        void* g_phi_q, float* d_s, float* d_z,
                        int64_t T, int BH, int K, int d, rfa_stream_t stream);

/* ------------------------------------------------------------------------
 * One incremental-decoding step, in place on the state:
 *   s += phi_k (x) v;  z += phi_k;  out = phi_q . s / max(phi_q . z, 1)
 * phi_q, phi_k [BH,K], v/out [BH,d] of in_dtype; s [BH,K,d], z [BH,K] of
 * state_dtype.  replaces the loop body of incremental_rfa,
 * causal_attention.py:42-50 (which allocates a new state every token).
 * ---------------------------------------------------------------------- */
int rfa_decode_step(const void* phi_q, const void* phi_k, const void* v, int in_dtype,
                    void* s, void* z, int state_dtype, void* out,
                    int BH, int K, int d, rfa_stream_t stream);

/* The same step from raw q,k [BH,d]: applies the feature map (W fp32 [H,D,d],
 * bh % H selects the head) inside the kernel.  K = 2*D. */
int rfa_decode_step_fused(const void* q, const void* k, const void* v, int in_dtype,
                          const float* w, float scale,
                          void* s, void* z, int state_dtype, void* out,
                          int BH, int H, int D, int d, rfa_stream_t stream);

/* One decoding step of cross attention for all L layers in one launch:
 *   out[l] = phi_q[l] . s_l / max(|phi_q[l] . z_l|, 1)
 * phi_q [L,BH,K], out [L,BH,d] of in_dtype; s_ptrs / z_ptrs: DEVICE arrays of L
 * pointers to the layers' fp32 states [BH,K,d] / [BH,K] (16-byte aligned; they do
 * not change while a sequence is decoded, so the arrays are built once).
 * replaces L calls of CrossAttention.rfa with tgt_len 1 (cross_attention.py:266-269). */
int rfa_cross_decode_step(const void* phi_q, int in_dtype,
                          const float* const* s_ptrs, const float* const* z_ptrs,
                          void* out, int L, int BH, int K, int d, rfa_stream_t stream);

/* Causal forward with the feature map inside the kernel: replaces
 * utils.random_project on q and k (utils.py:100-120, called at
 * causal_attention.py:241-248, with the masked_fill of padded keys at :137-143)
 * followed by RFA.forward (rfa.py:113-124, cuda/forward.cu:16-169).
 * x_q, x_k, v, out: [T, B*H, d] fp16, the head index fastest in the middle axis;
 * w [H, D, d] fp32 (the matrices build_random_matrices returns, sigma and 1/tau
 * folded in); row_mask [T, B] bytes, nonzero = padded key, or NULL; scale = the
 * feature scale (D^-1/2 upstream).  The features phi [T, B*H, 2D] are formed tile
 * by tile in shared memory and never written.  d = 64, D = 64 only.  One CTA per
 * (batch, head): meant for B*H of about the SM count or more.
 * s_in/z_in/s_out/z_out as in rfa_causal_fwd.  save_den != 0: the raw
 * denominators are left in `workspace` (rfa_causal_workspace_bytes(T, B*H, 2D, d))
 * where rfa_causal_bwd_saved(..., ws_has = RFA_WS_DEN) finds them, once the caller
 * has recomputed the features with rfa_feature_map_fwd[_masked]; otherwise the
 * workspace may be NULL. */
int rfa_causal_fwd_fused(const void* x_q, const void* x_k, const void* v,
                         const float* w, const uint8_t* row_mask, float scale,
                         void* out,
                         const float* s_in, const float* z_in,
                         float* s_out, float* z_out,
                         void* workspace, size_t workspace_bytes,
                         int64_t T, int B, int H, int d, int D,
                         int save_den, rfa_stream_t stream);

/* Measurement aid, no upstream counterpart: streams in [T, BH, 64*nb] fp16 through
 * shared memory with the tile pattern of the causal kernels (one CTA per (batch,
 * head), chunks of 128 tokens, nb boxes of 128 rows x 128 bytes per chunk, two
 * stages) and, with_store != 0, writes one [128][128] fp16 tile per chunk to out
 * [T, BH, 128].  No arithmetic: its time is the memory system's own for this
 * pattern; bench.py reports it beside the copy bandwidth. */
int rfa_stream_probe(const void* in, void* out, int64_t T, int BH, int nb, int with_store,
                     rfa_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* RFA_B200_H_ */
