// Measurement aid: what the memory system delivers for the access pattern of the causal kernels, with no arithmetic at
// all.  One CTA per (batch, head) walks its sequence in chunks of 128 tokens through a two-stage TMA ring exactly as
// the attention kernels do (rows of 128 bytes, one head's rows a whole [BH * width] row apart), optionally writing a
// [128][128] fp16 tile per chunk back with a TMA store.  bench.py times it to put a practical ceiling beside the copy
// bandwidth: a kernel that streams the same tiles cannot be faster than this.  No counterpart upstream.
#define RFA_TC_FAMILY 7
#include "tc_common.cuh"

namespace rfa {

// in [T][BH][64 * nb] fp16 is read as nb boxes of [128 rows][64 halves] per chunk; with_store: out [T][BH][128] written
__global__ void __launch_bounds__(128, 1)
stream_probe_kernel(const __grid_constant__ CUtensorMap tm_in, const __grid_constant__ CUtensorMap tm_out, int64_t T, int nb,
                    int with_store) {
  extern __shared__ unsigned char sp_raw[];
  unsigned char* sm = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(sp_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t bars[2];
  const int bh = blockIdx.x;
  const uint32_t stage_bytes = (uint32_t)nb * kBox;
  unsigned char* staging = sm + 2 * stage_bytes;
  if (threadIdx.x == 0) { mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_fence_init(); }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int nchunk = (int)((T + kTC - 1) / kTC);
  auto issue = [&](int c) {
    const int st = c & 1;
    mbar_arrive_expect_tx(&bars[st], stage_bytes);
    for (int b = 0; b < nb; ++b) tma_load_3d(sm + st * stage_bytes + b * kBox, &tm_in, &bars[st], b * 64, bh, c * kTC);
  };
  for (int c = 0; c < 2 && c < nchunk; ++c) issue(c);
  for (int c = 0; c < nchunk; ++c) {
    if (!mbar_wait(&bars[c & 1], (c >> 1) & 1)) { tc_fail(1); break; }
    if (with_store) {
      tma_store_wait_read<0>();
      tma_store_3d(&tm_out, staging, 0, bh, c * kTC);
      tma_store_3d(&tm_out, staging + kBox, 64, bh, c * kTC);
      tma_store_commit();
    }
    if (c + 2 < nchunk) issue(c + 2);
  }
  if (with_store) tma_store_wait<0>();
}

RFA_TC_UNIT(stream_probe)

}  // namespace rfa

using namespace rfa;

extern "C" int rfa_stream_probe(const void* in, void* out, int64_t T, int BH, int nb, int with_store, rfa_stream_t stream) {
  RFA_REQUIRE(in && (out || !with_store), RFA_EINVAL, "stream_probe: null pointer");
  RFA_REQUIRE(T > 0 && BH > 0 && BH <= 65535 && nb >= 1 && nb <= 6, RFA_EINVAL, "stream_probe: T=%lld BH=%d nb=%d (1..6)", (long long)T, BH, nb);
  RFA_REQUIRE(aligned16(in) && aligned16(out), RFA_EALIGN, "stream_probe: 16-byte alignment required");
  CUtensorMap ti, to;
  if (make_tmap_rows(&ti, in, T, BH, 64 * nb, kTC) || make_tmap_rows(&to, with_store ? out : in, T, BH, with_store ? 128 : 64 * nb, kTC))
    return fail(RFA_EDEVICE, "stream_probe: cuTensorMapEncodeTiled failed or is unavailable");
  const size_t smem = 2 * (size_t)nb * kBox + 2 * kBox + 1024;
  cudaError_t e = cudaFuncSetAttribute(stream_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail((int)e, "stream_probe: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
  stream_probe_kernel<<<BH, 128, smem, as_stream(stream)>>>(ti, to, T, nb, with_store);
  return check_launch("rfa_stream_probe");
}
