"""Tensor-level wrappers over the C ABI: allocate outputs, pass raw pointers and
the current stream, turn status codes into exceptions.  No arithmetic happens
here; every function launches kernels from ``librfa_b200.so``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from ._lib import check, dtype_code, ptr, require_half, stream_of

K_BUILT, D_BUILT = 128, 64      # geometry the attention kernels are built for


def _guard(t: Tensor):
    if not t.is_cuda:
        raise RuntimeError(f"rfa_b200 kernels take CUDA tensors only (there is no CPU path); got a {t.device} tensor")
    return _Guard(t.device)


class _Guard:
    """Make the tensor's device current for the call and, on first use of a device, switch on the status mirror."""

    def __init__(self, device):
        self.ctx = torch.cuda.device(device)
        self.index = device.index if device.index is not None else torch.cuda.current_device()

    def __enter__(self):
        self.ctx.__enter__()
        _lib.watch_device(self.index)
        return self

    def __exit__(self, *a):
        return self.ctx.__exit__(*a)


def _workspace(T: int, BH: int, K: int, d: int, like: Tensor) -> Tuple[Tensor, int]:
    n = _lib.load().rfa_causal_workspace_bytes(T, BH, K, d)
    ws = torch.empty(max(n, 256), dtype=torch.uint8, device=like.device)
    return ws, n


# --------------------------------------------------------------------------- feature map
def _row_mask(row_mask: Optional[Tensor], rows: int, dev) -> Optional[Tensor]:
    if row_mask is None:
        return None
    m = (row_mask.to(device=dev).reshape(-1) != 0).to(torch.uint8).contiguous()
    assert m.numel() == rows, (m.numel(), rows)
    return m


def feature_map_fwd(x: Tensor, w: Tensor, scale: float, out_dtype: Optional[torch.dtype] = None,
                    row_mask: Optional[Tensor] = None) -> Tensor:
    """x [..., H, d], w [H, D, d] fp32 -> phi [..., H, 2D].  row_mask (one entry per leading index, non-zero = masked):
    those rows get all-zero features."""
    H, D, d = w.shape
    assert x.shape[-2] == H and x.shape[-1] == d, (x.shape, w.shape)
    x = x.contiguous()
    w = w.contiguous().float()
    phi = torch.empty(*x.shape[:-1], 2 * D, dtype=out_dtype or x.dtype, device=x.device)
    rows = x.numel() // (H * d)
    m = _row_mask(row_mask, rows, x.device)
    with _guard(x):
        check(_lib.load().rfa_feature_map_fwd_masked(ptr(x), dtype_code(x), ptr(w), ptr(m), ptr(phi), dtype_code(phi),
                                                     rows, H, d, D, float(scale), stream_of(x)), "rfa_feature_map_fwd")
    return phi


def feature_map_bwd(x: Tensor, w: Tensor, g_phi: Tensor, scale: float, need_gw: bool,
                    row_mask: Optional[Tensor] = None) -> Tuple[Tensor, Optional[Tensor]]:
    H, D, d = w.shape
    x = x.contiguous()
    w = w.contiguous().float()
    g_phi = g_phi.contiguous().to(x.dtype)
    g_x = torch.empty_like(x)
    g_w = torch.zeros(H, D, d, dtype=torch.float32, device=x.device) if need_gw else None
    rows = x.numel() // (H * d)
    m = _row_mask(row_mask, rows, x.device)
    with _guard(x):
        check(_lib.load().rfa_feature_map_bwd_masked(ptr(x), dtype_code(x), ptr(w), ptr(m), ptr(g_phi), dtype_code(g_phi),
                                                     ptr(g_x), dtype_code(g_x), ptr(g_w), rows, H, d, D, float(scale),
                                                     stream_of(x)), "rfa_feature_map_bwd")
    return g_x, g_w


def feature_map_pair_supported(x_a: Tensor, x_b: Tensor, w: Tensor) -> bool:
    """Whether the one-launch feature map of two arrays takes these: same shape, fp16, head_dim = proj_dim = 64."""
    return (x_a.shape == x_b.shape and x_a.dtype == x_b.dtype == torch.float16 and x_a.is_cuda and x_b.is_cuda
            and tuple(w.shape[-2:]) == (64, 64))


def feature_map_fwd_pair(x_a: Tensor, x_b: Tensor, w: Tensor, scale: float, row_mask_a: Optional[Tensor] = None,
                         row_mask_b: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """phi of x_a and of x_b (same shape [..., H, 64], fp16; w [H, 64, 64]) in one launch."""
    H, D, d = w.shape
    assert x_a.shape == x_b.shape and x_a.shape[-2] == H and x_a.shape[-1] == d, (x_a.shape, x_b.shape, w.shape)
    require_half(x_a, x_b)
    x_a, x_b = x_a.contiguous(), x_b.contiguous()
    w = w.contiguous().float()
    phi_a = torch.empty(*x_a.shape[:-1], 2 * D, dtype=torch.float16, device=x_a.device)
    phi_b = torch.empty_like(phi_a)
    rows = x_a.numel() // (H * d)
    ma, mb = _row_mask(row_mask_a, rows, x_a.device), _row_mask(row_mask_b, rows, x_a.device)
    with _guard(x_a):
        check(_lib.load().rfa_feature_map_fwd_pair(ptr(x_a), ptr(x_b), ptr(w), ptr(ma), ptr(mb), ptr(phi_a), ptr(phi_b), rows, H, d, D,
                                                   float(scale), stream_of(x_a)), "rfa_feature_map_fwd_pair")
    return phi_a, phi_b


def feature_map_bwd_pair(x_a: Tensor, x_b: Tensor, w: Tensor, g_phi_a: Tensor, g_phi_b: Tensor, scale: float, need_gw: bool,
                         row_mask_a: Optional[Tensor] = None, row_mask_b: Optional[Tensor] = None):
    """Backward of ``feature_map_fwd_pair``: (g_x_a, g_x_b, g_w) with g_w the sum of both arrays' contributions (or None)."""
    H, D, d = w.shape
    require_half(x_a, x_b)
    x_a, x_b = x_a.contiguous(), x_b.contiguous()
    w = w.contiguous().float()
    g_phi_a, g_phi_b = g_phi_a.contiguous().to(torch.float16), g_phi_b.contiguous().to(torch.float16)
    g_x_a, g_x_b = torch.empty_like(x_a), torch.empty_like(x_b)
    g_w = torch.zeros(H, D, d, dtype=torch.float32, device=x_a.device) if need_gw else None
    rows = x_a.numel() // (H * d)
    ma, mb = _row_mask(row_mask_a, rows, x_a.device), _row_mask(row_mask_b, rows, x_a.device)
    with _guard(x_a):
        check(_lib.load().rfa_feature_map_bwd_pair(ptr(x_a), ptr(x_b), ptr(w), ptr(ma), ptr(mb), ptr(g_phi_a), ptr(g_phi_b), ptr(g_x_a),
                                                   ptr(g_x_b), ptr(g_w), rows, H, d, D, float(scale), stream_of(x_a)),
              "rfa_feature_map_bwd_pair")
    return g_x_a, g_x_b, g_w


def gather_random_matrices(bank: Tensor, picks: Tensor, sigma: Optional[Tensor] = None,
                           inv_tau: Optional[Tensor] = None) -> Tensor:
    """bank [N, D, d] (fp16 / fp32, on the device), picks [n] int64 -> [n, D, d] fp32 = sigma[i] * bank[picks[i]] * inv_tau[i]
    (sigma [n, d], inv_tau [n], both optional), one launch."""
    N, D, d = bank.shape
    bank = bank.contiguous()
    picks = picks.to(device=bank.device, dtype=torch.int64).contiguous()
    n = picks.numel()
    out = torch.empty(n, D, d, dtype=torch.float32, device=bank.device)
    if sigma is not None:
        sigma = sigma.to(device=bank.device, dtype=torch.float32).reshape(n, d).contiguous()
    if inv_tau is not None:
        inv_tau = inv_tau.to(device=bank.device, dtype=torch.float32).reshape(n).contiguous()
    bad = torch.zeros(1, dtype=torch.int32, device=bank.device)
    with _guard(bank):
        check(_lib.load().rfa_gather_random_matrices(ptr(bank), dtype_code(bank), N, ptr(picks), n, ptr(sigma), ptr(inv_tau),
                                                     ptr(out), D, d, ptr(bad), stream_of(bank)), "rfa_gather_random_matrices")
    return out, bad


# --------------------------------------------------------------------------- causal
def causal_fwd(q: Tensor, k: Tensor, v: Tensor, s_in: Optional[Tensor] = None, z_in: Optional[Tensor] = None,
               return_state: bool = False):
    """q,k [T,BH,K], v [T,BH,d] fp16 -> out [T,BH,d] (and the final state when asked)."""
    require_half(q, k, v)
    T, BH, K = q.shape
    d = v.shape[-1]
    assert k.shape == q.shape and v.shape[:2] == q.shape[:2]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty(T, BH, d, dtype=torch.float16, device=q.device)
    if s_in is not None:
        s_in, z_in = s_in.contiguous().float(), z_in.contiguous().float()
    if T == 0:      # nothing to launch (empty tensors have no address); the state passes through
        if not return_state:
            return out
        if s_in is None:
            return out, torch.zeros(BH, K, d, device=q.device), torch.zeros(BH, K, device=q.device)
        return out, s_in.clone(), z_in.clone()
    s_out = torch.empty(BH, K, d, dtype=torch.float32, device=q.device) if return_state else None
    z_out = torch.empty(BH, K, dtype=torch.float32, device=q.device) if return_state else None
    ws, n = _workspace(T, BH, K, d, q)
    with _guard(q):
        check(_lib.load().rfa_causal_fwd(ptr(q), ptr(k), ptr(v), ptr(out), ptr(s_in), ptr(z_in), ptr(s_out),
                                         ptr(z_out), ptr(ws), n, T, BH, K, d, stream_of(q)), "rfa_causal_fwd")
    return (out, s_out, z_out) if return_state else out


def causal_bwd(q: Tensor, k: Tensor, v: Tensor, g: Tensor, s_in: Optional[Tensor] = None,
               z_in: Optional[Tensor] = None, ds_in: Optional[Tensor] = None, dz_in: Optional[Tensor] = None):
    require_half(q, k, v, g)
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if T == 0:
        return gq, gk, gv
    ws, n = _workspace(T, BH, K, d, q)
    with _guard(q):
        check(_lib.load().rfa_causal_bwd(ptr(q), ptr(k), ptr(v), ptr(g), ptr(gq), ptr(gk), ptr(gv), ptr(s_in),
                                         ptr(z_in), ptr(ds_in), ptr(dz_in), ptr(ws), n, T, BH, K, d, stream_of(q)),
              "rfa_causal_bwd")
    return gq, gk, gv


# --------------------------------------------------------------------------- causal, staged (kept workspace / saved output)
STATE_N = K_BUILT * D_BUILT + K_BUILT      # floats of one packed state [S | z]


def causal_fwd_saved(q: Tensor, k: Tensor, v: Tensor, s_in: Optional[Tensor] = None, z_in: Optional[Tensor] = None,
                     ws: Optional[Tensor] = None, ws_has: int = 0):
    """Forward that keeps what the backward can reuse.  Returns (out, workspace, ws_has): the workspace then holds the
    raw denominators and, when the sequence is cut into segments, the states entering each of them.  ``ws`` / ``ws_has``
    hand in a workspace that ``shard_total`` has already filled for the same k, v."""
    require_half(q, k, v)
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    out = torch.empty(T, BH, d, dtype=torch.float16, device=q.device)
    if T == 0:
        return out, torch.empty(256, dtype=torch.uint8, device=q.device), 0
    if ws is None:
        ws, _ = _workspace(T, BH, K, d, q)
        ws_has = 0
    with _guard(q):
        check(_lib.load().rfa_causal_fwd_staged(ptr(q), ptr(k), ptr(v), ptr(out), ptr(s_in), ptr(z_in), None, None,
                                                ptr(ws), ws.numel(), T, BH, K, d, ws_has & _lib.WS_PARTIALS, 1, stream_of(q)),
              "rfa_causal_fwd_staged")
    return out, ws, _lib.WS_STATES | _lib.WS_DEN


def fused_forward_supported(x: Tensor, w: Tensor) -> bool:
    """Whether ``causal_fwd_fused`` takes these inputs: fp16 vectors of head_dim 64 with proj_dim 64 matrices, and enough
    (batch, head) sequences that one CTA each fills the GPU (the kernel does not cut a sequence into segments)."""
    T, B, H, d = x.shape
    return (x.dtype == torch.float16 and x.is_cuda and d == 64 and tuple(w.shape[-2:]) == (64, 64)
            and (B * H >= 120 or T < 1024))


def causal_fwd_fused(x_q: Tensor, x_k: Tensor, v: Tensor, w: Tensor, scale: float, row_mask: Optional[Tensor] = None,
                     s_in: Optional[Tensor] = None, z_in: Optional[Tensor] = None, return_state: bool = False,
                     save_den: bool = False):
    """Causal RFA forward from the raw per-head vectors: x_q, x_k, v [T, B, H, 64] fp16, w [H, 64, 64] fp32; the features
    scale * [sin | cos]((W x) / (|x| + 1e-3)) of q and k are formed inside the kernel.  row_mask [T, B] (or [T * B]) marks
    padded keys.  Returns out [T, B*H, 64] and, as asked, the final state (s, z) and the workspace holding the raw
    denominators for ``causal_bwd_saved(..., ws_has=WS_DEN)``: (out[, s, z][, ws])."""
    require_half(x_q, x_k, v)
    T, B, H, d = x_q.shape
    D = w.shape[-2]
    x_q, x_k, v = x_q.contiguous(), x_k.contiguous(), v.contiguous()
    w = w.contiguous().float()
    BH = B * H
    out = torch.empty(T, BH, d, dtype=torch.float16, device=x_q.device)
    m = _row_mask(row_mask, T * B, x_q.device)
    s_out = z_out = None
    if return_state:
        s_out = torch.empty(BH, 2 * D, d, dtype=torch.float32, device=x_q.device)
        z_out = torch.empty(BH, 2 * D, dtype=torch.float32, device=x_q.device)
    ws = None
    if save_den:
        ws, _ = _workspace(max(T, 1), BH, 2 * D, d, x_q)
    with _guard(x_q):
        check(_lib.load().rfa_causal_fwd_fused(ptr(x_q), ptr(x_k), ptr(v), ptr(w), ptr(m), float(scale), ptr(out), ptr(s_in),
                                               ptr(z_in), ptr(s_out), ptr(z_out), ptr(ws), ws.numel() if ws is not None else 0,
                                               T, B, H, d, D, 1 if save_den else 0, stream_of(x_q)), "rfa_causal_fwd_fused")
    res = (out,)
    if return_state:
        res += (s_out, z_out)
    if save_den:
        res += (ws,)
    return res if len(res) > 1 else out


def causal_bwd_saved(q: Tensor, k: Tensor, v: Tensor, g: Tensor, out: Tensor, ws: Tensor, ws_has: int,
                     s_in: Optional[Tensor] = None, z_in: Optional[Tensor] = None):
    """Backward from the forward's output and kept workspace (``causal_fwd_saved``)."""
    require_half(q, k, v, g, out)
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v, g, out = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous(), out.contiguous()
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    if T == 0:
        return gq, gk, gv
    with _guard(q):
        check(_lib.load().rfa_causal_bwd_saved(ptr(q), ptr(k), ptr(v), ptr(g), ptr(out), ptr(gq), ptr(gk), ptr(gv), ptr(s_in),
                                               ptr(z_in), None, None, ptr(ws), ws.numel(), T, BH, K, d, ws_has, stream_of(q)),
              "rfa_causal_bwd_saved")
    return gq, gk, gv


def shard_total(k: Tensor, v: Tensor, packed: Optional[Tensor] = None):
    """This shard's own [sum k (x) v | sum k], packed [BH, K*d + K] fp32 (into ``packed`` when given, e.g. a slice of an
    all-gather buffer), and the workspace holding the per-segment partial sums for ``causal_fwd_saved``."""
    require_half(k, v)
    T, BH, K = k.shape
    d = v.shape[-1]
    k, v = k.contiguous(), v.contiguous()
    if packed is None:
        packed = torch.empty(BH, K * d + K, dtype=torch.float32, device=k.device)
    if T == 0:
        packed.zero_()
        return packed, None
    ws, _ = _workspace(T, BH, K, d, k)
    with _guard(k):
        check(_lib.load().rfa_causal_shard_total(ptr(k), ptr(v), ptr(packed), ptr(ws), ws.numel(), T, BH, K, d, stream_of(k)),
              "rfa_causal_shard_total")
    return packed, ws


def scan_gathered(gathered: Tensor, rank: int, reverse: bool, K: int = K_BUILT, d: int = D_BUILT):
    """gathered [world, BH, K*d + K] fp32 (every shard's packed total) -> the carry of shard ``rank``: the sum over the
    shards before (``reverse``: after) it, as (s [BH,K,d], z [BH,K])."""
    world, BH, n = gathered.shape
    assert n == K * d + K and gathered.dtype == torch.float32 and gathered.is_contiguous()
    s = torch.empty(BH, K, d, dtype=torch.float32, device=gathered.device)
    z = torch.empty(BH, K, dtype=torch.float32, device=gathered.device)
    with _guard(gathered):
        check(_lib.load().rfa_exclusive_scan_gathered(ptr(gathered), world, rank, int(reverse), ptr(s), ptr(z), BH, K, d,
                                                      stream_of(gathered)), "rfa_exclusive_scan_gathered")
    return s, z


def causal_bwd_q_staged(q, k, v, g, out, s_in, z_in, ws: Tensor, ws_has: int, packed: Optional[Tensor] = None,
                        want_total: bool = True):
    """Forward-direction half of the backward on a kept workspace.  Returns (gq, packed reverse-state total or None)."""
    require_half(q, k, v, g)
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    gq = torch.empty_like(q)
    if want_total and packed is None:
        packed = torch.empty(BH, K * d + K, dtype=torch.float32, device=q.device)
    if T == 0:
        if want_total:
            packed.zero_()
        return gq, packed if want_total else None
    with _guard(q):
        check(_lib.load().rfa_causal_bwd_q_staged(ptr(q), ptr(k), ptr(v), ptr(g), ptr(out), ptr(gq), ptr(s_in), ptr(z_in),
                                                  ptr(packed) if want_total else None, ptr(ws), ws.numel(), T, BH, K, d, ws_has,
                                                  stream_of(q)), "rfa_causal_bwd_q_staged")
    return gq, packed if want_total else None


def causal_bwd_q(q, k, v, g, s_in, z_in, want_dseg: bool):
    """Forward-direction half of the backward.  Returns (gq, ds_seg, dz_seg, workspace)."""
    require_half(q, k, v, g)
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    gq = torch.empty_like(q)
    if T == 0:      # an empty shard: nothing to launch (empty tensors have no address); its reverse-state total is zero
        zeros = (torch.zeros(BH, K, d, device=q.device), torch.zeros(BH, K, device=q.device)) if want_dseg else (None, None)
        return gq, zeros[0], zeros[1], torch.empty(256, dtype=torch.uint8, device=q.device)
    ds = torch.empty(BH, K, d, dtype=torch.float32, device=q.device) if want_dseg else None
    dz = torch.empty(BH, K, dtype=torch.float32, device=q.device) if want_dseg else None
    ws, n = _workspace(T, BH, K, d, q)
    with _guard(q):
        check(_lib.load().rfa_causal_bwd_q(ptr(q), ptr(k), ptr(v), ptr(g), ptr(gq), ptr(s_in), ptr(z_in), ptr(ds),
                                           ptr(dz), ptr(ws), n, T, BH, K, d, stream_of(q)), "rfa_causal_bwd_q")
    return gq, ds, dz, ws


def causal_bwd_kv(q, k, v, g, ds_in, dz_in, ws: Tensor):
    T, BH, K = q.shape
    d = v.shape[-1]
    q, k, v, g = q.contiguous(), k.contiguous(), v.contiguous(), g.contiguous()
    gk, gv = torch.empty_like(k), torch.empty_like(v)
    if T == 0:
        return gk, gv
    with _guard(q):
        check(_lib.load().rfa_causal_bwd_kv(ptr(q), ptr(k), ptr(v), ptr(g), ptr(gk), ptr(gv), ptr(ds_in), ptr(dz_in),
                                            ptr(ws), ws.numel(), T, BH, K, d, stream_of(q)), "rfa_causal_bwd_kv")
    return gk, gv


# --------------------------------------------------------------------------- cross
def _mask_bytes(pad_mask: Optional[Tensor], B: int, T: int, dev) -> Optional[Tensor]:
    if pad_mask is None:
        return None
    m = pad_mask.to(device=dev).reshape(B, T)
    return (m != 0).to(torch.uint8).contiguous()


def cross_state_fwd(phi_k: Tensor, v: Tensor, pad_mask: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    """phi_k [T,B,H,K], v [T,B,H,d] fp16, pad_mask [B,T] (non-zero = pad) -> s [B,H,K,d], z [B,H,K] fp32."""
    require_half(phi_k, v)
    T, B, H, K = phi_k.shape
    d = v.shape[-1]
    phi_k, v = phi_k.contiguous(), v.contiguous()
    m = _mask_bytes(pad_mask, B, T, phi_k.device)
    s = torch.empty(B, H, K, d, dtype=torch.float32, device=phi_k.device)
    z = torch.empty(B, H, K, dtype=torch.float32, device=phi_k.device)
    with _guard(phi_k):
        check(_lib.load().rfa_cross_state_fwd(ptr(phi_k), ptr(v), ptr(m), ptr(s), ptr(z), T, B, H, K, d,
                                              stream_of(phi_k)), "rfa_cross_state_fwd")
    return s, z


def state_total(phi_k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor]:
    """phi_k [T,BH,K], v [T,BH,d] fp16 -> (sum_t k_t v_t^T [BH,K,d], sum_t k_t [BH,K]) fp32, with enough CTAs per
    sequence to fill the GPU when BH is small (partials over runs of tokens, summed here)."""
    require_half(phi_k, v)
    T, BH, K = phi_k.shape
    d = v.shape[-1]
    phi_k, v = phi_k.contiguous(), v.contiguous()
    if T == 0:      # an empty shard contributes nothing
        return torch.zeros(BH, K, d, device=phi_k.device), torch.zeros(BH, K, device=phi_k.device)
    sms = torch.cuda.get_device_properties(phi_k.device).multi_processor_count
    nseg = max(1, min(sms // max(BH, 1), T // 512))
    s = torch.empty(BH, nseg, K, d, dtype=torch.float32, device=phi_k.device)
    z = torch.empty(BH, nseg, K, dtype=torch.float32, device=phi_k.device)
    with _guard(phi_k):
        check(_lib.load().rfa_state_partials(ptr(phi_k), ptr(v), ptr(s), ptr(z), T, BH, K, d, nseg, stream_of(phi_k)),
              "rfa_state_partials")
    return (s[:, 0], z[:, 0]) if nseg == 1 else (s.sum(dim=1), z.sum(dim=1))


def cross_state_bwd(phi_k: Tensor, v: Tensor, pad_mask: Optional[Tensor], d_s: Tensor, d_z: Tensor):
    T, B, H, K = phi_k.shape
    d = v.shape[-1]
    phi_k, v = phi_k.contiguous(), v.contiguous()
    m = _mask_bytes(pad_mask, B, T, phi_k.device)
    d_s, d_z = d_s.contiguous().float(), d_z.contiguous().float()
    g_k, g_v = torch.empty_like(phi_k), torch.empty_like(v)
    with _guard(phi_k):
        check(_lib.load().rfa_cross_state_bwd(ptr(phi_k), ptr(v), ptr(m), ptr(d_s), ptr(d_z), ptr(g_k), ptr(g_v),
                                              T, B, H, K, d, stream_of(phi_k)), "rfa_cross_state_bwd")
    return g_k, g_v


def cross_query_fwd(phi_q: Tensor, s: Tensor, z: Tensor) -> Tensor:
    """phi_q [T,B,H,K] fp16, s [B,H,K,d], z [B,H,K] fp32 -> out [T,B,H,d] fp16."""
    require_half(phi_q)
    T, B, H, K = phi_q.shape
    d = s.shape[-1]
    phi_q = phi_q.contiguous()
    s, z = s.contiguous().float(), z.contiguous().float()
    out = torch.empty(T, B, H, d, dtype=torch.float16, device=phi_q.device)
    with _guard(phi_q):
        check(_lib.load().rfa_cross_query_fwd(ptr(phi_q), ptr(s), ptr(z), ptr(out), T, B * H, K, d,
                                              stream_of(phi_q)), "rfa_cross_query_fwd")
    return out


def cross_query_bwd(phi_q: Tensor, s: Tensor, z: Tensor, g: Tensor):
    require_half(phi_q, g)
    T, B, H, K = phi_q.shape
    d = s.shape[-1]
    phi_q, g = phi_q.contiguous(), g.contiguous()
    s, z = s.contiguous().float(), z.contiguous().float()
    g_q = torch.empty_like(phi_q)
    d_s, d_z = torch.empty_like(s), torch.empty_like(z)
    with _guard(phi_q):
        check(_lib.load().rfa_cross_query_bwd(ptr(phi_q), ptr(s), ptr(z), ptr(g), ptr(g_q), ptr(d_s), ptr(d_z),
                                              T, B * H, K, d, stream_of(phi_q)), "rfa_cross_query_bwd")
    return g_q, d_s, d_z


# --------------------------------------------------------------------------- decode
def decode_step(phi_q: Tensor, phi_k: Tensor, v: Tensor, s: Tensor, z: Tensor, out: Optional[Tensor] = None) -> Tensor:
    """One token, state updated IN PLACE.  phi_q,phi_k [B,H,K], v [B,H,d]; s [B,H,K,d], z [B,H,K]."""
    B, H, K = phi_q.shape
    d = v.shape[-1]
    phi_q, phi_k, v = phi_q.contiguous(), phi_k.contiguous(), v.contiguous()
    if not (s.is_contiguous() and z.is_contiguous()):
        raise ValueError("decode_step: state tensors must be contiguous (they are updated in place)")
    if not (phi_q.dtype == phi_k.dtype == v.dtype) or s.dtype != z.dtype:
        raise TypeError(f"decode_step: phi_q, phi_k, v must share a dtype and so must s, z (got {phi_q.dtype}, {phi_k.dtype}, "
                        f"{v.dtype}; {s.dtype}, {z.dtype})")
    if out is None:
        out = torch.empty(B, H, d, dtype=v.dtype, device=v.device)
    elif out.dtype != v.dtype or not out.is_contiguous():
        raise TypeError("decode_step: out must be contiguous and of v's dtype")
    with _guard(v):
        check(_lib.load().rfa_decode_step(ptr(phi_q), ptr(phi_k), ptr(v), dtype_code(v), ptr(s), ptr(z), dtype_code(s),
                                          ptr(out), B * H, K, d, stream_of(v)), "rfa_decode_step")
    return out


def decode_step_fused(q: Tensor, k: Tensor, v: Tensor, w: Tensor, scale: float, s: Tensor, z: Tensor,
                      out: Optional[Tensor] = None) -> Tensor:
    """One token from raw q,k [B,H,d]; w [H,D,d] fp32 contiguous; state updated IN PLACE."""
    B, H, d = q.shape
    D = w.shape[1]
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    if w.dtype != torch.float32 or not w.is_contiguous():
        raise ValueError("decode_step_fused: w must be a contiguous fp32 [H,D,d] tensor")
    if not (q.dtype == k.dtype == v.dtype) or s.dtype != z.dtype:
        raise TypeError(f"decode_step_fused: q, k, v must share a dtype and so must s, z (got {q.dtype}, {k.dtype}, {v.dtype}; "
                        f"{s.dtype}, {z.dtype})")
    if not (s.is_contiguous() and z.is_contiguous()):
        raise ValueError("decode_step_fused: state tensors must be contiguous (they are updated in place)")
    if out is None:
        out = torch.empty(B, H, d, dtype=v.dtype, device=v.device)
    elif out.dtype != v.dtype or not out.is_contiguous():
        raise TypeError("decode_step_fused: out must be contiguous and of v's dtype")
    with _guard(v):
        check(_lib.load().rfa_decode_step_fused(ptr(q), ptr(k), ptr(v), dtype_code(v), ptr(w), float(scale), ptr(s),
                                                ptr(z), dtype_code(s), ptr(out), B * H, H, D, d, stream_of(v)),
              "rfa_decode_step_fused")
    return out


class CrossDecodeStates:
    """The cross-attention states of all layers of a decoder, gathered once per sequence for ``cross_decode_step``:
    device arrays of pointers to each layer's ``s [B,H,K,d]`` and ``z [B,H,K]`` (fp32, contiguous).  The states are
    referenced, not copied; keep them alive and unchanged while this object is used."""

    def __init__(self, states):
        self.s = [st[0].contiguous() for st in states]
        self.z = [st[1].contiguous() for st in states]
        for t in self.s + self.z:
            if not t.is_cuda or t.dtype != torch.float32:
                raise TypeError("rfa_b200: cross-attention states must be fp32 CUDA tensors")
        self.L = len(self.s)
        B, H, self.K, self.d = self.s[0].shape
        self.BH = B * H
        dev = self.s[0].device
        self.s_ptrs = torch.tensor([t.data_ptr() for t in self.s], dtype=torch.int64, device=dev)
        self.z_ptrs = torch.tensor([t.data_ptr() for t in self.z], dtype=torch.int64, device=dev)


def cross_decode_step(phi_q: Tensor, states: CrossDecodeStates, out: Optional[Tensor] = None) -> Tensor:
    """phi_q [L, B, H, K] (one token's query features for every layer) -> out [L, B, H, d], one launch for all layers."""
    L, B, H, K = phi_q.shape
    assert (L, B * H, K) == (states.L, states.BH, states.K), (phi_q.shape, states.L, states.BH, states.K)
    phi_q = phi_q.contiguous()
    if out is None:
        out = torch.empty(L, B, H, states.d, dtype=phi_q.dtype, device=phi_q.device)
    with _guard(phi_q):
        check(_lib.load().rfa_cross_decode_step(ptr(phi_q), dtype_code(phi_q), ptr(states.s_ptrs), ptr(states.z_ptrs), ptr(out),
                                                L, B * H, K, states.d, stream_of(phi_q)), "rfa_cross_decode_step")
    return out
