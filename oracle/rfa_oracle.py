"""CPU oracle for the Random Feature Attention hot path.

TEST INFRASTRUCTURE ONLY.  This module is the checker that the CUDA kernels are
compared against.  It may be imported by the test-suite, by the smoke test and by
the CPU-baseline leg of the benchmark; the shipped package never imports it and
has no CPU fallback.

Every function restates, in plain PyTorch on the CPU, one piece of the upstream
project (Noahs-ARK/RFA, package ``random_feature_attention``).  The upstream
file:line each function follows is given in its docstring.  Parity of this file
with upstream is pinned by ``tests/golden/*.npz``: those fixtures were produced
by importing the upstream Python sources themselves (``tests/golden/make_golden.py``)
and ``tests/test_oracle_golden.py`` checks every function here against them.

The causal functions are written in a *streaming* form (the running state
``S = sum phi(k) v^T`` and ``z = sum phi(k)`` is carried from block to block)
so that they need O(block * K * d) memory instead of upstream's O(T * K * d)
cumulative-sum tensor; on small inputs the two forms agree to rounding.
"""

from __future__ import annotations

from typing import Optional, Tuple

import numpy as np
import torch
from torch import Tensor

EPS = 1.0      # rfa.py:17, utils.py:9 -- denominator clamp
SCALE = 0.1    # utils.py:10           -- constant feature scale (not 1/sqrt(D))
NORM_EPS = 1e-3  # utils.py:102        -- x / (||x|| + 1e-3)


# ---------------------------------------------------------------------------
# random matrices (construct_random_matrices.py)
# ---------------------------------------------------------------------------

def rrf(*, head_dim: int, proj_dim: int) -> np.ndarray:
    """Gaussian random features, construct_random_matrices.py:10-11.
    Consumes the global numpy RNG exactly like upstream."""
    return np.random.normal(loc=0.0, scale=1.0, size=(proj_dim, head_dim))


def orf(*, head_dim: int, proj_dim: int) -> np.ndarray:
    """Orthogonal random features, construct_random_matrices.py:14-21:
    reduced QR of a Gaussian [D, d] block, rows rescaled by chi(df=D) draws."""
    assert proj_dim >= head_dim
    g = np.random.normal(loc=0.0, scale=1.0, size=(proj_dim, head_dim))
    q, _ = np.linalg.qr(g)
    s = np.sqrt(np.random.chisquare(df=proj_dim, size=proj_dim))
    return q * s[:, None]


def draw_matrices(kind: str, n: int, head_dim: int, proj_dim: int, seed: int) -> np.ndarray:
    """n matrices stacked [n, D, d] after seeding the global numpy RNG, the way
    construct_random_matrices.py:60-66,77-79 builds its bank."""
    f = {"rrf": rrf, "orf": orf}[kind]
    np.random.seed(seed)
    return np.stack([f(head_dim=head_dim, proj_dim=proj_dim) for _ in range(n)], axis=0)


def build_random_matrices(w: Tensor, tau: float, sigma: Optional[Tensor] = None,
                          reparam_proj: bool = False) -> Tensor:
    """utils.py:90-97: W' = sigma * W / tau (sigma [H,1,d] only when reparam_proj)."""
    if reparam_proj:
        w = sigma * w
    return w / tau


# ---------------------------------------------------------------------------
# feature map (utils.py:100-120)
# ---------------------------------------------------------------------------

def random_project(x: Tensor, w: Tensor, scale: float = SCALE) -> Tensor:
    """phi(x) = scale * [sin(W xhat), cos(W xhat)],  xhat = x / (||x||_2 + 1e-3).

    x [..., H, d], w [H, D, d] -> [..., H, 2D].   utils.py:100-102 (normalise),
    :115 (per-head projection), :116-119 (sin | cos concatenation and scale)."""
    n = torch.linalg.vector_norm(x, ord=2, dim=-1, keepdim=True)
    xh = x / (n + NORM_EPS)
    u = torch.einsum("...hd,hkd->...hk", xh, w)
    return torch.cat([torch.sin(u), torch.cos(u)], dim=-1) * scale


def random_project_backward(x: Tensor, w: Tensor, g_phi: Tensor,
                            scale: float = SCALE) -> Tuple[Tensor, Tensor]:
    """Analytic gradient of :func:`random_project` w.r.t. x and W (what autograd
    produces through utils.py:100-120).  Returns (g_x, g_w)."""
    D = w.shape[-2]
    n = torch.linalg.vector_norm(x, ord=2, dim=-1, keepdim=True)
    xh = x / (n + NORM_EPS)
    u = torch.einsum("...hd,hkd->...hk", xh, w)
    g_u = scale * (g_phi[..., :D] * torch.cos(u) - g_phi[..., D:] * torch.sin(u))
    g_xh = torch.einsum("...hk,hkd->...hd", g_u, w)
    g_w = torch.einsum("...hk,...hd->hkd", g_u, xh)
    dot = (x * g_xh).sum(-1, keepdim=True)
    g_x = g_xh / (n + NORM_EPS) - x * dot / (n.clamp_min(1e-30) * (n + NORM_EPS) ** 2)
    return g_x, g_w


# ---------------------------------------------------------------------------
# causal RFA (rfa.py:47-103), streaming form
# ---------------------------------------------------------------------------

def _blocks(T: int, block: int):
    for lo in range(0, T, block):
        yield lo, min(T, lo + block)


def causal_forward(q: Tensor, k: Tensor, v: Tensor, *, block: int = 64,
                   s0: Optional[Tensor] = None, z0: Optional[Tensor] = None,
                   return_state: bool = False, return_den: bool = False):
    """rfa.py:57-64.  q,k [T,BH,K], v [T,BH,d] -> attn [T,BH,d].

    S_t = sum_{s<=t} k_s v_s^T, z_t = sum_{s<=t} k_s (inclusive prefix),
    attn_t = q_t^T S_t / max(q_t . z_t, EPS).  The optional carry-in (s0 [BH,K,d],
    z0 [BH,K]) is the state of all earlier tokens; used by the sequence-sharded
    path and by prefill -> decode."""
    T, BH, K = q.shape
    d = v.shape[-1]
    S = torch.zeros(BH, K, d, dtype=q.dtype) if s0 is None else s0.clone()
    z = torch.zeros(BH, K, dtype=q.dtype) if z0 is None else z0.clone()
    out = torch.empty(T, BH, d, dtype=q.dtype)
    den_raw = torch.empty(T, BH, dtype=q.dtype)
    for lo, hi in _blocks(T, block):
        kb, vb, qb = k[lo:hi], v[lo:hi], q[lo:hi]
        Sb = S.unsqueeze(0) + torch.cumsum(torch.einsum("tbk,tbd->tbkd", kb, vb), dim=0)
        zb = z.unsqueeze(0) + torch.cumsum(kb, dim=0)
        qs = torch.einsum("tbkd,tbk->tbd", Sb, qb)
        qz = torch.einsum("tbk,tbk->tb", qb, zb)
        den_raw[lo:hi] = qz
        out[lo:hi] = qs / qz.clamp_min(EPS).unsqueeze(-1)
        S, z = Sb[-1], zb[-1]
    res = (out,)
    if return_state:
        res += (S, z)
    if return_den:
        res += (den_raw,)
    return res[0] if len(res) == 1 else res


def causal_backward(q: Tensor, k: Tensor, v: Tensor, g: Tensor, *, block: int = 64,
                    s0: Optional[Tensor] = None, z0: Optional[Tensor] = None,
                    ds_in: Optional[Tensor] = None, dz_in: Optional[Tensor] = None,
                    return_dstate: bool = False):
    """rfa.py:79-101.  Returns (grad_q, grad_k, grad_v) for upstream gradient g.

    grad_qs = g / qz, grad_qz = -(g . qs) / qz^2 * [qz > EPS]   (strict >, :91)
    grad_q  = S grad_qs + grad_qz z                              (:93-94)
    grad_S  = reverse-cumsum(q (x) grad_qs); grad_k = grad_S v + reverse-cumsum(q grad_qz)
    grad_v  = grad_S^T k                                         (:96-101)

    (s0, z0) is the forward carry-in of earlier tokens; (ds_in, dz_in) the reverse
    carry-in (sum over *later* tokens of q (x) grad_qs and of q grad_qz)."""
    T, BH, K = q.shape
    d = v.shape[-1]
    S = torch.zeros(BH, K, d, dtype=q.dtype) if s0 is None else s0.clone()
    z = torch.zeros(BH, K, dtype=q.dtype) if z0 is None else z0.clone()
    gq = torch.empty_like(q)
    gk = torch.empty_like(k)
    gv = torch.empty_like(v)
    g_qs = torch.empty(T, BH, d, dtype=q.dtype)
    g_qz = torch.empty(T, BH, dtype=q.dtype)
    for lo, hi in _blocks(T, block):
        kb, vb, qb, gb = k[lo:hi], v[lo:hi], q[lo:hi], g[lo:hi]
        Sb = S.unsqueeze(0) + torch.cumsum(torch.einsum("tbk,tbd->tbkd", kb, vb), dim=0)
        zb = z.unsqueeze(0) + torch.cumsum(kb, dim=0)
        qs = torch.einsum("tbkd,tbk->tbd", Sb, qb)
        qz_raw = torch.einsum("tbk,tbk->tb", qb, zb)
        qz = qz_raw.clamp_min(EPS)
        gqs = gb / qz.unsqueeze(-1)
        gqz = -(gb * qs).sum(-1) / qz ** 2 * (qz > EPS)
        gq[lo:hi] = torch.einsum("tbd,tbkd->tbk", gqs, Sb) + gqz.unsqueeze(-1) * zb
        g_qs[lo:hi], g_qz[lo:hi] = gqs, gqz
        S, z = Sb[-1], zb[-1]
    dS = torch.zeros(BH, K, d, dtype=q.dtype) if ds_in is None else ds_in.clone()
    dz = torch.zeros(BH, K, dtype=q.dtype) if dz_in is None else dz_in.clone()
    starts = [lo for lo, _ in _blocks(T, block)]
    for lo in reversed(starts):
        hi = min(T, lo + block)
        qb, kb, vb = q[lo:hi], k[lo:hi], v[lo:hi]
        inc = torch.einsum("tbk,tbd->tbkd", qb, g_qs[lo:hi])
        dSb = dS.unsqueeze(0) + torch.flip(torch.cumsum(torch.flip(inc, [0]), 0), [0])
        incz = qb * g_qz[lo:hi].unsqueeze(-1)
        dzb = dz.unsqueeze(0) + torch.flip(torch.cumsum(torch.flip(incz, [0]), 0), [0])
        gk[lo:hi] = torch.einsum("tbkd,tbd->tbk", dSb, vb) + dzb
        gv[lo:hi] = torch.einsum("tbkd,tbk->tbd", dSb, kb)
        dS, dz = dSb[0], dzb[0]
    if return_dstate:
        return gq, gk, gv, dS, dz
    return gq, gk, gv


def causal_forward_literal(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """rfa.py:57-64 restated with the full [T,BH,K,d] cumulative sum (small inputs
    only); used to show that the streaming form above is the same function."""
    s = torch.cumsum(torch.einsum("tbk,tbd->tbkd", k, v), dim=0)
    qs = torch.einsum("tbkd,tbk->tbd", s, q)
    qz = torch.einsum("tbk,tbk->tb", q, torch.cumsum(k, dim=0)).clamp_min(EPS)
    return qs / qz.unsqueeze(-1)


def segment_state(k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor]:
    """Total state contributed by a run of tokens: (sum_s k_s v_s^T [BH,K,d],
    sum_s k_s [BH,K]) -- the last element of the cumulative sums of rfa.py:58,61."""
    return torch.einsum("tbk,tbd->bkd", k, v), k.sum(0)


# ---------------------------------------------------------------------------
# incremental decoding (causal_attention.py:17-54)
# ---------------------------------------------------------------------------

def incremental_rfa(phi_q: Tensor, phi_k: Tensor, v: Tensor,
                    s: Optional[Tensor] = None, z: Optional[Tensor] = None):
    """phi_q,phi_k [T,B,H,K], v [T,B,H,d]; state s [B,H,K,d], z [B,H,K] (zeros in
    v.dtype when absent, causal_attention.py:35-40).  Per token (:42-50):
    s += phi_k (x) v; z += phi_k; attn = phi_q.s / max(phi_q.z, EPS).
    Returns (attn [T,B,H*d], s, z)."""
    T, B, H, K = phi_q.shape
    d = v.shape[-1]
    if s is None:
        s = torch.zeros(B, H, K, d, dtype=v.dtype)
        z = torch.zeros(B, H, K, dtype=v.dtype)
    outs = []
    for i in range(T):
        s = s + phi_k[i].unsqueeze(-1) * v[i].unsqueeze(-2)
        z = z + phi_k[i]
        qs = (phi_q[i].unsqueeze(-1) * s).sum(-2)
        qz = (phi_q[i] * z).sum(-1).clamp_min(EPS)
        outs.append(qs / qz.unsqueeze(-1))
    return torch.stack(outs, 0).reshape(T, B, H * d), s, z


# ---------------------------------------------------------------------------
# cross attention (cross_attention.py:97-104 and :254-270)
# ---------------------------------------------------------------------------

def cross_state(phi_k: Tensor, v: Tensor, pad_mask: Optional[Tensor] = None):
    """cross_attention.py:97-104.  phi_k [Ts,B,H,K], v [Ts,B,H,d], pad_mask [B,Ts]
    bool (True = padding).  phi_k rows at padded positions are zeroed, then
    s = sum_s phi_k (x) v  [B,H,K,d],  z = sum_s phi_k  [B,H,K]."""
    if pad_mask is not None:
        m = pad_mask.to(torch.bool).transpose(0, 1)[:, :, None, None]
        phi_k = phi_k.masked_fill(m, 0.0)
    return torch.einsum("sbhk,sbhd->bhkd", phi_k, v), phi_k.sum(0)


def cross_query(phi_q: Tensor, s: Tensor, z: Tensor) -> Tensor:
    """cross_attention.py:266-269.  attn = phi_q.s / max(|phi_q.z|, EPS),
    phi_q [Tq,B,H,K] -> [Tq,B,H,d]."""
    qs = torch.einsum("tbhk,bhkd->tbhd", phi_q, s)
    qz = torch.einsum("tbhk,bhk->tbh", phi_q, z).abs().clamp_min(EPS)
    return qs / qz.unsqueeze(-1)


def cross_backward(phi_q: Tensor, phi_k: Tensor, v: Tensor, g: Tensor,
                   pad_mask: Optional[Tensor] = None):
    """Analytic gradients of cross_query(phi_q, *cross_state(phi_k, v, mask)) for
    upstream gradient g [Tq,B,H,d]: what autograd yields through
    cross_attention.py:97-104 and :266-269.  Returns (g_phi_q, g_phi_k, g_v);
    g_phi_k is zero at padded keys (masked_fill blocks the gradient), g_v there
    is zero because the zeroed phi_k multiplies it."""
    if pad_mask is not None:
        m = pad_mask.to(torch.bool).transpose(0, 1)[:, :, None, None]
        pk = phi_k.masked_fill(m, 0.0)
    else:
        m, pk = None, phi_k
    s = torch.einsum("sbhk,sbhd->bhkd", pk, v)
    z = pk.sum(0)
    qs = torch.einsum("tbhk,bhkd->tbhd", phi_q, s)
    raw = torch.einsum("tbhk,bhk->tbh", phi_q, z)
    den = raw.abs().clamp_min(EPS)
    g_qs = g / den.unsqueeze(-1)
    g_raw = -(g * qs).sum(-1) / den ** 2 * torch.sign(raw) * (raw.abs() > EPS)
    g_pq = torch.einsum("tbhd,bhkd->tbhk", g_qs, s) + g_raw.unsqueeze(-1) * z.unsqueeze(0)
    d_s = torch.einsum("tbhk,tbhd->bhkd", phi_q, g_qs)
    d_z = torch.einsum("tbhk,tbh->bhk", phi_q, g_raw)
    g_pk = torch.einsum("sbhd,bhkd->sbhk", v, d_s) + d_z.unsqueeze(0)
    g_v = torch.einsum("sbhk,bhkd->sbhd", pk, d_s)
    if m is not None:
        g_pk = g_pk.masked_fill(m, 0.0)
    return g_pq, g_pk, g_v


# ---------------------------------------------------------------------------
# error metrics used by every parity test
# ---------------------------------------------------------------------------

def rel_l2(a: Tensor, b: Tensor) -> float:
    a, b = a.double().flatten(), b.double().flatten()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs(a: Tensor, b: Tensor) -> float:
    return float((a.double() - b.double()).abs().max()) if a.numel() else 0.0
