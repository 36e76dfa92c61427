"""Causal RFA: functional forms and the ``CausalAttention`` layer, with upstream's
names, arguments and tensor layouts (``causal_attention.py``).  The three hot
functions run on the sm_100a kernels:

* ``cuda_causal_rfa``  -> chunked prefix-scan kernels through ``RFA.apply``
* ``incremental_rfa``  -> the state-streaming decode kernel (one token) or the
                          causal kernel with a state carry (several tokens)
* the feature map      -> ``utils.random_project``
"""
import math
from typing import Dict, Optional

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from . import ops
from .rfa import RFA
from .utils import (EPS, SCALE, build_random_matrices, normalize_attn_weights, random_project, random_project_pair,
                    upgrade_state_dict_named)


class _StatefulRFA(torch.autograd.Function):
    """Causal RFA over a run of tokens with the state carried in AND out, differentiable in all five inputs:
    (q, k, v [T,BH,.] fp16; s_in [BH,K,d], z_in [BH,K] fp32) -> (out, s_out, z_out).  The gradient with respect to the
    incoming state is the run's own reverse-state total (sum_t q_t (x) g_t/den_t, sum_t q_t gz_t) plus whatever flows
    back into the outgoing state, which is exactly the reverse carry of the second backward sweep."""

    @staticmethod
    def forward(ctx, q, k, v, s_in, z_in):
        out, s_out, z_out = ops.causal_fwd(q, k, v, s_in, z_in, return_state=True)
        ctx.save_for_backward(q, k, v, s_in, z_in)
        return out, s_out, z_out

    @staticmethod
    def backward(ctx, g_out, g_s, g_z):
        q, k, v, s_in, z_in = ctx.saved_tensors
        g = g_out.contiguous().to(q.dtype)
        gq, ds_tot, dz_tot, ws = ops.causal_bwd_q(q, k, v, g, s_in, z_in, True)
        ds_in = None if g_s is None else g_s.contiguous().float()
        dz_in = None if g_z is None else g_z.contiguous().float()
        if (ds_in is None) != (dz_in is None):          # the kernels take the reverse carry as a pair
            ds_in = torch.zeros_like(ds_tot) if ds_in is None else ds_in
            dz_in = torch.zeros_like(dz_tot) if dz_in is None else dz_in
        gk, gv = ops.causal_bwd_kv(q, k, v, g, ds_in, dz_in, ws)
        if ds_in is not None:
            ds_tot, dz_tot = ds_tot + ds_in, dz_tot + dz_in
        return gq, gk, gv, ds_tot, dz_tot


def incremental_rfa(*, phi_q: Tensor, phi_k: Tensor, v: Tensor,
                    s: Optional[Tensor] = None, z: Optional[Tensor] = None):
    """Advance the running state by ``tgt_len`` tokens and attend.

    phi_q, phi_k ``[tgt_len, bsz, num_heads, 2*proj_dim]``, v ``[tgt_len, bsz, num_heads,
    head_dim]``; state s ``[bsz, num_heads, 2*proj_dim, head_dim]``, z ``[bsz, num_heads,
    2*proj_dim]``.  Returns ``(attn [tgt_len, bsz, num_heads*head_dim], s, z)``.

    Differences from upstream (causal_attention.py:17-54), both for accuracy/speed:
    a fresh state is created in fp32 (upstream: v's dtype), and -- when no gradient
    is being recorded, the inference loop -- a state that is passed in is UPDATED IN
    PLACE and returned (upstream allocates a new one per token).  With autograd
    recording and an input that requires grad the call is differentiable like
    upstream's: it then returns NEW state tensors and leaves the ones passed in alone."""
    tgt_len, bsz, num_heads, feat = phi_q.shape
    head_dim = v.size(-1)
    if s is None:
        assert z is None
        s = torch.zeros(bsz, num_heads, feat, head_dim, device=v.device, dtype=torch.float32)
        z = torch.zeros(bsz, num_heads, feat, device=v.device, dtype=torch.float32)
    if torch.is_grad_enabled() and any(t.requires_grad for t in (phi_q, phi_k, v, s, z)):
        BH = bsz * num_heads
        h = lambda t: t.contiguous().view(tgt_len, BH, -1).to(torch.float16)
        attn, s_new, z_new = _StatefulRFA.apply(h(phi_q), h(phi_k), h(v), s.reshape(BH, feat, head_dim).float().contiguous(),
                                                z.reshape(BH, feat).float().contiguous())
        return (attn.to(v.dtype).reshape(tgt_len, bsz, num_heads * head_dim), s_new.view(bsz, num_heads, feat, head_dim),
                z_new.view(bsz, num_heads, feat))
    with torch.no_grad():
        if tgt_len == 1:
            attn = ops.decode_step(phi_q[0], phi_k[0], v[0], s, z).unsqueeze(0)
        else:   # several tokens at once: the causal kernel with (s, z) carried in and out
            BH = bsz * num_heads
            h = lambda t: t.contiguous().view(tgt_len, BH, -1).half()
            attn, s_new, z_new = ops.causal_fwd(h(phi_q), h(phi_k), h(v), s.view(BH, feat, head_dim).float(),
                                                z.view(BH, feat).float(), return_state=True)
            s.copy_(s_new.view_as(s))
            z.copy_(z_new.view_as(z))
            attn = attn.to(v.dtype)
    return attn.reshape(tgt_len, bsz, num_heads * head_dim), s, z


def masked_rfa(*, phi_q: Tensor, phi_k: Tensor, v: Tensor,
               key_padding_mask: Optional[Tensor] = None, attn_mask: Optional[Tensor] = None) -> Tensor:
    """Quadratic, explicitly masked variant selected by ``cuda_causal_rfa=False``
    (upstream causal_attention.py:57-109).  It is a different function from the
    kernel path -- weights are normalised by ``|row sum|`` clamped at 1e-3, not by
    ``max(row sum, 1)`` -- and stays in PyTorch exactly as upstream has it."""
    tgt_len, bsz, num_heads, _ = phi_q.shape
    head_dim = v.size(-1)
    if key_padding_mask is not None and key_padding_mask.dim() == 0:
        key_padding_mask = None
    scores = torch.einsum("tbhk,sbhk->bhts", phi_q, phi_k)
    if key_padding_mask is not None:
        assert key_padding_mask.shape == (bsz, tgt_len)
        scores = scores.masked_fill(key_padding_mask.to(torch.bool)[:, None, None, :], 0.0)
    if attn_mask is not None:
        scores = scores.masked_fill((attn_mask < 0.0)[None, None], 0.0)
    weights = normalize_attn_weights(scores, dtype=scores.dtype)
    attn = torch.einsum("bhts,sbhd->tbhd", weights, v)
    return attn.contiguous().view(tgt_len, bsz, num_heads * head_dim)


def cuda_causal_rfa(*, phi_q: Tensor, phi_k: Tensor, v: Tensor,
                    key_padding_mask: Optional[Tensor] = None) -> Tensor:
    """Kernel-backed causal RFA (upstream causal_attention.py:112-151).

    phi_q, phi_k ``[tgt_len, bsz, num_heads, 2*proj_dim]``, v ``[tgt_len, bsz, num_heads,
    head_dim]``; key_padding_mask ``[bsz, tgt_len]`` with 1 = padding: those keys'
    features are zeroed, so they add nothing to the running state.  Returns
    ``[tgt_len, bsz, num_heads*head_dim]``.  The kernels are fp16; other float
    dtypes are converted on the way in and the result converted back."""
    tgt_len, bsz, num_heads, _ = phi_q.shape
    head_dim = v.size(-1)
    if key_padding_mask is not None and key_padding_mask.dim() == 0:
        key_padding_mask = None
    if key_padding_mask is not None:
        assert key_padding_mask.shape == (bsz, tgt_len)
        pad = key_padding_mask.to(torch.bool).t()[:, :, None, None]
        phi_k = phi_k.masked_fill(pad, 0.0)
    dtype = v.dtype
    flat = lambda t: t.contiguous().view(tgt_len, bsz * num_heads, -1).to(torch.float16)
    attn = RFA.apply(flat(phi_q), flat(phi_k), flat(v))
    return attn.view(tgt_len, bsz, num_heads * head_dim).to(dtype)


class _FusedCausalRFA(torch.autograd.Function):
    """Causal RFA from the raw per-head q and k: the forward forms the features inside the attention kernel
    (``ops.causal_fwd_fused``), so phi_q and phi_k are neither written to memory nor kept for the backward; the backward
    recomputes them with the feature-map kernel and runs the saved-output sweeps from the forward's output and raw
    denominators, then the feature map's own backward.  Replaces, for the kernel path, upstream's random_project on q and
    k followed by RFA.apply (causal_attention.py:241-248, 137-147; rfa.py:113-145).  A trade of time for memory when a
    gradient is wanted: the step saves the two feature tensors and one launch in the forward and pays two feature-map
    launches in the backward."""

    @staticmethod
    def forward(ctx, x_q, x_k, v, w, scale, row_mask):
        out, ws = ops.causal_fwd_fused(x_q, x_k, v, w, scale, row_mask=row_mask, save_den=True)
        ctx.save_for_backward(x_q, x_k, v, w, out, ws)
        ctx.scale, ctx.row_mask = scale, row_mask
        return out

    @staticmethod
    def backward(ctx, g):
        from . import _lib
        x_q, x_k, v, w, out, ws = ctx.saved_tensors
        T, B, H, d = x_q.shape
        wf = w.float()
        phi_q, phi_k = ops.feature_map_fwd_pair(x_q, x_k, wf, ctx.scale, None, ctx.row_mask)      # one launch for both
        g_pq, g_pk, g_v = ops.causal_bwd_saved(phi_q.view(T, B * H, -1), phi_k.view(T, B * H, -1), v.view(T, B * H, d),
                                               g.contiguous().to(torch.float16), out, ws, _lib.WS_DEN)
        need_w = ctx.needs_input_grad[3]
        g_xq, g_xk, g_w = ops.feature_map_bwd_pair(x_q, x_k, wf, g_pq.view(T, B, H, -1), g_pk.view(T, B, H, -1), ctx.scale,
                                                   need_w, None, ctx.row_mask)
        return g_xq, g_xk, g_v.view(T, B, H, d), (g_w.to(w.dtype) if need_w else None), None, None


def fused_causal_rfa(*, q: Tensor, k: Tensor, v: Tensor, random_matrices: Tensor, scale: float = SCALE,
                     key_padding_mask: Optional[Tensor] = None) -> Tensor:
    """q, k, v ``[tgt_len, bsz, num_heads, head_dim]`` fp16 (before the feature map), random_matrices ``[num_heads,
    proj_dim, head_dim]`` -> ``[tgt_len, bsz, num_heads*head_dim]``: ``cuda_causal_rfa(random_project(q), random_project(k),
    v)`` in one kernel.  Use ``ops.fused_forward_supported`` to see whether the sizes are ones the kernel is built for."""
    tgt_len, bsz, num_heads, head_dim = q.shape
    row_mask = None
    if key_padding_mask is not None and key_padding_mask.dim() > 0:
        assert key_padding_mask.shape == (bsz, tgt_len)
        row_mask = key_padding_mask.to(torch.bool).t().contiguous()
    attn = _FusedCausalRFA.apply(q.contiguous(), k.contiguous(), v.contiguous(), random_matrices, scale, row_mask)
    return attn.view(tgt_len, bsz, num_heads * head_dim)


class CausalAttention(nn.Module):
    """Random feature causal self-attention layer (upstream causal_attention.py:154-280):
    q/k/v projections, per-head feature map with W' = sigma * W / tau, causal RFA,
    output projection.  Parameter names match upstream so its checkpoints load."""

    def __init__(self, *, embed_dim: int, num_heads: int, head_dim: int, proj_dim: int,
                 tau: float = 1.0, reparam_proj: bool = True, cuda_causal_rfa: bool = True):
        super().__init__()
        assert head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, head_dim
        self.proj_dim, self.tau = proj_dim, tau
        self.reparam_proj, self.cuda_causal_rfa = reparam_proj, cuda_causal_rfa
        # training with the feature map inside the attention kernel: phi_q, phi_k are then not kept for the backward (which
        # recomputes them), at the price of those two extra launches; an addition, off by default
        self.fuse_feature_map = False
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        if reparam_proj:
            self.sigma = Parameter(Tensor(num_heads, 1, head_dim))
        self.reset_parameters()
        self.upgrade_state_dict_named = upgrade_state_dict_named

    def reset_parameters(self):
        for lin in (self.q_proj, self.k_proj, self.v_proj, self.out_proj):
            nn.init.xavier_uniform_(lin.weight, gain=1 / math.sqrt(2))
        if self.reparam_proj:
            nn.init.constant_(self.sigma, 1.)
        if self.out_proj.bias is not None:
            nn.init.constant_(self.out_proj.bias, 0.0)

    @staticmethod
    def reorder_incremental_state(saved_state: Dict[str, Optional[Tensor]], new_order: Tensor) -> Dict[str, Optional[Tensor]]:
        """Beam search: keep, per new batch slot i, the running state of old slot ``new_order[i]`` -- one gather per
        state tensor along the batch axis of ``prev_s [bsz, heads, 2*proj_dim, head_dim]`` and ``prev_z``.  (Upstream
        keeps the state in a plain dict, causal_attention.py:249-265, and leaves the reordering to its decoder, which
        is not part of the shipped sources.)"""
        for key in ("prev_s", "prev_z"):
            t = saved_state.get(key)
            if t is not None:
                saved_state[key] = t.index_select(0, new_order.to(device=t.device, dtype=torch.long))
        return saved_state

    def _heads(self, t: Tensor) -> Tensor:
        return t.contiguous().view(t.size(0), t.size(1), self.num_heads, self.head_dim)

    def forward(self, x: Tensor, random_matrices: Tensor, key_padding_mask: Optional[Tensor] = None,
                attn_mask: Optional[Tensor] = None,
                saved_state: Optional[Dict[str, Optional[Tensor]]] = None) -> Tensor:
        """x ``[tgt_len, bsz, embed_dim]``, random_matrices ``[num_heads, proj_dim, head_dim]``
        -> ``[tgt_len, bsz, embed_dim]``.  With ``saved_state`` (a dict; keys ``prev_s``,
        ``prev_z`` are created on first use) the call is one incremental-decoding step
        and tgt_len must be 1; masks are ignored there, as upstream does."""
        tgt_len, bsz, embed_dim = x.size()
        assert embed_dim == self.embed_dim
        q, k, v = self._heads(self.q_proj(x)), self._heads(self.k_proj(x)), self._heads(self.v_proj(x))
        w = build_random_matrices(random_matrices=random_matrices, tau=self.tau,
                                  sigma=self.sigma if self.reparam_proj else None,
                                  reparam_proj=self.reparam_proj)
        recording = torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or self.q_proj.weight.requires_grad)
        if (saved_state is None and self.cuda_causal_rfa and ops.fused_forward_supported(q, w)
                and (self.fuse_feature_map if recording else True)):
            # head_dim 64, proj_dim 64, fp16, enough sequences to fill the GPU: features formed inside the kernel.  Always
            # when no gradient is recorded (prefill, evaluation: one launch instead of three); when one is, only on
            # request (fuse_feature_map), because the backward then has to form the features again
            attn = fused_causal_rfa(q=q, k=k, v=v, random_matrices=w, key_padding_mask=key_padding_mask)
            return self.out_proj(attn.to(x.dtype))
        # the padding mask of the kernel path is applied inside the feature map of k (no separate pass over phi_k)
        fused_mask = key_padding_mask if (saved_state is None and self.cuda_causal_rfa) else None
        phi_q, phi_k = random_project_pair(x_a=q, x_b=k, random_matrices=w, key_padding_mask_b=fused_mask)
        if saved_state is not None:
            assert tgt_len == 1
            prev_s, prev_z = saved_state.get("prev_s"), saved_state.get("prev_z")
            assert (prev_s is None) == (prev_z is None)
            attn, s, z = incremental_rfa(phi_q=phi_q, phi_k=phi_k, v=v, s=prev_s, z=prev_z)
            saved_state["prev_s"], saved_state["prev_z"] = s, z
        elif self.cuda_causal_rfa:
            attn = cuda_causal_rfa(phi_q=phi_q, phi_k=phi_k, v=v, key_padding_mask=None)
        else:
            attn = masked_rfa(phi_q=phi_q, phi_k=phi_k, v=v, attn_mask=attn_mask,
                              key_padding_mask=key_padding_mask)
        return self.out_proj(attn.to(x.dtype))
