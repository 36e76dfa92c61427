"""Cross RFA: encoder-side state projection and decoder-side attention, with
upstream's class names, constructor arguments and tensor layouts
(``cross_attention.py``).  The masked state reduction S = sum phi(k) v^T,
z = sum phi(k) and the query-side product phi(q).S / max(|phi(q).z|, 1) run on the
sm_100a kernels, forward and backward."""
import math
from typing import List, Optional, Tuple

import torch
from torch import Tensor, nn
from torch.nn import Parameter

from . import ops
from .utils import (EPS, CrossAttentionState, build_random_matrices, load_random_matrices,
                    random_project, sample_random_matrices, upgrade_state_dict_named)


class _CrossState(torch.autograd.Function):
    """(phi_k [Ts,B,H,K], v [Ts,B,H,d], pad [B,Ts] or None) -> (s [B,H,K,d], z [B,H,K]) fp32."""

    @staticmethod
    def forward(ctx, phi_k, v, pad):
        ctx.save_for_backward(phi_k, v)
        ctx.pad = pad
        s, z = ops.cross_state_fwd(phi_k, v, pad)
        return s, z

    @staticmethod
    def backward(ctx, d_s, d_z):
        phi_k, v = ctx.saved_tensors
        g_k, g_v = ops.cross_state_bwd(phi_k, v, ctx.pad, d_s, d_z)
        return g_k, g_v, None


class _CrossQuery(torch.autograd.Function):
    """(phi_q [Tq,B,H,K], s, z) -> attn [Tq,B,H,d]."""

    @staticmethod
    def forward(ctx, phi_q, s, z):
        ctx.save_for_backward(phi_q, s, z)
        return ops.cross_query_fwd(phi_q, s, z)

    @staticmethod
    def backward(ctx, g):
        phi_q, s, z = ctx.saved_tensors
        g_q, d_s, d_z = ops.cross_query_bwd(phi_q, s, z, g.contiguous())
        return g_q, d_s.to(s.dtype), d_z.to(z.dtype)


def cross_rfa_state(phi_k: Tensor, v: Tensor, pad: Optional[Tensor]) -> Tuple[Tensor, Tensor]:
    """Masked state reduction; ``pad`` is ``[bsz, src_len]`` with non-zero = padding."""
    return _CrossState.apply(phi_k.to(torch.float16), v.to(torch.float16), pad)


def cross_rfa_query(phi_q: Tensor, s: Tensor, z: Tensor) -> Tensor:
    return _CrossQuery.apply(phi_q.to(torch.float16), s, z)


def _xavier(*linears):
    for lin in linears:
        nn.init.xavier_uniform_(lin.weight, gain=1 / math.sqrt(2))


class CrossAttentionProjectLayer(nn.Module):
    """One decoder layer's view of the encoder output: k/v projections, feature map
    of the keys, and the reduction to the constant-size state (s, z)."""

    def __init__(self, *, embed_dim: int, num_heads: int, head_dim: int, proj_dim: int,
                 tau: float = 1.0, reparam_proj: bool = True):
        super().__init__()
        assert num_heads * head_dim == embed_dim
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, head_dim
        self.proj_dim, self.tau, self.reparam_proj = proj_dim, tau, reparam_proj
        self.k_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.v_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        if reparam_proj:
            self.sigma = Parameter(Tensor(num_heads, 1, head_dim))
        self.reset_parameters()
        self.upgrade_state_dict_named = upgrade_state_dict_named

    def reset_parameters(self):
        _xavier(self.k_proj, self.v_proj)
        if self.reparam_proj:
            nn.init.constant_(self.sigma, 1.)

    def project_and_reshape(self, *, encoder_output: Tensor, random_matrices: Tensor,
                            mask: Optional[Tensor] = None) -> Tuple[Tensor, Tensor, Tensor, float]:
        """encoder_output ``[src_len, bsz, embed_dim]``, random_matrices ``[num_heads,
        proj_dim, head_dim]``, mask ``[src_len, bsz, 1, 1]`` bool (True = padding).
        Returns ``(s [bsz, num_heads, 2*proj_dim, head_dim], z [bsz, num_heads, 2*proj_dim],
        effective random matrices, tau)``; s and z are fp32 (upstream
        cross_attention.py:52-106 keeps them in the activation dtype)."""
        src_len, bsz, _ = encoder_output.size()
        shape = (src_len, bsz, self.num_heads, self.head_dim)
        k = self.k_proj(encoder_output).contiguous().view(shape)
        v = self.v_proj(encoder_output).contiguous().view(shape)
        w = build_random_matrices(random_matrices=random_matrices, tau=self.tau,
                                  sigma=self.sigma if self.reparam_proj else None,
                                  reparam_proj=self.reparam_proj)
        phi_k = random_project(x=k, random_matrices=w)
        pad = None if mask is None else mask.reshape(src_len, bsz).t()
        s, z = cross_rfa_state(phi_k, v, pad)
        return s, z, w, self.tau

    def forward(self, *, encoder_output: Tensor, random_matrices: Tensor,
                mask: Optional[Tensor] = None) -> CrossAttentionState:
        assert encoder_output.size(-1) == self.embed_dim
        return CrossAttentionState(*self.project_and_reshape(
            encoder_output=encoder_output, random_matrices=random_matrices, mask=mask))


class CrossAttentionProject(nn.Module):
    """Encoder-output projection for every decoder layer: holds the bank of random
    matrices, samples per-layer matrices (training) or takes the first
    ``num_heads`` (evaluation), and returns one ``CrossAttentionState`` per layer."""

    def __init__(self, *, num_layers: int, embed_dim: int, num_heads: int, head_dim: int,
                 proj_dim: int, tau: float = 1.0, reparam_proj: bool = True):
        super().__init__()
        self.num_layers, self.embed_dim, self.num_heads = num_layers, embed_dim, num_heads
        self.head_dim, self.proj_dim, self.tau, self.reparam_proj = head_dim, proj_dim, tau, reparam_proj
        self.layers = nn.ModuleList([
            CrossAttentionProjectLayer(embed_dim=embed_dim, num_heads=num_heads, head_dim=head_dim,
                                       proj_dim=proj_dim, tau=tau, reparam_proj=reparam_proj)
            for _ in range(num_layers)])
        self.random_matrices = load_random_matrices(head_dim=head_dim, proj_dim=proj_dim, dtype=torch.half)
        self.random_matrices_eval = nn.Parameter(
            sample_random_matrices(num_layers=num_layers, num_heads=num_heads,
                                   random_matrices=self.random_matrices, is_training=False).clone(),
            requires_grad=False)

    def forward(self, encoder_output: Tensor, key_padding_mask: Optional[Tensor] = None
                ) -> List[CrossAttentionState]:
        """encoder_output ``[src_len, bsz, embed_dim]``; key_padding_mask ``[bsz, src_len]``
        with 1 = padding."""
        src_len, bsz, _ = encoder_output.size()
        if self.training:
            per_layer = sample_random_matrices(num_layers=self.num_layers, num_heads=self.num_heads,
                                               random_matrices=self.random_matrices, is_training=True)
        else:
            per_layer = [self.random_matrices_eval] * self.num_layers
        mask = None
        if key_padding_mask is not None and key_padding_mask.dim() > 0:
            assert key_padding_mask.shape == (bsz, src_len)
            mask = key_padding_mask.to(torch.bool).t()[:, :, None, None]
        return [layer(encoder_output=encoder_output, random_matrices=w, mask=mask)
                for layer, w in zip(self.layers, per_layer)]


class CrossAttention(nn.Module):
    """Decoder-side random feature cross attention: attends a query to the encoder
    state (s, z) produced by ``CrossAttentionProject``."""

    def __init__(self, *, embed_dim: int, num_heads: int, head_dim: int, proj_dim: int,
                 tau: float = 1.0, reparam_proj: bool = True):
        super().__init__()
        assert head_dim * num_heads == embed_dim, "embed_dim must be divisible by num_heads"
        self.embed_dim, self.num_heads, self.head_dim = embed_dim, num_heads, head_dim
        self.proj_dim, self.tau, self.reparam_proj = proj_dim, tau, reparam_proj
        self.q_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.out_proj = nn.Linear(embed_dim, embed_dim, bias=True)
        self.reset_parameters()
        self.upgrade_state_dict_named = upgrade_state_dict_named

    def reset_parameters(self):
        _xavier(self.q_proj, self.out_proj)
        nn.init.constant_(self.out_proj.bias, 0.0)
        nn.init.constant_(self.q_proj.bias, 0.0)

    def rfa(self, query: Tensor, s: Tensor, z: Tensor, random_matrices: Tensor) -> Tensor:
        """query ``[tgt_len, bsz, num_heads, head_dim]`` -> ``[tgt_len, bsz, num_heads, head_dim]``:
        phi(q).s / max(|phi(q).z|, EPS)  (upstream cross_attention.py:254-270)."""
        phi_q = random_project(x=query, random_matrices=random_matrices)
        return cross_rfa_query(phi_q, s, z).to(query.dtype)

    def forward(self, query: Tensor, state: CrossAttentionState) -> Tensor:
        """query ``[tgt_len, bsz, embed_dim]`` -> ``[tgt_len, bsz, embed_dim]``."""
        s, z, random_matrices, tau = state
        tgt_len, bsz, embed_dim = query.size()
        assert embed_dim == self.embed_dim
        q = self.q_proj(query).contiguous().view(tgt_len, bsz, self.num_heads, self.head_dim)
        attn = self.rfa(q, s, z, random_matrices)
        return self.out_proj(attn.contiguous().view(tgt_len, bsz, embed_dim))
