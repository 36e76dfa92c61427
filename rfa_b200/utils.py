"""RFA utilities -- same names and meaning as upstream ``utils.py``; the feature
map runs as one fused sm_100a kernel (forward and backward) instead of a chain
of PyTorch ops."""
import os
from typing import List, NamedTuple, Optional, Tuple

import numpy as np
import torch
from torch import Tensor

from . import ops

EPS = 1.0
SCALE = 0.1
RANDOM_MATRICES_PATH = os.path.join(os.path.dirname(__file__), '../random_matrices')


class CrossAttentionState(NamedTuple):
    s: Tensor
    z: Tensor
    random_matrices: List[Tensor]
    tau: float


def upgrade_state_dict_named(*args, **kwargs):
    """Checkpoint-upgrade hook the modules expose; parameter names are unchanged
    from upstream, so there is nothing to rewrite."""
    return None


_DEFAULTS = dict(cross_proj_dim=64, causal_proj_dim=64, cross_tau=1.0, causal_tau=1.0,
                 reparam_proj=True, cuda_causal_rfa=True)


def get_rfa_attr(args):
    """Fill in defaults for the RFA options on an argparse namespace (upstream
    utils.py:20-28).  Upstream stores the ``use_rfa`` flag under the misspelt name
    ``use_linfa``; both names are set here."""
    args.use_rfa = getattr(args, "use_rfa", False)
    args.use_linfa = args.use_rfa
    for name, default in _DEFAULTS.items():
        setattr(args, name, getattr(args, name, default))
    return args


def add_rfa_args(parser):
    flag, num = dict(action='store_true'), dict(metavar='N', type=int)
    parser.add_argument('--use-rfa', help='whether or not to use rfa', **flag)
    parser.add_argument('--cross-proj-dim', help='projection size for cross rfa', **num)
    parser.add_argument('--causal-proj-dim', help='projection size for causal rfa', **num)
    parser.add_argument('--cross-tau', type=float, metavar='D', help='tau for rfa')
    parser.add_argument('--causal-tau', type=float, metavar='D', help='tau for rfa')
    parser.add_argument('--reparam-proj', help='whether or not to reparameterze random matrices in rfa', **flag)
    parser.add_argument('--cuda-causal-rfa', help='whether or not to use custom cuda kernel for causal rfa', **flag)
    return parser


def load_random_matrices(*, head_dim: int, proj_dim: int, dtype: torch.dtype = torch.half) -> Tensor:
    """Bank ``[num_random_matrices, proj_dim, head_dim]`` from
    ``RANDOM_MATRICES_PATH/{head_dim}_{proj_dim}.npy`` as a frozen Parameter.  Build
    the file with ``python -m rfa_b200.construct_random_matrices orf head_dim proj_dim``."""
    path = f"{RANDOM_MATRICES_PATH}/{head_dim}_{proj_dim}.npy"
    bank = torch.tensor(np.load(path), dtype=dtype)
    return torch.nn.Parameter(bank, requires_grad=False)


def sample_matrix_indices(*, num_layers: int, num_heads: int, bank_size: int,
                          generator: Optional[torch.Generator] = None) -> Tensor:
    """``num_layers * num_heads`` distinct indices into the bank.  With a ``torch.Generator`` the draw is reproducible
    and identical on every rank that seeds it alike; without one it consumes numpy's global RNG exactly as upstream
    does (utils.py:73-76), which differs from rank to rank unless the caller seeds numpy everywhere."""
    n = num_layers * num_heads
    if generator is None:
        return torch.from_numpy(np.random.choice(bank_size, size=n, replace=False)).to(torch.int64)
    return torch.randperm(bank_size, generator=generator, device=generator.device)[:n].to(torch.int64)


def sample_random_matrices(*, num_layers: int, num_heads: int, random_matrices: Tensor,
                           is_training: bool = True, generator: Optional[torch.Generator] = None):
    """Training: ``num_layers * num_heads`` distinct matrices drawn from the bank, returned as a list of
    ``[num_heads, proj_dim, head_dim]`` per layer.  Evaluation: the first ``num_heads`` matrices (one tensor shared by
    all layers).  (upstream utils.py:62-87; ``generator`` is an addition, see ``sample_matrix_indices``)"""
    if not is_training:
        return random_matrices[list(range(num_heads))]
    picks = sample_matrix_indices(num_layers=num_layers, num_heads=num_heads, bank_size=random_matrices.size(0),
                                  generator=generator)
    chosen = random_matrices[picks.to(random_matrices.device)]
    return list(chosen.split(num_heads, dim=0))


class _GatherMatrices(torch.autograd.Function):
    """out[i] = sigma[i] * bank[picks[i]] * inv_tau[i] in one kernel; differentiable in sigma (the layers' learnable
    per-head scales), whose gradient is a small reduction done with tensor ops."""

    @staticmethod
    def forward(ctx, bank, picks, sigma, inv_tau):
        out, bad = ops.gather_random_matrices(bank, picks, sigma, inv_tau)
        ctx.save_for_backward(bank, picks, inv_tau)
        ctx.bad = bad
        return out

    @staticmethod
    def backward(ctx, g_out):
        bank, picks, inv_tau = ctx.saved_tensors
        g_sigma = None
        if ctx.needs_input_grad[2]:
            w = bank[picks.to(bank.device)].float()
            if inv_tau is not None:
                w = w * inv_tau.to(w.device).view(-1, 1, 1)
            g_sigma = (g_out * w).sum(dim=1)
        return None, None, g_sigma, None


def sample_effective_matrices(*, num_layers: int, num_heads: int, random_matrices: Tensor, taus, sigmas=None,
                              is_training: bool = True, generator: Optional[torch.Generator] = None) -> Tensor:
    """Sampling and ``build_random_matrices`` for ALL layers of a step in one kernel launch on a device-resident bank:
    returns ``[num_layers, num_heads, proj_dim, head_dim]`` fp32 with layer l holding ``sigma_l * W / tau_l`` -- what
    each layer would otherwise compute itself from the list ``sample_random_matrices`` returns (upstream utils.py:62-97,
    cross_attention.py:166-176).  ``taus``: one float per layer; ``sigmas``: per layer ``[num_heads, 1, head_dim]`` or
    None.  Pass the result's slices to layers built with ``reparam_proj=False, tau=1``-style calls of ``random_project``."""
    bank = random_matrices
    if not bank.is_cuda:
        raise RuntimeError("rfa_b200: sample_effective_matrices wants the bank on the device (there is no CPU path)")
    n = num_layers * num_heads
    if is_training:
        picks = sample_matrix_indices(num_layers=num_layers, num_heads=num_heads, bank_size=bank.size(0), generator=generator)
    else:
        picks = torch.arange(num_heads, dtype=torch.int64).repeat(num_layers)
    head_dim = bank.size(-1)
    inv_tau = torch.tensor([1.0 / float(t) for t in taus], dtype=torch.float32).repeat_interleave(num_heads)
    sigma = None
    if sigmas is not None:
        sigma = torch.stack([s.reshape(num_heads, head_dim) for s in sigmas]).reshape(n, head_dim)
    out = _GatherMatrices.apply(bank, picks.to(bank.device), sigma, inv_tau.to(bank.device))
    return out.view(num_layers, num_heads, bank.size(1), head_dim)


def build_random_matrices(random_matrices: Tensor, tau: float, sigma: Optional[Tensor] = None,
                          reparam_proj: bool = False) -> Tensor:
    """Effective projection ``sigma * W / tau`` (``sigma`` [H,1,d] only when reparam_proj)."""
    w = sigma * random_matrices if reparam_proj else random_matrices
    return w / tau


def _normalize(x: Tensor) -> Tuple[Tensor, Tensor]:
    norm = torch.linalg.vector_norm(x, ord=2, dim=-1, keepdim=True)
    return x / (norm + 1e-3), norm


class _FeatureMap(torch.autograd.Function):
    """phi(x) = SCALE * [sin(W xhat) | cos(W xhat)] with xhat = x / (|x| + 1e-3)."""

    @staticmethod
    def forward(ctx, x, w, scale, row_mask):
        ctx.save_for_backward(x, w)
        ctx.scale, ctx.row_mask = scale, row_mask
        return ops.feature_map_fwd(x, w, scale, row_mask=row_mask)

    @staticmethod
    def backward(ctx, g_phi):
        x, w = ctx.saved_tensors
        need_w = ctx.needs_input_grad[1]
        g_x, g_w = ops.feature_map_bwd(x, w, g_phi, ctx.scale, need_w, row_mask=ctx.row_mask)
        return g_x, (g_w.to(w.dtype) if need_w else None), None, None


class _FeatureMapPair(torch.autograd.Function):
    """The feature maps of two arrays that share W (q and k of a self-attention layer) as one launch each way."""

    @staticmethod
    def forward(ctx, x_a, x_b, w, scale, row_mask_a, row_mask_b):
        ctx.save_for_backward(x_a, x_b, w)
        ctx.scale, ctx.masks = scale, (row_mask_a, row_mask_b)
        return ops.feature_map_fwd_pair(x_a, x_b, w, scale, row_mask_a, row_mask_b)

    @staticmethod
    def backward(ctx, g_a, g_b):
        x_a, x_b, w = ctx.saved_tensors
        need_w = ctx.needs_input_grad[2]
        g_x_a, g_x_b, g_w = ops.feature_map_bwd_pair(x_a, x_b, w, g_a, g_b, ctx.scale, need_w, ctx.masks[0], ctx.masks[1])
        return g_x_a, g_x_b, (g_w.to(w.dtype) if need_w else None), None, None, None


def random_project_pair(*, x_a: Tensor, x_b: Tensor, random_matrices: Tensor, scale: float = SCALE,
                        key_padding_mask_b: Optional[Tensor] = None) -> Tuple[Tensor, Tensor]:
    """``random_project`` of two arrays of one shape with the same matrices -- the q and k of a self-attention layer
    (upstream calls it twice, causal_attention.py:241-248) -- in one launch when the sizes allow (fp16, head_dim =
    proj_dim = 64), else as two calls.  ``key_padding_mask_b`` ``[bsz, seq_len]`` zeroes the features of x_b's padded
    positions."""
    if not ops.feature_map_pair_supported(x_a, x_b, random_matrices):
        return (random_project(x=x_a, random_matrices=random_matrices, scale=scale),
                random_project(x=x_b, random_matrices=random_matrices, scale=scale, key_padding_mask=key_padding_mask_b))
    row_mask = None
    if key_padding_mask_b is not None and key_padding_mask_b.dim() > 0:
        assert key_padding_mask_b.shape == (x_b.size(1), x_b.size(0)), (key_padding_mask_b.shape, x_b.shape)
        row_mask = key_padding_mask_b.to(torch.bool).t().contiguous()
    return _FeatureMapPair.apply(x_a, x_b, random_matrices, scale, None, row_mask)


def random_project(*, x: Tensor, random_matrices: Tensor, scale: float = SCALE,
                   key_padding_mask: Optional[Tensor] = None) -> Tensor:
    """x ``[seq_len, bsz, num_heads, head_dim]``, random_matrices ``[num_heads, proj_dim,
    head_dim]`` -> phi ``[seq_len, bsz, num_heads, 2 * proj_dim]`` in x's dtype
    (upstream utils.py:105-120; ``scale`` defaults to upstream's constant 0.1).

    ``key_padding_mask`` ``[bsz, seq_len]`` (1 = padding; an addition): the features of padded positions come out as
    zeros, inside the kernel -- what upstream's ``cuda_causal_rfa`` does to phi_k with a separate ``masked_fill`` pass
    (causal_attention.py:137-143)."""
    row_mask = None
    if key_padding_mask is not None and key_padding_mask.dim() > 0:
        assert key_padding_mask.shape == (x.size(1), x.size(0)), (key_padding_mask.shape, x.shape)
        row_mask = key_padding_mask.to(torch.bool).t().contiguous()          # [seq_len, bsz]: one entry per row of x
    return _FeatureMap.apply(x, random_matrices, scale, row_mask)


def normalize_attn_weights(x: Tensor, dim: int = -1, dtype: torch.dtype = torch.float32) -> Tensor:
    x = x.float()
    total = x.sum(dim=dim, keepdim=True).abs().clamp(1e-3)
    return (x / total).type(dtype)
