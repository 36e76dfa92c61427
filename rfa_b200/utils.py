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


def sample_random_matrices(*, num_layers: int, num_heads: int, random_matrices: Tensor,
                           is_training: bool = True):
    """Training: ``num_layers * num_heads`` distinct matrices drawn from the bank with
    numpy's global RNG, returned as a list of ``[num_heads, proj_dim, head_dim]`` per
    layer.  Evaluation: the first ``num_heads`` matrices (one tensor shared by all
    layers).  (upstream utils.py:62-87)"""
    if not is_training:
        return random_matrices[list(range(num_heads))]
    picks = np.random.choice(random_matrices.size(0), size=num_layers * num_heads, replace=False)
    chosen = random_matrices[picks]
    return list(chosen.split(num_heads, dim=0))


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
    def forward(ctx, x, w, scale):
        ctx.save_for_backward(x, w)
        ctx.scale = scale
        return ops.feature_map_fwd(x, w, scale)

    @staticmethod
    def backward(ctx, g_phi):
        x, w = ctx.saved_tensors
        need_w = ctx.needs_input_grad[1]
        g_x, g_w = ops.feature_map_bwd(x, w, g_phi, ctx.scale, need_w)
        return g_x, (g_w.to(w.dtype) if need_w else None), None


def random_project(*, x: Tensor, random_matrices: Tensor, scale: float = SCALE) -> Tensor:
    """x ``[seq_len, bsz, num_heads, head_dim]``, random_matrices ``[num_heads, proj_dim,
    head_dim]`` -> phi ``[seq_len, bsz, num_heads, 2 * proj_dim]`` in x's dtype
    (upstream utils.py:105-120; ``scale`` defaults to upstream's constant 0.1)."""
    return _FeatureMap.apply(x, random_matrices, scale)


def normalize_attn_weights(x: Tensor, dim: int = -1, dtype: torch.dtype = torch.float32) -> Tensor:
    x = x.float()
    total = x.sum(dim=dim, keepdim=True).abs().clamp(1e-3)
    return (x / total).type(dtype)
