"""rfa_b200 -- Random Feature Attention hot path on NVIDIA B200 (sm_100a).

Same Python surface as upstream's ``random_feature_attention`` package for the
path it accelerates; all compute happens in ``csrc/librfa_b200.so`` (hand-written
CUDA, loaded through its C ABI).  There is no CPU or PyTorch fallback: importing
the kernels without the built library raises.

``install_aliases()`` makes ``import random_feature_attention`` and
``import rfa_cuda`` resolve to this package, for code written against upstream.
"""
import sys

from .utils import CrossAttentionState
from .causal_attention import CausalAttention
from .cross_attention import CrossAttention, CrossAttentionProject

__all__ = ["CausalAttention", "CrossAttention", "CrossAttentionState", "CrossAttentionProject",
           "install_aliases"]


def install_aliases() -> None:
    """Register this package under upstream's import names."""
    from . import causal_attention, construct_random_matrices, cross_attention, rfa, rfa_cuda, utils
    me = sys.modules[__name__]
    sys.modules.setdefault("random_feature_attention", me)
    for name, mod in (("rfa", rfa), ("utils", utils), ("causal_attention", causal_attention),
                      ("cross_attention", cross_attention),
                      ("construct_random_matrices", construct_random_matrices)):
        sys.modules.setdefault(f"random_feature_attention.{name}", mod)
    sys.modules.setdefault("rfa_cuda", rfa_cuda)
