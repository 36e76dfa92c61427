"""Stand-in for upstream's pybind11 extension module ``rfa_cuda``
(cuda/rfa_cuda.cpp:39-42): the same two functions with the same signatures,
implemented as thin calls into the sm_100a library through its C ABI.

``rfa_b200.install_aliases()`` registers this module under the top-level name
``rfa_cuda`` so that ``import rfa_cuda`` in unmodified upstream code finds it.
"""
from typing import List

from torch import Tensor

from . import ops


def forward(q: Tensor, k: Tensor, v: Tensor) -> Tensor:
    """q,k [tgt_len, bsz*num_heads, 2*proj_dim], v [tgt_len, bsz*num_heads, head_dim],
    all fp16 CUDA -> attn [tgt_len, bsz*num_heads, head_dim]
    (cuda/rfa_cuda.cpp:22-27).  Unlike upstream, a non-fp16 tensor is rejected
    instead of being reinterpreted."""
    return ops.causal_fwd(q, k, v)


def backward(q: Tensor, k: Tensor, v: Tensor, grad_attn: Tensor) -> List[Tensor]:
    """-> [grad_q, grad_k, grad_v]  (cuda/rfa_cuda.cpp:29-36)."""
    return list(ops.causal_bwd(q, k, v, grad_attn))
