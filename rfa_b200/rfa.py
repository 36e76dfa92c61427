"""Causal RFA autograd boundary -- same surface as upstream ``rfa.py``.

``RFA.apply(q, k, v)`` with q,k ``[tgt_len, bsz*num_heads, 2*proj_dim]`` and v
``[tgt_len, bsz*num_heads, head_dim]`` (fp16, CUDA) returns
``attn[t] = q_t^T S_t / max(q_t . z_t, EPS)`` with the inclusive running sums
``S_t = sum_{s<=t} k_s v_s^T`` and ``z_t = sum_{s<=t} k_s`` (upstream rfa.py:57-64).

``forward_cuda`` / ``backward_cuda`` run the sm_100a kernels; ``forward_torch`` /
``backward_torch`` are the PyTorch twins upstream keeps beside them for
checking (any device, any float dtype).  ``forward``/``backward`` always use the
kernels -- there is no fallback.
"""
import torch

from . import rfa_cuda

EPS = 1.0


def reverse_cumsum(x, dim):
    """Suffix sums along ``dim`` (upstream rfa.py:20-21)."""
    total = x.sum(dim=dim, keepdim=True)
    return total - torch.cumsum(x, dim=dim) + x


def _running_state(k, v):
    """Inclusive prefix sums of k (x) v and of k along time."""
    kv = k.unsqueeze(-1) * v.unsqueeze(-2)            # [T,B,K,d]
    return torch.cumsum(kv, dim=0), torch.cumsum(k, dim=0)


def rfa_debug(q, k, v):
    """Same function as ``RFA.forward_torch`` (upstream rfa.py:24-41)."""
    return RFA.forward_torch(q, k, v)


class RFA(torch.autograd.Function):

    @staticmethod
    def forward_torch(q, k, v):
        """PyTorch twin of the forward kernel (upstream rfa.py:47-64)."""
        s, z = _running_state(k, v)
        num = (s * q.unsqueeze(-1)).sum(dim=-2)
        den = (q * z).sum(dim=-1, keepdim=True).clamp_min(EPS)
        return num / den

    @staticmethod
    def backward_torch(q, k, v, grad_attn):
        """PyTorch twin of the backward kernel (upstream rfa.py:67-103).
        Returns (grad_q, grad_k, grad_v)."""
        s, z = _running_state(k, v)
        num = (s * q.unsqueeze(-1)).sum(dim=-2)
        den = (q * z).sum(dim=-1, keepdim=True).clamp_min(EPS)
        g_num = grad_attn / den
        g_den = -(grad_attn * num).sum(dim=-1, keepdim=True) / den.square()
        g_den = g_den * (den > EPS)
        grad_q = (s * g_num.unsqueeze(-2)).sum(dim=-1) + g_den * z
        g_s = reverse_cumsum(q.unsqueeze(-1) * g_num.unsqueeze(-2), dim=0)
        grad_k = (g_s * v.unsqueeze(-2)).sum(dim=-1) + reverse_cumsum(q * g_den, dim=0)
        grad_v = (g_s * k.unsqueeze(-1)).sum(dim=-2)
        return grad_q, grad_k, grad_v

    @staticmethod
    def forward_cuda(q, k, v):
        return rfa_cuda.forward(q, k, v)

    @staticmethod
    def backward_cuda(q, k, v, grad_attn):
        return rfa_cuda.backward(q, k, v, grad_attn)

    @staticmethod
    def forward(ctx, q, k, v):
        ctx.save_for_backward(q, k, v)
        return RFA.forward_cuda(q, k, v)

    @staticmethod
    def backward(ctx, grad_attn):
        q, k, v = ctx.saved_tensors
        grad_q, grad_k, grad_v = RFA.backward_cuda(q, k, v, grad_attn.contiguous())
        return grad_q, grad_k, grad_v
