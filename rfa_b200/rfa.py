"""Causal RFA autograd boundary -- same surface as upstream ``rfa.py``.

``RFA.apply(q, k, v)`` with q,k ``[tgt_len, bsz*num_heads, 2*proj_dim]`` and v
``[tgt_len, bsz*num_heads, head_dim]`` (fp16, CUDA) returns
``attn[t] = q_t^T S_t / max(q_t . z_t, EPS)`` with the inclusive running sums
``S_t = sum_{s<=t} k_s v_s^T`` and ``z_t = sum_{s<=t} k_s`` (upstream rfa.py:57-64).

``forward_cuda`` / ``backward_cuda`` run the sm_100a kernels with upstream's signatures
(the backward recomputes everything from q, k, v, as upstream's does); ``forward_torch`` /
``backward_torch`` are the PyTorch twins upstream keeps beside them for checking (any
device, any float dtype).  ``RFA.apply`` itself keeps the forward's output, raw
denominators and segment states for its backward, which then skips the recomputation
(upstream saves q, k, v only, rfa.py:116); there is no fallback to PyTorch.
"""
import torch

from . import ops, rfa_cuda

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
        if not (ctx.needs_input_grad[0] or ctx.needs_input_grad[1] or ctx.needs_input_grad[2]):
            return RFA.forward_cuda(q, k, v)
        out, ws, has = ops.causal_fwd_saved(q, k, v)
        ctx.save_for_backward(q, k, v, out, ws)
        ctx.ws_has = has
        return out

    @staticmethod
    def backward(ctx, grad_attn):
        q, k, v, out, ws = ctx.saved_tensors
        grad_q, grad_k, grad_v = ops.causal_bwd_saved(q, k, v, grad_attn.contiguous().to(q.dtype), out, ws, ctx.ws_has)
        return grad_q, grad_k, grad_v
