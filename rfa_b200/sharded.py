"""Causal RFA with the SEQUENCE split across the ranks of a process group.

Each rank holds a contiguous run of tokens of every (batch, head) sequence it owns:
``q, k [T_local, BH, K]``, ``v [T_local, BH, d]``, rank r of the group holding the r-th run.
Because the attention state is a plain sum over past tokens, one exchange per direction
suffices (upstream has no multi-device path; its kernel walks the whole sequence in one
CTA, cuda/forward.cu:112-125):

forward   1. every rank reduces its own tokens to (S_r, z_r)          -- no dependency
          2. exclusive prefix sum over ranks: carry_r = sum_{j<r} (S_j, z_j)   (one all-gather)
          3. the local causal kernel runs with that carry
backward  1. the forward-direction sweep runs with the saved carry and also yields this
             rank's own reverse-state total (dS_r, dz_r)
          2. exclusive SUFFIX sum over ranks: carry_r = sum_{j>r} (dS_j, dz_j)  (one all-gather)
          3. the reverse sweep runs with that carry

Heads shard trivially (slice BH); combine both by giving each head group its own
sequence process group.  The states are small (33 KB per head), so the exchange is
latency-bound; it is an all-gather followed by a local masked sum.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


class InProcessShards:
    """Stands in for a process group when the shards of one sequence run ONE AFTER ANOTHER in a single process (a
    sequence whose activations do not fit the device at once; a one-GPU check of the sharded path).  Set ``rank``
    before each shard's call.  Forward calls must come in rank order 0, 1, ... and backward calls in the opposite
    order, because a shard's carry is the sum of what the shards before (backward: after) it have deposited here."""

    def __init__(self, world: int):
        self.world, self.rank = int(world), 0
        self._deposits = {False: {}, True: {}}

    def exclusive_scan(self, local: Tensor, reverse: bool) -> Tensor:
        box = self._deposits[reverse]
        box[self.rank] = local.detach().clone()
        need = range(self.rank + 1, self.world) if reverse else range(self.rank)
        missing = [r for r in need if r not in box]
        if missing:
            raise RuntimeError(f"InProcessShards: shard {self.rank} ran before shard(s) {missing} "
                               f"({'backward' if reverse else 'forward'} order violated)")
        total = torch.zeros_like(local)
        for r in need:
            total += box[r]
        return total


def exclusive_scan_over_ranks(local: Tensor, group=None, reverse: bool = False) -> Tensor:
    """Sum of ``local`` over the ranks strictly before (``reverse``: strictly after) this
    rank in ``group``.  One all-gather of the per-rank tensors, then a local sum."""
    if isinstance(group, InProcessShards):
        return group.exclusive_scan(local, reverse)
    if not (dist.is_available() and dist.is_initialized()):
        return torch.zeros_like(local)            # single process: nothing comes before or after
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    if world == 1:
        return torch.zeros_like(local)
    local = local.contiguous()
    flat = local.reshape(1, -1)
    gathered = torch.empty((world, flat.shape[1]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered, flat, group=group)
    gathered = gathered.view((world,) + tuple(local.shape))
    sel = gathered[rank + 1:] if reverse else gathered[:rank]
    if sel.shape[0] == 0:
        return torch.zeros_like(local)
    return sel.sum(dim=0)


def _group_size(group) -> int:
    if isinstance(group, InProcessShards):
        return group.world
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


class _CudaKernels:
    """The four local steps on the sm_100a kernels."""

    @staticmethod
    def segment_state(k: Tensor, v: Tensor) -> Tuple[Tensor, Tensor]:
        from . import ops
        return ops.state_total(k, v)

    @staticmethod
    def forward(q, k, v, s_in, z_in):
        from . import ops
        return ops.causal_fwd(q, k, v, s_in, z_in)

    @staticmethod
    def backward_q(q, k, v, g, s_in, z_in):
        from . import ops
        gq, ds, dz, ws = ops.causal_bwd_q(q, k, v, g, s_in, z_in, True)
        return gq, ds, dz, ws

    @staticmethod
    def backward_kv(q, k, v, g, ds_in, dz_in, ctx):
        from . import ops
        return ops.causal_bwd_kv(q, k, v, g, ds_in, dz_in, ctx)

    @staticmethod
    def backward_full(q, k, v, g):
        from . import ops
        return ops.causal_bwd(q, k, v, g, None, None, None, None)


class SequenceShardedRFA(torch.autograd.Function):
    """``SequenceShardedRFA.apply(q, k, v, group)`` -- attention output for this rank's tokens."""

    kernels = _CudaKernels

    @staticmethod
    def forward(ctx, q, k, v, group=None):
        kern = SequenceShardedRFA.kernels
        ctx.group = group
        ctx.alone = _group_size(group) == 1
        if ctx.alone:                              # the whole sequence is here: no carry in either direction
            ctx.save_for_backward(q, k, v)
            return kern.forward(q, k, v, None, None)
        s_loc, z_loc = kern.segment_state(k, v)
        packed = torch.cat([s_loc.reshape(s_loc.shape[0], -1), z_loc], dim=1)          # [BH, K*d + K]
        carry = exclusive_scan_over_ranks(packed, group)
        n = s_loc[0].numel()
        s_in = carry[:, :n].reshape(s_loc.shape).contiguous()
        z_in = carry[:, n:].contiguous()
        ctx.group = group
        ctx.save_for_backward(q, k, v, s_in, z_in)
        return kern.forward(q, k, v, s_in, z_in)

    @staticmethod
    def backward(ctx, g):
        kern = SequenceShardedRFA.kernels
        g = g.contiguous()
        if ctx.alone:
            q, k, v = ctx.saved_tensors
            if hasattr(kern, "backward_full"):
                return tuple(kern.backward_full(q, k, v, g)) + (None,)
            gq, _, _, sweep_ctx = kern.backward_q(q, k, v, g, None, None)
            gk, gv = kern.backward_kv(q, k, v, g, None, None, sweep_ctx)
            return gq, gk, gv, None
        q, k, v, s_in, z_in = ctx.saved_tensors
        gq, ds_loc, dz_loc, sweep_ctx = kern.backward_q(q, k, v, g, s_in, z_in)
        packed = torch.cat([ds_loc.reshape(ds_loc.shape[0], -1), dz_loc], dim=1)
        carry = exclusive_scan_over_ranks(packed, ctx.group, reverse=True)
        n = ds_loc[0].numel()
        ds_in = carry[:, :n].reshape(ds_loc.shape).contiguous()
        dz_in = carry[:, n:].contiguous()
        gk, gv = kern.backward_kv(q, k, v, g, ds_in, dz_in, sweep_ctx)
        return gq, gk, gv, None


def sequence_sharded_causal_rfa(q: Tensor, k: Tensor, v: Tensor, group=None) -> Tensor:
    """q,k ``[T_local, BH, 2*proj_dim]``, v ``[T_local, BH, head_dim]`` (fp16 CUDA): this rank's
    slice of the sequence; returns ``[T_local, BH, head_dim]``.  Differentiable."""
    return SequenceShardedRFA.apply(q, k, v, group)


def shard_bounds(T: int, world: int, rank: int, align: int = 128) -> Tuple[int, int]:
    """Token range [lo, hi) of ``rank`` when T tokens are cut into ``world`` contiguous runs of
    equal length rounded up to ``align`` (the kernels' chunk length); trailing ranks may be short."""
    per = -(-T // world)
    per = -(-per // align) * align
    lo = min(T, rank * per)
    return lo, min(T, lo + per)
