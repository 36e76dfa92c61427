"""Causal RFA with the SEQUENCE split across the ranks of a process group.

Each rank holds a contiguous run of tokens of every (batch, head) sequence it owns:
``q, k [T_local, BH, K]``, ``v [T_local, BH, d]``, rank r of the group holding the r-th run.
Because the attention state is a plain sum over past tokens, one exchange per direction
suffices (upstream has no multi-device path; its kernel walks the whole sequence in one
CTA, cuda/forward.cu:112-125):

forward   1. every rank reduces its own tokens to (S_r, z_r)          -- no dependency; the per-segment
             partial sums stay in the workspace, so the local kernel does not read k, v a second time for them
          2. exclusive prefix sum over ranks: carry_r = sum_{j<r} (S_j, z_j)   (one all-gather + one small kernel)
          3. the local causal kernel runs with that carry and keeps its output, raw denominators and segment
             states for the backward
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
    gathered = _all_gather(local, group, world)
    sel = gathered[rank + 1:] if reverse else gathered[:rank]
    if sel.shape[0] == 0:
        return torch.zeros_like(local)
    return sel.sum(dim=0)


def _all_gather(local: Tensor, group, world: int) -> Tensor:
    local = local.contiguous()
    gathered = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(gathered.view(world, -1), local.view(1, -1), group=group)
    return gathered


def _group_size(group) -> int:
    if isinstance(group, InProcessShards):
        return group.world
    if not (dist.is_available() and dist.is_initialized()):
        return 1
    return dist.get_world_size(group)


def _carry(kern, packed: Tensor, group, reverse: bool, K: int, d: int):
    """The exchange step: every shard's packed total [BH, K*d + K] -> this shard's carry (s [BH,K,d], z [BH,K]).
    With a real process group the gathered totals are reduced by one kernel when the kernel set has one."""
    if not isinstance(group, InProcessShards) and hasattr(kern, "scan_gathered") and kern.packed_kernels(K, d):
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        return kern.scan_gathered(_all_gather(packed, group, world), rank, reverse)
    total = exclusive_scan_over_ranks(packed, group, reverse)
    n = K * d
    return total[:, :n].reshape(-1, K, d).contiguous(), total[:, n:].contiguous()


class _CudaKernels:
    """The local steps on the sm_100a kernels.  Totals travel packed ``[BH, K*d + K]`` (S then z).  What a step keeps for
    a later one is a tuple of tensors (the kept workspace: per-segment sums, then segment-entry states and raw
    denominators, then the per-token scalars of the first backward sweep; and the forward's output) plus one plain
    value; the autograd function stores the tensors with ``save_for_backward``."""

    @staticmethod
    def packed_kernels(K: int, d: int) -> bool:
        """The packed-total / kept-workspace entry points exist for the tensor-core geometry only; other geometries take
        the plain entry points (same results, a few more launches)."""
        from . import ops
        return (K, d) == (ops.K_BUILT, ops.D_BUILT)

    @staticmethod
    def local_total(k: Tensor, v: Tensor):
        from . import ops
        if not _CudaKernels.packed_kernels(k.shape[-1], v.shape[-1]):
            s, z = ops.state_total(k, v)
            return torch.cat([s.reshape(s.shape[0], -1), z], dim=1), None
        return ops.shard_total(k, v)

    @staticmethod
    def scan_gathered(gathered: Tensor, rank: int, reverse: bool):
        from . import ops
        return ops.scan_gathered(gathered, rank, reverse)

    @staticmethod
    def forward(q, k, v, s_in, z_in, ws):
        from . import _lib, ops
        if not _CudaKernels.packed_kernels(q.shape[-1], v.shape[-1]):
            return ops.causal_fwd(q, k, v, s_in, z_in), (), None
        out, ws, has = ops.causal_fwd_saved(q, k, v, s_in, z_in, ws, _lib.WS_PARTIALS if ws is not None else 0)
        return out, (out, ws), has

    @staticmethod
    def backward_q(q, k, v, g, s_in, z_in, kept, has):
        from . import ops
        if not kept:
            gq, ds, dz, ws = ops.causal_bwd_q(q, k, v, g, s_in, z_in, True)
            return gq, torch.cat([ds.reshape(ds.shape[0], -1), dz], dim=1), ws
        out, ws = kept
        gq, dpacked = ops.causal_bwd_q_staged(q, k, v, g, out, s_in, z_in, ws, has)
        return gq, dpacked, ws

    @staticmethod
    def backward_kv(q, k, v, g, ds_in, dz_in, ws):
        from . import ops
        return ops.causal_bwd_kv(q, k, v, g, ds_in, dz_in, ws)

    @staticmethod
    def forward_alone(q, k, v):
        from . import ops
        out, ws, has = ops.causal_fwd_saved(q, k, v)
        return out, (out, ws), has

    @staticmethod
    def backward_alone(q, k, v, g, kept, has):
        from . import ops
        out, ws = kept
        return ops.causal_bwd_saved(q, k, v, g, out, ws, has)


class SequenceShardedRFA(torch.autograd.Function):
    """``SequenceShardedRFA.apply(q, k, v, group)`` -- attention output for this rank's tokens."""

    kernels = _CudaKernels

    @staticmethod
    def forward(ctx, q, k, v, group=None):
        kern = SequenceShardedRFA.kernels
        ctx.group = group
        ctx.alone = _group_size(group) == 1
        K, d = q.shape[-1], v.shape[-1]
        if ctx.alone:                              # the whole sequence is here: no carry in either direction
            out, kept, ctx.meta = kern.forward_alone(q, k, v)
            ctx.save_for_backward(q, k, v, *kept)
            return out
        packed, fwd_ctx = kern.local_total(k, v)
        s_in, z_in = _carry(kern, packed, group, False, K, d)
        out, kept, ctx.meta = kern.forward(q, k, v, s_in, z_in, fwd_ctx)
        ctx.save_for_backward(q, k, v, s_in, z_in, *kept)
        return out

    @staticmethod
    def backward(ctx, g):
        kern = SequenceShardedRFA.kernels
        g = g.contiguous()
        if ctx.alone:
            q, k, v, *kept = ctx.saved_tensors
            return tuple(kern.backward_alone(q, k, v, g, tuple(kept), ctx.meta)) + (None,)
        q, k, v, s_in, z_in, *kept = ctx.saved_tensors
        K, d = q.shape[-1], v.shape[-1]
        gq, dpacked, sweep_ctx = kern.backward_q(q, k, v, g, s_in, z_in, tuple(kept), ctx.meta)
        ds_in, dz_in = _carry(kern, dpacked, ctx.group, True, K, d)
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
