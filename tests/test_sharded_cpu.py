"""The sequence-sharded scan on CPU ranks (gloo, world size 2 and 3): the rank-level logic of
rfa_b200.sharded -- local reduction, exclusive prefix / suffix scan over ranks, carries --
with the CPU oracle standing in for the local kernels.  The sharded result must equal the
unsharded oracle on the full sequence, outputs and all gradients."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import rfa_oracle as O


class OracleKernels:
    """Same steps as rfa_b200.sharded._CudaKernels, computed by the oracle in fp64 (it keeps nothing between steps)."""

    @staticmethod
    def local_total(k, v):
        s, z = O.segment_state(k, v)
        return torch.cat([s.reshape(s.shape[0], -1), z], dim=1), None

    @staticmethod
    def forward(q, k, v, s_in, z_in, fwd_ctx):
        return O.causal_forward(q, k, v, s0=s_in, z0=z_in), (), None

    @staticmethod
    def backward_q(q, k, v, g, s_in, z_in, kept, meta):
        gq, _, _, ds, dz = O.causal_backward(q, k, v, g, s0=s_in, z0=z_in, return_dstate=True)
        return gq, torch.cat([ds.reshape(ds.shape[0], -1), dz], dim=1), (s_in, z_in)

    @staticmethod
    def backward_kv(q, k, v, g, ds_in, dz_in, ctx):
        s_in, z_in = ctx
        _, gk, gv = O.causal_backward(q, k, v, g, s0=s_in, z0=z_in, ds_in=ds_in, dz_in=dz_in)
        return gk, gv

    @staticmethod
    def forward_alone(q, k, v):
        return O.causal_forward(q, k, v), (), None

    @staticmethod
    def backward_alone(q, k, v, g, kept, meta):
        return O.causal_backward(q, k, v, g)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, T, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from rfa_b200 import sharded
        sharded.SequenceShardedRFA.kernels = OracleKernels
        out_q.put((rank, _run(rank, world, T, sharded)))
    except Exception as e:  # noqa: BLE001 -- report instead of leaving the parent waiting
        out_q.put((rank, [repr(e)]))
    finally:
        dist.destroy_process_group()


def _run(rank, world, T, sharded):
    if True:
        gen = torch.Generator().manual_seed(0)
        BH, K, d = 3, 16, 8
        q = (torch.rand(T, BH, K, generator=gen, dtype=torch.float64) * 0.4)
        k = (torch.rand(T, BH, K, generator=gen, dtype=torch.float64) * 0.4)
        v = torch.randn(T, BH, d, generator=gen, dtype=torch.float64)
        g = torch.randn(T, BH, d, generator=gen, dtype=torch.float64)
        lo, hi = sharded.shard_bounds(T, world, rank, align=8)
        ql, kl, vl = (t[lo:hi].clone().requires_grad_(True) for t in (q, k, v))
        out = sharded.sequence_sharded_causal_rfa(ql, kl, vl)
        out.backward(g[lo:hi])
        ro = O.causal_forward(q, k, v)
        rq, rk, rv = O.causal_backward(q, k, v, g)
        errs = [float((out.detach() - ro[lo:hi]).abs().max()) if hi > lo else 0.0]
        for a, b in ((ql.grad, rq), (kl.grad, rk), (vl.grad, rv)):
            errs.append(float((a - b[lo:hi]).abs().max()) if hi > lo else 0.0)
        # the scan primitive itself
        x = torch.full((2, 3), float(rank + 1))
        pre = sharded.exclusive_scan_over_ranks(x)
        suf = sharded.exclusive_scan_over_ranks(x, reverse=True)
        errs.append(float((pre - sum(range(1, rank + 1))).abs().max()))
        errs.append(float((suf - sum(range(rank + 2, world + 1))).abs().max()))
        return errs


# (4, 20): runs of 8 tokens leave the last rank an EMPTY shard, which must still join both exchanges
@pytest.mark.parametrize("world,T", [(2, 64), (3, 50), (4, 20)])
def test_sequence_sharded_equals_unsharded(world, T):
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, T, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=120) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, errs in results:
        assert all(isinstance(e, float) for e in errs), (rank, errs)
        assert max(errs) < 1e-10, (rank, errs)


def test_shard_bounds_cover_the_sequence():
    from rfa_b200.sharded import shard_bounds
    for T, world in ((131072, 8), (1000, 3), (5, 4), (0, 2)):
        spans = [shard_bounds(T, world, r) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == T
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
        assert all((lo % 128 == 0) or lo == T for lo, _ in spans)


def test_a_lone_shard_skips_the_exchange():
    """Without a process group (or in a group of one) the whole sequence is local: no shard total is computed, no
    carry is exchanged, and the result equals the plain oracle."""
    from rfa_b200 import sharded

    calls = []

    class Counting(OracleKernels):
        @staticmethod
        def local_total(k, v):
            calls.append("local_total")
            return OracleKernels.local_total(k, v)

    saved = sharded.SequenceShardedRFA.kernels
    sharded.SequenceShardedRFA.kernels = Counting
    try:
        gen = torch.Generator().manual_seed(3)
        T, BH = 70, 2
        q = (torch.rand(T, BH, 128, generator=gen, dtype=torch.float64) * 0.2).requires_grad_(True)
        k = (torch.rand(T, BH, 128, generator=gen, dtype=torch.float64) * 0.2).requires_grad_(True)
        v = torch.randn(T, BH, 64, generator=gen, dtype=torch.float64).requires_grad_(True)
        g = torch.randn(T, BH, 64, generator=gen, dtype=torch.float64)
        out = sharded.sequence_sharded_causal_rfa(q, k, v, None)
        out.backward(g)
        assert calls == []
        ro = O.causal_forward(q.detach(), k.detach(), v.detach())
        rq, rk, rv = O.causal_backward(q.detach(), k.detach(), v.detach(), g)
        for a, b in ((out.detach(), ro), (q.grad, rq), (k.grad, rk), (v.grad, rv)):
            assert torch.allclose(a, b, rtol=1e-10, atol=1e-12)
    finally:
        sharded.SequenceShardedRFA.kernels = saved


def test_in_process_shards_equal_the_unsharded_oracle():
    """Shards of one sequence run one after another in one process (forward in rank order, backward in reverse)."""
    from rfa_b200 import sharded
    saved = sharded.SequenceShardedRFA.kernels
    sharded.SequenceShardedRFA.kernels = OracleKernels
    try:
        gen = torch.Generator().manual_seed(5)
        T, BH, K, d, world = 40, 2, 16, 8, 3
        q = torch.rand(T, BH, K, generator=gen, dtype=torch.float64) * 0.4
        k = torch.rand(T, BH, K, generator=gen, dtype=torch.float64) * 0.4
        v = torch.randn(T, BH, d, generator=gen, dtype=torch.float64)
        g = torch.randn(T, BH, d, generator=gen, dtype=torch.float64)
        group = sharded.InProcessShards(world)
        bounds = [sharded.shard_bounds(T, world, r, align=8) for r in range(world)]
        leaves, outs = [], []
        for r, (lo, hi) in enumerate(bounds):
            group.rank = r
            leaves.append(tuple(t[lo:hi].clone().requires_grad_(True) for t in (q, k, v)))
            outs.append(sharded.sequence_sharded_causal_rfa(*leaves[-1], group))
        group.rank = 0
        with pytest.raises(RuntimeError, match="order violated"):       # shard 0 cannot go backward before the later shards
            outs[0].backward(g[bounds[0][0]:bounds[0][1]], retain_graph=True)
        for r in reversed(range(world)):
            group.rank = r
            outs[r].backward(g[bounds[r][0]:bounds[r][1]])
        ro = O.causal_forward(q, k, v)
        want = (ro,) + tuple(O.causal_backward(q, k, v, g))
        got = (torch.cat([o.detach() for o in outs]),) + tuple(torch.cat([l[i].grad for l in leaves]) for i in range(3))
        for a, b in zip(got, want):
            assert torch.allclose(a, b, rtol=1e-10, atol=1e-12)
    finally:
        sharded.SequenceShardedRFA.kernels = saved
