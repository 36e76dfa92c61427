"""Sequence-sharded causal RFA on 2 and 4 GPUs over NCCL (skipped with fewer devices):
rfa_b200.sharded with the real kernels must equal the unsharded kernels and the oracle."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from oracle import rfa_oracle as O
        from rfa_b200 import sharded
        gen = torch.Generator().manual_seed(0)
        T, BH = 1024 * world // 2, 3
        q = (torch.rand(T, BH, 128, generator=gen) * 0.2).half()
        k = (torch.rand(T, BH, 128, generator=gen) * 0.2).half()
        v = torch.randn(T, BH, 64, generator=gen).half()
        g = torch.randn(T, BH, 64, generator=gen).half()
        lo, hi = sharded.shard_bounds(T, world, rank)
        ql, kl, vl = (t[lo:hi].to(dev).requires_grad_(True) for t in (q, k, v))
        out = sharded.sequence_sharded_causal_rfa(ql, kl, vl)
        out.backward(g[lo:hi].to(dev))
        torch.cuda.synchronize()
        ro = O.causal_forward(q.float(), k.float(), v.float())
        rq, rk, rv = O.causal_backward(q.float(), k.float(), v.float(), g.float())
        errs = [O.rel_l2(out.detach().float().cpu(), ro[lo:hi]), O.rel_l2(ql.grad.float().cpu(), rq[lo:hi]),
                O.rel_l2(kl.grad.float().cpu(), rk[lo:hi]), O.rel_l2(vl.grad.float().cpu(), rv[lo:hi])]
        out_q.put((rank, errs))
    except Exception as e:  # noqa: BLE001
        out_q.put((rank, [repr(e)]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_multi_gpu_sequence_sharding_matches_oracle(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    out_q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, out_q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [out_q.get(timeout=300) for _ in range(world)]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in results:
        assert all(isinstance(e, float) for e in errs), (rank, errs)
        assert max(errs) <= 2e-3, (rank, errs)
