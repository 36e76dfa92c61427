"""Parity at the sizes the benchmark reports (BASELINE configs 2-5), through the C ABI, against the CPU
oracle: the headline launch plan (one segment x 16 chunks x 128 CTAs), cross attention in two waves with key
masks that end inside a chunk, decoding from a prefilled state replayed from a CUDA graph, the long sequence
(all heads on the GPU, two of them against the fp64 streaming oracle, late tokens checked separately), and the
sequence split into 2, 4 and 8 shards run in one process.

Gate as everywhere: fp16 outputs and gradients within rel-L2 <= 2e-3 and max-abs <= 1e-2 of the fp32 (fp64 for
the long sequence) oracle on identical fp16-valued inputs."""
import pytest
import torch

from conftest import assert_close
from oracle import rfa_oracle as O

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- config 2 (headline)
def test_headline_workload_all_heads_vs_oracle(dev):
    """B8 H16 T2048, inputs exactly as bench.make_inputs builds them (seeds 0 / 1): every one of the 128
    (batch, head) sequences, out and all three gradients."""
    import bench
    from rfa_b200 import ops
    q, k, v, up, _ = bench.make_inputs(0, dev)
    T, BH = q.shape[0], q.shape[1]
    assert (T, BH) == (2048, 128)
    out, ws, has = ops.causal_fwd_saved(q, k, v)              # what RFA.apply and the benchmark run
    gq, gk, gv = ops.causal_bwd_saved(q, k, v, up, out, ws, has)
    rec = (ops.causal_fwd(q, k, v),) + tuple(ops.causal_bwd(q, k, v, up))      # upstream's signature: recompute from q, k, v
    torch.cuda.synchronize()
    for name, a, b in zip(("out", "gq", "gk", "gv"), (out, gq, gk, gv), rec):
        assert_close(a, b.float().cpu(), f"c2 {name}: saved-output path vs recomputing path", rel=1e-3)
    worst = {}
    for lo in range(0, BH, 32):
        sl = slice(lo, lo + 32)
        qf, kf, vf, gf = (t[:, sl].float().cpu() for t in (q, k, v, up))
        ro = O.causal_forward(qf, kf, vf)
        rq, rk, rv = O.causal_backward(qf, kf, vf, gf)
        for name, a, b in (("out", out, ro), ("gq", gq, rq), ("gk", gk, rk), ("gv", gv, rv)):
            r, m = assert_close(a[:, sl], b, f"c2 heads {lo}..{lo + 31} {name}")
            worst[name] = max(worst.get(name, (0, 0)), (r, m))
    print("c2 worst (rel-L2, max-abs) per output:", {n: (f"{r:.2e}", f"{m:.2e}") for n, (r, m) in worst.items()})


# ----------------------------------------------------------------------------- config 3 (cross attention)
def test_cross_workload_full_size_vs_oracle(dev):
    """B16 H16 Tq = Tk = 1024, key lengths U[512, 1024] from seed 2 (256 CTAs; masks end mid-chunk)."""
    from rfa_b200 import ops
    Bc, Hc, Tq = 16, 16, 1024
    g = torch.Generator().manual_seed(2)
    lens = torch.randint(512, 1025, (Bc,), generator=g)
    pad = torch.arange(Tq)[None] >= lens[:, None]
    w = torch.from_numpy(O.draw_matrices("orf", Hc, 64, 64, 1)).float()
    xq, xk = torch.randn(Tq, Bc, Hc, 64, generator=g), torch.randn(Tq, Bc, Hc, 64, generator=g)
    pq = O.random_project(xq, w).half().float()
    pk = O.random_project(xk, w).half().float()
    v = torch.randn(Tq, Bc, Hc, 64, generator=g).half().float()
    up = torch.randn(Tq, Bc, Hc, 64, generator=g).half().float()
    assert any(int(n) % 128 for n in lens)
    dq, dk, dv, dup, dpad = pq.half().to(dev), pk.half().to(dev), v.half().to(dev), up.half().to(dev), pad.to(dev)
    s, z = ops.cross_state_fwd(dk, dv, dpad)
    attn = ops.cross_query_fwd(dq, s, z)
    gq, d_s, d_z = ops.cross_query_bwd(dq, s, z, dup)
    gk, gv = ops.cross_state_bwd(dk, dv, dpad, d_s, d_z)
    torch.cuda.synchronize()
    rs, rz = O.cross_state(pk, v, pad)
    assert_close(s, rs, "c3 s", rel=1e-4); assert_close(z, rz, "c3 z", rel=1e-4)
    assert_close(attn, O.cross_query(pq, rs, rz), "c3 attn")
    rq, rk, rv = O.cross_backward(pq, pk, v, up, pad)
    assert_close(gq, rq, "c3 g_phi_q"); assert_close(gk, rk, "c3 g_phi_k"); assert_close(gv, rv, "c3 g_v")
    assert (gk.cpu()[pad.T] == 0).all() and (gv.cpu()[pad.T] == 0).all()


# ----------------------------------------------------------------------------- config 4 (decode)
def test_decode_workload_prefill_then_graph_replayed_steps(dev):
    """B64 H16: a 512-token prompt prefilled by the causal kernel (state handed over through s_out / z_out),
    then 256 fused single-token steps replayed from CUDA graphs of 128 steps, as the benchmark issues them;
    every step's output and the final state against the oracle's token-by-token loop."""
    from rfa_b200 import ops
    Bd, Hd, Tp, steps, chunk = 64, 16, 512, 256, 128
    g = torch.Generator().manual_seed(3)
    w = torch.from_numpy(O.draw_matrices("orf", Hd, 64, 64, 1)).float()
    pre = [torch.randn(Tp, Bd, Hd, 64, generator=g).half() for _ in range(3)]
    wd = w.to(dev)
    pq = ops.feature_map_fwd(pre[0].to(dev), wd, 0.1).view(Tp, Bd * Hd, 128)
    pk = ops.feature_map_fwd(pre[1].to(dev), wd, 0.1).view(Tp, Bd * Hd, 128)
    _, s, z = ops.causal_fwd(pq, pk, pre[2].to(dev).view(Tp, Bd * Hd, 64), return_state=True)
    rs, rz = O.segment_state(pk.float().cpu(), pre[2].float().view(Tp, Bd * Hd, 64))
    assert_close(s, rs, "c4 prefilled S", rel=1e-4); assert_close(z, rz, "c4 prefilled z", rel=1e-4)
    s, z = s.view(Bd, Hd, 128, 64), z.view(Bd, Hd, 128)
    rs, rz = s.float().cpu().clone(), z.float().cpu().clone()      # the oracle continues from the SAME state
    outs, refs = [], []
    qs, ks, vs = (torch.empty(chunk, Bd, Hd, 64, dtype=torch.half, device=dev) for _ in range(3))
    o = torch.empty(chunk, Bd, Hd, 64, dtype=torch.half, device=dev)

    def run_chunk():
        for i in range(chunk):
            ops.decode_step_fused(qs[i], ks[i], vs[i], wd, 0.1, s, z, o[i])
    keep_s, keep_z = s.clone(), z.clone()
    run_chunk()                                                    # warm-up outside capture (restored below)
    torch.cuda.synchronize()
    s.copy_(keep_s); z.copy_(keep_z)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_chunk()
    s.copy_(keep_s); z.copy_(keep_z)
    for c in range(steps // chunk):
        hq, hk, hv = (torch.randn(chunk, Bd, Hd, 64, generator=g).half() for _ in range(3))
        qs.copy_(hq); ks.copy_(hk); vs.copy_(hv)
        graph.replay()
        torch.cuda.synchronize()
        outs.append(o.cpu().clone())
        fq, fk = O.random_project(hq.float(), w).half().float(), O.random_project(hk.float(), w).half().float()
        for i in range(chunk):
            ref, rs, rz = O.incremental_rfa(fq[i:i + 1], fk[i:i + 1], hv[i:i + 1].float(), rs, rz)
            refs.append(ref)
    got = torch.cat(outs).view(steps, Bd, -1)
    want = torch.cat(refs).view(steps, Bd, -1)
    assert_close(got, want, "c4 decode outputs")
    assert_close(got[-16:], want[-16:], "c4 decode outputs (last 16 steps)")
    assert_close(s, rs, "c4 final S", rel=2e-3); assert_close(z, rz, "c4 final z", rel=2e-3)


# ----------------------------------------------------------------------------- config 5 (long sequence)
def _long_inputs(T, H, dev, seed=4):
    gen = torch.Generator().manual_seed(seed)
    w = torch.from_numpy(O.draw_matrices("orf", H, 64, 64, 1)).float().to(dev)
    from rfa_b200 import ops
    xq = torch.randn(T, 1, H, 64, generator=gen).half().to(dev)
    xk = torch.randn(T, 1, H, 64, generator=gen).half().to(dev)
    q = ops.feature_map_fwd(xq, w, 0.1).view(T, H, 128)
    k = ops.feature_map_fwd(xk, w, 0.1).view(T, H, 128)
    v = torch.randn(T, H, 64, generator=gen).half().to(dev)
    g = torch.randn(T, H, 64, generator=gen).half().to(dev)
    return q, k, v, g


def test_long_sequence_workload_vs_fp64_oracle(dev):
    """B1 H32 T131072 on the GPU for all 32 heads (the segmented plan: 4 segments x 256 chunks per head); two heads
    against the fp64 streaming oracle, the last eighth of the sequence (denominators in the thousands, g/den in the
    fp16 subnormal range) held to the same gate on its own; every head finite."""
    from rfa_b200 import ops
    T, H = 131072, 32
    q, k, v, g = _long_inputs(T, H, dev)
    out = ops.causal_fwd(q, k, v)
    gq, gk, gv = ops.causal_bwd(q, k, v, g)
    torch.cuda.synchronize()
    for t in (out, gq, gk, gv):
        assert torch.isfinite(t).all()
    heads = [0, 21]
    qd, kd, vd, gd = (t[:, heads].double().cpu() for t in (q, k, v, g))
    ro = O.causal_forward(qd, kd, vd, block=256)
    rq, rk, rv = O.causal_backward(qd, kd, vd, gd, block=256)
    tail = slice(T - T // 8, T)
    for name, a, b in (("out", out, ro), ("gq", gq, rq), ("gk", gk, rk), ("gv", gv, rv)):
        assert_close(a[:, heads], b, f"c5 {name}")
        assert_close(a[tail][:, heads], b[tail], f"c5 {name} (last eighth)")


@pytest.mark.parametrize("shards", [2, 4, 8])
def test_sequence_shards_in_one_process_equal_the_unsharded_run(dev, shards):
    """The sequence-sharded path (rfa_b200.sharded.SequenceShardedRFA: shard totals, exclusive scan over shards, local
    kernels with carries) driven with 2, 4 and 8 shards of one sequence run one after another on one GPU: outputs and
    gradients must equal the unsharded kernels' (same gate; the two differ only in where fp32 partial sums are cut)
    and the oracle's."""
    from rfa_b200 import ops, sharded
    T, H = 8192, 4
    q, k, v, g = _long_inputs(T, H, dev, seed=40 + shards)
    whole = (ops.causal_fwd(q, k, v),) + tuple(ops.causal_bwd(q, k, v, g))
    group = sharded.InProcessShards(shards)
    bounds = [sharded.shard_bounds(T, shards, r) for r in range(shards)]
    leaves, outs = [], []
    for r, (lo, hi) in enumerate(bounds):                       # forward in rank order
        group.rank = r
        ql, kl, vl = (t[lo:hi].clone().requires_grad_(True) for t in (q, k, v))
        leaves.append((ql, kl, vl))
        outs.append(sharded.sequence_sharded_causal_rfa(ql, kl, vl, group))
    for r in reversed(range(shards)):                           # backward in reverse rank order
        group.rank = r
        lo, hi = bounds[r]
        outs[r].backward(g[lo:hi])
    torch.cuda.synchronize()
    got = (torch.cat([o.detach() for o in outs]),) + tuple(torch.cat([l[i].grad for l in leaves]) for i in range(3))
    qf, kf, vf, gf = (t.float().cpu() for t in (q, k, v, g))
    want = (O.causal_forward(qf, kf, vf),) + tuple(O.causal_backward(qf, kf, vf, gf))
    for name, a, b, c in zip(("out", "gq", "gk", "gv"), got, whole, want):
        assert_close(a, b.float().cpu(), f"{shards} shards {name} vs unsharded kernels")
        assert_close(a, c, f"{shards} shards {name} vs oracle")


def test_empty_shard_calls_launch_nothing(dev):
    """A trailing shard can be empty (T = 300 over 4 ranks): its local steps return zero totals and empty gradients
    without touching the library, so that the rank still joins both exchanges."""
    from rfa_b200 import ops
    e = lambda w: torch.empty(0, 3, w, dtype=torch.half, device=dev)
    s, z = ops.state_total(e(128), e(64))
    assert s.shape == (3, 128, 64) and not s.any() and z.shape == (3, 128) and not z.any()
    gq, ds, dz, ws = ops.causal_bwd_q(e(128), e(128), e(64), e(64), None, None, True)
    assert gq.shape == (0, 3, 128) and not ds.any() and not dz.any()
    gk, gv = ops.causal_bwd_kv(e(128), e(128), e(64), e(64), None, None, ws)
    assert gk.shape == (0, 3, 128) and gv.shape == (0, 3, 64)


def test_decode_rejects_odd_feature_width_without_launching(dev):
    from rfa_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(4096, dtype=torch.float32, device=dev)
    p = x.data_ptr()
    assert lib.rfa_decode_step(p, p, p, 1, p, p, 1, p, 1, 127, 64, None) == -3
    assert b"multiple of 4" in lib.rfa_last_error()
    assert lib.rfa_decode_step(p, p, p, 1, p, p, 0, p, 1, 128, 64, None) == -3      # fp32 inputs with an fp16 state
