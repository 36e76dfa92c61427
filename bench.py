#!/usr/bin/env python
"""Benchmark of the RFA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--no-extras]

One "step" = causal RFA forward + backward at the upstream kernel boundary
(``RFA.apply`` on given features and its gradient) on one batch of synthetic input:
batch 8, heads 16, seq 2048, head_dim 64, proj_dim 64 (phi width 128), fp16.
Metric: tokens/s with tokens = batch * seq per step; with N GPUs every rank runs
its own batch (weak scaling over batch x heads, no collective on the data path).

Prints ONE JSON line (rank 0).  ``--impl reference`` instead times the CPU
restatement of upstream's PyTorch path (oracle/rfa_oracle.py) on the host cores,
on a bounded slice of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

B, H, T, D_HEAD, D_PROJ = 8, 16, 2048, 64, 64
K_FEAT = 2 * D_PROJ
BH = B * H
TOKENS_PER_STEP = B * T
# algorithmic bytes per (token, head): fwd reads q,k (2*K*2) + v (d*2), writes out (d*2);
# bwd reads q,k,v,g and writes gq,gk (2*K*2) + gv (d*2)
BYTES_FWD = 2 * K_FEAT * 2 + 2 * D_HEAD * 2                       # 768
BYTES_BWD_Q = K_FEAT * 2 + 3 * D_HEAD * 2 + K_FEAT * 2              # 896   (k,v,g and the saved out in; gq out: q is not read)
BYTES_BWD_KV = 2 * K_FEAT * 2 + 2 * D_HEAD * 2 + K_FEAT * 2 + D_HEAD * 2   # 1152  (q,k,v,g in; gk,gv out)
BYTES_PATH = 2176                                                 # fwd 768 + bwd (768 in + 640 out)
LAUNCHES_PER_STEP = 3                                             # causal_fwd, causal_bwd_q, causal_bwd_kv
WORKLOAD = f"causal RFA fwd+bwd, B{B} H{H} T{T} d{D_HEAD} D{D_PROJ} fp16, RFA.apply boundary"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def make_inputs(seed, device):
    """q,k,v,g for the workload.  Features come from the feature map of N(0,1) vectors
    (seed 0) with one orthogonal random matrix per head (numpy seed 1), v and the upstream
    gradient are N(0,1); everything rounded to fp16."""
    from rfa_b200 import ops
    from rfa_b200.construct_random_matrices import orf
    import numpy as np
    np.random.seed(1)
    w = torch.tensor(np.stack([orf(head_dim=D_HEAD, proj_dim=D_PROJ) for _ in range(H)]), dtype=torch.float32)
    g = torch.Generator().manual_seed(seed)
    xq = torch.randn(T, B, H, D_HEAD, generator=g).half()
    xk = torch.randn(T, B, H, D_HEAD, generator=g).half()
    v = torch.randn(T, B, H, D_HEAD, generator=g).half()
    up = torch.randn(T, B, H, D_HEAD, generator=g).half()
    wd = w.to(device)
    q = ops.feature_map_fwd(xq.to(device), wd, 0.1).view(T, BH, K_FEAT)
    k = ops.feature_map_fwd(xk.to(device), wd, 0.1).view(T, BH, K_FEAT)
    return q, k, v.to(device).view(T, BH, D_HEAD), up.to(device).view(T, BH, D_HEAD), (xq, xk, w)


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.proc, self.lines, self.reader = index, None, [], None

    def __enter__(self):
        """Starts nvidia-smi and returns once it has printed its first line (its start-up takes a few hundred
        milliseconds, longer with one per rank): the lines kept are those printed from then on, i.e. under load as long as
        the caller keeps the GPU busy (``busy_until_sampled``)."""
        import threading
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-i", str(self.index), "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return self
        first = threading.Event()

        def pump():
            for line in self.proc.stdout:
                if first.is_set():
                    self.lines.append(line)
                first.set()
        self.reader = threading.Thread(target=pump, daemon=True)
        self.reader.start()
        first.wait(timeout=10.0)
        return self

    def busy_until_sampled(self, work, want=3, limit_s=2.0):
        """Keeps the GPU on ``work`` (untimed) until ``want`` lines have been printed since the start."""
        t_end = time.time() + limit_s
        while self.proc is not None and len(self.lines) < want and time.time() < t_end:
            work()
            torch.cuda.synchronize()

    def __exit__(self, *a):
        self.summary = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        if self.reader is not None:
            self.reader.join(timeout=2.0)
        out = "".join(self.lines)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for n, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        if sm:
            self.summary = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                            "samples": len(sm)}


def timed(fn, iters, stream):
    """Average device milliseconds per call of fn over iters calls (CUDA events on stream)."""
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for _ in range(iters):
        fn()
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def timed_replayed(fn, iters, stream):
    """Device milliseconds per call of fn with the iters calls captured in one CUDA graph and replayed, which is how a
    training step made of a few short launches is run when host time must not show; eager timing if capture fails.
    Returns (ms, "graph" | "eager")."""
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for _ in range(iters):
                fn()
        graph.replay()
        ms = timed(graph.replay, 3, stream) / iters
        del graph
        return ms, "graph"
    except Exception:  # noqa: BLE001
        torch.cuda.synchronize()
        return timed(fn, iters, stream), "eager"


def host_threads():
    """All the host cores this process may use.  A launcher that starts one process per GPU exports
    OMP_NUM_THREADS=1, which would make the CPU arm a one-core number: set the count explicitly."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def cpu_port_sample():
    """Upstream's PyTorch path restated on the CPU (oracle), fwd+bwd, on a BH slice of the workload: the first 32 of the
    128 (batch, head) sequences of make_inputs-style features at full T.
    Returns (tokens_per_s for the FULL workload by linear scaling in BH, cores, description, seconds)."""
    from oracle import rfa_oracle as O
    cores = host_threads()
    bh = 32
    g = torch.Generator().manual_seed(0)
    q = torch.randn(T, bh, K_FEAT, generator=g) * 0.1
    k = torch.randn(T, bh, K_FEAT, generator=g) * 0.1
    v = torch.randn(T, bh, D_HEAD, generator=g)
    up = torch.randn(T, bh, D_HEAD, generator=g)
    O.causal_forward(q[:256], k[:256], v[:256])     # warm the thread pool
    t0 = time.perf_counter()
    O.causal_forward(q, k, v)
    O.causal_backward(q, k, v, up)
    dt = time.perf_counter() - t0
    full = dt * (BH / bh)
    return TOKENS_PER_STEP / full, cores, f"BH={bh} of {BH} heads at full T={T}, fp32, scaled linearly in BH", dt


def cpu_config1():
    """BASELINE config 1 exactly as specified, on the host cores: batch 2, heads 4, seq 512, head dim 64, D = 64, fp32;
    q,k,v ~ N(0,1) from seed 0, W = 4 orthogonal 64x64 matrices (numpy seed 1), features by random_project (which
    L2-normalises), loss = sum(out * seeded N(0,1)); feature map + forward + backward (upstream utils.py:100-120,
    rfa.py:47-103 restated by the oracle).  Median of 5 runs after one warm-up."""
    from oracle import rfa_oracle as O
    cores = host_threads()
    b, h, t = 2, 4, 512
    torch.manual_seed(0)
    xq, xk, v = (torch.randn(t, b, h, D_HEAD) for _ in range(3))
    w = torch.from_numpy(O.draw_matrices("orf", h, D_HEAD, D_PROJ, 1)).float()
    up = torch.randn(t, b * h, D_HEAD)
    times = []
    for i in range(6):
        t0 = time.perf_counter()
        q = O.random_project(xq, w).view(t, b * h, K_FEAT)
        k = O.random_project(xk, w).view(t, b * h, K_FEAT)
        O.causal_forward(q, k, v.view(t, b * h, D_HEAD))
        O.causal_backward(q, k, v.view(t, b * h, D_HEAD), up)
        if i:
            times.append(time.perf_counter() - t0)
    sec = statistics.median(times)
    return {"workload": "config 1: B2 H4 T512 d64 D64 fp32, seeds 0/1, feature map + causal fwd + bwd", "seconds": sec,
            "tokens_per_s": b * t / sec, "cores": cores, "kind": "port"}


def workload_config(world):
    """The `config` object of the JSON line: the same keys and values for both arms."""
    return {"workload": WORKLOAD, "per_gpu_batch": B, "global_batch": B * world, "heads": H, "seq_len": T,
            "l2": "inputs+outputs 570 MB per step, larger than the 126 MB L2; no flush",
            "parallelism": f"batch x heads sharded over {world} GPU(s), no collective"}


def run_reference(args, rank):
    """The CPU arm: upstream's PyTorch path (restated by the oracle; the upstream package is Python and its checkout
    does not travel to the GPU box) on all host cores, each step a bounded sample of the workload."""
    if rank != 0:
        return
    samples = []
    for i in range(args.warmup + args.steps):
        tps, cores, desc, dt = cpu_port_sample()
        if i >= args.warmup:
            samples.append((tps, dt))
    tps = statistics.median(s[0] for s in samples)
    ms = statistics.median(s[1] for s in samples) * 1e3         # what one step of THIS arm took: the bounded sample
    line = {"impl": "reference", "metric": "causal_rfa_fwd_bwd_tokens_per_s", "value": tps, "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(args.gpus),
            "note": "CPU restatement of upstream rfa.py:47-103 (PyTorch) on the host cores; one step = the bounded sample "
                    "(a quarter of the workload's heads), value = tokens/s of the full workload by linear scaling in heads",
            "sample_fraction": 32 / BH,
            "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc,
                             "sample_seconds": statistics.median(s[1] for s in samples), "config1": cpu_config1()},
            "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def check_timed_buffers(q, k, v, up, out, gq, gk, gv, heads=(0, 37, 77, 127)):
    """The buffers the timed steps have just written, compared with the CPU oracle on a subset of the (batch, head)
    sequences: rel-L2 and max-abs per output (gate: 2e-3 / 1e-2)."""
    from oracle import rfa_oracle as O
    idx = list(heads)
    qf, kf, vf, gf = (t[:, idx].float().cpu() for t in (q, k, v, up))
    ro = O.causal_forward(qf, kf, vf)
    rq, rk, rv = O.causal_backward(qf, kf, vf, gf)
    res = {"heads": idx, "gate": {"rel_l2": 2e-3, "max_abs": 1e-2}}
    ok = True
    for name, a, b in (("out", out, ro), ("gq", gq, rq), ("gk", gk, rk), ("gv", gv, rv)):
        a = a[:, idx].float().cpu()
        r, m = O.rel_l2(a, b), O.max_abs(a, b)
        res[name] = {"rel_l2": r, "max_abs": m}
        ok = ok and r <= 2e-3 and m <= 1e-2 and bool(torch.isfinite(a).all())
    res["ok"] = ok
    return res


# DRAM bytes per launch of the three kernels at this workload (dram__bytes_read.sum + dram__bytes_write.sum of one ncu
# capture each; the summaries with the commands are in profiles/causal_tc_kernels_B8H16T2048.md)
NCU_TRAFFIC = {"causal_fwd": 182.5e6, "causal_bwd_q": 204.7e6, "causal_bwd_kv": 268.9e6}


def upstream_cuda_leg(q, k, v, up, stream, ours_ms):
    """Upstream's own CUDA kernels (oracle/_ref, compiled unmodified for this GPU) on the same inputs."""
    try:
        from oracle import ref_cuda
        mod = ref_cuda.load()
        if mod is None:
            return {"unavailable": "oracle/_ref/rfa_cuda_ref.so not built"}
        legacy = torch.cuda.default_stream()          # upstream launches on the legacy default stream
        with torch.cuda.stream(legacy):
            for _ in range(2):
                mod.forward(q, k, v); mod.backward(q, k, v, up)
            ms_f = timed(lambda: mod.forward(q, k, v), 5, legacy)
            ms_b = timed(lambda: mod.backward(q, k, v, up), 5, legacy)
        return {"fwd_ms": ms_f, "bwd_ms": ms_b, "tokens_per_s": TOKENS_PER_STEP / ((ms_f + ms_b) * 1e-3),
                "speedup_of_new_kernels": (ms_f + ms_b) / ours_ms,
                "note": "includes upstream's own output allocation + zero fill, as its API does"}
    except Exception as e:  # noqa: BLE001
        return {"error": repr(e)}


def tile_stream_ceiling(device, stream, hbm):
    """What the memory system gives for the causal kernels' own access pattern with no arithmetic (rfa_stream_probe): the
    headline geometry (128 CTAs walking T in chunks of 128 rows of 128 bytes, two stages), reading 64 KB per chunk, alone
    and with a 32 KB tile written back per chunk -- the read : write mix of the backward's first sweep."""
    from rfa_b200 import ops
    lib = ops._lib.load()
    Tp, nb = 8 * T, 4                               # 1.07 GB read per launch: far beyond L2
    src = torch.zeros(Tp, BH, 64 * nb, dtype=torch.half, device=device)
    dst = torch.empty(Tp, BH, 128, dtype=torch.half, device=device)
    res = {"workload": f"{BH} CTAs x {Tp // 128} chunks, {16 * nb} KB read (+32 KB written) per chunk, two stages"}
    for name, store in (("read_only", 0), ("read_and_write_2_to_1", 1)):
        fn = lambda: ops.check(lib.rfa_stream_probe(ops.ptr(src), ops.ptr(dst), Tp, BH, nb, store, stream.cuda_stream), "probe")
        for _ in range(2):
            fn()
        ms = timed(fn, 5, stream)
        nbytes = Tp * BH * (128 * nb + (256 if store else 0))
        res[name] = {"ms": ms, "GBps": nbytes / (ms * 1e-3) / 1e9, "frac_of_copy_peak": nbytes / (ms * 1e-3) / 1e9 / hbm}
    return res


def extras(device, stream, hbm):
    """Secondary measurements: decode (config 4), cross attention (config 3), feature map."""
    from rfa_b200 import ops
    out = {}
    try:
        out["tile_stream_ceiling"] = tile_stream_ceiling(device, stream, hbm)
    except Exception as e:  # noqa: BLE001
        out["tile_stream_ceiling"] = {"error": repr(e)}
    # ---- incremental decoding: B64 H16, fp32 state, prefill 512 tokens, 4096 fused steps
    try:
        Bd, Hd, steps, chunk = 64, 16, 4096, 128
        g = torch.Generator().manual_seed(3)
        import numpy as np
        from rfa_b200.construct_random_matrices import orf
        np.random.seed(1)
        w = torch.tensor(np.stack([orf(head_dim=64, proj_dim=64) for _ in range(Hd)]), dtype=torch.float32, device=device)
        pre = [torch.randn(512, Bd, Hd, 64, generator=g).half().to(device) for _ in range(3)]
        pq = ops.feature_map_fwd(pre[0], w, 0.1).view(512, Bd * Hd, 128)
        pk = ops.feature_map_fwd(pre[1], w, 0.1).view(512, Bd * Hd, 128)
        _, s, z = ops.causal_fwd(pq, pk, pre[2].view(512, Bd * Hd, 64), return_state=True)
        s, z = s.view(Bd, Hd, 128, 64), z.view(Bd, Hd, 128)
        qs, ks, vs = (torch.randn(chunk, Bd, Hd, 64, generator=g).half().to(device) for _ in range(3))
        o = torch.empty(chunk, Bd, Hd, 64, dtype=torch.half, device=device)

        def run_chunk():
            for i in range(chunk):
                ops.decode_step_fused(qs[i], ks[i], vs[i], w, 0.1, s, z, o[i])
        run_chunk()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            run_chunk()
        stream = torch.cuda.current_stream()
        graph.replay()
        ms = timed(graph.replay, steps // chunk, stream) / chunk           # per decode step
        per_step_bytes = Bd * Hd * 67328
        out["decode"] = {"workload": "decode B64 H16 d64 D64, fp32 state, fused feature map, CUDA graph of 128 steps",
                         "tokens_per_s": Bd / (ms * 1e-3), "us_per_step": ms * 1e3,
                         "algorithmic_GBps": per_step_bytes / (ms * 1e-3) / 1e9,
                         "frac_of_hbm": per_step_bytes / (ms * 1e-3) / 1e9 / hbm,
                         "note": "state (34 MB) fits in L2; algorithmic bytes, not DRAM bytes"}
        del graph
    except Exception as e:  # noqa: BLE001
        out["decode"] = {"error": repr(e)}
    # ---- cross attention fwd+bwd: B16 H16 Tq=Tk=1024, key lengths U[512,1024]
    try:
        Bc, Hc, Tq = 16, 16, 1024
        g = torch.Generator().manual_seed(2)
        lens = torch.randint(512, 1025, (Bc,), generator=g)
        pad = (torch.arange(Tq)[None] >= lens[:, None]).to(device)
        pq = (torch.randn(Tq, Bc, Hc, 128, generator=g) * 0.1).half().to(device)
        pk = (torch.randn(Tq, Bc, Hc, 128, generator=g) * 0.1).half().to(device)
        v = torch.randn(Tq, Bc, Hc, 64, generator=g).half().to(device)
        up = torch.randn(Tq, Bc, Hc, 64, generator=g).half().to(device)

        def cross_step():
            s, z = ops.cross_state_fwd(pk, v, pad)
            ops.cross_query_fwd(pq, s, z)
            _, d_s, d_z = ops.cross_query_bwd(pq, s, z, up)
            ops.cross_state_bwd(pk, v, pad, d_s, d_z)
        for _ in range(3):
            cross_step()
        ms, how = timed_replayed(cross_step, 10, stream)
        nbytes = Tq * Bc * Hc * BYTES_PATH
        out["cross"] = {"workload": "cross RFA fwd+bwd B16 H16 Tq=Tk=1024 fp16, given features; 4 launches per step, 10 steps "
                                    "per " + how + " timing",
                        "query_tokens_per_s": Bc * Tq / (ms * 1e-3), "ms": ms,
                        "frac_of_hbm": nbytes / (ms * 1e-3) / 1e9 / hbm}
    except Exception as e:  # noqa: BLE001
        out["cross"] = {"error": repr(e)}
    # ---- feature map alone at the causal workload's shape
    try:
        g = torch.Generator().manual_seed(0)
        x = torch.randn(T, B, H, 64, generator=g).half().to(device)
        w = torch.randn(H, 64, 64, generator=g).to(device)
        gp = torch.randn(T, B, H, 128, generator=g).half().to(device)
        for _ in range(3):
            ops.feature_map_fwd(x, w, 0.1)
        ms_f, how = timed_replayed(lambda: ops.feature_map_fwd(x, w, 0.1), 10, stream)
        ms_b, _ = timed_replayed(lambda: ops.feature_map_bwd(x, w, gp, 0.1, True), 10, stream)
        ms_pf, _ = timed_replayed(lambda: ops.feature_map_fwd_pair(x, x, w, 0.1), 10, stream)
        ms_pb, _ = timed_replayed(lambda: ops.feature_map_bwd_pair(x, x, w, gp, gp, 0.1, True), 10, stream)
        nb = T * BH * 384
        out["feature_map_pair"] = {"workload": "q and k of one layer in one launch each way, same shape as feature_map",
                                   "fwd_ms": ms_pf, "fwd_frac_of_hbm": 2 * nb / (ms_pf * 1e-3) / 1e9 / hbm,
                                   "bwd_ms": ms_pb, "bwd_frac_of_hbm": 2 * T * BH * 512 / (ms_pb * 1e-3) / 1e9 / hbm}
        out["feature_map"] = {"timing": how + ", 10 calls", "fwd_ms": ms_f, "fwd_GBps": nb / (ms_f * 1e-3) / 1e9, "fwd_frac_of_hbm": nb / (ms_f * 1e-3) / 1e9 / hbm,
                              "bwd_ms": ms_b, "bwd_GBps": T * BH * 512 / (ms_b * 1e-3) / 1e9,
                              "bwd_frac_of_hbm": T * BH * 512 / (ms_b * 1e-3) / 1e9 / hbm}
    except Exception as e:  # noqa: BLE001
        out["feature_map"] = {"error": repr(e)}
    # ---- forward from the raw q, k (feature map inside the attention kernel) against the two launches it replaces
    try:
        g = torch.Generator().manual_seed(0)
        xq, xk, xv = (torch.randn(T, B, H, 64, generator=g).half().to(device) for _ in range(3))
        w = torch.randn(H, 64, 64, generator=g).to(device)

        def two_step():
            pq = ops.feature_map_fwd(xq, w, 0.1).view(T, BH, K_FEAT)
            pk = ops.feature_map_fwd(xk, w, 0.1).view(T, BH, K_FEAT)
            return ops.causal_fwd(pq, pk, xv.view(T, BH, D_HEAD))
        for _ in range(3):
            ops.causal_fwd_fused(xq, xk, xv, w, 0.1)
            two_step()
        ms_1, how = timed_replayed(lambda: ops.causal_fwd_fused(xq, xk, xv, w, 0.1), 10, stream)
        ms_2, _ = timed_replayed(two_step, 10, stream)
        nb = T * BH * 512                 # x_q, x_k, v in and the output out: 4 x 128 bytes per (token, head)
        out["fused_forward"] = {"workload": "causal forward from raw q, k (feature map inside the kernel), B8 H16 T2048 d64 D64 fp16",
                                "timing": how + ", 10 calls", "ms": ms_1, "frac_of_hbm": nb / (ms_1 * 1e-3) / 1e9 / hbm,
                                "algorithmic_bytes": nb, "two_step_ms": ms_2,
                                "two_step_algorithmic_bytes": T * BH * (2 * 384 + 768)}
    except Exception as e:  # noqa: BLE001
        out["fused_forward"] = {"error": repr(e)}
    # ---- one CausalAttention layer, forward + backward, at the headline shape (embed 1024 = 16 heads x 64): the four
    # projections (cuBLAS), the paired feature map, the causal kernels and the feature map's backward
    try:
        from rfa_b200.causal_attention import CausalAttention
        torch.manual_seed(0)
        layer = CausalAttention(embed_dim=H * D_HEAD, num_heads=H, head_dim=D_HEAD, proj_dim=D_PROJ).to(device).half()
        xm = torch.randn(T, B, H * D_HEAD, device=device).half().requires_grad_(True)
        wm = torch.randn(H, D_PROJ, D_HEAD, device=device).half()
        upm = torch.randn(T, B, H * D_HEAD, device=device).half()

        def layer_step():
            xm.grad = None
            for p_ in layer.parameters():
                p_.grad = None
            layer(xm, wm).backward(upm)
        for _ in range(3):
            layer_step()
        side = torch.cuda.Stream(device)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            layer_step()
        stream.wait_stream(side)
        ms_l, how = timed_replayed(layer_step, 5, stream)
        with torch.no_grad():
            for _ in range(3):
                layer(xm, wm)
            ms_i, _ = timed_replayed(lambda: layer(xm, wm), 5, stream)
        out["layer"] = {"workload": "CausalAttention layer B8 T2048 embed 1024 (16 heads x 64), proj_dim 64, fp16: forward + backward, "
                                    "and the forward alone without a gradient (feature map inside the attention kernel)",
                        "timing": how + ", 5 calls", "fwd_bwd_ms": ms_l, "tokens_per_s": B * T / (ms_l * 1e-3),
                        "no_grad_fwd_ms": ms_i}
    except Exception as e:  # noqa: BLE001
        out["layer"] = {"error": repr(e)}
    return out


LONG_H, LONG_T = 32, 131072


def long_sequence(steps, warmup, rank, world, device, use_graph=True):
    """Long-sequence causal fwd+bwd (BASELINE config 5): batch 1, heads 32, seq 131072, sharded over heads at 2 GPUs and
    over heads x sequence at 4 and 8 (sequence shards exchange boundary states: rfa_b200.sharded).  The process group,
    if any, is already initialised.  Returns (result dict on rank 0 / None elsewhere, release) -- call release() before
    the process group is destroyed: it drops the captured graph, which holds the communicator's collectives."""
    import torch.distributed as dist
    from rfa_b200 import sharded
    Hh, Tt = LONG_H, LONG_T
    group = None
    g_h = 2 if world >= 2 else 1
    g_s = world // g_h
    if world > 1:
        for i in range(g_h):
            grp = dist.new_group(list(range(i * g_s, (i + 1) * g_s)))
            if rank // g_s == i:
                group = grp
    h_loc = Hh // g_h
    lo, hi = sharded.shard_bounds(Tt, g_s, rank % g_s)
    t_loc = hi - lo
    gen = torch.Generator(device=device).manual_seed(4 + rank)
    mk = lambda w, s: (torch.rand(t_loc, h_loc, w, device=device, generator=gen) * s).half()
    q, k = mk(K_FEAT, 0.2).requires_grad_(True), mk(K_FEAT, 0.2).requires_grad_(True)
    v = (torch.randn(t_loc, h_loc, D_HEAD, device=device, generator=gen)).half().requires_grad_(True)
    up = torch.randn(t_loc, h_loc, D_HEAD, device=device, generator=gen).half()
    stream = torch.cuda.current_stream()

    def step():
        q.grad = k.grad = v.grad = None
        out = sharded.sequence_sharded_causal_rfa(q, k, v, group)
        out.backward(up)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
    for _ in range(max(warmup, 3)):
        step()
    barrier()
    # The step is a handful of short launches around two all-gathers: issued eagerly its host time shows.  Capture it in
    # a CUDA graph (kernels, NCCL all-gathers and the autograd backward alike); measure eagerly if capture fails.
    held = {"run": step, "graph": None}
    mode = "eager"
    if use_graph:
        try:
            side = torch.cuda.Stream(device)
            side.wait_stream(stream)
            with torch.cuda.stream(side):
                step()
            stream.wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
            graph.replay()
            torch.cuda.synchronize()
            held["graph"], held["run"], mode = graph, graph.replay, "cuda graph"
        except Exception as e:                      # noqa: BLE001 -- report and measure eagerly
            mode = f"eager (graph capture failed: {type(e).__name__})"
            torch.cuda.synchronize()
    with ClockSampler(device.index) as clk:
        barrier()                                   # after the sampler's start-up, which differs from rank to rank
        ms = timed(held["run"], steps, stream)
        barrier()
        t = torch.tensor([ms], device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        # the sampler's period is 100 ms: the same step keeps running (untimed) for about 0.35 s so that the clocks
        # reported are clocks under this load -- the same number of replays on every rank (the step holds collectives)
        for _ in range(min(2000, int(350.0 / max(ms, 1e-3)) + 1)):
            held["run"]()
        barrier()

    def release():
        held["run"] = None
        held["graph"] = None            # the graph's destructor runs here, before any communicator is torn down
        torch.cuda.synchronize()

    if rank != 0:
        return None, release
    hbm, peak_src = peaks()
    nbytes = Tt * Hh * BYTES_PATH
    return {
        "metric": "long_causal_rfa_fwd_bwd_tokens_per_s", "value": Tt / (ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": steps, "warmup": max(warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"causal RFA fwd+bwd, B1 H{Hh} T{Tt} d64 D64 fp16", "heads_x_sequence_shards": [g_h, g_s],
                   "l2": "9.1 GB per step, far larger than L2", "issue": mode},
        "clocks": clk.summary,
        "roofline": {"bound": "hbm", "achieved": nbytes / (ms * 1e-3) / 1e9 / world, "peak": hbm, "unit": "GB/s per GPU",
                     "frac": nbytes / (ms * 1e-3) / 1e9 / world / hbm, "peak_source": peak_src, "traffic": None}}, release


def leave(world, releases=()):
    """Orderly exit of a multi-rank run: drop captured graphs first (a communicator whose collectives a live graph
    still holds does not tear down), then destroy the process group; if that still does not return within 30 s,
    every rank has finished and rank 0 has printed, so leave without the destructors."""
    import threading
    import torch.distributed as dist
    for r in releases:
        r()
    if world <= 1:
        return
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    giveup = threading.Timer(30.0, lambda: os._exit(0))
    giveup.daemon = True
    giveup.start()
    dist.destroy_process_group()
    giveup.cancel()


def run_long(args, rank, local_rank, world):
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    res, release = long_sequence(args.steps, args.warmup, rank, world, device, use_graph=not args.no_graph)
    if rank == 0:
        print(json.dumps(res), flush=True)
    leave(world, [release])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-extras", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="long workload: issue the step eagerly instead of as a CUDA graph")
    ap.add_argument("--workload", default="headline", choices=["headline", "long"],
                    help="headline = B8 H16 T2048 (the metric's config); long = B1 H32 T131072, sequence-sharded")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "long":
        run_long(args, rank, local_rank, world)
        return

    import torch.distributed as dist
    from rfa_b200 import ops
    from rfa_b200.rfa import RFA
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path); use --impl reference for the CPU baseline")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    hbm, peak_src = peaks()
    stream = torch.cuda.current_stream()
    # pinned buffers and the copy-issuing thread next to the GPU's PCIe root (undone before the CPU baseline is timed)
    # (the CPU worker threads are started first, so that they keep the full core set for the CPU baseline)
    from rfa_b200.host_pipeline import bind_to_gpu_numa_node
    if world == 1:
        host_threads()
        torch.randn(1 << 22).sum().item()
    affinity_before = bind_to_gpu_numa_node(local_rank)
    q, k, v, up, _ = make_inputs(rank, device)
    gq, gk, gv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    out = torch.empty_like(v)
    lib = ops._lib.load()
    nws = lib.rfa_causal_workspace_bytes(T, BH, K_FEAT, D_HEAD)
    ws = torch.empty(max(nws, 256), dtype=torch.uint8, device=device)
    P, st = ops.ptr, stream.cuda_stream

    # what RFA.apply runs: the forward keeps its raw denominators (and segment states) in the workspace, the backward's
    # first sweep reads them and the forward's output instead of recomputing scores and numerators
    kept = ops._lib.WS_STATES | ops._lib.WS_DEN

    def fwd():
        ops.check(lib.rfa_causal_fwd_staged(P(q), P(k), P(v), P(out), None, None, None, None, P(ws), nws, T, BH, K_FEAT, D_HEAD,
                                            0, 1, st), "fwd")

    def bwd_q():
        ops.check(lib.rfa_causal_bwd_q_staged(P(q), P(k), P(v), P(up), P(out), P(gq), None, None, None, P(ws), nws, T, BH, K_FEAT,
                                              D_HEAD, kept, st), "bwd_q")

    def bwd_kv():
        ops.check(lib.rfa_causal_bwd_kv(P(q), P(k), P(v), P(up), P(gk), P(gv), None, None, P(ws), nws, T, BH, K_FEAT, D_HEAD, st), "bwd_kv")

    def step():
        fwd(); bwd_q(); bwd_kv()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    with ClockSampler(local_rank) as clk:
        barrier()                                   # after the sampler's start-up, which differs from rank to rank
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(args.steps):
            step()
        e1.record(stream)
        barrier()
        total_ms = e0.elapsed_time(e1)
        # per-kernel durations, also inside the sampled region
        per = {"causal_fwd": timed(fwd, args.steps, stream), "causal_bwd_q": timed(bwd_q, args.steps, stream),
               "causal_bwd_kv": timed(bwd_kv, args.steps, stream)}
        # the timed region lasts a few milliseconds and the sampler's period is 100 ms: the same step keeps running
        # (untimed) until the sampler has printed a few lines, so that the clocks reported are clocks under this load
        clk.busy_until_sampled(lambda: [step() for _ in range(50)])
    t = torch.tensor([total_ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    value = world * TOKENS_PER_STEP / (ms_per_step * 1e-3)

    # ---- end to end through the public API with host buffers (pinned), copies inside the timed region
    e2e_steps = min(args.steps, 8)
    hq, hk, hv, hg = (x.cpu().pin_memory() for x in (q, k, v, up))
    ho = [torch.empty_like(x, device="cpu").pin_memory() for x in (out, q, k, v)]

    from rfa_b200.host_pipeline import HostPipelinedRFA
    pipe = HostPipelinedRFA(device)

    def e2e_step():
        pipe.step(hq, hk, hv, hg, ho)
    e2e_step()
    pipe.join(stream)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    pipe.up.wait_stream(stream)
    e0.record(stream)
    for _ in range(e2e_steps):
        e2e_step()
    pipe.join(stream)                      # every upload, kernel and download of the timed steps has finished
    e1.record(stream)
    torch.cuda.synchronize()
    e2e_ms = e0.elapsed_time(e1) / e2e_steps
    t = torch.tensor([e2e_ms], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    # the host link's own ceiling, measured the same way on every rank at once: the step's uploads and downloads with no
    # kernel between them (full duplex: uploads on one stream, downloads on another)
    dev_in = pipe.slots[0]["in"]
    dev_out = pipe.slots[0]["out"]

    def copies_only():
        with torch.cuda.stream(pipe.up):
            for dst, h in zip(dev_in, (hq, hk, hv, hg)):
                dst.copy_(h, non_blocking=True)
        with torch.cuda.stream(pipe.down):
            for h, src in zip(ho, dev_out):
                h.copy_(src, non_blocking=True)
    barrier()
    e0.record(stream)
    pipe.up.wait_stream(stream); pipe.down.wait_stream(stream)
    for _ in range(e2e_steps):
        copies_only()
    pipe.join(stream)
    e1.record(stream)
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / e2e_steps], device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    copy_ms = float(t.item())
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hg))
    d2h = sum(x.numel() * x.element_size() for x in ho)

    if affinity_before is not None:
        os.sched_setaffinity(0, affinity_before)
    parity = check_timed_buffers(q, k, v, up, out, gq, gk, gv) if rank == 0 else None

    # ---- the long-sequence workload (config 5) at this N: the sequence-sharded path with its exchange of states
    long_res, release = None, (lambda: None)
    if not args.no_extras:
        hq = hk = hv = hg = ho = pipe = None      # the pinned buffers and the pipeline's device buffers are no longer needed
        torch.cuda.empty_cache()
        try:
            long_res, release = long_sequence(min(args.steps, 10), 3, rank, world, device, use_graph=not args.no_graph)
        except Exception as e:  # noqa: BLE001
            long_res = {"error": repr(e)}

    if rank == 0:
        units = T * BH
        kbytes = {"causal_fwd": BYTES_FWD, "causal_bwd_q": BYTES_BWD_Q, "causal_bwd_kv": BYTES_BWD_KV}
        dom = max(per, key=per.get)
        achieved = units * kbytes[dom] / (per[dom] * 1e-3) / 1e9
        line = {
            "metric": "causal_rfa_fwd_bwd_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config(world),
            "clocks": clk.summary,
            "e2e": {"value": world * TOKENS_PER_STEP / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "h2d_GBps_per_rank": h2d / (e2e_ms * 1e-3) / 1e9, "d2h_GBps_per_rank": d2h / (e2e_ms * 1e-3) / 1e9,
                    "copies_only_ms_per_step": copy_ms, "frac_of_copy_ceiling": copy_ms / e2e_ms,
                    "numa_bound": affinity_before is not None,
                    "api": "rfa_b200.host_pipeline.HostPipelinedRFA.step (upload / compute / download streams), pinned host buffers"},
            "gpu_launches": LAUNCHES_PER_STEP * args.steps,
            "parity": parity,
            "roofline": {"bound": "hbm", "kernel": dom, "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm, "peak_source": peak_src, "traffic": NCU_TRAFFIC.get(dom),
                         "traffic_source": "ncu dram__bytes_read.sum + dram__bytes_write.sum, one capture of this kernel at this "
                                           "workload (profiles/)",
                         "algorithmic_bytes_per_launch": units * kbytes[dom], "ms_per_launch": per[dom],
                         "per_kernel_ms": per,
                         "path": {"bytes_per_step": units * BYTES_PATH,
                                  "achieved": units * BYTES_PATH / (ms_per_step * 1e-3) / 1e9,
                                  "frac": units * BYTES_PATH / (ms_per_step * 1e-3) / 1e9 / hbm}},
        }
        if not args.no_extras:
            line["extra"] = {"long_sequence": long_res}
        if world == 1:
            tps, cores, desc, dt = cpu_port_sample()
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": desc,
                                    "seconds": dt, "config1": cpu_config1()}
            if not args.no_extras:
                line["extra"].update(extras(device, stream, hbm))
                line["extra"]["upstream_cuda_kernels"] = upstream_cuda_leg(q, k, v, up, stream, ms_per_step)
        print(json.dumps(line), flush=True)
    leave(world, [release])


if __name__ == "__main__":
    main()
