"""The allocation-free backward entry point (rfa_causal_bwd_noalloc) against the regular one.

Some callers of the library cannot bring a workspace: a serving process that handed all
device memory to its own pools and bans cudaMalloc while running, or a C program with no
device allocator.  For them the library keeps the backward's scratch in a fixed array of
its own.  This file checks, through the C ABI, that the entry point gives the same
gradients as rfa_causal_bwd -- on two calls in a row of different sizes, so that what the
first call left in the shared array cannot leak into the second -- and that it refuses
problems larger than the array.  It is collected last on purpose: a run that stops at the
first failure has then already run every other test.
"""
import pytest
import torch

from conftest import assert_close

pytestmark = pytest.mark.gpu


def _inputs(T, BH, seed, dev):
    gen = torch.Generator().manual_seed(seed)
    q = (torch.rand(T, BH, 128, generator=gen) * 0.2 - 0.05).half().to(dev)
    k = (torch.rand(T, BH, 128, generator=gen) * 0.2 - 0.05).half().to(dev)
    v = torch.randn(T, BH, 64, generator=gen).half().to(dev)
    g = torch.randn(T, BH, 64, generator=gen).half().to(dev)
    return q, k, v, g


def _noalloc_bwd(q, k, v, g, check_mem=True):
    from rfa_b200 import _lib
    lib = _lib.load()
    T, BH, _ = q.shape
    gq, gk, gv = torch.full_like(q, float("nan")), torch.full_like(k, float("nan")), torch.full_like(v, float("nan"))
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()      # the driver's own count: sees a cudaMalloc made inside the library too
    status = lib.rfa_causal_bwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(), gq.data_ptr(),
                                        gk.data_ptr(), gv.data_ptr(), T, BH, 128, 64,
                                        torch.cuda.current_stream().cuda_stream)
    assert status == 0, _lib.last_error()
    assert torch.cuda.memory_allocated() == before
    torch.cuda.synchronize()
    if check_mem:       # (the very first launch of a kernel may make the driver load its code, which takes device memory)
        assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the call"
    return gq, gk, gv


def test_noalloc_backward_matches_regular_backward_twice_in_a_row(dev):
    from oracle import rfa_oracle as O
    from rfa_b200 import ops
    _noalloc_bwd(*_inputs(8, 1, 0, dev), check_mem=False)              # first call on the device and thread: one-time set-up, not measured
    for T, BH, seed in ((700, 3, 1), (130, 5, 2)):      # the second call is smaller: stale scratch lies beyond and inside it
        q, k, v, g = _inputs(T, BH, seed, dev)
        ref = ops.causal_bwd(q, k, v, g)
        got = _noalloc_bwd(q, k, v, g)
        want = O.causal_backward(*(t.float().cpu() for t in (q, k, v, g)))
        for name, a, b, c in zip(("gq", "gk", "gv"), got, ref, want):
            assert_close(a, b, f"T={T} {name} vs rfa_causal_bwd")
            assert_close(a, c, f"T={T} {name} vs oracle")


def test_noalloc_backward_refuses_sizes_beyond_its_scratch(dev):
    from rfa_b200 import _lib
    lib = _lib.load()
    limit = lib.rfa_causal_bwd_noalloc_max_token_heads()
    assert limit == 512 * 1024
    x = torch.zeros(16, dtype=torch.half, device=dev)
    p = x.data_ptr()
    assert lib.rfa_causal_bwd_noalloc(p, p, p, p, p, p, p, limit // 4 + 1, 4, 128, 64, None) == -4
    assert b"exceeds the built-in scratch" in lib.rfa_last_error()
    assert lib.rfa_causal_bwd_noalloc(p, p, p, p, p, p, p, 8, 2, 96, 64, None) == -3
