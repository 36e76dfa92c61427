"""Upstream's own CUDA kernels (compiled unmodified for the B200 by oracle/build_ref.py) beside
the new kernels, on upstream's own check shapes and criterion (grad_check.py:13-50: squared
difference < 1e-4 elementwise), plus a looser look at a longer sequence where upstream's
fp16-accumulated state has drifted.  Skipped when oracle/_ref/rfa_cuda_ref.so is absent."""
import pytest
import torch

from conftest import golden
from oracle import ref_cuda
from oracle import rfa_oracle as O

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def upstream():
    mod = ref_cuda.load()
    if mod is None:
        pytest.skip("oracle/_ref/rfa_cuda_ref.so not built (python oracle/build_ref.py)")
    return mod


@pytest.mark.parametrize("name", ["causal_fwd_gradcheck", "causal_bwd_gradcheck"])
def test_same_answers_as_upstream_kernels_on_upstream_check_shapes(dev, upstream, name):
    from rfa_b200 import ops
    g = golden(name)
    q, k, v = (g[n].half().to(dev).contiguous() for n in ("q", "k", "v"))
    up = (g["g"] if "g" in g else torch.ones_like(g["v"])).half().to(dev).contiguous()
    ref_out = upstream.forward(q, k, v)
    ref_gq, ref_gk, ref_gv = upstream.backward(q, k, v, up)
    torch.cuda.synchronize()
    out = ops.causal_fwd(q, k, v)
    gq, gk, gv = ops.causal_bwd(q, k, v, up)
    # Upstream's criterion (grad_check.py:13-14) is |difference| < 1e-2 against its fp32 twin.  On the
    # unit-norm fixture both kernel sets meet it against each other.  On the first fixture (unnormalised
    # rows, outputs up to 6) upstream's own fp16-accumulating kernel is 0.038 away from its fp32 twin --
    # it fails its own check there -- so the new kernels are held to: inside the criterion against fp32,
    # and no further from upstream's kernel than upstream's kernel is from fp32.
    if name == "causal_bwd_gradcheck":
        for a, b in ((out, ref_out), (gq, ref_gq), (gk, ref_gk), (gv, ref_gv)):
            assert ((a.float() - b.float()) ** 2 < 1e-4).all()
    else:
        want = g["attn"].to(dev)
        mine, theirs = (out.float() - want).abs().max(), (ref_out.float() - want).abs().max()
        assert mine < 1e-2 and mine <= theirs
        assert (out.float() - ref_out.float()).abs().max() <= mine + theirs


def test_upstream_kernels_drift_where_new_kernels_do_not(dev, upstream):
    """T = 2048 on real features: both against the fp32 oracle.  Reported, and the new kernels
    must be the closer of the two."""
    from rfa_b200 import ops
    gen = torch.Generator().manual_seed(0)
    T, BH = 2048, 4
    w = torch.from_numpy(O.draw_matrices("orf", 1, 64, 64, 1)).float()
    q = O.random_project(torch.randn(T, BH, 1, 64, generator=gen), w).view(T, BH, 128).half()
    k = O.random_project(torch.randn(T, BH, 1, 64, generator=gen), w).view(T, BH, 128).half()
    v = torch.randn(T, BH, 64, generator=gen).half()
    ref = O.causal_forward(q.float(), k.float(), v.float())
    mine = ops.causal_fwd(q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    theirs = upstream.forward(q.to(dev), k.to(dev), v.to(dev)).float().cpu()
    e_mine, e_theirs = O.rel_l2(mine, ref), O.rel_l2(theirs, ref)
    print(f"rel-L2 vs fp32 oracle at T=2048: new kernels {e_mine:.2e}, upstream kernels {e_theirs:.2e}")
    assert e_mine <= 2e-3 and e_mine <= e_theirs
