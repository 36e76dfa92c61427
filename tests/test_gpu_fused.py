"""Parity of the causal forward that forms the feature map inside the kernel (rfa_causal_fwd_fused) with the CPU oracle
(random_project of q and k, then the causal forward: upstream utils.py:100-120 + rfa.py:57-64) and with this library's own
two-step path (feature map kernel, then the forward on ready-made features).

Gate: relative L2 <= 2e-3 and max-abs <= 1e-2 against the fp32 oracle evaluated on the same fp16-valued inputs."""
import pytest
import torch

from conftest import assert_close
from oracle import rfa_oracle as O

pytestmark = pytest.mark.gpu

SCALE = 64 ** -0.5


def h16(t):
    return t.half().float()


def raw_inputs(T, B, H, seed):
    gen = torch.Generator().manual_seed(seed)
    w = torch.from_numpy(O.draw_matrices("orf", H, 64, 64, seed + 7)).float()
    xq, xk = h16(torch.randn(T, B, H, 64, generator=gen)), h16(torch.randn(T, B, H, 64, generator=gen))
    v, g = h16(torch.randn(T, B, H, 64, generator=gen)), h16(torch.randn(T, B, H, 64, generator=gen))
    return xq, xk, v, g, w


def oracle_features(xq, xk, w, mask):
    T, B, H, _ = xq.shape
    pq = O.random_project(xq, w, SCALE).reshape(T, B * H, 128)
    pk = O.random_project(xk, w, SCALE)
    if mask is not None:
        pk = pk.masked_fill(mask.reshape(T, B, 1, 1), 0.0)
    return pq, pk.reshape(T, B * H, 128)


@pytest.mark.parametrize("T,B,H,masked", [(1, 1, 1, False), (128, 1, 1, False), (129, 2, 1, True), (300, 2, 3, False),
                                          (300, 2, 3, True), (1000, 2, 4, True), (77, 3, 2, False)])
def test_fused_forward_against_oracle(dev, T, B, H, masked):
    from rfa_b200 import ops
    xq, xk, v, _, w = raw_inputs(T, B, H, 11)
    mask = None
    if masked:                       # padded keys: the tail of each sequence, a different length per batch element
        lens = torch.tensor([max(1, T - 17 * (b + 1)) for b in range(B)])
        mask = torch.arange(T)[:, None] >= lens[None, :]
    pq, pk = oracle_features(xq, xk, w, mask)
    want, s_w, z_w = O.causal_forward(pq, pk, v.reshape(T, B * H, 64), return_state=True)
    out, s, z = ops.causal_fwd_fused(xq.half().to(dev), xk.half().to(dev), v.half().to(dev), w.to(dev), SCALE,
                                     row_mask=None if mask is None else mask.to(dev), return_state=True)
    assert_close(out, want, "attn")
    assert_close(s, s_w, "S", rel=1e-3, mabs=1e-2)
    assert_close(z, z_w, "z", rel=1e-3, mabs=1e-2)


def test_fused_forward_matches_two_step_path_and_carries_state(dev):
    from rfa_b200 import ops
    T, B, H = 520, 2, 4
    xq, xk, v, _, w = raw_inputs(T, B, H, 5)
    cu = lambda t: t.half().to(dev)
    wd = w.to(dev)
    pq = ops.feature_map_fwd(cu(xq), wd, SCALE).view(T, B * H, 128)
    pk = ops.feature_map_fwd(cu(xk), wd, SCALE).view(T, B * H, 128)
    two, s2, z2 = ops.causal_fwd(pq, pk, cu(v).view(T, B * H, 64), return_state=True)
    one, s1, z1 = ops.causal_fwd_fused(cu(xq), cu(xk), cu(v), wd, SCALE, return_state=True)
    assert_close(one, two, "fused vs two-step attn", rel=5e-4)
    assert_close(s1, s2, "fused vs two-step S", rel=1e-4, mabs=1e-3)
    assert_close(z1, z2, "fused vs two-step z", rel=1e-4, mabs=1e-3)
    # a sequence run in two calls, the second carrying the first's state, equals one call
    cut = 256
    a, sa, za = ops.causal_fwd_fused(cu(xq[:cut]), cu(xk[:cut]), cu(v[:cut]), wd, SCALE, return_state=True)
    b, sb, zb = ops.causal_fwd_fused(cu(xq[cut:]), cu(xk[cut:]), cu(v[cut:]), wd, SCALE, s_in=sa, z_in=za, return_state=True)
    assert_close(torch.cat([a, b]), one, "two calls vs one", rel=5e-4)
    assert_close(sb, s1, "carried S", rel=1e-4, mabs=1e-3)
    assert_close(zb, z1, "carried z", rel=1e-4, mabs=1e-3)


def test_fused_forward_leaves_denominators_for_the_saved_backward(dev):
    from rfa_b200 import _lib, ops
    T, B, H = 384, 2, 2
    xq, xk, v, g, w = raw_inputs(T, B, H, 21)
    cu = lambda t: t.half().to(dev)
    wd = w.to(dev)
    out, ws = ops.causal_fwd_fused(cu(xq), cu(xk), cu(v), wd, SCALE, save_den=True)
    pq = ops.feature_map_fwd(cu(xq), wd, SCALE).view(T, B * H, 128)
    pk = ops.feature_map_fwd(cu(xk), wd, SCALE).view(T, B * H, 128)
    gq, gk, gv = ops.causal_bwd_saved(pq, pk, cu(v).view(T, B * H, 64), cu(g).view(T, B * H, 64), out, ws, _lib.WS_DEN)
    fq, fk = oracle_features(xq, xk, w, None)
    wq, wk, wv = O.causal_backward(fq, fk, v.reshape(T, B * H, 64), g.reshape(T, B * H, 64))
    assert_close(gq, wq, "g_phi_q")
    assert_close(gk, wk, "g_phi_k")
    assert_close(gv, wv, "g_v")


def test_fused_forward_at_the_benchmark_shape(dev):
    """B8 H16 T2048: 128 CTAs of 16 chunks, every head against the two-step path, four heads against the oracle."""
    from rfa_b200 import ops
    T, B, H = 2048, 8, 16
    xq, xk, v, _, w = raw_inputs(T, B, H, 0)
    cu = lambda t: t.half().to(dev)
    wd = w.to(dev)
    one = ops.causal_fwd_fused(cu(xq), cu(xk), cu(v), wd, SCALE)
    pq = ops.feature_map_fwd(cu(xq), wd, SCALE).view(T, B * H, 128)
    pk = ops.feature_map_fwd(cu(xk), wd, SCALE).view(T, B * H, 128)
    two = ops.causal_fwd(pq, pk, cu(v).view(T, B * H, 64))
    assert_close(one, two, "fused vs two-step attn", rel=5e-4)
    heads = [0, 37, 90, 127]
    fq, fk = oracle_features(xq, xk, w, None)
    want = O.causal_forward(fq[:, heads], fk[:, heads], v.reshape(T, B * H, 64)[:, heads])
    want = want[0] if isinstance(want, tuple) else want
    assert_close(one[:, heads], want, "attn")
    assert _status() == 0


def _status():
    from rfa_b200 import _lib
    return _lib.load().rfa_debug_status()


def test_causal_attention_module_uses_the_fused_forward(dev, monkeypatch):
    """A half-precision CausalAttention layer (head_dim 64, proj_dim 64, many heads): without a gradient, and on request
    with one, the forward goes through the fused kernel; output and every gradient agree with the same layer run through
    the two-step path."""
    from rfa_b200 import causal_attention as CA
    from rfa_b200 import ops
    T, B, E, H = 256, 4, 512, 8
    torch.manual_seed(3)
    layer = CA.CausalAttention(embed_dim=E, num_heads=H, head_dim=64, proj_dim=64, tau=1.0, reparam_proj=True).to(dev).half()
    w = torch.from_numpy(O.draw_matrices("orf", H, 64, 64, 9)).half().to(dev).requires_grad_(True)
    x = torch.randn(T, B, E, device=dev).half().requires_grad_(True)
    pad = torch.zeros(B, T, dtype=torch.bool, device=dev)
    pad[1, 200:] = True
    pad[3, 77:] = True
    up = torch.randn(T, B, E, device=dev).half()

    calls = []
    real = ops.causal_fwd_fused
    monkeypatch.setattr(ops, "causal_fwd_fused", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    # without a gradient the layer takes the fused kernel by itself; with one, only when asked to
    with torch.no_grad():
        y0 = layer(x, w, key_padding_mask=pad)
    assert len(calls) == 1
    y1 = layer(x, w, key_padding_mask=pad)
    assert len(calls) == 1
    assert_close(y0, y1, "module out, no-grad fused vs recorded two-step", rel=2e-3)
    calls.clear()
    layer.fuse_feature_map = True

    def run():
        for p in list(layer.parameters()) + [w, x]:
            p.grad = None
        y = layer(x, w, key_padding_mask=pad)
        y.backward(up)
        return [y.detach().clone(), x.grad.clone(), w.grad.clone()] + [p.grad.clone() for p in layer.parameters()]

    fused = run()
    assert calls, "the fused forward was not used"
    monkeypatch.setattr(ops, "fused_forward_supported", lambda *_: False)
    n = len(calls)
    two = run()
    assert len(calls) == n
    names = ["out", "g_x", "g_w"] + ["g_" + k for k, _ in layer.named_parameters()]
    for a, b, name in zip(fused, two, names):
        assert_close(a, b, "module " + name, rel=2e-3)
