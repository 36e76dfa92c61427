"""The CPU oracle against fixtures produced by the upstream Python sources
(tests/golden/make_golden.py).  fp32 vs fp32: tolerances are rounding-level."""
import numpy as np
import torch

from oracle import rfa_oracle as O
from conftest import golden

TIGHT = dict(rtol=2e-5, atol=2e-6)


def close(a, b, **kw):
    kw = {**TIGHT, **kw}
    assert a.shape == b.shape
    assert torch.allclose(a.float(), b.float(), **kw), float((a.float() - b.float()).abs().max())


def test_matrices_match_upstream_generators():
    g = golden("matrices")
    close(torch.from_numpy(O.draw_matrices("orf", 4, 64, 64, 1)), g["orf_seed1"], rtol=0, atol=0)
    close(torch.from_numpy(O.draw_matrices("rrf", 2, 64, 64, 7)), g["rrf_seed7"], rtol=0, atol=0)
    close(torch.from_numpy(O.draw_matrices("orf", 2, 32, 48, 11)), g["orf_wide_seed11"], rtol=0, atol=0)


def test_feature_map_forward_and_backward():
    g = golden("feature_map")
    w_eff = O.build_random_matrices(g["w"], float(g["tau"]), g["sigma"], True)
    close(w_eff, g["w_eff"])
    close(O.random_project(g["x"], w_eff), g["phi"])
    close(O.random_project(g["x"], g["w"]), g["phi_plain"])
    gx, gw = O.random_project_backward(g["x"], w_eff, g["g_phi"])
    close(gx, g["g_x"], atol=2e-5)
    close(gw, g["g_w"], atol=2e-5)


def test_causal_forward_gradcheck_shapes():
    g = golden("causal_fwd_gradcheck")
    for blk in (1, 7, 64):
        close(O.causal_forward(g["q"], g["k"], g["v"], block=blk), g["attn"])
    close(O.causal_forward_literal(g["q"], g["k"], g["v"]), g["attn_debug"])


def test_causal_backward_gradcheck_shapes():
    g = golden("causal_bwd_gradcheck")
    close(O.causal_forward(g["q"], g["k"], g["v"]), g["attn"])
    for blk in (13, 64):
        gq, gk, gv = O.causal_backward(g["q"], g["k"], g["v"], g["g"], block=blk)
        close(gq, g["gq"], atol=1e-5); close(gk, g["gk"], atol=1e-5); close(gv, g["gv"], atol=1e-5)


def test_causal_on_features_both_clamp_branches():
    g = golden("causal_features")
    out, den = O.causal_forward(g["q"], g["k"], g["v"], return_den=True)
    close(out, g["attn"], atol=1e-5)
    close(den, g["qz"], atol=1e-5)
    gq, gk, gv = O.causal_backward(g["q"], g["k"], g["v"], g["g"])
    close(gq, g["gq"], atol=2e-5); close(gk, g["gk"], atol=2e-5); close(gv, g["gv"], atol=2e-5)


def test_causal_carry_in_equals_unsplit():
    """Splitting the sequence and carrying (S,z) forward / (dS,dz) backward is the
    same function -- the property the sequence-sharded path relies on."""
    g = golden("causal_features")
    q, k, v, gr = (g[n].double() for n in ("q", "k", "v", "g"))
    cut = 70
    o1, S, z = O.causal_forward(q[:cut], k[:cut], v[:cut], return_state=True)
    o2 = O.causal_forward(q[cut:], k[cut:], v[cut:], s0=S, z0=z)
    full = O.causal_forward(q, k, v)
    close(torch.cat([o1, o2]), full, rtol=1e-12, atol=1e-13)
    S_seg, z_seg = O.segment_state(k[:cut], v[:cut])
    close(S_seg, S, rtol=1e-12, atol=1e-13); close(z_seg, z, rtol=1e-12, atol=1e-13)
    gq2, gk2, gv2, dS, dz = O.causal_backward(q[cut:], k[cut:], v[cut:], gr[cut:], s0=S, z0=z,
                                              return_dstate=True)
    gq1, gk1, gv1 = O.causal_backward(q[:cut], k[:cut], v[:cut], gr[:cut], ds_in=dS, dz_in=dz)
    fq, fk, fv = O.causal_backward(q, k, v, gr)
    for a, b in ((torch.cat([gq1, gq2]), fq), (torch.cat([gk1, gk2]), fk), (torch.cat([gv1, gv2]), fv)):
        close(a, b, rtol=1e-10, atol=1e-12)


def test_incremental_decoding():
    g = golden("incremental")
    a1, s1, z1 = O.incremental_rfa(g["phi_q"][:6], g["phi_k"][:6], g["v"][:6])
    close(a1, g["attn_a"]); close(z1, g["z_a"])
    a2, s2, z2 = O.incremental_rfa(g["phi_q"][6:], g["phi_k"][6:], g["v"][6:], s1, z1)
    close(a2, g["attn_b"]); close(s2, g["s_b"]); close(z2, g["z_b"])
    close(torch.cat([a1, a2]), g["attn_full"], atol=1e-5)


def test_cross_attention():
    g = golden("cross")
    s, z = O.cross_state(g["phi_k"], g["v"], g["pad"])
    close(s, g["s"]); close(z, g["z"])
    close(O.cross_query(g["phi_q"], s, z), g["attn"])
    close(O.cross_query(O.random_project(g["xq"], golden("matrices")["orf_seed1"][:2].float()), s, z),
          g["attn_module"], atol=2e-4)   # module fixture used un-rounded phi_q
    gq, gk, gv = O.cross_backward(g["phi_q"], g["phi_k"], g["v"], g["g"], g["pad"])
    close(gq, g["g_phi_q"], atol=2e-5); close(gk, g["g_phi_k"], atol=2e-5); close(gv, g["g_v"], atol=2e-5)
    assert (gk[g["pad"].T] == 0).all() and (gv[g["pad"].T] == 0).all()


def test_cross_attention_signed_denominator():
    g = golden("cross_signed")
    s, z = O.cross_state(g["phi_k"], g["v"])
    close(O.cross_query(g["phi_q"], s, z), g["attn"], atol=1e-5)
    gq, gk, gv = O.cross_backward(g["phi_q"], g["phi_k"], g["v"], g["g"])
    close(gq, g["g_phi_q"], atol=5e-5); close(gk, g["g_phi_k"], atol=5e-5); close(gv, g["g_v"], atol=5e-5)


def test_config1_cpu_case():
    """BASELINE config 1: B2 H4 T512 d64 D64 fp32, seeds 0 (inputs) / 1 (W)."""
    g = golden("config1")
    torch.manual_seed(0)
    T, B, H = 512, 2, 4
    q, k, v = torch.randn(T, B, H, 64), torch.randn(T, B, H, 64), torch.randn(T, B, H, 64)
    gup = torch.randn(T, B * H, 64)
    digest = torch.tensor([float(t.double().sum()) for t in (q, k, v, gup)], dtype=torch.float64)
    assert torch.allclose(digest, g["digest"].double(), rtol=0, atol=1e-9), "torch RNG stream differs from fixture"
    w = golden("matrices")["orf_seed1"].float()
    pq = O.random_project(q, w).view(T, B * H, 128)
    pk = O.random_project(k, w).view(T, B * H, 128)
    vv = v.view(T, B * H, 64)
    out = O.causal_forward(pq, pk, vv)
    gq, gk, gv = O.causal_backward(pq, pk, vv, gup)
    sl = slice(0, T, 16)
    close(out[sl], g["attn"], atol=2e-5); close(gq[sl], g["gq"], atol=1e-4)
    close(gk[sl], g["gk"], atol=1e-4); close(gv[sl], g["gv"], atol=1e-4)
    norms = torch.tensor([float(t.double().norm()) for t in (out, gq, gk, gv)], dtype=torch.float64)
    assert torch.allclose(norms, g["norms"].double(), rtol=1e-5)
    assert abs(float((out.double() * gup.double()).sum()) - float(g["loss"])) < 1e-3
