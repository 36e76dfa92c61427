"""Generate the golden fixtures in this directory from the upstream Python sources.

Run once, in a container that has the upstream checkout (set ``RFA_REFERENCE`` to its
``random_feature_attention`` directory if it is not at the default location):

    python tests/golden/make_golden.py

The upstream package does not import as shipped, so its modules are loaded one
file at a time, unmodified, with four small accommodations: (1) a synthetic
parent package so ``__init__.py`` (which imports files that were never
published) is not executed; (2) ``typing.NamedTuple`` made visible to
``utils.py``, which uses it without importing it; (3) a no-op
``upgrade_state_dict_named`` attribute on ``utils``, which two modules import
but nothing defines; (4) a stand-in ``rfa_cuda`` module so ``rfa.py`` imports
without the CUDA extension; its ``forward``/``backward`` are bound to upstream's own
fp32 twins ``RFA.forward_torch``/``RFA.backward_torch`` so that the module-level
fixture can run ``CausalAttention`` end to end.  Only pure-PyTorch code runs.

All inputs are rounded to fp16-representable values (stored as fp16) so that the
fp16 CUDA kernels and the fp32 oracle see identical numbers; outputs are what the
upstream fp32 code returns on those inputs.
"""

import importlib.util
import os
import sys
import types
import typing

import numpy as np
import torch

OUT = os.path.dirname(os.path.abspath(__file__))
# the upstream package directory: RFA_REFERENCE, or a checkout named "reference" beside this repository
REF = os.environ.get("RFA_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(OUT))), "reference",
                                                      "random_feature_attention")


def load_upstream():
    pkg = types.ModuleType("random_feature_attention")
    pkg.__path__ = [REF]
    sys.modules["random_feature_attention"] = pkg
    sys.modules["rfa_cuda"] = types.ModuleType("rfa_cuda")

    def load(name, pre=None):
        full = f"random_feature_attention.{name}"
        spec = importlib.util.spec_from_file_location(full, os.path.join(REF, f"{name}.py"))
        mod = importlib.util.module_from_spec(spec)
        sys.modules[full] = mod
        if pre:
            pre(mod)
        spec.loader.exec_module(mod)
        setattr(pkg, name, mod)
        return mod

    utils = load("utils", pre=lambda m: setattr(m, "NamedTuple", typing.NamedTuple))
    utils.upgrade_state_dict_named = lambda *a, **k: None
    rfa = load("rfa")
    sys.modules["rfa_cuda"].forward = rfa.RFA.forward_torch
    sys.modules["rfa_cuda"].backward = lambda q, k, v, g: list(rfa.RFA.backward_torch(q, k, v, g))
    causal = load("causal_attention")
    cross = load("cross_attention")
    crm = load("construct_random_matrices")
    return utils, rfa, causal, cross, crm


def h(x):
    """Round to fp16-representable values, keep fp32 dtype."""
    return x.half().float()


def save(name, **arrs):
    out = {}
    for k, v in arrs.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = v
    path = os.path.join(OUT, name + ".npz")
    np.savez_compressed(path, **out)
    print(f"{name}: {os.path.getsize(path) / 1024:.1f} KiB")


def main():
    utils, rfa, causal, cross, crm = load_upstream()
    RFA = rfa.RFA
    torch.set_num_threads(8)

    # --- W: the upstream orf/rrf generators (construct_random_matrices.py:10-21)
    np.random.seed(1)
    w_orf = np.stack([crm.orf(head_dim=64, proj_dim=64) for _ in range(4)], 0)
    np.random.seed(7)
    w_rrf = np.stack([crm.rrf(head_dim=64, proj_dim=64) for _ in range(2)], 0)
    np.random.seed(11)
    w_orf_wide = np.stack([crm.orf(head_dim=32, proj_dim=48) for _ in range(2)], 0)
    save("matrices", orf_seed1=w_orf, rrf_seed7=w_rrf, orf_wide_seed11=w_orf_wide)

    # --- feature map (utils.py:90-120), with and without the sigma reparam
    torch.manual_seed(10)
    x = h(torch.randn(24, 2, 4, 64) * 1.7)
    w = torch.tensor(w_orf, dtype=torch.float32)
    sigma = h(1.0 + 0.25 * torch.randn(4, 1, 64))
    w_eff = utils.build_random_matrices(w, 0.8, sigma, True)
    x_ = x.clone().requires_grad_(True)
    w_ = w_eff.clone().requires_grad_(True)
    phi = utils.random_project(x=x_, random_matrices=w_)
    g_phi = h(torch.randn_like(phi))
    (phi * g_phi).sum().backward()
    phi_plain = utils.random_project(x=x, random_matrices=w)
    save("feature_map", x=x.half(), w=w_orf.astype(np.float32), sigma=sigma.half(), tau=np.float32(0.8),
         w_eff=w_eff, phi=phi, g_phi=g_phi.half(), g_x=x_.grad, g_w=w_.grad, phi_plain=phi_plain)

    # --- causal forward, the shapes of grad_check.py:17-28 (seed 3, T=50, rand-0.5)
    torch.manual_seed(3)
    q = h(torch.rand(50, 1, 128) - .5)
    k = h(torch.rand(50, 1, 128) - .5)
    v = h(torch.rand(50, 1, 64) - .5)
    save("causal_fwd_gradcheck", q=q.half(), k=k.half(), v=v.half(),
         attn=RFA.forward_torch(q, k, v), attn_debug=rfa.rfa_debug(q, k, v))

    # --- causal backward, the shapes of grad_check.py:31-50 (bsz 5, T=100, unit rows)
    torch.manual_seed(3)
    nz = lambda t: t / t.norm(p=2, dim=-1, keepdim=True)
    q = h(nz(torch.rand(100, 5, 128) - .5))
    k = h(nz(torch.rand(100, 5, 128) - .5))
    v = h(nz(torch.rand(100, 5, 64) - .5))
    g = h(nz(torch.rand(100, 5, 64)))
    gq, gk, gv = RFA.backward_torch(q, k, v, g)
    save("causal_bwd_gradcheck", q=q.half(), k=k.half(), v=v.half(), g=g.half(),
         attn=RFA.forward_torch(q, k, v), gq=gq, gk=gk, gv=gv)

    # --- causal fwd+bwd on real features: both clamp branches are live (qz crosses 1)
    torch.manual_seed(5)
    T, B, H = 160, 1, 2
    xq, xk = h(torch.randn(T, B, H, 64)), h(torch.randn(T, B, H, 64))
    pq = h(utils.random_project(x=xq, random_matrices=w[:2])).view(T, B * H, 128)
    pk = h(utils.random_project(x=xk, random_matrices=w[:2])).view(T, B * H, 128)
    v = h(torch.randn(T, B * H, 64))
    g = h(torch.randn(T, B * H, 64))
    attn = RFA.forward_torch(pq, pk, v)
    gq, gk, gv = RFA.backward_torch(pq, pk, v, g)
    qz = torch.einsum("tbk,tbk->tb", pq, torch.cumsum(pk, 0))
    assert (qz > 1).any() and (qz < 1).any()
    save("causal_features", q=pq.half(), k=pk.half(), v=v.half(), g=g.half(),
         attn=attn, gq=gq, gk=gk, gv=gv, qz=qz)

    # --- incremental decoding (causal_attention.py:17-54): 6 tokens, then 3 more with state
    torch.manual_seed(6)
    T, B, H = 9, 2, 2
    pq = h(utils.random_project(x=h(torch.randn(T, B, H, 64)), random_matrices=w[:2]))
    pk = h(utils.random_project(x=h(torch.randn(T, B, H, 64)), random_matrices=w[:2]))
    v = h(torch.randn(T, B, H, 64))
    a1, s1, z1 = causal.incremental_rfa(phi_q=pq[:6], phi_k=pk[:6], v=v[:6])
    a2, s2, z2 = causal.incremental_rfa(phi_q=pq[6:], phi_k=pk[6:], v=v[6:], s=s1, z=z1)
    full = RFA.forward_torch(pq.view(T, B * H, 128), pk.view(T, B * H, 128), v.view(T, B * H, 64))
    save("incremental", phi_q=pq.half(), phi_k=pk.half(), v=v.half(), attn_a=a1, z_a=z1,
         attn_b=a2, s_b=s2, z_b=z2, attn_full=full.view(T, B, H * 64))

    # --- cross attention (cross_attention.py:97-104, :254-270) with ragged key lengths
    torch.manual_seed(8)
    Ts, Tq, B, H = 37, 21, 3, 2
    w2 = w[:2]
    lens = torch.tensor([37, 20, 5])
    pad = torch.arange(Ts)[None, :] >= lens[:, None]                  # [B,Ts] True = pad
    xq = h(torch.randn(Tq, B, H, 64))
    pk0 = h(utils.random_project(x=h(torch.randn(Ts, B, H, 64)), random_matrices=w2))
    v = h(torch.randn(Ts, B, H, 64))
    g = h(torch.randn(Tq, B, H, 64))
    pk_ = pk0.clone().requires_grad_(True)
    v_ = v.clone().requires_grad_(True)
    pkm = pk_.masked_fill(pad.transpose(0, 1)[:, :, None, None], 0.0)     # :97-100
    s = torch.einsum("sbhk,sbhd->bhkd", pkm, v_)                         # :103
    z = torch.sum(pkm, dim=0)                                            # :104
    pq_ = h(utils.random_project(x=xq, random_matrices=w2)).requires_grad_(True)
    qs = torch.einsum("tbhk,bhkd->tbhd", pq_, s)                         # :266
    qz = torch.einsum("tbhk,bhk->tbh", pq_, z).abs().clamp_min(utils.EPS)  # :267
    attn = qs / qz.unsqueeze(-1)                                         # :269
    (attn * g).sum().backward()
    # the same through the module method itself (no Linear layers involved in .rfa)
    ca = cross.CrossAttention(embed_dim=128, num_heads=2, head_dim=64, proj_dim=64)
    attn_mod = ca.rfa(xq, s.detach(), z.detach(), w2)
    save("cross", xq=xq.half(), phi_q=pq_.detach().half(), phi_k=pk0.half(), v=v.half(), g=g.half(),
         pad=pad.numpy(), s=s, z=z, attn=attn, attn_module=attn_mod,
         g_phi_q=pq_.grad, g_phi_k=pk_.grad, g_v=v_.grad)

    # --- cross attention where phi_q.z goes negative (abs / sign branch)
    torch.manual_seed(9)
    pq = h(torch.randn(16, 2, 2, 128) * 0.3).requires_grad_(True)
    pk = h(torch.randn(12, 2, 2, 128) * 0.6).requires_grad_(True)
    v = h(torch.randn(12, 2, 2, 64)).requires_grad_(True)
    g = h(torch.randn(16, 2, 2, 64))
    s = torch.einsum("sbhk,sbhd->bhkd", pk, v)
    z = pk.sum(0)
    raw = torch.einsum("tbhk,bhk->tbh", pq, z)
    assert (raw < -1).any() and (raw > 1).any() and (raw.abs() < 1).any()
    attn = torch.einsum("tbhk,bhkd->tbhd", pq, s) / raw.abs().clamp_min(utils.EPS).unsqueeze(-1)
    (attn * g).sum().backward()
    save("cross_signed", phi_q=pq.detach().half(), phi_k=pk.detach().half(), v=v.detach().half(),
         g=g.half(), attn=attn, g_phi_q=pq.grad, g_phi_k=pk.grad, g_v=v.grad, raw=raw)

    # --- whole modules (projection weights included), fp32: CausalAttention in its
    #     teacher-forced and incremental modes, CrossAttentionProjectLayer + CrossAttention
    torch.manual_seed(12)
    E, H = 128, 2
    wm = torch.tensor(w_orf[:2], dtype=torch.float32)
    mod = causal.CausalAttention(embed_dim=E, num_heads=H, head_dim=64, proj_dim=64, tau=0.9)
    with torch.no_grad():
        mod.sigma.copy_(1.0 + 0.1 * torch.randn_like(mod.sigma))
        for p in mod.parameters():
            p.copy_(h(p))
    x = h(torch.randn(33, 2, E))
    kpm = torch.zeros(2, 33, dtype=torch.bool)
    kpm[1, 25:] = True
    y = mod(x, wm, key_padding_mask=kpm)
    st = {}
    ys = [mod(x[i:i + 1], wm, saved_state=st) for i in range(4)]
    sd = {"causal." + k_: v_ for k_, v_ in mod.state_dict().items()}
    layer = cross.CrossAttentionProjectLayer(embed_dim=E, num_heads=H, head_dim=64, proj_dim=64, tau=1.1)
    dec = cross.CrossAttention(embed_dim=E, num_heads=H, head_dim=64, proj_dim=64, tau=1.1)
    with torch.no_grad():
        for m_ in (layer, dec):
            for p in m_.parameters():
                p.copy_(h(p))
    enc = h(torch.randn(19, 2, E))
    emask = torch.zeros(19, 2, 1, 1, dtype=torch.bool)
    emask[11:, 0] = True
    state = layer(encoder_output=enc, random_matrices=wm, mask=emask)
    torch.manual_seed(13)
    query = h(torch.randn(7, 2, E))
    yq = dec(query, state)
    sd.update({"xlayer." + k_: v_ for k_, v_ in layer.state_dict().items()})
    sd.update({"xdec." + k_: v_ for k_, v_ in dec.state_dict().items()})
    save("modules", w=wm, x=x, kpm=kpm.numpy(), y=y, y_inc=torch.cat(ys, 0),
         prev_s=st["prev_s"], prev_z=st["prev_z"], enc=enc, emask=emask.numpy(),
         xs=state.s, xz=state.z, xw=state.random_matrices, query=query, yq=yq, **sd)

    # --- BASELINE config 1 (B2 H4 T512 d64 D64 fp32, seeds 0/1): inputs are regenerated from
    #     the seeds by the tests; stored are a digest of the inputs and a strided sample of outputs
    torch.manual_seed(0)
    T, B, H = 512, 2, 4
    q, k, v = torch.randn(T, B, H, 64), torch.randn(T, B, H, 64), torch.randn(T, B, H, 64)
    gup = torch.randn(T, B * H, 64)
    pq = utils.random_project(x=q, random_matrices=w).view(T, B * H, 128)
    pk = utils.random_project(x=k, random_matrices=w).view(T, B * H, 128)
    vv = v.view(T, B * H, 64)
    attn = RFA.forward_torch(pq, pk, vv)
    gq, gk, gv = RFA.backward_torch(pq, pk, vv, gup)
    sl = slice(0, T, 16)
    save("config1", digest=np.array([float(q.double().sum()), float(k.double().sum()),
                                      float(v.double().sum()), float(gup.double().sum())]),
         attn=attn[sl], gq=gq[sl], gk=gk[sl], gv=gv[sl],
         loss=np.float64((attn.double() * gup.double()).sum()),
         norms=np.array([float(t.double().norm()) for t in (attn, gq, gk, gv)]))


if __name__ == "__main__":
    main()
