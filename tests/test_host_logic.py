"""Host-side mirrors of upstream's Python helpers, checked on CPU against the oracle
and the upstream-generated fixtures."""
import argparse

import numpy as np
import torch

from conftest import golden
from oracle import rfa_oracle as O


def test_matrix_generators_match_upstream_bitwise():
    from rfa_b200 import construct_random_matrices as crm
    g = golden("matrices")
    np.random.seed(1)
    mine = np.stack([crm.orf(head_dim=64, proj_dim=64) for _ in range(4)])
    assert np.array_equal(mine, g["orf_seed1"].numpy())
    np.random.seed(7)
    assert np.array_equal(np.stack([crm.rrf(head_dim=64, proj_dim=64) for _ in range(2)]), g["rrf_seed7"].numpy())
    np.random.seed(11)
    assert np.array_equal(np.stack([crm.orf(head_dim=32, proj_dim=48) for _ in range(2)]), g["orf_wide_seed11"].numpy())


def test_matrix_bank_cli(tmp_path):
    from rfa_b200 import construct_random_matrices as crm
    out = tmp_path / "64_64.npy"
    crm.NUM_MATRICES, keep = 3, crm.NUM_MATRICES
    try:
        crm.main(["prog", "orf", "64", "64", str(out)])
    finally:
        crm.NUM_MATRICES = keep
    bank = np.load(out)
    assert bank.shape == (3, 64, 64)
    assert np.array_equal(bank, O.draw_matrices("orf", 3, 64, 64, 31415))
    assert crm.test(64, 64, bank[0].copy(), num_ites=5) < 0.5     # kernel approximation quality is sane


def test_torch_twins_match_oracle():
    from rfa_b200.rfa import RFA, reverse_cumsum, rfa_debug
    g = golden("causal_bwd_gradcheck")
    q, k, v, up = g["q"], g["k"], g["v"], g["g"]
    assert torch.allclose(RFA.forward_torch(q, k, v), g["attn"], atol=2e-6)
    assert torch.allclose(rfa_debug(q, k, v), g["attn"], atol=2e-6)
    for a, b in zip(RFA.backward_torch(q, k, v, up), (g["gq"], g["gk"], g["gv"])):
        assert torch.allclose(a, b, atol=1e-5)
    x = torch.arange(12.).view(3, 4)
    assert torch.equal(reverse_cumsum(x, 0), torch.flip(torch.cumsum(torch.flip(x, [0]), 0), [0]))


def test_utils_helpers():
    from rfa_b200 import utils
    g = golden("feature_map")
    w = utils.build_random_matrices(g["w"], float(g["tau"]), g["sigma"], True)
    assert torch.allclose(w, g["w_eff"], rtol=1e-6)
    assert torch.equal(utils.build_random_matrices(g["w"], 1.0), g["w"])
    xn, n = utils._normalize(g["x"])
    assert torch.allclose(xn, g["x"] / (g["x"].norm(dim=-1, keepdim=True) + 1e-3))
    bank = torch.arange(10 * 2 * 3.).view(10, 2, 3)
    ev = utils.sample_random_matrices(num_layers=3, num_heads=2, random_matrices=bank, is_training=False)
    assert torch.equal(ev, bank[:2])
    np.random.seed(0)
    tr = utils.sample_random_matrices(num_layers=3, num_heads=2, random_matrices=bank, is_training=True)
    np.random.seed(0)
    idx = np.random.choice(10, size=6, replace=False)
    assert len(tr) == 3 and all(torch.equal(tr[i], bank[idx[2 * i:2 * i + 2]]) for i in range(3))
    p = utils.add_rfa_args(argparse.ArgumentParser())
    a = utils.get_rfa_attr(p.parse_args(["--use-rfa", "--causal-proj-dim", "32"]))
    assert a.use_rfa and a.use_linfa and a.causal_proj_dim == 32 and a.cross_tau is None
    a = utils.get_rfa_attr(argparse.Namespace())
    assert (a.cross_proj_dim, a.causal_tau, a.reparam_proj, a.cuda_causal_rfa) == (64, 1.0, True, True)
    wts = utils.normalize_attn_weights(torch.tensor([[1., 3.], [0., 0.]]))
    assert torch.allclose(wts, torch.tensor([[.25, .75], [0., 0.]]))
    st = utils.CrossAttentionState(torch.zeros(1), torch.zeros(1), [], 1.0)
    assert st.tau == 1.0 and st._fields == ("s", "z", "random_matrices", "tau")


def test_masked_rfa_is_upstreams_quadratic_variant():
    from rfa_b200.causal_attention import masked_rfa
    gen = torch.Generator().manual_seed(0)
    T, B, H = 12, 2, 2
    pq, pk = torch.rand(T, B, H, 16, generator=gen), torch.rand(T, B, H, 16, generator=gen)
    v = torch.randn(T, B, H, 8, generator=gen)
    causal = torch.triu(torch.full((T, T), float("-inf")), 1)
    out = masked_rfa(phi_q=pq, phi_k=pk, v=v, attn_mask=causal)
    # with positive features every row sum exceeds 1e-3, so this equals sum-normalised causal attention
    a = torch.einsum("tbhk,sbhk->bhts", pq, pk) * torch.tril(torch.ones(T, T))
    ref = torch.einsum("bhts,sbhd->tbhd", a / a.sum(-1, keepdim=True), v).reshape(T, B, H * 8)
    assert torch.allclose(out, ref, atol=1e-5)


def test_cpu_list_parsing_for_numa_binding():
    from rfa_b200.host_pipeline import _cpulist, gpu_numa_cpus
    assert _cpulist("0-3,8,10-11\n") == [0, 1, 2, 3, 8, 10, 11]
    assert _cpulist("") == []
    assert gpu_numa_cpus(0, sysfs="/nonexistent") is None       # no GPU / no sysfs entry: nothing to bind to


def test_matrix_sampling_with_a_generator_is_reproducible():
    from rfa_b200.utils import sample_matrix_indices, sample_random_matrices
    mk = lambda: torch.Generator().manual_seed(7)
    a = sample_matrix_indices(num_layers=3, num_heads=4, bank_size=50, generator=mk())
    b = sample_matrix_indices(num_layers=3, num_heads=4, bank_size=50, generator=mk())
    assert torch.equal(a, b) and a.numel() == 12 and len(set(a.tolist())) == 12 and int(a.max()) < 50
    bank = torch.arange(50.).view(50, 1, 1).expand(50, 2, 3).contiguous()
    layers = sample_random_matrices(num_layers=3, num_heads=4, random_matrices=bank, generator=mk())
    assert len(layers) == 3 and torch.equal(torch.cat(layers)[:, 0, 0].long(), a)
    import numpy as np
    np.random.seed(3)
    x = sample_matrix_indices(num_layers=2, num_heads=2, bank_size=9)        # upstream's way: numpy's global RNG
    np.random.seed(3)
    assert x.tolist() == np.random.choice(9, size=4, replace=False).tolist()
