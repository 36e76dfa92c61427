"""Draw banks of random projection matrices W [n, proj_dim, head_dim]
(upstream construct_random_matrices.py).

    python -m rfa_b200.construct_random_matrices {rrf|orf} head_dim proj_dim [out.npy]

The draws consume numpy's global RNG in the same order as upstream, so the same
seed gives the same bank.  Differences from upstream: sizes are passed
explicitly instead of being read from module globals, and the output path is an
argument (default ``random_matrices/{head_dim}_{proj_dim}.npy`` next to the
package) instead of a hard-coded home directory.
"""
import os
import sys

import numpy as np

SEED = 31415            # upstream construct_random_matrices.py:77
NUM_MATRICES = 500      # upstream :79


def normal(size, mean, std):
    return np.random.normal(loc=mean, scale=std, size=size)


def rrf(*, head_dim, proj_dim):
    """Plain Gaussian features: W ~ N(0,1)^{proj_dim x head_dim}."""
    return normal(size=(proj_dim, head_dim), mean=0., std=1)


def orf(*, head_dim, proj_dim):
    """Orthogonal features: the Q factor of a Gaussian block, row i rescaled by an
    independent chi(proj_dim) draw so row norms are distributed as for ``rrf``."""
    assert proj_dim >= head_dim
    basis, _ = np.linalg.qr(normal(size=(proj_dim, head_dim), mean=0., std=1.))
    lengths = np.sqrt(np.random.chisquare(df=proj_dim, size=proj_dim))
    return basis * lengths[:, None]


def normalize(x):
    return x / np.linalg.norm(x, ord=2, axis=-1, keepdims=True)


def random_proj(q, k, random_matrix):
    """numpy feature map with the 1/sqrt(proj_dim) scale used by the quality check."""
    def phi(x):
        u = x @ random_matrix.T
        return np.concatenate([np.sin(u), np.cos(u)], axis=-1) * u.shape[-1] ** -0.5
    return phi(q), phi(k)


def test(head_dim, proj_dim, random_matrix, num_ites=100, tau=0.7, b=100):
    """Mean relative L2 error of phi(q).phi(k) e^{1/tau^2} against exp(q.k / tau^2)
    over random unit vectors; prints and returns it."""
    w = random_matrix / tau
    err = 0.
    for _ in range(num_ites):
        q = normalize(3 * (normal((b, head_dim), 0., 1.) - 0.5))
        k = normalize(10 * (normal((b, head_dim), 0., 1.) - 0.7))
        gold = np.exp(np.sum(q * k, axis=-1) / tau ** 2)
        pq, pk = random_proj(q, k, w)
        pred = np.sum(pq * pk, axis=-1) * np.exp(1. / tau ** 2)
        err += np.linalg.norm(gold - pred) / np.linalg.norm(gold)
    err /= num_ites
    print(err)
    return err


def construct_random_matrices(feature_func, num_random_matrices, *, head_dim, proj_dim):
    return np.stack([feature_func(head_dim=head_dim, proj_dim=proj_dim)
                     for _ in range(num_random_matrices)], axis=0)


def main(argv):
    if len(argv) < 4 or argv[1] not in ("rrf", "orf"):
        raise SystemExit(__doc__)
    feature_func = {"rrf": rrf, "orf": orf}[argv[1]]
    head_dim, proj_dim = int(argv[2]), int(argv[3])
    out = argv[4] if len(argv) > 4 else os.path.join(
        os.path.dirname(os.path.abspath(__file__)), "..", "random_matrices", f"{head_dim}_{proj_dim}.npy")
    np.random.seed(SEED)
    bank = construct_random_matrices(feature_func, NUM_MATRICES, head_dim=head_dim, proj_dim=proj_dim)
    os.makedirs(os.path.dirname(os.path.abspath(out)), exist_ok=True)
    np.save(out, bank)
    print(f"wrote {bank.shape} to {out}")


if __name__ == "__main__":
    main(sys.argv)
