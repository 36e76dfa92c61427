import os
import sys

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")

# Tolerances of the parity gate for fp16 kernels against the fp32 oracle on
# identical fp16-valued inputs (outputs and every gradient).
REL_L2_TOL = 2e-3
MAX_ABS_TOL = 1e-2


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def golden(name):
    """Load tests/golden/<name>.npz as a dict of torch tensors (fp16 arrays -> fp32)."""
    out = {}
    with np.load(os.path.join(GOLDEN, name + ".npz")) as f:
        for k in f.files:
            a = f[k]
            t = torch.from_numpy(np.ascontiguousarray(a)) if a.ndim else torch.tensor(a.item())
            out[k] = t.float() if t.dtype == torch.float16 else t
    return out


@pytest.fixture(scope="session")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda:0")


PARITY_LOG = []     # (test id, what, rel-L2, max-abs, max-abs gate used, largest |reference|) of every comparison made


def assert_close(got, want, what, rel=REL_L2_TOL, mabs=MAX_ABS_TOL):
    from oracle.rfa_oracle import max_abs, rel_l2
    got = got.detach().float().cpu()
    want = want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    r, m = rel_l2(got, want), max_abs(got, want)
    # values far above 1 cannot be held to an absolute 1e-2 with fp16 operands and outputs (spacing
    # 2^-10 * magnitude, and the fp16 copy of the state is rounded once more): the absolute bound scales
    # with the largest reference magnitude once that exceeds ~5; the relative-L2 bound always binds
    plain = mabs
    mabs = max(mabs, float(want.abs().max()) * 2.0 ** -8) if want.numel() else mabs      # 8 fp16 ulps of the largest value
    PARITY_LOG.append((os.environ.get("PYTEST_CURRENT_TEST", "").split(" ")[0], what, r, m, plain, mabs,
                       float(want.abs().max()) if want.numel() else 0.0))
    assert r <= rel and m <= mabs, f"{what}: rel-L2 {r:.3e} (tol {rel}), max-abs {m:.3e} (tol {mabs})"
    return r, m


@pytest.fixture(autouse=True)
def _device_health(request):
    """After every GPU test: no bounded wait inside a tensor-core kernel may have run out."""
    yield
    if request.node.get_closest_marker("gpu") and torch.cuda.is_available():
        from rfa_b200 import _lib
        status = _lib.load().rfa_debug_status()
        assert status == 0, f"a bounded wait inside a kernel ran out (site code {status})"


def pytest_terminal_summary(terminalreporter):
    """Achieved errors of every comparison, with the plain absolute gate beside the scaled one, and a list of the
    comparisons that needed the scaled gate."""
    if not PARITY_LOG:
        return
    tr = terminalreporter
    tr.section("parity: achieved rel-L2 / max-abs per comparison")
    worst_rel = max(PARITY_LOG, key=lambda e: e[2])
    tr.write_line(f"{len(PARITY_LOG)} comparisons; worst rel-L2 {worst_rel[2]:.3e} ({worst_rel[0]} :: {worst_rel[1]})")
    over = [e for e in PARITY_LOG if e[3] > e[4]]
    tr.write_line(f"{len(over)} comparison(s) above the plain max-abs gate (they passed the gate scaled by |reference|max * 2^-8):")
    for tid, what, r, m, plain, used, big in over:
        tr.write_line(f"  {tid} :: {what}: max-abs {m:.3e} > {plain:g}; gate used {used:.3e}; largest |reference| {big:.3g}; rel-L2 {r:.3e}")
    if os.environ.get("RFA_PARITY_VERBOSE"):
        for tid, what, r, m, plain, used, big in PARITY_LOG:
            tr.write_line(f"  {tid} :: {what}: rel-L2 {r:.3e} max-abs {m:.3e}")
