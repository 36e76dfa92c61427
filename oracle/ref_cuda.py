"""Loader for upstream's own CUDA extension as built by oracle/build_ref.py.
TEST / BASELINE INFRASTRUCTURE ONLY: the product never imports this.

``load()`` returns the extension module (functions ``forward(q,k,v)`` and
``backward(q,k,v,grad_attn)``, upstream cuda/rfa_cuda.cpp:39-42) or None when
oracle/_ref/rfa_cuda_ref.so has not been built.  Upstream's kernels launch on the legacy
default stream, take fp16 contiguous CUDA tensors and check nothing; its backward needs
18 432 + 4*T bytes of shared memory without opting in, so T must stay <= 7680
(cuda/backward.cu:490-493, 567).
"""
import importlib.machinery
import importlib.util
import os

_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "rfa_cuda_ref.so")
_mod = None


def load():
    global _mod
    if _mod is not None:
        return _mod
    if not os.path.exists(_PATH):
        return None
    import torch  # noqa: F401  (libtorch must be loaded before the extension)
    loader = importlib.machinery.ExtensionFileLoader("rfa_cuda_ref", _PATH)
    spec = importlib.util.spec_from_loader("rfa_cuda_ref", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    _mod = mod
    return mod
