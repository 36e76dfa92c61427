"""The C-ABI library loads on a machine without a GPU, exports every function the header
declares, and rejects bad arguments on the host before touching a device."""
import ctypes as C
import os
import re

import pytest

from conftest import ROOT


def header_functions():
    text = open(os.path.join(ROOT, "include", "rfa_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(rfa_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from rfa_b200 import _lib
    lib = _lib.load()
    declared = header_functions()
    assert len(declared) >= 15
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/rfa_b200.h but not exported"
    assert sorted(_lib.SIGNATURES) == declared, "ctypes signature table and header disagree"
    assert lib.rfa_version() == 100


def test_host_side_argument_checks_need_no_gpu():
    from rfa_b200 import _lib
    lib = _lib.load()
    # wrong geometry: rejected before any CUDA call
    assert lib.rfa_causal_fwd(16, 16, 16, 16, None, None, None, None, None, 0, 8, 2, 100, 64, None) == -3   # K not a multiple of 8
    assert b"multiples of 8" in lib.rfa_last_error()
    assert lib.rfa_causal_fwd(None, None, None, None, None, None, None, None, None, 0, 8, 2, 128, 64, None) == -1
    assert lib.rfa_causal_fwd(8, 16, 16, 16, None, None, None, None, None, 0, 8, 2, 128, 64, None) == -2   # misaligned q
    assert lib.rfa_decode_step(16, 16, 16, 0, 16, 16, 1, 16, 4, 128, 63, None) == -3
    assert lib.rfa_decode_step(16, 16, 16, 7, 16, 16, 1, 16, 4, 128, 64, None) == -3                      # bad dtype code
    assert lib.rfa_feature_map_fwd(16, 0, 16, 16, 0, 10, 2, 60, 64, C.c_float(0.1), None) == -3
    assert lib.rfa_cross_query_fwd(16, 16, 16, None, 10, 2, 128, 64, None) == -1
    assert lib.rfa_causal_bwd_q(16, 16, 16, 16, 16, None, None, None, None, None, 0, 8, 2, 128, 64, None) == -4  # no workspace


def test_workspace_query_is_a_pure_function_of_the_geometry():
    from rfa_b200 import _lib
    lib = _lib.load()
    a = lib.rfa_causal_workspace_bytes(2048, 128, 128, 64)
    assert a == lib.rfa_causal_workspace_bytes(2048, 128, 128, 64) and a >= 2 * 2048 * 128 * 4
    assert lib.rfa_causal_workspace_bytes(2048, 128, 100, 64) == 0          # no kernel for K % 8 != 0
    assert lib.rfa_causal_workspace_bytes(2048, 128, 96, 64) >= 2 * 2048 * 128 * 4   # generic kernels: the per-token scalars
    # few heads + long sequence -> segmented plan needs room for boundary states
    assert lib.rfa_causal_workspace_bytes(131072, 32, 128, 64) > 2 * 131072 * 32 * 4 + 32 * 2 * 128 * 65 * 4


def test_cpu_tensors_are_refused_loudly():
    import torch
    from rfa_b200 import ops
    from rfa_b200.rfa import RFA
    q = torch.zeros(4, 1, 128, dtype=torch.half)
    v = torch.zeros(4, 1, 64, dtype=torch.half)
    with pytest.raises(RuntimeError, match="no CPU path"):
        RFA.apply(q, q, v)
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.feature_map_fwd(torch.zeros(4, 1, 64), torch.zeros(1, 64, 64), 0.1)


def test_upstream_import_names_resolve():
    import rfa_b200
    rfa_b200.install_aliases()
    import random_feature_attention as up
    import rfa_cuda
    from random_feature_attention.rfa import RFA, EPS, reverse_cumsum, rfa_debug
    from random_feature_attention.causal_attention import CausalAttention, cuda_causal_rfa, incremental_rfa, masked_rfa
    from random_feature_attention.cross_attention import CrossAttention, CrossAttentionProject, CrossAttentionProjectLayer
    from random_feature_attention.utils import (CrossAttentionState, SCALE, add_rfa_args, build_random_matrices,
                                                get_rfa_attr, load_random_matrices, normalize_attn_weights,
                                                random_project, sample_random_matrices, _normalize)
    assert EPS == 1.0 and SCALE == 0.1
    assert callable(rfa_cuda.forward) and callable(rfa_cuda.backward)
    assert up.CausalAttention is CausalAttention
