"""ctypes binding of ``librfa_b200.so`` (the C ABI declared in ``include/rfa_b200.h``).

The library is the only compute path of this package: if it cannot be loaded
the import fails with an error that says how to build it.  Nothing here falls
back to PyTorch ops.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "librfa_b200.so")

RFA_F16, RFA_F32 = 0, 1
WS_EMPTY, WS_PARTIALS, WS_STATES, WS_DEN = 0, 1, 2, 4      # what a kept workspace holds (include/rfa_b200.h)
_DTYPE_CODE = {torch.float16: RFA_F16, torch.float32: RFA_F32}

_i64, _int, _f32, _vp, _sz = C.c_int64, C.c_int, C.c_float, C.c_void_p, C.c_size_t

# name -> (restype, argtypes); mirrors include/rfa_b200.h one to one
SIGNATURES = {
    "rfa_version": (_int, []),
    "rfa_last_error": (C.c_char_p, []),
    "rfa_debug_status": (_int, []),
    "rfa_status_mirror_enable": (_int, []),
    "rfa_status_peek": (_int, []),
    "rfa_feature_map_fwd": (_int, [_vp, _int, _vp, _vp, _int, _i64, _int, _int, _int, _f32, _vp]),
    "rfa_feature_map_bwd": (_int, [_vp, _int, _vp, _vp, _int, _vp, _int, _vp, _i64, _int, _int, _int, _f32, _vp]),
    "rfa_feature_map_fwd_pair": (_int, [_vp] * 7 + [_i64, _int, _int, _int, _f32, _vp]),
    "rfa_feature_map_bwd_pair": (_int, [_vp] * 10 + [_i64, _int, _int, _int, _f32, _vp]),
    "rfa_feature_map_fwd_masked": (_int, [_vp, _int, _vp, _vp, _vp, _int, _i64, _int, _int, _int, _f32, _vp]),
    "rfa_feature_map_bwd_masked": (_int, [_vp, _int, _vp, _vp, _vp, _int, _vp, _int, _vp, _i64, _int, _int, _int, _f32, _vp]),
    "rfa_gather_random_matrices": (_int, [_vp, _int, _i64, _vp, _i64, _vp, _vp, _vp, _int, _int, _vp, _vp]),
    "rfa_causal_workspace_bytes": (_sz, [_i64, _int, _int, _int]),
    "rfa_causal_fwd": (_int, [_vp] * 4 + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _vp]),
    "rfa_causal_bwd": (_int, [_vp] * 4 + [_vp] * 3 + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _vp]),
    "rfa_causal_bwd_q": (_int, [_vp] * 4 + [_vp] + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _vp]),
    "rfa_causal_bwd_kv": (_int, [_vp] * 4 + [_vp] * 2 + [_vp] * 2 + [_vp, _sz, _i64, _int, _int, _int, _vp]),
    "rfa_causal_fwd_staged": (_int, [_vp] * 4 + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _int, _int, _vp]),
    "rfa_causal_fwd_fused": (_int, [_vp] * 3 + [_vp, _vp, _f32, _vp] + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _int, _int, _vp]),
    "rfa_causal_shard_total": (_int, [_vp] * 3 + [_vp, _sz, _i64, _int, _int, _int, _vp]),
    "rfa_exclusive_scan_gathered": (_int, [_vp, _int, _int, _int, _vp, _vp, _int, _int, _int, _vp]),
    "rfa_causal_bwd_q_staged": (_int, [_vp] * 6 + [_vp] * 3 + [_vp, _sz, _i64, _int, _int, _int, _int, _vp]),
    "rfa_causal_bwd_saved": (_int, [_vp] * 8 + [_vp] * 4 + [_vp, _sz, _i64, _int, _int, _int, _int, _vp]),
    "rfa_causal_bwd_noalloc_max_token_heads": (_i64, []),
    "rfa_causal_bwd_noalloc": (_int, [_vp] * 4 + [_vp] * 3 + [_i64, _int, _int, _int, _vp]),
    "rfa_cross_state_fwd": (_int, [_vp] * 5 + [_i64, _int, _int, _int, _int, _vp]),
    "rfa_state_partials_run_length": (_i64, [_i64, _int]),
    "rfa_state_partials": (_int, [_vp] * 4 + [_i64, _int, _int, _int, _int, _vp]),
    "rfa_cross_state_bwd": (_int, [_vp] * 7 + [_i64, _int, _int, _int, _int, _vp]),
    "rfa_cross_query_fwd": (_int, [_vp] * 4 + [_i64, _int, _int, _int, _vp]),
    "rfa_cross_query_bwd": (_int, [_vp] * 7 + [_i64, _int, _int, _int, _vp]),
    "rfa_decode_step": (_int, [_vp, _vp, _vp, _int, _vp, _vp, _int, _vp, _int, _int, _int, _vp]),
    "rfa_stream_probe": (_int, [_vp, _vp, _i64, _int, _int, _int, _vp]),
    "rfa_cross_decode_step": (_int, [_vp, _int, _vp, _vp, _vp, _int, _int, _int, _int, _vp]),
    "rfa_decode_step_fused": (_int, [_vp, _vp, _vp, _int, _vp, _f32, _vp, _vp, _int, _vp, _int, _int, _int, _int, _vp]),
}

_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the shared library once; raise loudly if it is absent."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing. rfa_b200 has no fallback path: build the CUDA library with "
            "`python -m rfa_b200.build` (needs nvcc; cross-compiles for sm_100a without a GPU).")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)       # AttributeError here = header and library disagree
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def last_error() -> str:
    return load().rfa_last_error().decode("utf-8", "replace")


_mirrored = set()


def watch_device(index: int) -> None:
    """Once per device (with that device current): have the kernels mirror a bounded wait that ran out into a word of
    mapped host memory, which ``check`` looks at after every call."""
    if index in _mirrored:
        return
    status = load().rfa_status_mirror_enable()
    if status != 0:
        raise RuntimeError(f"rfa_status_mirror_enable failed with status {status}: {last_error()}")
    _mirrored.add(index)


def check(status: int, what: str) -> None:
    if status == 0:
        code = load().rfa_status_peek()         # a plain host read: no synchronisation
        if code:
            load().rfa_debug_status()           # synchronise and clear, so that the error is reported once
            raise RuntimeError(
                f"rfa_b200: a bounded wait inside a kernel launched before or by {what} ran out (site code {code}); "
                "results computed since are invalid")
        return
    msg = f"{what} failed with status {status}: {last_error()}"
    if status < 0 and status != -5:
        raise ValueError(msg)
    raise RuntimeError(msg)


def ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise RuntimeError("rfa_b200 kernels take CUDA tensors only (there is no CPU path); got a "
                           f"{t.device} tensor")
    if not t.is_contiguous():
        raise ValueError("rfa_b200: tensor must be contiguous")
    return t.data_ptr()


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise TypeError(f"rfa_b200: unsupported dtype {t.dtype} (fp16 and fp32 only)") from None


def stream_of(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def require_half(*ts: torch.Tensor) -> None:
    for t in ts:
        if t.dtype != torch.float16:
            raise TypeError(f"rfa_b200: this kernel is fp16-only, got {t.dtype}")
