"""ctypes binding of libcrb_b200.so (the C ABI declared in include/crb_b200.h).

There is no fallback: if the shared library is missing or a call returns an
error, an exception is raised.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_lib", "libcrb_b200.so")

BLOCK = 128
TRACE_DOUBLES = 320
TECHNIQUES = {"braq": 0, "crbog": 1, "crb": 2, "crb_norefine": 3, "crb_symdamp": 4,
              "crb_symdamp_norefine": 5}
ORDERS_DEFAULT = 112
METRICS = {"hessian": 0, "magnitude": 1}
DTYPES = {"float32": 0, "float16": 1, "bfloat16": 2}

FLAG_NONFINITE = 1
FLAG_BAD_PIVOT = 2
FLAG_WAIT_LIMIT = 4

_vp, _i, _i64, _f, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_float, C.c_size_t

# name -> (restype, argtypes); mirrors include/crb_b200.h one to one
SIGNATURES = {
    "crb_version": (_i, []),
    "crb_arch": (C.c_char_p, []),
    "crb_status_string": (C.c_char_p, [_i]),
    "crb_hessian_workspace_bytes": (_sz, [_i, _i64, _i]),
    "crb_hessian_accumulate": (_i, [_vp, _i, _i64, _i, _i64, _vp, _vp, _sz, _vp]),
    "crb_hessian_finalize": (_i, [_vp, _i, _f, _vp]),
    "crb_hessian_packed_floats": (_sz, [_i]),
    "crb_hessian_pack": (_i, [_vp, _i, _vp, _vp]),
    "crb_hessian_unpack": (_i, [_vp, _i, _vp, _vp]),
    "crb_factor_workspace_bytes": (_sz, [_i]),
    "crb_hinv_upper_factor": (_i, [_vp, _i, _vp, _i, _i64, _f, _i, _vp, _sz, _vp, _vp]),
    "crb_block_workspace_bytes": (_sz, [_i]),
    "crb_block_step": (_i, [_vp, _i, _i64, _vp, _i64, _i, _i, _i, _f, _f, _i, _vp, _vp, _vp, _vp, _vp,
                            _vp, _sz, _vp]),
    "crb_block_step_static_max_rows": (_i, []),
    "crb_block_step_static": (_i, [_vp, _i, _i64, _vp, _i64, _i, _i, _i, _f, _f, _i, _vp, _vp, _vp, _vp, _vp,
                                   _vp, _vp]),
    "crb_binarize_group": (_i, [_vp, _i, _i64, _vp, _i64, _i, _i, _f, _f, _vp, _i64, _vp]),
    "crb_trailing_update": (_i, [_vp, _i, _i, _i64, _vp, _vp, _i64, _i, _vp]),
    "crb_gemm_f32": (_i, [_i, _i, _i, _i, _i, _f, _vp, _i64, _vp, _i64, _f, _vp, _i64, _vp, _vp]),
    "crb_linear_workspace_bytes": (_sz, [_i]),
    "crb_quantize_linear": (_i, [_vp, _i, _i, _i64, _vp, _i64, _i, _i, _f, _f, _i, _vp, _vp, _vp, _vp,
                                 _vp, _sz, _vp]),
    "crb_dequantize": (_i, [_vp, _i, _i, _i64, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp]),
    "crb_read_status": (_i, [_vp, _vp]),
    "crb_launch_count": (C.c_ulonglong, []),
    "crb_set_dependent_launch": (_i, [_i]),
    "crb_set_fused_selection": (_i, [_i]),
    "crb_set_trailing_lookahead": (_i, [_i]),
    "crb_set_factor_lookahead": (_i, [_i]),
    "crb_selftest_wait_limit": (_i, [_vp, _sz, C.c_uint, _vp, _vp]),
}

_lib = None


class CrbError(RuntimeError):
    pass


def lib():
    """The loaded library (loads it on first use)."""
    global _lib
    if _lib is None:
        path = os.environ.get("CRB_B200_LIBRARY", LIB_PATH)      # another build of the same library
        if not os.path.exists(path):
            raise CrbError(
                f"{path} is missing: build it with `python -m crb_b200.build` "
                "(there is no CPU or PyTorch fallback for the CUDA path)")
        handle = C.CDLL(path)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)       # AttributeError if the export is missing
            fn.restype, fn.argtypes = res, args
        _lib = handle
    return _lib


def orders_code(orders) -> int:
    """(low, mid, salient) expansion counts -> the decimal-digit code of the C ABI (112 = (1, 1, 2))."""
    o = tuple(int(v) for v in orders)
    if len(o) != 3 or any(v not in (1, 2) for v in o):
        raise NotImplementedError(f"orders {orders!r}: three values, each 1 or 2, are implemented")
    return 100 * o[0] + 10 * o[1] + o[2]


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().crb_status_string(rc).decode()
        raise CrbError(f"{what} failed: {msg} ({rc})")


def ptr(t):
    """Device pointer of a torch tensor (None -> NULL)."""
    return None if t is None else C.c_void_p(t.data_ptr())


def stream_ptr(stream=None):
    import torch
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)
