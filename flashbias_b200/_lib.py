"""ctypes binding of libflashbias_b200.so (the C ABI declared in include/flashbias_b200.h).

The library is the only compute path of the package: if it is missing, loading raises and
every operator fails loudly.  There is no CPU or eager fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libflashbias_b200.so")

FB_DTYPE_F16, FB_DTYPE_BF16, FB_DTYPE_F32 = 0, 1, 2
FB_MASK_NONE, FB_MASK_VECTOR, FB_MASK_MATRIX = 0, 1, 2
FB_FLAG_FORCE_GENERAL = 1
FB_FLAG_BWD_QUERY_MAJOR = 2
FB_FLAG_BWD_ONE_ITEM = 4
FB_FLAG_BWD_PERSISTENT = 8

I64x3 = C.c_int64 * 3


class FbParams(C.Structure):
    """Mirror of ``struct fb_params``; field order and types must match the header."""
    _fields_ = [
        ("B", C.c_int32), ("H", C.c_int32), ("Sq", C.c_int32), ("Sk", C.c_int32), ("D", C.c_int32), ("R", C.c_int32),
        ("dtype", C.c_int32), ("causal", C.c_int32), ("mask_kind", C.c_int32), ("mask_dtype", C.c_int32),
        ("flags", C.c_int32), ("softmax_scale", C.c_float),
        ("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p),
        ("q_bias", C.c_void_p), ("k_bias", C.c_void_p), ("mask", C.c_void_p),
        ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3),
        ("q_bias_stride", I64x3), ("k_bias_stride", I64x3), ("mask_stride", I64x3),
        ("o", C.c_void_p), ("o_stride", I64x3),
        ("lse", C.c_void_p), ("lse_stride_bh", C.c_int64),
        ("dout", C.c_void_p), ("dout_stride", I64x3),
        ("delta", C.c_void_p),
        ("dq", C.c_void_p), ("dk", C.c_void_p), ("dv", C.c_void_p), ("dq_bias", C.c_void_p), ("dk_bias", C.c_void_p),
        ("dq_stride", I64x3), ("dk_stride", I64x3), ("dv_stride", I64x3),
        ("dq_bias_stride", I64x3), ("dk_bias_stride", I64x3),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
        ("status", C.c_void_p),
        ("alibi_slopes", C.c_void_p),
        ("mask_batch_period", C.c_int32),
    ]


EXPORTS = {
    "fb_version": (C.c_int, []),
    "fb_params_size": (C.c_size_t, []),
    "fb_strerror": (C.c_char_p, [C.c_int]),
    "fb_fwd_uses_tensor_path": (C.c_int, [C.POINTER(FbParams)]),
    "fb_bwd_uses_tensor_path": (C.c_int, [C.POINTER(FbParams)]),
    "fb_fwd_workspace_bytes": (C.c_size_t, [C.POINTER(FbParams)]),
    "fb_fwd": (C.c_int, [C.POINTER(FbParams), C.c_void_p]),
    "fb_fwd_noalloc": (C.c_int, [C.POINTER(FbParams), C.c_void_p]),
    "fb_fwd_noalloc_capacity": (C.c_size_t, []),
    "fb_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(FbParams)]),
    "fb_bwd_preprocess": (C.c_int, [C.POINTER(FbParams), C.c_void_p]),
    "fb_bwd": (C.c_int, [C.POINTER(FbParams), C.c_void_p]),
    "fb_read_status": (C.c_int, [C.c_void_p, C.POINTER(C.c_int32), C.c_void_p]),
    "fb_status_string": (C.c_char_p, [C.c_int32]),
    "fb_prepare_rows": (C.c_int, [C.c_void_p, C.c_int32, C.POINTER(C.c_int64), C.c_void_p, C.c_int32,
                                  C.POINTER(C.c_int64), C.c_int32, C.c_int32, C.c_int32, C.c_int32, C.c_int32,
                                  C.c_void_p, C.c_float, C.c_void_p]),
    "fb_launch_count": (C.c_longlong, []),
    "fb_prof_begin": (C.c_int, [C.c_int]),
    "fb_prof_end": (C.c_int, [C.POINTER(C.c_float), C.POINTER(C.c_int)]),
    "fb_selftest_count": (C.c_int, []),
    "fb_selftest_info": (C.c_int, [C.c_int] + [C.POINTER(C.c_int32)] * 7),
    "fb_selftest_run": (C.c_int, [C.c_int, C.c_int32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
}

_lock = threading.Lock()
_lib = None


def load() -> C.CDLL:
    """Load the shared library once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python -m flashbias_b200.build` "
                    "(needs nvcc; there is no fallback path)")
            lib = C.CDLL(LIB_PATH)
            for name, (res, args) in EXPORTS.items():
                fn = getattr(lib, name)  # AttributeError if the symbol is not exported
                fn.restype = res
                fn.argtypes = args
            if lib.fb_params_size() != C.sizeof(FbParams):
                raise RuntimeError("fb_params layout mismatch between the Python binding and the built library")
            _lib = lib
    return _lib


def strerror(code: int) -> str:
    return load().fb_strerror(code).decode()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed: [{code}] {strerror(code)}")
