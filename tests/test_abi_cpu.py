"""The C-ABI library loads, exports every symbol the public header declares, and rejects bad
arguments on the host before touching a device (no compute calls here)."""
import ctypes as C
import os
import re

import pytest

from flashbias_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "flashbias_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fb_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _declared_functions()
    assert "fb_fwd" in names and "fb_bwd" in names and "fb_bwd_preprocess" in names
    for n in names:
        assert hasattr(lib, n), f"{n} declared in the header but not exported"
    assert set(names) == set(_lib.EXPORTS), "binding table and header disagree"


def test_struct_mirror_matches():
    assert _lib.load().fb_params_size() == C.sizeof(_lib.FbParams)


def _valid_params():
    p = _lib.FbParams()
    p.B, p.H, p.Sq, p.Sk, p.D, p.R = 1, 2, 128, 128, 32, 0
    p.dtype = _lib.FB_DTYPE_BF16
    p.softmax_scale = 0.25
    for name in ("q", "k", "v", "o", "lse"):
        setattr(p, name, 0x1000)  # never dereferenced on the host
    for name in ("q_stride", "k_stride", "v_stride", "o_stride"):
        setattr(p, name, _lib.I64x3(128 * 64, 32, 64))
    p.lse_stride_bh = 128
    return p


@pytest.mark.parametrize("mutate,code", [
    (lambda p: setattr(p, "q", None), -1),
    (lambda p: setattr(p, "D", 129), -2),
    (lambda p: setattr(p, "Sq", 0), -2),
    (lambda p: setattr(p, "dtype", 2), -3),
    (lambda p: setattr(p, "q_stride", _lib.I64x3(-1, 32, 64)), -4),
    (lambda p: setattr(p, "mask_kind", 1), -5),
    (lambda p: setattr(p, "R", 4), -7),
    (lambda p: setattr(p, "lse_stride_bh", 64), -8),
])
def test_host_side_validation(mutate, code):
    lib = _lib.load()
    p = _valid_params()
    mutate(p)
    assert lib.fb_fwd(C.byref(p), None) == code
    assert _lib.strerror(code)


def test_backward_requires_gradient_buffers():
    lib = _lib.load()
    p = _valid_params()
    assert lib.fb_bwd(C.byref(p), None) == -1
    assert lib.fb_bwd_preprocess(C.byref(p), None) == -1


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", "/nonexistent/libflashbias_b200.so")
    with pytest.raises(RuntimeError, match="no fallback"):
        _lib.load()
