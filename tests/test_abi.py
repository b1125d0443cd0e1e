"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

import pytest

from conftest import ROOT


def header_symbols():
    text = open(os.path.join(ROOT, "include", "qlm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qlmb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    syms = header_symbols()
    for must in ("qlmb_encode", "qlmb_step", "qlmb_linear_fwd", "qlmb_moe_forward", "qlmb_gemv_decode"):
        assert must in syms


def test_library_exports_every_declared_symbol():
    import cudalm_c_b200
    from cudalm_c_b200._lib import PROTOTYPES
    L = ctypes.CDLL(cudalm_c_b200.lib_path())
    for name in header_symbols():
        assert hasattr(L, name), "missing export " + name
        assert name in PROTOTYPES, "no ctypes prototype for " + name
    assert cudalm_c_b200.lib().qlmb_version() >= 1


def test_argument_errors_are_reported_not_fatal():
    import cudalm_c_b200 as q
    L = q.lib()
    rc = L.qlmb_encode(None, None, None, None, None, 0, 0, 128, 7, 1, None)
    assert rc == 1
    assert b"qlmb_encode" in L.qlmb_last_error()
    with pytest.raises(q.QlmbError):
        q.check(rc)


def test_no_fallback_when_library_missing(monkeypatch):
    import cudalm_c_b200._lib as m
    monkeypatch.setattr(m, "_lib", None)
    monkeypatch.setattr(m, "lib_path", lambda: "/nonexistent/libqlm_b200.so")
    with pytest.raises(m.QlmbError):
        m.lib()
