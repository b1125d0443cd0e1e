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


def test_shape_errors_of_the_step_operators():
    """The attention / block / decoder entry points check their shapes before touching a device: a bad call returns a
    status and a message (the reference would exit), so it can be tried without a GPU."""
    import cudalm_c_b200 as q
    L = q.lib()
    one = ctypes.c_void_p(16)                              # any non-NULL pointer; the checks come first
    cases = [
        (lambda: L.qlmb_attn_fwd(one, one, one, one, one, 1, 128, 2, 2, 32, 0, None), b"head dimension"),
        (lambda: L.qlmb_attn_fwd(one, one, one, one, one, 1, 128, 3, 2, 64, 0, None), b"bad shape"),
        (lambda: L.qlmb_attn_bwd(one, one, one, one, one, one, one, one, one, one, 1, 128, 2, 2, 128, 0, None), b"head dimension"),
        (lambda: L.qlmb_rope(one, 1, one, one, 8, 2, 63, 16, 0, None), b"qlmb_rope"),
        (lambda: L.qlmb_rmsnorm_fwd(one, 1, one, one, 1, one, 8, 30, None), b"multiple of 4"),
        (lambda: L.qlmb_gemm_nt(one, 0, one, one, 8, 100, 128, 0.0, None), b"qlmb_gemm_nt"),
        (lambda: L.qlmb_dec_attn(one, one, one, one, one, 0, 1, 8192, 2, 2, 64, None), b"qlmb_dec_attn"),
        (lambda: L.qlmb_gemv_decode_stack(one, one, one, one, 3, 100, 768, 768, 1, None), b"qlmb_gemv_decode_stack"),
        (lambda: L.qlmb_ng_touched(one, one, one, one, 8, 32, 100, 4, None), b"qlmb_ng_touched"),
        (lambda: L.qlmb_softmax_ce(one, 5, one, one, one, 0, 4, 16, 4, None), b"qlmb_softmax_ce"),
        (lambda: L.qlmb_router_bias_update(one, one, 64, 300, 2, 1, 0.001, 1, None), b"qlmb_router_bias_update"),
        (lambda: L.qlmb_router_bias_update(None, one, 64, 32, 2, 1, 0.001, 1, None), b"NULL"),
        (lambda: L.qlmb_nggate_fwd(one, one, one, one, 1, one, one, one, 8, 30, None), b"multiple of 4"),
        (lambda: L.qlmb_nggate_bwd(one, one, one, one, 7, one, one, one, one, one, 8, 32, None), b"qlmb_nggate_bwd"),
        (lambda: L.qlmb_gemv_decode_res_norm(one, one, one, one, one, one, one, 4, 768, 4096, None), b"qlmb_gemv_decode_res_norm"),
        (lambda: L.qlmb_gemv_decode_norm_stack(one, one, None, one, one, 3, 4, 768, 768, 1, None), b"qlmb_gemv_decode_norm_stack"),
        (lambda: L.qlmb_dec_qkv(one, one, one, one, one, one, one, one, one, one, 4, 768, 63, 128, None), b"qlmb_dec_qkv"),
    ]
    for call, needle in cases:
        rc = call()
        assert rc != 0
        assert needle in L.qlmb_last_error(), (needle, L.qlmb_last_error())


def test_no_fallback_when_library_missing(monkeypatch):
    import cudalm_c_b200._lib as m
    monkeypatch.setattr(m, "_lib", None)
    monkeypatch.setattr(m, "lib_path", lambda: "/nonexistent/libqlm_b200.so")
    with pytest.raises(m.QlmbError):
        m.lib()


def test_new_entry_points_reject_bad_arguments_without_a_gpu():
    """Argument checks of the entry points added for the engram table, the exact 4-bit export and the native
    communicator run before any CUDA call: status 1 and a message, nothing fatal."""
    import cudalm_c_b200 as q
    L = q.lib()
    assert L.qlmb_eg_key(None, None, None, None, None, None, 8, 4, 2, 16, None) == 1 and b"qlmb_eg_key" in L.qlmb_last_error()
    assert L.qlmb_eg_gather(None, None, None, 8, 2, 32, None) == 1
    assert L.qlmb_q4n_export(None, 0, None, None, 1024, 128, None, None) == 1
    assert L.qlmb_q4n_decode(None, None, None, 1024, 128, None) == 1
    assert L.qlmb_q4n_work_bytes(1024, 128) >= 8 * 9 + 8 * 8 and L.qlmb_q4n_max_bytes(1000, 128) == 8 * 4 + 4000
    assert L.qlmb_q4n_work_bytes(1024, 0) == 0
    assert L.qlmb_comm_init(None, None, 0, 1) == 1 and b"qlmb_comm_init" in L.qlmb_last_error()
    assert L.qlmb_comm_rank(None) == -1 and L.qlmb_comm_world(None) == 0
    assert L.qlmb_comm_destroy(None) == 0
    assert L.qlmb_selftest_stream_read(None, 256, 8, 1, None) == 1


def test_header_is_plain_c_and_links_from_c(tmp_path):
    """include/qlm_b200.h compiles as C99 with warnings as errors and a C program linked against the library runs the
    argument-error paths (status + message, no exit) on a machine without a GPU."""
    import shutil
    import subprocess
    import cudalm_c_b200
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    libdir = os.path.dirname(cudalm_c_b200.lib_path())
    exe = str(tmp_path / "probe")
    subprocess.check_call(["gcc", "-std=c99", "-Wall", "-Werror", "-pedantic", "-I", os.path.join(ROOT, "include"),
                           os.path.join(ROOT, "tests", "c_abi", "probe.c"), "-L", libdir, "-lqlm_b200", "-Wl,-rpath," + libdir, "-o", exe])
    out = subprocess.run([exe], capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stdout + out.stderr
    assert out.stdout.startswith("ok ")
