"""QLMH optimizer-state file (the reference's qlm_save / qlm_load, qlm.cuh:703-788): the library's
host-side reader and writer against a file written by the reference itself
(tests/golden/qlmh_small.opt.q, made by tests/golden/make_golden.py)."""
import os
import shutil

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden", "qlmh_small.opt.q")


def make_state():
    from cudalm_c_b200 import qlm
    g = np.load(os.path.join(HERE, "golden", "qlmh_small.npz"))
    # two quantised spans of 640 and 300 elements; 40 float parameters between and after them
    Q = qlm.Qlm([(0, 640), (660, 300)], 640 + 20 + 300 + 20, "cpu")
    assert (Q.nq, Q.ngrp, Q.nfloat, Q.nspan) == (940, 8, 40, 2)
    return Q, g


def fill(Q, g):
    for name in ("d", "r", "m8", "v8", "s", "m8s", "v8s"):
        getattr(Q, name)[:g[name].size].copy_(torch.from_numpy(g[name]))
    Q.Mc.copy_(torch.from_numpy(g["Mc"].view(np.int16))); Q.Vc.copy_(torch.from_numpy(g["Vc"].view(np.int16)))
    Q.spanH["sref"] = g["sref"]


def test_reads_the_reference_file():
    Q, g = make_state()
    it, pg = Q.load(GOLD)
    assert it == 1234 and pg == pytest.approx(2.5)
    for name in ("d", "r", "m8", "v8", "s", "m8s", "v8s"):
        assert np.array_equal(getattr(Q, name)[:g[name].size].numpy(), g[name]), name
    assert np.array_equal(Q.Mc.numpy().view(np.uint16), g["Mc"]) and np.array_equal(Q.Vc.numpy().view(np.uint16), g["Vc"])
    assert np.array_equal(Q.spanH["sref"], g["sref"])


def test_writes_the_same_bytes_as_the_reference(tmp_path):
    Q, g = make_state()
    fill(Q, g)
    out = tmp_path / "mine.opt.q"
    Q.save(out, 1234, prev_gn=2.5)
    assert not os.path.exists(str(out) + ".tmp")
    assert open(out, "rb").read() == open(GOLD, "rb").read()


def test_refuses_another_shape_and_damaged_files(tmp_path):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import qlm
    other = qlm.Qlm([(0, 640), (660, 428)], 1108, "cpu")           # other element count
    with pytest.raises(q.QlmbError):
        other.load(GOLD)
    lion = qlm.Qlm([(0, 640), (660, 300)], 980, "cpu", adam=0)      # other optimizer
    with pytest.raises(q.QlmbError):
        lion.load(GOLD)
    raw = open(GOLD, "rb").read()
    cut = tmp_path / "cut.opt.q"
    cut.write_bytes(raw[:1000])
    Q, _ = make_state()
    with pytest.raises(q.QlmbError):
        Q.load(cut)
    bad = tmp_path / "bad.opt.q"
    bad.write_bytes(b"XXXX" + raw[4:])
    with pytest.raises(q.QlmbError):
        Q.load(bad)
    with pytest.raises(q.QlmbError):
        Q.load(tmp_path / "missing.opt.q")


def test_file_without_trailers_keeps_the_reference_scales(tmp_path):
    """Files written before the SREF / PGN1 trailers existed end after the scale arrays."""
    Q, g = make_state()
    raw = open(GOLD, "rb").read()
    old = tmp_path / "old.opt.q"
    old.write_bytes(raw[:raw.index(b"SREF")])
    Q.spanH["sref"] = np.array([0.125, 0.25], np.float32)
    it, pg = Q.load(old)
    assert it == 1234 and pg is None
    assert np.array_equal(Q.spanH["sref"], np.array([0.125, 0.25], np.float32))
    assert np.array_equal(Q.r[:940].numpy(), g["r"])


def test_round_trip_through_the_reference_loader(tmp_path):
    """A file written by this library is accepted by the reference's own qlm_load (when its CPU
    build is present next to the tests) and yields the same arrays."""
    from oracle import loader
    ref = loader.reference(exact=True)
    if ref is None or not hasattr(ref.lib, "ref_qlm_load"):
        pytest.skip("compiled reference not available")
    Q, g = make_state()
    fill(Q, g)
    path = tmp_path / "mine.opt.q"
    Q.save(path, 77, prev_gn=3.25)
    sp, nq, ng = loader.make_spans([640, 300], 128)
    st = dict(dmax=7, group=128, adam=1, packed=1, d=np.zeros(470, np.int8), r=np.zeros(940, np.int8),
              m8=np.zeros(940, np.int8), v8=np.zeros(940, np.uint8), s=np.zeros(8, np.float32), m8s=np.zeros(8, np.float32),
              v8s=np.zeros(8, np.float32), Mc=np.zeros(40, np.uint16), Vc=np.zeros(40, np.uint16))
    ok, it, pg = ref.qlm_load(str(path), st, sp)
    assert ok == 1 and it == 77 and pg == pytest.approx(3.25)
    for name in ("d", "r", "m8", "v8", "s", "m8s", "v8s", "Mc", "Vc"):
        assert np.array_equal(st[name], g[name]), name
    assert np.array_equal(sp["sref"], g["sref"])


def test_model_file_interchange(tmp_path):
    """TLM4 model files (model_save_bundle / model_load_full, cudalm.cu:554-565, 431-466): what the library
    writes the reference loads, what the reference writes the library reads, and both write the same bytes.
    Also pins the parameter layout of cudalm_c_b200/model.py to the reference's calc_offsets."""
    import ctypes as C
    import numpy as np
    import cudalm_c_b200 as q
    from oracle import loader
    ref = loader.reference()
    if ref is None:
        import pytest
        pytest.skip("compiled reference not present (make -C oracle ref)")
    L = q.lib()
    hdr = np.array([64, 32, 2, 2, 2, 48, 16, 3, 0, 0, 4, 0, 0], np.int32)     # V D L H KV F T eot tmpl n_mtp n_exp win full_every
    n = ref.param_count(hdr)
    from cudalm_c_b200 import model
    cfg = model.Config(L=2, D=32, H=2, KV=2, hd=16, E=4, K=2, F=48, V=64, T=16, B=1)
    assert model.Offsets(cfg).total == n
    rng = np.random.default_rng(0)
    P = rng.standard_normal(n).astype(np.float32)
    mine, theirs = str(tmp_path / "mine.bin"), str(tmp_path / "theirs.bin")
    p = lambda a: a.ctypes.data_as(C.c_void_p)
    q.check(L.qlmb_modelfile_write(mine.encode(), p(hdr), p(P), n, None, 0))
    ref.model_save(theirs, hdr, P)
    assert open(mine, "rb").read() == open(theirs, "rb").read()
    h2, P2 = ref.model_load(mine, n)
    assert (h2 == hdr).all() and (P2 == P).all()
    h3 = np.zeros(13, np.int32); cap = C.c_ulonglong(0); tb = C.c_int(0)
    q.check(L.qlmb_modelfile_read_header(theirs.encode(), p(h3), C.byref(cap), C.byref(tb)))
    assert (h3 == hdr).all() and cap.value >= n
    P3 = np.zeros(n, np.float32)
    q.check(L.qlmb_modelfile_read(theirs.encode(), p(P3), n, None, 0, C.byref(tb)))
    assert (P3 == P).all() and tb.value == 0
    assert L.qlmb_modelfile_read(theirs.encode(), p(np.zeros(n + 8, np.float32)), n + 8, None, 0, None) != 0   # truncated body is refused
