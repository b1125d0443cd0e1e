"""Exact 4-bit export (q4n) and the engram table's keys, gather and compact scatter.

Fixtures (tests/golden/q4n.npz, engram.npz) were written by the reference's own quantize_params / dequantize_params
(cudalm.cu:639-656, 688-695) and its CPU kernels k_eg_key, k_eg_gather, k_eg_scatter_c (cpu_kern.h:665-688).
CPU tests cover the host walk over a stream and the container file; GPU tests are bit-exact parity."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import golden

f32 = np.float32


def test_index_walks_the_reference_stream():
    from cudalm_c_b200 import q4n
    g = golden("q4n")
    P, q, group = g["P"], g["q"], int(g["group"][0])
    off = q4n.index(q, P.size, group)
    assert int(off[-1]) == q.size
    sizes = np.diff(off.astype(np.int64))
    scales = np.array([np.frombuffer(q[int(o):int(o) + 4].tobytes(), f32)[0] for o in off[:-1]])
    raw = np.isnan(scales)
    assert raw.sum() == 2 and (sizes[raw] == 4 + 4 * group).all()
    assert (sizes[~raw][:-1] == 4 + group // 2).all() and sizes[-1] == 4 + 35          # short last group of 70
    import cudalm_c_b200 as cq
    with pytest.raises(cq.QlmbError):
        q4n.index(q[:-3].copy(), P.size, group)


def test_container_file_round_trip(tmp_path):
    from cudalm_c_b200 import q4n
    from cudalm_c_b200._lib import check, lib
    g = golden("q4n")
    q, group = g["q"], int(g["group"][0])
    for win, magic, nh in ((0, b"TLQ1", 11), (256, b"TLQ2", 13)):
        hdr = np.array([500, 64, 2, 4, 2, 128, 32, 7, 0, 0, 8, win, 4 if win else 0], np.int32)
        blob = np.frombuffer(b"tokenizer-bytes", np.uint8)
        path = tmp_path / ("m%d.bin" % win)
        check(lib().qlmb_qfile_write(str(path).encode(), hdr.ctypes.data_as(C.c_void_p), 3, group, q.ctypes.data_as(C.c_void_p),
                                     q.size, blob.ctypes.data_as(C.c_void_p), blob.size))
        raw = open(path, "rb").read()
        # the reference's layout (cudalm.cu:9783-9793): magic, header ints, qtype, group, body, blob length, blob
        assert raw[:4] == magic and np.array_equal(np.frombuffer(raw[4:4 + 4 * nh], np.int32), hdr[:nh])
        assert np.array_equal(np.frombuffer(raw[4 + 4 * nh:12 + 4 * nh], np.int32), [3, group])
        assert raw[12 + 4 * nh:12 + 4 * nh + q.size] == q.tobytes()
        assert raw[12 + 4 * nh + q.size:] == np.int32(blob.size).tobytes() + blob.tobytes()
        h2, qt, gr, buf = q4n.read(path)
        assert np.array_equal(h2[:nh], hdr[:nh]) and (qt, gr) == (3, group)
        assert buf.size == q.size + 4 + blob.size and np.array_equal(buf[:q.size], q)


def test_reference_reads_our_container(tmp_path):
    """model_load_full (cudalm.cu:438-450) on a TLQ1 file written by this library."""
    from oracle import loader
    from cudalm_c_b200._lib import check, lib
    R = loader.reference(True)
    if R is None:
        pytest.skip("compiled reference not present (make -C oracle ref)")
    rm = R.model_new(64, 32, 1, 2, 1, 64, 16, 4, 2, 1)
    n = rm.np
    rng = np.random.default_rng(5)
    ng = (n + 127) // 128
    P = (np.repeat((np.exp(rng.uniform(-8, -3, ng))).astype(f32), 128)[:n] * rng.integers(-7, 8, n).astype(f32)).astype(f32)
    q = R.q4n_export(P, 128)
    hdr = np.array([64, 32, 1, 2, 1, 64, 16, 0, 0, 0, 4, 0, 0], np.int32)
    path = tmp_path / "m.bin"
    check(lib().qlmb_qfile_write(str(path).encode(), hdr.ctypes.data_as(C.c_void_p), 3, 128, q.ctypes.data_as(C.c_void_p), q.size, None, 0))
    h2, P2 = R.model_load(str(path), n + 16)
    assert np.array_equal(h2[:7], hdr[:7]) and P2.size == n and np.array_equal(P2.view(np.uint32), P.view(np.uint32))


@pytest.mark.gpu
def test_export_is_byte_identical_and_decodes_exactly(cuda, tmp_path):
    from cudalm_c_b200 import q4n
    g = golden("q4n")
    P, q, group = g["P"], g["q"], int(g["group"][0])
    Pd = torch.from_numpy(P).to(cuda)
    out, raw = q4n.export(Pd, group)
    assert raw == 2
    assert np.array_equal(out.cpu().numpy(), q)
    back = q4n.decode(q, P.size, cuda, group)
    assert np.array_equal(back.cpu().numpy().view(np.uint32), P.view(np.uint32))
    hdr = np.array([1, 2, 3, 4, 5, 6, 7, 8, 0, 0, 9, 0, 0], np.int32)
    nb, _ = q4n.save(tmp_path / "x.bin", hdr, Pd, b"blob", group)
    h2, P2, blob = q4n.load(tmp_path / "x.bin", P.size, cuda)
    assert nb == q.size and blob == b"blob" and np.array_equal(h2, hdr)
    assert np.array_equal(P2.cpu().numpy().view(np.uint32), P.view(np.uint32))


@pytest.mark.gpu
def test_export_of_rendered_state_is_lossless_at_size(cuda):
    """8.4 M parameters rendered from random digits and scales: no group falls back to raw fp32, the stream has the
    fixed size 68 bytes per 128 and decodes to the same bits; against the reference's export when it is present."""
    from cudalm_c_b200 import q4n
    gen = torch.Generator(device=cuda); gen.manual_seed(3)
    ng, group = 65536, 128
    d = torch.randint(-7, 8, (ng, group), device=cuda, generator=gen).float()
    s = torch.exp(torch.rand(ng, 1, device=cuda, generator=gen) * 10 - 12)
    P = (d * s).reshape(-1).contiguous()
    out, raw = q4n.export(P, group)
    assert raw == 0 and out.numel() == ng * 68
    oh = out.cpu().numpy()
    back = q4n.decode(oh, P.numel(), cuda, group)
    assert torch.equal(back.view(torch.int32), P.view(torch.int32))
    from oracle import loader
    R = loader.reference(True)
    if R is not None:
        n = 4096 * group
        assert np.array_equal(R.q4n_export(P[:n].cpu().numpy(), group), oh[:4096 * 68])


@pytest.mark.gpu
def test_engram_keys_gather_and_compact_scatter(cuda):
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    g = golden("engram")
    V, T, B, De, grp, Rraw, Rp = [int(x) for x in g["cfg"]]
    ords, prime, mult = g["ords"], g["prime"], g["mult"]
    S, N = ords.size, B * T
    L = lib()
    dv = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    tok, ordd, primed, multd = dv(g["tok"]), dv(ords), dv(prime), dv(mult.view(np.int64))
    canon = dv(g["canon"].view(np.int16))
    key = torch.zeros(S * N, dtype=torch.int32, device=cuda)
    check(L.qlmb_eg_key(ptr(key), ptr(tok), None, ptr(ordd), ptr(primed), ptr(multd), N, T, S, Rp, stream_ptr()))
    keyc = torch.zeros_like(key)
    check(L.qlmb_eg_key(ptr(keyc), ptr(tok), ptr(canon), ptr(ordd), ptr(primed), ptr(multd), N, T, S, Rp, stream_ptr()))
    assert np.array_equal(key.cpu().numpy(), g["key"]) and np.array_equal(keyc.cpu().numpy(), g["keyc"])
    tbl = dv(g["tbl"])
    buf = torch.full((N, S * De), float("nan"), device=cuda)
    check(L.qlmb_eg_gather(ptr(buf), ptr(tbl), ptr(key), N, S, De, stream_ptr()))
    assert np.array_equal(buf.cpu().numpy(), g["buf"])
    ngrp = S * Rp * De // grp
    flag = torch.zeros(ngrp, dtype=torch.int32, device=cuda)
    count = torch.zeros(1, dtype=torch.int32, device=cuda)
    cap = min(S * N, ngrp)
    tgi = torch.zeros(cap, dtype=torch.int32, device=cuda)
    Gc = torch.full((cap * grp,), float("nan"), device=cuda)
    db = dv(g["db"])
    check(L.qlmb_ng_touched(ptr(tgi), ptr(count), ptr(flag), ptr(key), S * N, De, grp, ngrp, stream_ptr()))
    check(L.qlmb_eg_scatter_compact(ptr(Gc), ptr(key), ptr(tgi), ptr(count), ptr(db), N, S, De, grp, cap, stream_ptr()))
    n = int(count[0])
    assert np.array_equal(tgi[:n].cpu().numpy(), g["touched"])
    assert np.array_equal(Gc[:n * grp].reshape(n, grp).cpu().numpy(), g["Gc"])
