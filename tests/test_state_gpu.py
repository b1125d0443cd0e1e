"""CUDA integer-state kernels through the C ABI vs the golden vectors of the
reference and vs the oracle on random inputs.  Bar: bit-exact."""
import numpy as np
import pytest
import torch

from conftest import golden
from oracle import loader

pytestmark = pytest.mark.gpu
f32 = np.float32


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


class DevState:
    def __init__(self, cuda, sizes, group, dmax, packed, pofs=None):
        from cudalm_c_b200 import qlm
        self.q, self.cuda = qlm, cuda
        self.sp, self.nq, self.ng = loader.make_spans(sizes, group, pofs)
        self.group, self.dmax, self.packed = group, dmax, packed
        z = lambda n, dt: torch.zeros(n, dtype=dt, device=cuda)
        self.d = z((self.nq + 1) // 2 if packed else self.nq, torch.int8)
        self.r = z(self.nq, torch.int8); self.m8 = z(self.nq, torch.int8); self.v8 = z(self.nq, torch.uint8)
        self.s = z(self.ng, torch.float32); self.m8s = z(self.ng, torch.float32); self.v8s = z(self.ng, torch.float32)
        self.push_spans()

    def push_spans(self):
        self.spd = self.q.spans_to_device(self.sp, self.cuda)

    def encode(self, P):
        self.q.qlm_encode(P, self.d, self.r, self.s, self.spd, len(self.sp), self.group, self.dmax, self.packed)

    def step(self, P, G, t, gscale=1.0, gsp=None, lrmode=0, adam=1, stat=None, gi_base=0, ng=None):
        bc1 = f32(1) - f32(np.power(f32(0.9), f32(t))); bc2 = f32(1) - f32(np.power(f32(0.95), f32(t)))
        self.q.qlm_step_launch(P, G, self.d, self.r, self.s, self.m8, self.m8s, self.v8, self.v8s, self.spd,
                               len(self.sp), self.group, self.dmax, 3e-4, 0.9, 0.95, 0.1, gscale, gsp,
                               float(f32(1) / bc1), float(f32(1) / np.sqrt(bc2)), lrmode, t, adam, stat,
                               self.packed, gi_base, self.ng if ng is None else ng)

    def host(self):
        return {k: getattr(self, k).cpu().numpy() for k in ("d", "r", "s", "m8", "v8", "m8s", "v8s")}


def test_one_group_known_answers(cuda):
    g = golden("one_group")
    st = DevState(cuda, [128], 128, 7, 1)
    st.encode(dev(g["P"], cuda))
    h = st.host()
    assert (h["d"] == g["d0"]).all() and (h["r"] == g["r0"]).all() and (h["s"] == g["s0"]).all()
    st.sp[0]["sref"] = h["s"][0]; st.push_spans()
    P = torch.zeros(128, device=cuda); G = dev(g["G"], cuda)
    for t in (1, 2):
        st.step(P, G, t)
        h = st.host(); h["P"] = P.cpu().numpy()
        for k in ("d", "r", "m8", "v8", "m8s", "v8s", "P"):
            assert (h[k] == g["%s_t%d" % (k, t)]).all(), (k, t)


@pytest.mark.parametrize("name", ["state_g128", "state_g64_abs", "state_g96_int8", "state_g256_lion"])
def test_state_sequences_match_reference(cuda, name):
    g = golden(name)
    group, dmax, packed, steps, lrmode, adam = [int(x) for x in g["cfg"]]
    st = DevState(cuda, [int(x) for x in g["sizes"]], group, dmax, packed)
    st.encode(dev(g["P"], cuda))
    h = st.host()
    assert (h["d"] == g["d0"]).all() and (h["r"] == g["r0"]).all() and (h["s"] == g["s0"]).all()
    st.sp["sref"] = g["sref"]; st.push_spans()
    P = torch.zeros(st.nq, device=cuda)
    for t in range(1, steps + 1):
        stat = torch.zeros(4, dtype=torch.int64, device=cuda)
        st.step(P, dev(g["G"][t - 1], cuda), t, gscale=float(g["gscale"][t - 1]), lrmode=lrmode, adam=adam, stat=stat)
        if t == 3:
            st.q.qlm_servo(st.d, st.r, st.s, st.spd, len(st.sp), group, dmax, 0.9 / group, 0.2 / group, packed)
        h = st.host(); h["stat"] = stat.cpu().numpy()
        for k in ("d", "r", "s", "m8", "v8", "m8s", "v8s", "stat"):
            assert (h[k] == g["%s_t%d" % (k, t)]).all(), (k, t)
    st.q.qlm_render(P, st.d, st.s, st.spd, len(st.sp), group, packed)
    assert (P.cpu().numpy() == g["P_final"]).all()


@pytest.mark.parametrize("with_p,use_gsp", [(True, False), (False, True)])
def test_fast_step_matches_oracle(cuda, oracle, with_p, use_gsp):
    """The vectorised group-128 kernel (no stat, aligned spans) vs the oracle over
    10 steps on 2.1M elements, including a short tail group and an unaligned span
    that take the in-kernel fallback."""
    rng = np.random.default_rng(5)
    sizes = [128 * 8192, 128 * 8000 + 40, 128 * 100]
    st = DevState(cuda, sizes, 128, 7, 1)
    P0 = (rng.standard_normal(st.nq) * 0.02).astype(f32)
    st.encode(dev(P0, cuda))
    h = st.host()
    d, r, s = h["d"].copy(), h["r"].copy(), h["s"].copy()
    d2, r2, s2 = np.zeros_like(d), np.zeros_like(r), np.zeros_like(s)
    oracle.encode(P0, d2, r2, s2, st.sp)
    assert (d == d2).all() and (r == r2).all() and (s == s2).all()
    for i in range(len(st.sp)):
        g0 = int(st.sp[i]["gi0"]); st.sp[i]["sref"] = f32(s[g0:g0 + int(st.sp[i]["ngrp"])].astype(np.float64).mean())
    st.push_spans()
    m8 = np.zeros(st.nq, np.int8); v8 = np.zeros(st.nq, np.uint8)
    m8s = np.zeros(st.ng, f32); v8s = np.zeros(st.ng, f32)
    Ph = np.zeros(st.nq, f32)
    P = torch.zeros(st.nq, device=cuda) if with_p else None
    for t in range(1, 11):
        G = (rng.standard_normal(st.nq) * 1e-3).astype(f32)
        gsc = 0.61 if t % 3 == 0 else 1.0
        gsp = torch.tensor([gsc], dtype=torch.float32, device=cuda) if use_gsp else None
        st.step(P, dev(G, cuda), t, gscale=(7.0 if use_gsp else gsc), gsp=gsp)
        bc1 = f32(1) - f32(np.power(f32(0.9), f32(t))); bc2 = f32(1) - f32(np.power(f32(0.95), f32(t)))
        oracle.step(Ph, G, d, r, s, m8, m8s, v8, v8s, st.sp, lr=3e-4, b1=0.9, b2=0.95, wd=0.1, gscale=gsc,
                    inv_bc1=float(f32(1) / bc1), inv_sqrt_bc2=float(f32(1) / np.sqrt(bc2)), t=t)
        h = st.host()
        for k, v in dict(d=d, r=r, m8=m8, v8=v8, m8s=m8s, v8s=v8s).items():
            assert (h[k] == v).all(), (k, t, int((h[k] != v).sum()))
        if with_p:
            assert (P.cpu().numpy() == Ph).all()


def test_step_sharded_equals_whole(cuda):
    """ZeRO-1 style split: stepping group ranges separately gives the same bytes."""
    rng = np.random.default_rng(6)
    sizes = [128 * 300, 128 * 212]
    a = DevState(cuda, sizes, 128, 7, 1); b = DevState(cuda, sizes, 128, 7, 1)
    P0 = dev((rng.standard_normal(a.nq) * 0.02).astype(f32), cuda)
    a.encode(P0); b.encode(P0)
    for t in (1, 2, 3):
        G = dev((rng.standard_normal(a.nq) * 1e-3).astype(f32), cuda)
        a.step(None, G, t)
        for lo, n in ((0, 100), (100, 313), (413, 99)):
            b.step(None, G, t, gi_base=lo, ng=n)
        ha, hb = a.host(), b.host()
        for k in ha:
            assert (ha[k] == hb[k]).all(), (k, t)


def test_config3_full_size_properties(cuda):
    """BASELINE config 3's size (125 829 120 parameters, 983 040 groups), where the CPU oracle is too
    slow: properties that do not depend on the size.  (1) encode -> render -> encode reproduces the
    digits and scales exactly and leaves no residual (every rendered value is digit x scale);
    (2) two optimizer steps taken as four group ranges give the same bytes as taken whole;
    (3) the weights written by the step kernel equal a render of the state it left."""
    n = 125829120
    gen = torch.Generator(device=cuda); gen.manual_seed(3)
    a = DevState(cuda, [n], 128, 7, 1); b = DevState(cuda, [n], 128, 7, 1)
    P0 = torch.randn(n, device=cuda, generator=gen) * 0.02
    a.encode(P0)
    R = torch.empty_like(P0)
    a.q.qlm_render(R, a.d, a.s, a.spd, 1)
    b.encode(R)
    assert torch.equal(a.d, b.d)
    # the re-derived scale is |max digit| x scale / 7, which is the scale again only up to one rounding
    assert float(((a.s - b.s).abs() / a.s).max()) < 2e-7
    assert int(b.r.abs().max()) <= 1
    del R
    for st in (a, b):
        st.sp[0]["sref"] = f32(float(a.s.double().mean())); st.push_spans()
    b.d.copy_(a.d); b.r.copy_(a.r); b.s.copy_(a.s)
    P = torch.zeros(n, device=cuda)
    ng = a.ng
    cuts = [0, ng // 4 + 3, ng // 2, ng - 5, ng]
    for t in (1, 2):
        G = torch.randn(n, device=cuda, generator=gen) * 1e-3
        a.step(P, G, t)
        for lo, hi in zip(cuts[:-1], cuts[1:]):
            b.step(None, G, t, gi_base=lo, ng=hi - lo)
        for k in ("d", "r", "m8", "v8", "m8s", "v8s"):
            assert torch.equal(getattr(a, k), getattr(b, k)), (k, t)
    R = torch.empty(n, device=cuda)
    a.q.qlm_render(R, a.d, a.s, a.spd, 1)
    assert torch.equal(R, P)


def test_config3_ten_steps_match_reference(cuda):
    """BASELINE config 3 as written: a flat span of 125 829 120 parameters ~ N(0, 0.02) encoded by the reference,
    moments from zero, ten steps with a fresh seeded gradient ~ N(0, 1e-3) each (lr 3e-4, betas 0.9 / 0.95,
    wd 0.1, relative learning rate against the frozen mean scale).  After every step the digits, residuals, both
    moment arrays and their scales must equal the compiled reference's (qlm_step_launch of its CPU build) bit
    for bit, and so must the fp32 view after the last one."""
    ref = loader.reference(True)
    if ref is None:
        pytest.skip("compiled reference not present (make -C oracle ref)")
    n = 125829120
    rng = np.random.default_rng(2024)
    P0 = rng.standard_normal(n, dtype=np.float32) * f32(0.02)
    sp, nq, ng = loader.make_spans([n])
    h = dict(d=np.zeros(n // 2, np.int8), r=np.zeros(n, np.int8), s=np.zeros(ng, np.float32), m8=np.zeros(n, np.int8),
             v8=np.zeros(n, np.uint8), m8s=np.zeros(ng, np.float32), v8s=np.zeros(ng, np.float32))
    ref.encode(P0, h["d"], h["r"], h["s"], sp)
    st = DevState(cuda, [n], 128, 7, 1)
    st.encode(dev(P0, cuda))
    sref = f32(np.cumsum(h["s"].astype(np.float64))[-1] / float(ng))       # qlm_gpu_init's double mean (qlm.cuh:528-533)
    sp[0]["sref"] = sref; st.sp[0]["sref"] = sref; st.push_spans()
    for k in ("d", "r", "s"):
        assert torch.equal(getattr(st, k), dev(h[k], cuda)), ("encode", k)
    Ph = P0                                                                # the reference renders into it
    P = torch.zeros(n, device=cuda)
    G = torch.empty(n, device=cuda)
    for t in range(1, 11):
        Gh = rng.standard_normal(n, dtype=np.float32) * f32(1e-3)
        bc1 = f32(1) - f32(np.power(f32(0.9), f32(t))); bc2 = f32(1) - f32(np.power(f32(0.95), f32(t)))
        ref.step(Ph, Gh, h["d"], h["r"], h["s"], h["m8"], h["m8s"], h["v8"], h["v8s"], sp, lr=3e-4, b1=0.9, b2=0.95, wd=0.1,
                 inv_bc1=float(f32(1) / bc1), inv_sqrt_bc2=float(f32(1) / np.sqrt(bc2)), t=t)
        G.copy_(torch.from_numpy(Gh))
        st.step(P if t == 10 else None, G, t)
        for k in ("d", "r", "m8", "v8", "m8s", "v8s"):
            assert torch.equal(getattr(st, k), dev(h[k], cuda)), (k, t)
    assert torch.equal(P, dev(Ph, cuda))


def test_empty_and_bad_arguments(cuda):
    import cudalm_c_b200 as q
    st = DevState(cuda, [256], 128, 7, 1)
    P = torch.zeros(256, device=cuda)
    st.step(P, P, 1, ng=0)                       # empty range: no launch, no error
    with pytest.raises(q.QlmbError):
        q.qlm.qlm_encode(P, st.d, st.r, st.s, st.spd, 1, group=31)
    with pytest.raises(q.QlmbError):
        q.qlm.qlm_encode(P, st.d, st.r, st.s, st.spd, 1, dmax=127, packed=1)


def test_gnorm_matches_reference(cuda, oracle):
    from cudalm_c_b200 import qlm
    g = golden("gnorm")
    G, side, small = dev(g["G"], cuda), dev(g["side"], cuda), dev(g["small"], cuda)
    assert (qlm.gnorm(G).cpu().numpy() == g["gs_plain"]).all()
    assert (qlm.gnorm(G, [side], 1).cpu().numpy() == g["gs_side"]).all()
    assert (qlm.gnorm(G, [side], 0).cpu().numpy() == g["gs_noclip"]).all()
    assert (qlm.gnorm(small).cpu().numpy() == g["gs_small"]).all()
    bad = side.clone(); bad[5] = float("inf")
    assert np.isnan(qlm.gnorm(G, [bad], 0).cpu().numpy()[1])
    rng = np.random.default_rng(9)
    big = (rng.standard_normal(30_000_001) * 1e-3).astype(f32)
    assert (qlm.gnorm(dev(big, cuda)).cpu().numpy() == oracle.gnorm(big)).all()


def test_adamw_float_spans(cuda, oracle):
    from cudalm_c_b200 import qlm
    rng = np.random.default_rng(10)
    n = 100_003
    P = rng.standard_normal(n).astype(f32); G = (rng.standard_normal(n) * 1e-2).astype(f32)
    M = np.zeros(n, np.uint16); V = np.zeros(n, np.uint16)
    Pd, Md, Vd = dev(P, cuda), dev(M.view(np.int16), cuda), dev(V.view(np.int16), cuda)
    gs = np.array([0.5, 2.0], f32)
    for t in range(1, 4):
        bc1, bc2 = qlm.bias_corrections(0.9, 0.95, t)
        qlm.adamw(Pd, dev(G, cuda), Md, Vd, 3e-4, 0.9, 0.95, 0.1, bc1, bc2, dev(gs, cuda))
        oracle.adamw(P, G, M, V, 3e-4, 0.9, 0.95, 0.1, bc1, bc2, gs)
    assert (Pd.cpu().numpy() == P).all()
    assert (Md.cpu().numpy().view(np.uint16) == M).all() and (Vd.cpu().numpy().view(np.uint16) == V).all()


def test_qlm_class_update_with_servo(cuda, oracle):
    """Qlm mirror: init, 3 updates (servo every 2) over two matrices with float gaps."""
    from cudalm_c_b200 import qlm
    rng = np.random.default_rng(12)
    mats = [(100, 128 * 20), (100 + 128 * 20 + 50, 128 * 12)]
    total = mats[1][0] + mats[1][1] + 30
    Q = qlm.Qlm(mats, total, cuda, servo_every=2)
    P0 = (rng.standard_normal(total) * 0.02).astype(f32)
    P = dev(P0, cuda)
    Q.init_from(P)
    sp, nq, ng = loader.make_spans([m[1] for m in mats], 128, [m[0] for m in mats])
    d = np.zeros(nq // 2, np.int8); r = np.zeros(nq, np.int8); s = np.zeros(ng, f32)
    oracle.encode(P0, d, r, s, sp)
    for i in range(2):
        g0 = int(sp[i]["gi0"]); sp[i]["sref"] = f32(np.cumsum(s[g0:g0 + int(sp[i]["ngrp"])].astype(np.float64))[-1] / float(sp[i]["ngrp"]))
    assert (Q.spanH["sref"] == sp["sref"]).all()
    Ph = P0.copy(); oracle.render(Ph, d, s, sp)
    assert (P.cpu().numpy() == Ph).all()
    m8 = np.zeros(nq, np.int8); v8 = np.zeros(nq, np.uint8); m8s = np.zeros(ng, f32); v8s = np.zeros(ng, f32)
    Mc = np.zeros(Q.nfloat, np.uint16); Vc = np.zeros(Q.nfloat, np.uint16)
    for t in (1, 2, 3):
        G = (rng.standard_normal(total) * 1e-3).astype(f32)
        gsd = qlm.gnorm(dev(G * 100, cuda))
        gs = oracle.gnorm(G * 100)
        assert (gsd.cpu().numpy() == gs).all()
        Q.update(P, dev(G * 100, cuda), 3e-4, 0.9, 0.95, 0.1, t, gs=gsd)
        bc1, bc2 = qlm.bias_corrections(0.9, 0.95, t)
        oracle.step(Ph, G * 100, d, r, s, m8, m8s, v8, v8s, sp, lr=3e-4, b1=0.9, b2=0.95, wd=0.1, gscale=float(gs[0]),
                    inv_bc1=float(f32(1) / f32(bc1)), inv_sqrt_bc2=float(f32(1) / np.sqrt(f32(bc2))), t=t)
        for off, n, cs in Q.fs:
            oracle.adamw(Ph[off:off + n], (G * 100)[off:off + n], Mc[cs:cs + n], Vc[cs:cs + n], 3e-4, 0.9, 0.95, 0.1, bc1, bc2, gs)
        if t % 2 == 0:
            oracle.servo(d, r, s, sp, 128, 7, Q.f_hi, Q.f_lo, 1)
        assert (Q.d.cpu().numpy() == d).all() and (Q.r.cpu().numpy() == r).all() and (Q.s.cpu().numpy() == s).all()
        assert (P.cpu().numpy() == Ph).all()


def test_state_sequence_v4(cuda):
    """QLM_V4 (qlm.cuh:62-72) through qlmb_set_v4: same bytes as the reference with d_qv4 = 1."""
    import cudalm_c_b200 as q
    q.check(q.lib().qlmb_set_v4(1))
    try:
        test_state_sequences_match_reference(cuda, "state_g128_v4")
    finally:
        q.check(q.lib().qlmb_set_v4(0))


def test_fused_per_layer_update_matches_reference(cuda):
    """qlm_fused_layer / qlm_fused_tail (cudalm.cu:6105-6187): layers share one gradient block, each is
    consumed as soon as it is complete, the clip multiplier is the previous step's and stays on the
    device.  Fixture: the reference's own kernels composed the same way, three steps."""
    from cudalm_c_b200 import qlm
    g = golden("fused_update")
    lay = loader.fused_layout(3, 20, 4, 32, 32)
    Q = qlm.Qlm(list(zip(lay["q_pofs"], lay["q_sizes"])), lay["np"], cuda)
    P = dev(g["P0"], cuda)
    Q.init_from(P, render=False)
    assert (Q.spanH["sref"] == g["out_sref"]).all()
    fu = qlm.FusedUpdate(Q, lay["L"], lay["layer_g0"], lay["layer_gn"],
                         [[(p, go, n, 0.0) for p, go, n in fl] for fl in lay["layer_float"]],
                         [(p, go, n, 0.0) for p, go, n in lay["tail_float"]])
    fu.set_gof(lay["q_gofs"])
    G = torch.zeros(lay["ng_total"], device=cuda)
    g0, gn = lay["layer_g0"], lay["layer_gn"]
    for t in (1, 2, 3):
        blocks = g["g%d_layers" % (t - 1)].astype(f32)
        for l in range(lay["L"] - 1, -1, -1):
            G[g0:g0 + gn] = dev(blocks[l], cuda)
            fu.layer(P, G, l, 3e-4, t)
        emb, nf = g["g%d_emb" % (t - 1)].astype(f32), g["g%d_nf" % (t - 1)].astype(f32)
        G[0:emb.size] = dev(emb, cuda); G[emb.size:emb.size + nf.size] = dev(nf, cuda)
        fu.tail(P, G, 3e-4, t)
        assert fu.gs.cpu().numpy()[1] == g["out_norms"][t - 1], t
    for k in ("d", "r", "s", "m8", "v8", "m8s", "v8s"):
        assert (getattr(Q, k).cpu().numpy() == g["out_" + k]).all(), k
    assert (Q.Mc.cpu().numpy().view(np.uint16) == g["out_Mc"]).all()
    assert (Q.Vc.cpu().numpy().view(np.uint16) == g["out_Vc"]).all()
    assert (P.cpu().numpy() == g["out_P"]).all()


def test_ngram_q4_table_update(cuda):
    """NGRAM_Q4_FOLD (cudalm.cu:4465-4530, 4673-4745): touched-group map, compact gradient scatter and the
    list-driven integer AdamW step, three steps, against the reference's CPU kernels: same touched groups, same
    bytes of state and the same rendered table.  The device never learns the touched count on the host."""
    import cudalm_c_b200 as q
    from cudalm_c_b200 import qlm
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    g = golden("ngram_q4")
    R, De, group, dmax = [int(x) for x in g["cfg"]]
    nt = R * De
    st = DevState(cuda, [nt], group, dmax, 1)
    st.encode(dev(g["Praw"], cuda))
    h = st.host()
    assert (h["d"] == g["d0"]).all() and (h["r"] == g["r0"]).all() and (h["s"] == g["s0"]).all()
    P = dev(g["P0"], cuda)                                               # the rendered table the gather reads
    sref = float(g["sref"][0])
    ngrp = st.ng
    flag = torch.zeros(ngrp, dtype=torch.int32, device=cuda)
    count = torch.zeros(1, dtype=torch.int32, device=cuda)
    L = lib()
    for t in (1, 2, 3):
        key = dev(g["key%d" % t], cuda); dbuf = dev(g["dbuf%d" % t], cuda); gs = dev(g["gs%d" % t], cuda)
        NK, Nd = key.numel(), dbuf.shape[0]
        cap = min(NK, ngrp)
        tgi = torch.zeros(cap, dtype=torch.int32, device=cuda)
        Gc = torch.full((cap * group,), float("nan"), device=cuda)          # every live element must be overwritten
        check(L.qlmb_ng_touched(ptr(tgi), ptr(count), ptr(flag), ptr(key), NK, De, group, ngrp, stream_ptr()))
        check(L.qlmb_ng_scatter_compact(ptr(Gc), ptr(key), ptr(tgi), ptr(count), ptr(dbuf), NK, De, group, Nd, cap, stream_ptr()))
        bc1 = f32(1) - f32(np.power(f32(0.9), f32(t))); bc2 = f32(1) - f32(np.power(f32(0.95), f32(t)))
        check(L.qlmb_ng_step(ptr(P), ptr(Gc), ptr(st.d), ptr(st.r), ptr(st.s), ptr(st.m8), ptr(st.m8s), ptr(st.v8), ptr(st.v8s),
                             ptr(tgi), ptr(count), cap, group, dmax, 3e-3, 0.9, 0.95, 0.0, sref, float(f32(1) / bc1),
                             float(f32(1) / np.sqrt(bc2)), t, nt, ptr(gs), stream_ptr()))
        n = int(count[0])
        assert (tgi[:n].cpu().numpy() == g["touched%d" % t]).all()
        assert int(flag.sum()) == 0
    h = st.host()
    for k in ("d", "r", "m8", "v8", "m8s", "v8s"):
        assert (h[k] == g[k]).all(), k
    assert (P.cpu().numpy() == g["P"]).all()
    q.check(q.lib().qlmb_check_device(None))
