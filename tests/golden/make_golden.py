"""Generate tests/golden/*.npz by running the UNMODIFIED reference.

Needs oracle/_ref/libcudalm_ref_exact.so (make -C oracle ref), i.e. a checkout
of the reference; the produced vectors are committed so the tests run without
it.  Every array an op reads is stored next to what the reference wrote, so a
fixture is self-contained and does not depend on any RNG staying stable.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import loader  # noqa: E402

OUT = os.path.dirname(os.path.abspath(__file__))
f32 = np.float32


def bias_corr(b1, b2, t):
    """inv_bc1, inv_sqrt_bc2 as the reference derives them (cudalm.cu:6454, 6085)."""
    bc1 = f32(1) - f32(np.power(f32(b1), f32(t)))
    bc2 = f32(1) - f32(np.power(f32(b2), f32(t)))
    return float(f32(1) / bc1), float(f32(1) / np.sqrt(bc2))


def set_sref(sp, s):
    for i in range(len(sp)):
        g0 = int(sp[i]["gi0"])
        sp[i]["sref"] = f32(s[g0:g0 + int(sp[i]["ngrp"])].astype(np.float64).mean())


def golden_hash(ref):
    xs = np.array([0, 1, 2, 0x0123456789ABCDEF, 0xFFFFFFFFFFFFFFFF, 12345678901234567], np.uint64)
    hs = np.array([ref.hash(int(x)) for x in xs], np.uint32)
    vals = np.array([0.5, -0.5, 2.25, -47.75, 0.001, -0.999, 7.5, 126.99], f32)
    idx = np.arange(16, dtype=np.uint64) * np.uint64(1000003) + np.uint64(5)
    ts = np.array([1, 2, 3, 1000, 1 + 0x5EED, 1 + 0xBEEF], np.uint64)
    sr = np.zeros((len(vals), len(idx), len(ts)), np.int32)
    for a, v in enumerate(vals):
        for b, i in enumerate(idx):
            for c, t in enumerate(ts):
                sr[a, b, c] = ref.sround(float(v), int(i), int(t))
    np.savez_compressed(os.path.join(OUT, "hash.npz"), xs=xs, hs=hs, vals=vals, idx=idx, ts=ts, sr=sr)


def golden_one_group(ref):
    """The single 128-element group of the reference survey's known-answer table."""
    j = np.arange(128)
    P = ((j - 64).astype(f32) * f32(0.001)).astype(f32)
    G = (f32(1e-3) * ((j % 7) - 3).astype(f32)).astype(f32)
    sp, nq, ng = loader.make_spans([128])
    d = np.zeros(64, np.int8); r = np.zeros(128, np.int8); s = np.zeros(1, f32)
    ref.encode(P, d, r, s, sp)
    out = dict(P=P, G=G, d0=d.copy(), r0=r.copy(), s0=s.copy())
    sp[0]["sref"] = s[0]
    m8 = np.zeros(128, np.int8); v8 = np.zeros(128, np.uint8)
    m8s = np.zeros(1, f32); v8s = np.zeros(1, f32); Pv = np.zeros(128, f32)
    for t in (1, 2):
        i1, i2 = bias_corr(0.9, 0.95, t)
        ref.step(Pv, G, d, r, s, m8, m8s, v8, v8s, sp, lr=3e-4, b1=0.9, b2=0.95, wd=0.1,
                 inv_bc1=i1, inv_sqrt_bc2=i2, t=t)
        for k, v in dict(d=d, r=r, m8=m8, v8=v8, m8s=m8s, v8s=v8s, P=Pv).items():
            out["%s_t%d" % (k, t)] = v.copy()
    # the values the table quotes
    assert s.view(np.uint32)[0] == 0x3C15CBED
    assert out["m8s_t1"].view(np.uint32)[0] == 0x361E8661
    assert out["v8s_t2"].view(np.uint32)[0] == 0x367686BE
    np.savez_compressed(os.path.join(OUT, "one_group.npz"), **out)


def golden_state(ref, name, sizes, group, dmax, packed, steps, seed, lrmode=0, adam=1):
    """Ragged multi-span state: encode, `steps` optimiser steps with a servo
    tick after step 3 (thresholds widened so it fires) and a final render."""
    rng = np.random.default_rng(seed)
    sp, nq, ng = loader.make_spans(sizes, group)
    P = (rng.standard_normal(nq) * 0.02).astype(f32)
    P[:7] = 0.0
    d = np.zeros((nq + 1) // 2 if packed else nq, np.int8)
    r = np.zeros(nq, np.int8); s = np.zeros(ng, f32)
    ref.encode(P, d, r, s, sp, group, dmax, packed)
    set_sref(sp, s)
    out = dict(P=P, sizes=np.array(sizes), cfg=np.array([group, dmax, packed, steps, lrmode, adam]),
               sref=sp["sref"].copy(), d0=d.copy(), r0=r.copy(), s0=s.copy())
    m8 = np.zeros(nq, np.int8); v8 = np.zeros(nq, np.uint8)
    m8s = np.zeros(ng, f32); v8s = np.zeros(ng, f32); Pv = np.zeros(nq, f32)
    Gs = []
    gsc = []
    for t in range(1, steps + 1):
        G = (rng.standard_normal(nq) * 1e-3).astype(f32)
        if t == 2:
            G[::5] *= 300.0          # multi-carry steps and the +-8 clamp
        Gs.append(G)
        gscale = 0.37 if t % 2 == 0 else 1.0
        gsc.append(gscale)
        i1, i2 = bias_corr(0.9, 0.95, t)
        stat = np.zeros(4, np.int64)
        ref.step(Pv, G, d, r, s, m8, m8s, v8, v8s, sp, group=group, dmax=dmax, lr=3e-4, b1=0.9,
                 b2=0.95, wd=0.1, gscale=gscale, inv_bc1=i1, inv_sqrt_bc2=i2, lrmode=lrmode, t=t,
                 adam=adam, stat=stat, packed=packed)
        if t == 3:
            ref.servo(d, r, s, sp, group, dmax, 0.9 / group, 0.2 / group, packed)
        for k, v in dict(d=d, r=r, s=s, m8=m8, v8=v8, m8s=m8s, v8s=v8s, stat=stat).items():
            out["%s_t%d" % (k, t)] = v.copy()
    ref.render(Pv, d, s, sp, group, packed)
    out["P_final"] = Pv.copy()
    out["G"] = np.stack(Gs); out["gscale"] = np.array(gsc, f32)
    np.savez_compressed(os.path.join(OUT, name + ".npz"), **out)


def golden_gnorm(ref):
    rng = np.random.default_rng(11)
    G = (rng.standard_normal(60007) * 7e-3).astype(f32)
    side = (rng.standard_normal(1234) * 0.1).astype(f32)
    small = (rng.standard_normal(1000) * 1e-3).astype(f32)
    np.savez_compressed(os.path.join(OUT, "gnorm.npz"), G=G, side=side, small=small,
                        gs_plain=ref.gnorm(G), gs_side=ref.gnorm(G, [side], 1),
                        gs_noclip=ref.gnorm(G, [side], 0), gs_small=ref.gnorm(small))


def golden_router(ref):
    rng = np.random.default_rng(21)
    out = {}
    for tag, (N, E, K) in dict(a=(300, 32, 2), b=(257, 7, 3), c=(64, 4, 1), d=(100, 256, 8)).items():
        rt = (rng.standard_normal((N, E)) * 2.0).astype(f32)
        rt[3] = rt[3, 0]                   # exact ties: first index must win
        bias = (rng.standard_normal((K, E)) * 0.01).astype(f32)
        for bt, (b, bs) in dict(nb=(None, 0), wb=(bias, E)).items():
            rp, asg, gt = ref.router_topk(rt, K, b, bs)
            out["%s_%s_rprobs" % (tag, bt)] = rp
            out["%s_%s_assign" % (tag, bt)] = asg
            out["%s_%s_gate" % (tag, bt)] = gt
        out[tag + "_rt"] = rt
        out[tag + "_bias"] = bias
    np.savez_compressed(os.path.join(OUT, "router.npz"), **out)


def golden_linear(ref):
    """g_ab / g_abt / g_atb on a rendered 4-bit weight (the selftest's odd shapes
    rounded up to whole groups)."""
    rng = np.random.default_rng(31)
    M, K, N = 67, 128, 256
    X = rng.standard_normal((M, K)).astype(f32)
    dY = rng.standard_normal((M, N)).astype(f32)
    W = (rng.standard_normal(K * N) * 0.02).astype(f32)
    sp, nq, ng = loader.make_spans([K * N])
    d = np.zeros(nq // 2, np.int8); r = np.zeros(nq, np.int8); s = np.zeros(ng, f32)
    ref.encode(W, d, r, s, sp)
    Wr = np.zeros(nq, f32); ref.render(Wr, d, s, sp)
    out = dict(X=X, dY=dY, d=d, s=s)
    Wkn = Wr.reshape(K, N)                 # layout KN: Y = X @ W
    out["Y_kn"] = ref.g_ab(X, Wkn); out["dX_kn"] = ref.g_abt(dY, Wkn)
    out["dW_kn"] = ref.g_atb(X, dY, np.zeros((K, N), f32))
    Wnk = Wr.reshape(N, K)                 # layout NK: Y = X @ W^T
    out["Y_nk"] = ref.g_abt(X, Wnk); out["dX_nk"] = ref.g_ab(dY, Wnk)
    out["dW_nk"] = ref.g_atb(dY, X, np.zeros((N, K), f32))
    np.savez_compressed(os.path.join(OUT, "linear.npz"), **out)


def golden_moe(ref):
    """One MoE layer forward+backward through the reference's moe_forward /
    moe_backward (top-2, selection bias off, aux 0.03, stash on)."""
    rng = np.random.default_rng(41)
    N, D, F, E, K = 160, 128, 256, 4, 2

    def quant(n):
        sp, nq, ng = loader.make_spans([n])
        W = (rng.standard_normal(n) * 0.02).astype(f32)
        d = np.zeros(n // 2, np.int8); r = np.zeros(n, np.int8); s = np.zeros(ng, f32)
        ref.encode(W, d, r, s, sp)
        Wv = np.zeros(n, f32); ref.render(Wv, d, s, sp)
        return d, s, Wv

    d1, s1, P1 = quant(E * D * F); d3, s3, P3 = quant(E * D * F); d2, s2, P2 = quant(E * F * D)
    Wr = (rng.standard_normal((D, E)) * 0.02).astype(f32)
    # activations are bf16-representable so a bf16 path sees identical inputs
    def bf(x):
        u = x.astype(f32).view(np.uint32)
        return (((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16).astype(np.uint32).view(f32)
    fn = bf(rng.standard_normal((N, D))); fi = bf(rng.standard_normal((N, D)))
    dout = bf(rng.standard_normal((N, D)))
    L = ref.moe_new(N, D, F, E, K, 0.03)
    P = L.buf("P", (L.np,))
    for nm, v in (("wr", Wr.ravel()), ("w1", P1), ("w3", P3), ("w2", P2)):
        P[L.off(nm):L.off(nm) + v.size] = v
    L.buf("f_norm", (N, D))[:] = fn; L.buf("f_in", (N, D))[:] = fi; L.buf("dout", (N, D))[:] = dout
    L.forward(); L.backward()
    G = L.buf("G", (L.np,))
    np.savez_compressed(
        os.path.join(OUT, "moe.npz"), shape=np.array([N, D, F, E, K]), aux=f32(0.03),
        d1=d1, s1=s1, d3=d3, s3=s3, d2=d2, s2=s2, Wr=Wr, fn=fn, fi=fi, dout=dout,
        out=L.buf("out", (N, D)).copy(), rt=L.buf("rt", (N, E)).copy(),
        rprobs=L.buf("rprobs", (N, E)).copy(), assign=L.buf("assign", (K, N), np.int32).copy(),
        gate=L.buf("gate", (K, N)).copy(), perm=L.buf("perm", (K, N), np.int32).copy(),
        hoff=L.buf("hoff", (K, E + 1), np.int32).copy(), d_gate=L.buf("d_gate", (K, N)).copy(),
        dfnorm=L.buf("dfnorm", (N, D)).copy(),
        dW1=G[L.off("w1"):L.off("w1") + E * D * F].astype(np.float16),
        dW3=G[L.off("w3"):L.off("w3") + E * D * F].astype(np.float16),
        dW2=G[L.off("w2"):L.off("w2") + E * D * F].astype(np.float16),
        dWr=G[L.off("wr"):L.off("wr") + D * E].copy())


def golden_statefile(ref):
    """A QLMH optimizer-state file written by the reference's own qlm_save (two ragged spans,
    3 optimizer steps, 40 float-span moments), plus the arrays that went into it."""
    rng = np.random.default_rng(11)
    group, dmax, packed = 128, 7, 1
    sp, nq, ng = loader.make_spans([128 * 5, 300], group)
    P = (rng.standard_normal(nq) * 0.02).astype(f32)
    d = np.zeros((nq + 1) // 2, np.int8); r = np.zeros(nq, np.int8); s = np.zeros(ng, f32)
    ref.encode(P, d, r, s, sp, group, dmax, packed)
    set_sref(sp, s)
    m8 = np.zeros(nq, np.int8); v8 = np.zeros(nq, np.uint8); m8s = np.zeros(ng, f32); v8s = np.zeros(ng, f32)
    Pv = np.zeros(nq, f32)
    for t in range(1, 4):
        G = (rng.standard_normal(nq) * 1e-3).astype(f32)
        i1, i2 = bias_corr(0.9, 0.95, t)
        ref.step(Pv, G, d, r, s, m8, m8s, v8, v8s, sp, group=group, dmax=dmax, lr=3e-4, b1=0.9, b2=0.95, wd=0.1,
                 inv_bc1=i1, inv_sqrt_bc2=i2, t=t, packed=packed)
    Mc = rng.integers(0, 65536, 40).astype(np.uint16); Vc = rng.integers(0, 32768, 40).astype(np.uint16)
    st = dict(dmax=dmax, group=group, adam=1, packed=packed, d=d, r=r, m8=m8, v8=v8, s=s, m8s=m8s, v8s=v8s, Mc=Mc, Vc=Vc)
    path = os.path.join(OUT, "qlmh_small.opt.q")
    assert ref.qlm_save(path, st, sp, 1234, 2.5) == 1
    np.savez_compressed(os.path.join(OUT, "qlmh_small.npz"), d=d, r=r, m8=m8, v8=v8, s=s, m8s=m8s, v8s=v8s, Mc=Mc, Vc=Vc,
                        sref=sp["sref"].copy(), cfg=np.array([dmax, group, 1, len(sp), packed, 1234]), prev_gn=np.float32(2.5))


def fused_case(impl, P0, grads16):
    """Three fused-update steps on the small model of the fused fixture with `impl`'s primitives."""
    lay = loader.fused_layout(3, 20, 4, 32, 32)
    sp, nq, ng = loader.make_spans(lay["q_sizes"], 128, lay["q_pofs"])
    P = P0.copy()
    st = dict(sp=sp, d=np.zeros((nq + 1) // 2, np.int8), r=np.zeros(nq, np.int8), s=np.zeros(ng, f32),
              m8=np.zeros(nq, np.int8), v8=np.zeros(nq, np.uint8), m8s=np.zeros(ng, f32), v8s=np.zeros(ng, f32))
    impl.encode(P, st["d"], st["r"], st["s"], sp, 128, 7, 1)
    set_sref(sp, st["s"])
    sp["gof"] = lay["q_gofs"]
    # compact offsets of the float spans: the gaps between the quantised spans in ascending order
    gaps, cur, acc = [], 0, 0
    for pof, n in zip(lay["q_pofs"], lay["q_sizes"]):
        if pof > cur:
            gaps.append((cur, pof - cur, acc)); acc += pof - cur
        cur = pof + n
    if cur < lay["np"]:
        gaps.append((cur, lay["np"] - cur, acc)); acc += lay["np"] - cur
    def cs_of(p_off):
        for off, n, cs in gaps:
            if off <= p_off < off + n:
                return cs + p_off - off
        raise ValueError(p_off)
    Mc = np.zeros(acc, np.uint16); Vc = np.zeros(acc, np.uint16)
    grads = [([b.astype(f32) for b in blocks], e.astype(f32), n.astype(f32)) for blocks, e, n in grads16]
    norms = loader.fused_steps(impl, lay, P, st, Mc, Vc, cs_of, grads, wdf=0.0)
    return dict(P=P, d=st["d"], r=st["r"], s=st["s"], m8=st["m8"], v8=st["v8"], m8s=st["m8s"], v8s=st["v8s"],
                Mc=Mc, Vc=Vc, norms=norms, sref=sp["sref"].copy())


def fused_inputs(seed=11):
    lay = loader.fused_layout(3, 20, 4, 32, 32)
    rng = np.random.default_rng(seed)
    P0 = (rng.standard_normal(lay["np"]) * 0.02).astype(f32)
    grads16 = []
    for t in range(3):
        sc = (0.02, 0.004, 0.05)[t]                      # norms above and below 1: the clip switches on and off
        blocks = [(rng.standard_normal(lay["per"]) * sc).astype(np.float16) for _ in range(lay["L"])]
        grads16.append((blocks, (rng.standard_normal(32 * 20) * sc).astype(np.float16),
                        (rng.standard_normal(20) * sc).astype(np.float16)))
    return P0, grads16


def golden_fused(ref):
    """qlm_fused_layer / qlm_fused_tail composed from the reference's own kernels (cudalm.cu:6105-6187)."""
    P0, grads16 = fused_inputs()
    out = fused_case(ref, P0, grads16)
    out = {"out_" + k: v for k, v in out.items()}
    out["P0"] = P0
    for t, (blocks, e, n) in enumerate(grads16):
        out["g%d_layers" % t] = np.stack(blocks); out["g%d_emb" % t] = e; out["g%d_nf" % t] = n
    np.savez_compressed(os.path.join(OUT, "fused_update.npz"), **out)


def golden_state_v4(ref):
    """QLM_V4 (qlm.cuh:62-72): the same ragged state sequence with v8 holding the fourth root of the second moment."""
    ref.set_v4(1)
    try:
        golden_state(ref, "state_g128_v4", [128 * 12, 1000, 78], 128, 7, 1, 5, seed=6)
    finally:
        ref.set_v4(0)


def golden_ngram(ref):
    """The 4-bit n-gram table update (NGRAM_Q4_FOLD; ng_build_touched, k_ng_scatter_compact, k_ng_q4_step,
    cudalm.cu:4465-4530, 4673-4745) through the reference's CPU kernels: three steps on a table of 1024 rows x 32."""
    rng = np.random.default_rng(21)
    R, De, group, dmax = 1024, 32, 128, 7
    nt = R * De
    sp, nq, ng = loader.make_spans([nt], group)
    P = (rng.standard_normal(nt) * 0.02).astype(f32)
    d = np.zeros(nt // 2, np.int8); r = np.zeros(nt, np.int8); s = np.zeros(ng, f32)
    Praw = P.copy()
    ref.encode(P, d, r, s, sp, group, dmax, 1)
    sref = f32(s.astype(np.float64).sum() / ng)
    ref.render(P, d, s, sp, group, 1)
    out = dict(Praw=Praw, P0=P.copy(), d0=d.copy(), r0=r.copy(), s0=s.copy(), sref=np.array([sref], f32), cfg=np.array([R, De, group, dmax]))
    m8 = np.zeros(nt, np.int8); v8 = np.zeros(nt, np.uint8); m8s = np.zeros(ng, f32); v8s = np.zeros(ng, f32)
    Nd = 300
    for t in (1, 2, 3):
        key = rng.integers(0, R, 2 * Nd).astype(np.int32)
        key[rng.integers(0, 2 * Nd, 40)] = -1                       # masked positions
        key[100:140] = key[50]                                      # one heavily repeated row
        dbuf = (rng.standard_normal((Nd, De)) * 1e-3).astype(f32)
        gs = np.array([0.5 if t == 2 else 1.0, 0.0], f32)
        tgi, cidx = ref.ng_touched(key, De, group, ng)
        Gc = np.zeros(tgi.size * group, f32)
        ref.ng_scatter_compact(Gc, key, cidx, dbuf, De, group, Nd)
        i1, i2 = bias_corr(0.9, 0.95, t)
        ref.ng_step(P, Gc, d, r, s, m8, m8s, v8, v8s, tgi, group, dmax, 3e-3, 0.9, 0.95, 0.0, float(sref), i1, i2, t, nt, gs)
        out["key%d" % t] = key; out["dbuf%d" % t] = dbuf; out["gs%d" % t] = gs
        out["touched%d" % t] = np.sort(tgi)
    out.update(P=P, d=d, r=r, m8=m8, v8=v8, m8s=m8s, v8s=v8s)
    np.savez_compressed(os.path.join(OUT, "ngram_q4.npz"), **out)


def golden_router_bias(ref):
    """The selection-bias update after a step's routing (mbias_upd, cudalm.cu:3793-3802, called as at 4385): three
    updates in a row for the per-pass and the combined form, proportional and sign rule, u = 0.001 x a layer multiplier."""
    out = {}
    N, E, K = 4096, 64, 2
    for per_slot in (1, 0):
        for prop in (1, 0):
            rng = np.random.default_rng(31 + 2 * per_slot + prop)
            rows = K if per_slot else 1
            b = (rng.standard_normal((rows, E)) * 0.01).astype(f32)
            tag = "s%d_p%d" % (per_slot, prop)
            out["b0_" + tag] = b.copy()
            for it in range(3):
                asg = rng.integers(0, E, (K, N)).astype(np.int32)
                asg[0, : N // 4] = 3                       # a hot expert
                if per_slot:
                    asg[1] = np.arange(N) % E              # every expert exactly at the target load
                cs = (np.stack([np.bincount(asg[k], minlength=E) for k in range(K)]) if per_slot
                      else np.bincount(asg.ravel(), minlength=E)[None]).astype(np.int32)
                m = f32(N) / f32(E) if per_slot else f32(K) * f32(N) / f32(E)
                ref.mbias_upd(b, np.ascontiguousarray(cs), float(m), 0.001, 1.5, prop)
                out["asg%d_%s" % (it, tag)] = asg
            out["b_" + tag] = b.copy()
    out["cfg"] = np.array([N, E, K])
    out["u"] = np.array([f32(0.001) * f32(1.5)], f32)
    np.savez_compressed(os.path.join(OUT, "router_bias.npz"), **out)


def golden_nggate(ref):
    """The n-gram table's context gate through the reference's CPU kernels (k_nggate_f / k_nggate_b, cpu_kern.h:573-589):
    12 rows of 256, keys correlated with the stream so that the gates spread."""
    rng = np.random.default_rng(9)
    N, D = 12, 256
    h, v, k, dy = [rng.standard_normal((N, D)).astype(f32) for _ in range(4)]
    k = (3.0 * k).astype(f32)
    k[:, :64] += 4.0 * h[:, :64] * np.linspace(-1, 1, N, dtype=f32)[:, None]
    out = dict(h0=h.copy(), v=v, k0=k.copy(), dy0=dy.copy())
    hn, g, rh, rk = ref.nggate_f(h, v, k)
    dv, dk = ref.nggate_b(dy, v, hn, k, g, rh, rk)
    out.update(h=h, k=k, hn=hn, g=g, rh=rh, rk=rk, dy=dy, dv=dv, dk=dk)
    np.savez_compressed(os.path.join(OUT, "nggate.npz"), **out)


def golden_engram(ref):
    """Sparse engram (cudalm.cu:4963-5098): keys of S = 2 orders x 2 heads sub-tables (with and without a canonical
    token map), the gather, and the compact gradient rows of the touched groups."""
    rng = np.random.default_rng(31)
    V, T, B, De, grp = 500, 32, 6, 32, 128
    ords = np.array([2, 2, 3, 3], np.int32); S = ords.size
    Rraw = 257; al = 128 // De; Rp = (Rraw + al - 1) // al * al
    prime, mult = ref.eg_tables(Rraw, ords)
    N = B * T
    tok = rng.integers(0, V, N).astype(np.int32)
    tok[40:60] = tok[8:28]                                              # repeated context: shared rows
    canon = rng.integers(0, V, V).astype(np.uint16)
    key = ref.eg_key(tok, None, T, S, Rp); keyc = ref.eg_key(tok, canon, T, S, Rp)
    tbl = (rng.standard_normal((S * Rp, De)) * 0.02).astype(f32)
    buf = ref.eg_gather(tbl, key, N, S, De)
    ngrp = S * Rp * De // grp
    tgi, cidx = ref.ng_touched(key, De, grp, ngrp)
    db = (rng.standard_normal((N, S * De)) * 1e-3).astype(f32)
    Gc = np.zeros(tgi.size * grp, f32)
    ref.eg_scatter_c(Gc, key, cidx, db, N, S, De, grp)
    order = np.argsort(tgi)                                             # rows in ascending group order
    np.savez_compressed(os.path.join(OUT, "engram.npz"), cfg=np.array([V, T, B, De, grp, Rraw, Rp]), ords=ords, prime=prime,
                        mult=mult, tok=tok, canon=canon, key=key, keyc=keyc, tbl=tbl, buf=buf, db=db, touched=tgi[order],
                        Gc=Gc.reshape(-1, grp)[order])


def golden_q4n(ref):
    """Exact 4-bit export (quantize_params / dequantize_params qtype 3, cudalm.cu:639-656, 688-695) of a vector whose
    groups are: rendered 4-bit digits with full range, with small digits only, all zero, tiny scales, a float span
    (no grid: stored raw), one value off the grid, and a short last group."""
    rng = np.random.default_rng(41)
    group = 128
    parts = []
    for g in range(24):
        sc = f32(np.exp(rng.uniform(-12, -2)))
        hi = 7 if g % 3 else int(rng.integers(1, 7))
        parts.append((rng.integers(-hi, hi + 1, group).astype(f32) * sc).astype(f32))
    parts.append(np.zeros(group, f32))
    parts.append((rng.integers(-7, 8, group).astype(f32) * f32(3e-41)).astype(f32))      # subnormal scale
    parts.append((rng.standard_normal(group) * 0.02).astype(f32))                           # no grid
    on = (rng.integers(-7, 8, group).astype(f32) * f32(0.0123)).astype(f32); on[77] = np.nextafter(on[77], f32(1))
    parts.append(on)
    parts.append(np.ones(group, f32))                                                       # gains
    parts.append((rng.integers(-7, 8, 70).astype(f32) * f32(0.004)).astype(f32))           # short tail
    P = np.concatenate(parts)
    q = ref.q4n_export(P, group)
    back = ref.q4n_decode(q, P.size, group)
    assert back is not None and (back.view(np.uint32) == P.view(np.uint32)).all()
    np.savez_compressed(os.path.join(OUT, "q4n.npz"), P=P, q=q, group=np.array([group]))


def main():
    ref = loader.reference(exact=True)
    if ref is None:
        sys.exit("oracle/_ref/libcudalm_ref_exact.so missing: run `make -C oracle ref` first")
    single = {"router_bias": golden_router_bias, "nggate": golden_nggate, "engram": golden_engram, "q4n": golden_q4n}
    if len(sys.argv) == 2 and sys.argv[1] in single:       # one fixture alone: python make_golden.py router_bias
        single[sys.argv[1]](ref)
        return
    golden_hash(ref)
    golden_one_group(ref)
    golden_state(ref, "state_g128", [128 * 40, 1000, 78, 128 * 3 + 2], 128, 7, 1, 6, seed=1)
    golden_state(ref, "state_g64_abs", [640, 130, 64], 64, 3, 1, 4, seed=2, lrmode=1)
    golden_state(ref, "state_g96_int8", [960, 100], 96, 127, 0, 4, seed=3)
    golden_state(ref, "state_g256_lion", [2560, 300], 256, 1, 1, 4, seed=4, adam=0)
    golden_gnorm(ref)
    golden_router(ref)
    golden_linear(ref)
    golden_moe(ref)
    golden_statefile(ref)
    golden_fused(ref)
    golden_state_v4(ref)
    golden_ngram(ref)
    golden_router_bias(ref)
    golden_nggate(ref)
    golden_engram(ref)
    golden_q4n(ref)
    for f in sorted(os.listdir(OUT)):
        if f.endswith(".npz"):
            print("%-24s %8d B" % (f, os.path.getsize(os.path.join(OUT, f))))


if __name__ == "__main__":
    main()
