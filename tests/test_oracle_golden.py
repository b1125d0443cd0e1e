"""Pins the C restatement (oracle/qlm_oracle.c) to vectors produced by the
unmodified reference (tests/golden/make_golden.py).  Integer state: bit-exact."""
import numpy as np
import pytest

from conftest import golden
from oracle import loader

f32 = np.float32


def bias_corr(b1, b2, t):
    bc1 = f32(1) - f32(np.power(f32(b1), f32(t)))
    bc2 = f32(1) - f32(np.power(f32(b2), f32(t)))
    return float(f32(1) / bc1), float(f32(1) / np.sqrt(bc2))


def test_hash_and_stochastic_rounding(oracle):
    g = golden("hash")
    assert [oracle.hash(int(x)) for x in g["xs"]] == list(g["hs"])
    # the reference survey's table
    assert oracle.hash(0) == 0x7B1DCDAF and oracle.hash(0xFFFFFFFFFFFFFFFF) == 0x1B652C20
    assert [oracle.sround(0.5, i, 1) for i in range(8)] == [0, 0, 0, 1, 0, 1, 1, 1]
    assert [oracle.sround(-0.5, i, 1) for i in range(8)] == [-1, -1, -1, 0, -1, 0, 0, 0]
    for a, v in enumerate(g["vals"]):
        for b, i in enumerate(g["idx"]):
            for c, t in enumerate(g["ts"]):
                assert oracle.sround(float(v), int(i), int(t)) == g["sr"][a, b, c]


def test_one_group_known_answers(oracle):
    g = golden("one_group")
    sp, nq, ng = loader.make_spans([128])
    d = np.zeros(64, np.int8); r = np.zeros(128, np.int8); s = np.zeros(1, f32)
    oracle.encode(g["P"], d, r, s, sp)
    assert s.view(np.uint32)[0] == 0x3C15CBED
    assert bytes(d[:16].view(np.uint8)).hex() == "9999a9aaaaaaaabbbbbbbbcbcccccccc"
    assert list(r[:16]) == [0, 14, 28, 42, 56, -58, -44, -30, -16, -2, 12, 26, 40, 54, -60, -46]
    assert (d == g["d0"]).all() and (r == g["r0"]).all()
    sp[0]["sref"] = s[0]
    m8 = np.zeros(128, np.int8); v8 = np.zeros(128, np.uint8)
    m8s = np.zeros(1, f32); v8s = np.zeros(1, f32); P = np.zeros(128, f32)
    for t in (1, 2):
        i1, i2 = bias_corr(0.9, 0.95, t)
        oracle.step(P, g["G"], d, r, s, m8, m8s, v8, v8s, sp, lr=3e-4, b1=0.9, b2=0.95, wd=0.1,
                    inv_bc1=i1, inv_sqrt_bc2=i2, t=t)
        for k, v in dict(d=d, r=r, m8=m8, v8=v8, m8s=m8s, v8s=v8s, P=P).items():
            assert (v == g["%s_t%d" % (k, t)]).all(), (k, t)
    assert list(m8[:8]) == [-127, -84, -43, 0, 42, 84, 127, -127]


@pytest.mark.parametrize("name", ["state_g128", "state_g64_abs", "state_g96_int8", "state_g256_lion"])
def test_state_sequences(oracle, name):
    g = golden(name)
    group, dmax, packed, steps, lrmode, adam = [int(x) for x in g["cfg"]]
    sp, nq, ng = loader.make_spans([int(x) for x in g["sizes"]], group)
    d = np.zeros_like(g["d0"]); r = np.zeros_like(g["r0"]); s = np.zeros_like(g["s0"])
    oracle.encode(g["P"], d, r, s, sp, group, dmax, packed)
    assert (d == g["d0"]).all() and (r == g["r0"]).all() and (s == g["s0"]).all()
    sp["sref"] = g["sref"]
    m8 = np.zeros(nq, np.int8); v8 = np.zeros(nq, np.uint8)
    m8s = np.zeros(ng, f32); v8s = np.zeros(ng, f32); P = np.zeros(nq, f32)
    for t in range(1, steps + 1):
        i1, i2 = bias_corr(0.9, 0.95, t)
        stat = np.zeros(4, np.int64)
        oracle.step(P, g["G"][t - 1], d, r, s, m8, m8s, v8, v8s, sp, group=group, dmax=dmax, lr=3e-4,
                    b1=0.9, b2=0.95, wd=0.1, gscale=float(g["gscale"][t - 1]), inv_bc1=i1, inv_sqrt_bc2=i2,
                    lrmode=lrmode, t=t, adam=adam, stat=stat, packed=packed)
        if t == 3:
            oracle.servo(d, r, s, sp, group, dmax, 0.9 / group, 0.2 / group, packed)
        for k, v in dict(d=d, r=r, s=s, m8=m8, v8=v8, m8s=m8s, v8s=v8s, stat=stat).items():
            assert (v == g["%s_t%d" % (k, t)]).all(), (k, t)
    oracle.render(P, d, s, sp, group, packed)
    assert (P == g["P_final"]).all()


def test_state_sequence_v4(oracle):
    """QLM_V4 (qlm.cuh:62-72): v8 holds the fourth root of the second moment."""
    oracle.set_v4(1)
    try:
        test_state_sequences(oracle, "state_g128_v4")
    finally:
        oracle.set_v4(0)


def test_gnorm(oracle):
    g = golden("gnorm")
    assert (oracle.gnorm(g["G"]) == g["gs_plain"]).all()
    assert (oracle.gnorm(g["G"], [g["side"]], 1) == g["gs_side"]).all()
    assert (oracle.gnorm(g["G"], [g["side"]], 0) == g["gs_noclip"]).all()
    assert (oracle.gnorm(g["small"]) == g["gs_small"]).all()
    assert oracle.gnorm(g["small"])[0] == 1.0          # norm below 1: no clipping
    bad = g["side"].copy(); bad[5] = np.inf
    assert np.isnan(oracle.gnorm(g["G"], [bad], 0)[1])  # a non-finite side poisons the norm


def test_router(oracle):
    g = golden("router")
    for tag, K in dict(a=2, b=3, c=1, d=8).items():
        rt = g[tag + "_rt"]
        for bt, bias in (("nb", None), ("wb", g[tag + "_bias"])):
            rp, asg, gt = oracle.router_topk(rt, K, bias, rt.shape[1] if bias is not None else 0)
            assert (rp == g["%s_%s_rprobs" % (tag, bt)]).all()
            assert (asg == g["%s_%s_assign" % (tag, bt)]).all()
            assert (gt == g["%s_%s_gate" % (tag, bt)]).all()
    # ties go to the lowest index
    assert golden("router")["a_nb_assign"][0, 3] == 0


def test_perm_matches_reference_layer():
    g = golden("moe")
    o = loader.restatement()
    N, D, F, E, K = [int(x) for x in g["shape"]]
    perm, inv, off, bad = o.perm_build(g["assign"], E, merged=0)
    assert bad == 0
    assert (perm.reshape(K, N) == g["perm"]).all()
    assert (off.reshape(K, E + 1) == g["hoff"]).all()
    # merged form: inverse really inverts, experts ascending, stable inside an expert
    perm, inv, off, bad = o.perm_build(g["assign"], E, merged=1)
    flat = g["assign"].reshape(-1)
    assert (perm[inv] == np.arange(K * N)).all()
    assert (np.diff(flat[perm]) >= 0).all()
    for e in range(E):
        seg = perm[off[e]:off[e + 1]]
        assert (np.diff(seg) > 0).all()
    asg_bad = g["assign"].copy(); asg_bad[0, 7] = E + 3
    assert o.perm_build(asg_bad, E, merged=0)[3] == 1 + E + 3


def test_linear_restatement(oracle):
    g = golden("linear")
    X, dY, d, s = g["X"], g["dY"], g["d"], g["s"]
    M, K = X.shape
    N = dY.shape[1]
    rel = lambda a, b: np.abs(a - b).max() / np.abs(b).max()
    assert rel(oracle.linear_fwd(X, d, s, 0, N), g["Y_kn"]) < 1e-5
    assert rel(oracle.linear_fwd(X, d, s, 1, N), g["Y_nk"]) < 1e-5
    assert rel(oracle.linear_dgrad(dY, d, s, 0, K), g["dX_kn"]) < 1e-5
    assert rel(oracle.linear_dgrad(dY, d, s, 1, K), g["dX_nk"]) < 1e-5
    assert rel(oracle.linear_wgrad(np.zeros((K, N), f32), dY, X, 0), g["dW_kn"]) < 1e-5
    assert rel(oracle.linear_wgrad(np.zeros((N, K), f32), dY, X, 1), g["dW_nk"]) < 1e-5


def test_moe_restatement(oracle):
    g = golden("moe")
    N, D, F, E, K = [int(x) for x in g["shape"]]
    q1, q3, q2 = (g["d1"], g["s1"]), (g["d3"], g["s3"]), (g["d2"], g["s2"])
    fw = oracle.moe_fwd(g["fi"], g["fn"], g["Wr"], q1, q3, q2, F, K)
    rel = lambda a, b: np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)
    assert (fw["assign"] == g["assign"]).all()
    assert rel(fw["rprobs"], g["rprobs"]) < 1e-5 and rel(fw["gate"], g["gate"]) < 1e-5
    assert rel(fw["out"], g["out"]) < 1e-5
    bw = oracle.moe_bwd(g["dout"], g["fn"], g["Wr"], q1, q3, q2, F, K, fw, aux=float(g["aux"]))
    assert rel(bw["dfnorm"], g["dfnorm"]) < 1e-5
    assert rel(bw["d_gate"], g["d_gate"]) < 1e-5
    assert rel(bw["dWr"].ravel(), g["dWr"]) < 1e-5
    for k in ("dW1", "dW3", "dW2"):            # stored as fp16 in the fixture
        assert rel(bw[k].ravel(), g[k].astype(f32)) < 2e-3


def test_fused_per_layer_update(oracle):
    """The restatement's sqsum / step / adamw composed as qlm_fused_layer / qlm_fused_tail
    (cudalm.cu:6105-6187) reproduce the reference's bytes on the fused fixture."""
    import os
    import sys
    sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
    import make_golden as mg
    g = golden("fused_update")
    grads16 = [(list(g["g%d_layers" % t]), g["g%d_emb" % t], g["g%d_nf" % t]) for t in range(3)]
    out = mg.fused_case(oracle, g["P0"], grads16)
    for k, v in out.items():
        assert np.array_equal(v, g["out_" + k]), k
    assert out["norms"][0] > 1.0 > out["norms"][1]          # the clip switches on for step 2 and off for step 3


def test_router_bias_update_restatement():
    """The float32 restatement of mbias_upd (oracle/loader.py, cudalm.cu:3793-3798, 4385) against the reference's own
    function on the same assignments: per-pass and combined counts, proportional and sign rule, three updates each."""
    g = golden("router_bias")
    N, E, K = [int(x) for x in g["cfg"]]
    u = float(g["u"][0])
    for per_slot in (1, 0):
        for prop in (1, 0):
            tag = "s%d_p%d" % (per_slot, prop)
            b = g["b0_" + tag].copy()
            for it in range(3):
                b = loader.bias_update_np(b, g["asg%d_%s" % (it, tag)], E, per_slot, u, prop)
            assert np.array_equal(b, g["b_" + tag]), tag
            assert not np.array_equal(b, g["b0_" + tag])


def test_router_bias_update_c_restatement(oracle):
    """qo_bias_update (oracle/qlm_oracle.c) on the fixture's counts: the reference's rows bit for bit."""
    g = golden("router_bias")
    N, E, K = [int(x) for x in g["cfg"]]
    u = float(g["u"][0])
    for per_slot in (1, 0):
        for prop in (1, 0):
            tag = "s%d_p%d" % (per_slot, prop)
            b = g["b0_" + tag].copy()
            for it in range(3):
                asg = g["asg%d_%s" % (it, tag)]
                cs = (np.stack([np.bincount(asg[k], minlength=E) for k in range(K)]) if per_slot
                      else np.bincount(asg.ravel(), minlength=E)[None]).astype(np.int32)
                m = np.float32(N) / np.float32(E) if per_slot else np.float32(K) * np.float32(N) / np.float32(E)
                oracle.bias_update(b, np.ascontiguousarray(cs), float(m), u, prop)
            assert np.array_equal(b, g["b_" + tag]), tag


def test_ngram_context_gate_restatement(oracle):
    """qo_nggate_f / qo_nggate_b against the reference's CPU kernels (fixture): 1e-5 relative, the row sums are taken in
    double here and in the kernels' own float orders there."""
    g = golden("nggate")
    rel = lambda a, b: float(np.abs(a - b).max() / np.abs(b).max())
    h, k, dy = g["h0"].copy(), g["k0"].copy(), g["dy0"].copy()
    hn, gg, rh, rk = oracle.nggate_f(h, g["v"], k)
    assert g["g"].std() > 0.05
    for a, b in ((gg, g["g"]), (rh, g["rh"]), (rk, g["rk"]), (hn, g["hn"]), (k, g["k"]), (h, g["h"])):
        assert rel(a, b) < 1e-5
    dv, dk = oracle.nggate_b(dy, g["v"], g["hn"], g["k"], g["g"], g["rh"], g["rk"])
    for a, b in ((dv, g["dv"]), (dk, g["dk"]), (dy, g["dy"])):
        assert rel(a, b) < 1e-5
