"""Router top-k and the expert-grouping permutation through the C ABI.
Bar: bit-exact against the reference's vectors and the oracle."""
import numpy as np
import pytest
import torch

from conftest import golden

pytestmark = pytest.mark.gpu
f32 = np.float32


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def test_router_topk_golden(cuda):
    from cudalm_c_b200 import moe
    g = golden("router")
    for tag, K in dict(a=2, b=3, c=1, d=8).items():
        rt = g[tag + "_rt"]
        for bt, bias in (("nb", None), ("wb", g[tag + "_bias"])):
            b = dev(bias, cuda) if bias is not None else None
            _, rp, asg, gt = moe.router_topk(rt=dev(rt, cuda), K=K, bias=b, bias_stride=rt.shape[1] if b is not None else 0)
            assert (rp.cpu().numpy() == g["%s_%s_rprobs" % (tag, bt)]).all(), (tag, bt)
            assert (asg.cpu().numpy() == g["%s_%s_assign" % (tag, bt)]).all(), (tag, bt)
            assert (gt.cpu().numpy() == g["%s_%s_gate" % (tag, bt)]).all(), (tag, bt)


def test_router_logits_fused(cuda, oracle):
    """Logits computed on the device (fp32 accumulate) agree with X@Wr to 1e-5 rel;
    given those logits the selection equals the oracle's exactly."""
    from cudalm_c_b200 import moe
    rng = np.random.default_rng(3)
    N, D, E, K = 1000, 768, 32, 2
    X = rng.standard_normal((N, D)).astype(f32)
    Wr = (rng.standard_normal((D, E)) * 0.02).astype(f32)
    for xdt in (torch.float32, torch.bfloat16):
        Xd = dev(X, cuda).to(xdt)
        rt, rp, asg, gt = moe.router_topk(X=Xd, Wr=dev(Wr, cuda), K=K)
        ref = Xd.float().cpu().numpy().astype(np.float64) @ Wr.astype(np.float64)
        assert np.abs(rt.cpu().numpy() - ref).max() / np.abs(ref).max() < 1e-5
        rp2, asg2, gt2 = oracle.router_topk(rt.cpu().numpy(), K)
        assert (rp.cpu().numpy() == rp2).all() and (asg.cpu().numpy() == asg2).all() and (gt.cpu().numpy() == gt2).all()


@pytest.mark.parametrize("E,K", [(33, 2), (48, 3), (64, 8), (100, 2), (128, 1), (200, 4), (256, 8)])
def test_router_topk_wide_matches_oracle(cuda, oracle, E, K):
    """More than 32 experts (one warp per token, several experts per lane): probabilities, choices and gates equal
    the oracle's bit for bit, with and without a selection bias, including exact ties between logits."""
    from cudalm_c_b200 import moe
    rng = np.random.default_rng(E * 10 + K)
    N = 777
    rt = (rng.standard_normal((N, E)) * 2.0).astype(f32)
    rt[:50, 5] = rt[:50, 40 % E]                     # exact ties: the lower index must win
    rt[50:60] = 0.25                                 # a whole row of ties
    bias = (rng.standard_normal((K, E)) * 0.01).astype(f32)
    for b in (None, bias):
        db = dev(b, cuda) if b is not None else None
        _, rp, asg, gt = moe.router_topk(rt=dev(rt, cuda), K=K, bias=db, bias_stride=E if b is not None else 0)
        rp2, asg2, gt2 = oracle.router_topk(rt, K, bias=b, bs=E if b is not None else 0)
        assert (rp.cpu().numpy() == rp2).all()
        assert (asg.cpu().numpy() == asg2).all()
        assert (gt.cpu().numpy() == gt2).all()


@pytest.mark.parametrize("N,E,K", [(5000, 7, 2), (8192, 32, 2), (64, 4, 1), (1500, 256, 8), (1, 3, 1), (16384, 32, 8), (33, 2, 1),
                                   (4097, 5, 2), (65536, 64, 2)])
def test_perm_matches_oracle(cuda, oracle, N, E, K):
    from cudalm_c_b200 import moe
    rng = np.random.default_rng(N + E)
    asg = rng.integers(0, E, size=(K, N)).astype(np.int32)
    if N > 100:
        asg[:, : N // 3] = 1 % E                    # a heavily loaded expert and (for E>2) empty ones
    for merged in (False, True):
        perm, inv, off, counts, bad = moe.moe_perm_all(dev(asg, cuda), E, merged=merged, pad=1)
        p2, i2, o2, b2 = oracle.perm_build(asg, E, merged=1 if merged else 0)
        assert int(bad.item()) == 0 and b2 == 0
        assert (perm.cpu().numpy().reshape(-1) == p2).all()
        assert (inv.cpu().numpy().reshape(-1) == i2).all()
        assert (off.cpu().numpy().reshape(-1) == o2).all()


def test_perm_matches_reference_layer(cuda):
    from cudalm_c_b200 import moe
    g = golden("moe")
    N, D, F, E, K = [int(x) for x in g["shape"]]
    perm, inv, off, counts, bad = moe.moe_perm_all(dev(g["assign"], cuda), E, merged=False, pad=1)
    assert (perm.cpu().numpy() == g["perm"]).all()
    assert (off.cpu().numpy() == g["hoff"]).all()


def test_perm_padded(cuda, oracle):
    """pad=128: every expert segment starts on a 128-row boundary, filler rows are
    -1, real rows keep the stable order, inv points at the padded positions."""
    from cudalm_c_b200 import moe
    rng = np.random.default_rng(77)
    N, E, K = 3000, 32, 2
    asg = rng.integers(0, E, size=(K, N)).astype(np.int32)
    asg[asg == 5] = 6                               # expert 5 empty
    perm, inv, off, counts, bad = moe.moe_perm_all(dev(asg, cuda), E, merged=True, pad=128)
    perm, inv, off, counts = [x.cpu().numpy().reshape(-1) for x in (perm, inv, off, counts)]
    p2, i2, o2, _ = oracle.perm_build(asg, E, merged=1)
    assert (counts == np.diff(o2)).all()
    assert (off % 128 == 0).all() and off[0] == 0
    assert (np.diff(off) == (counts + 127) // 128 * 128).all()
    for e in range(E):
        seg = perm[off[e]:off[e + 1]]
        assert (seg[:counts[e]] == p2[o2[e]:o2[e + 1]]).all()
        assert (seg[counts[e]:] == -1).all()
    assert (perm[inv] == np.arange(K * N)).all()


def test_perm_out_of_range_expert_is_flagged(cuda):
    from cudalm_c_b200 import moe
    asg = np.zeros((2, 100), np.int32); asg[1, 17] = 9
    perm, inv, off, counts, bad = moe.moe_perm_all(dev(asg, cuda), 4, merged=False, pad=1)
    assert int(bad.item()) == (9 | 0x40000000)
    import cudalm_c_b200 as q
    with pytest.raises(q.QlmbError):
        q.check(q.lib().qlmb_check_device(None))     # the error word was set ...
    q.check(q.lib().qlmb_check_device(None))         # ... and cleared by the read


@pytest.mark.parametrize("per_slot,prop", [(True, True), (True, False), (False, True), (False, False)])
def test_router_bias_update(cuda, per_slot, prop):
    """mbias_upd (cudalm.cu:3793-3798) restated in numpy float32; three updates in a row, bit-exact."""
    from cudalm_c_b200 import moe
    rng = np.random.default_rng(31 + 2 * per_slot + prop)
    N, E, K = 4096, 64, 2
    u = f32(0.001) * f32(1.5)
    rows = K if per_slot else 1
    b = (rng.standard_normal((rows, E)) * 0.01).astype(f32)
    db = dev(b, cuda)
    for it in range(3):
        asg = rng.integers(0, E, (K, N)).astype(np.int32)
        asg[0, : N // 4] = 3                       # a hot expert, and one that gets exactly the target load
        if per_slot:
            asg[1] = np.arange(N) % E
        moe.router_bias_update(db, dev(asg, cuda), E, per_slot=per_slot, u=float(u), proportional=prop)
        m = f32(N) / f32(E) if per_slot else f32(K) * f32(N) / f32(E)
        for s in range(rows):
            c = np.bincount((asg[s] if per_slot else asg.ravel()), minlength=E).astype(f32)
            d = (m - c) / m if prop else np.where(c < m, f32(1), np.where(c > m, f32(-1), f32(0))).astype(f32)
            b[s] = b[s] + (u * d.astype(f32)).astype(f32)
    assert np.array_equal(db.cpu().numpy(), b)


def test_router_bias_update_matches_reference(cuda):
    """qlmb_router_bias_update against the bias rows the reference's mbias_upd leaves (fixture): bit-exact."""
    from cudalm_c_b200 import moe
    g = golden("router_bias")
    N, E, K = [int(x) for x in g["cfg"]]
    u = float(g["u"][0])
    for per_slot in (1, 0):
        for prop in (1, 0):
            tag = "s%d_p%d" % (per_slot, prop)
            db = dev(g["b0_" + tag], cuda)
            for it in range(3):
                moe.router_bias_update(db, dev(g["asg%d_%s" % (it, tag)], cuda), E, per_slot=bool(per_slot), u=u,
                                       proportional=bool(prop))
            assert np.array_equal(db.cpu().numpy(), g["b_" + tag]), tag
