"""Embedding, RMSNorm, RoPE and softmax cross-entropy through the C ABI against the reference's CPU
kernels (cpu_kern.h:87-152, 489-503, compiled from the reference's sources).  fp32 activations: 1e-5
relative (summation order inside a row differs), the embedding gradient bit-exact (same order);
bf16 activations: compared after the same rounding of the inputs, 1e-2."""
import numpy as np
import pytest
import torch

from oracle import loader

pytestmark = pytest.mark.gpu


def rel(a, b):
    a, b = np.asarray(a, np.float64), np.asarray(b, np.float64)
    return np.abs(a - b).max() / max(np.abs(b).max(), 1e-30)


@pytest.fixture(scope="module")
def ref():
    r = loader.reference()
    if r is None:
        pytest.skip("compiled reference not present (make -C oracle ref)")
    return r


def test_embed_and_gradient(cuda, ref):
    from cudalm_c_b200 import block
    rng = np.random.default_rng(0)
    V, D, N = 300, 768, 4096
    emb = rng.standard_normal((V, D)).astype(np.float32)
    tok = rng.integers(0, V, N).astype(np.int32); tok[:50] = 7          # one heavily repeated token
    dout = rng.standard_normal((N, D)).astype(np.float32)
    X = block.embed(torch.from_numpy(emb).to(cuda), torch.from_numpy(tok).to(cuda))
    assert (X.cpu().numpy() == ref.embed(emb, tok)).all()
    G0 = rng.standard_normal((V, D)).astype(np.float32)
    G = torch.from_numpy(G0.copy()).to(cuda)
    block.embed_bwd(G, torch.from_numpy(dout).to(cuda), torch.from_numpy(tok).to(cuda))
    Gr = G0.copy(); ref.embed_bwd(Gr, dout, tok)
    got = G.cpu().numpy()
    # the reference adds row by row into G; the device sums a token's rows first and adds once
    assert rel(got, Gr) < 1e-5
    Gb = torch.zeros(V, D, device=cuda)
    block.embed_bwd(Gb, torch.from_numpy(dout).to(cuda).bfloat16(), torch.from_numpy(tok).to(cuda))
    Gr = np.zeros((V, D), np.float32); ref.embed_bwd(Gr, torch.from_numpy(dout).bfloat16().float().numpy(), tok)
    assert rel(Gb.cpu().numpy(), Gr) < 1e-5


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rmsnorm(cuda, ref, dt):
    from cudalm_c_b200 import block
    rng = np.random.default_rng(1)
    N, D = 1000, 768
    X = torch.from_numpy(rng.standard_normal((N, D)).astype(np.float32)).to(dt)
    dy = torch.from_numpy(rng.standard_normal((N, D)).astype(np.float32)).to(dt)
    gamma = (1.0 + 0.1 * rng.standard_normal(D)).astype(np.float32)
    Xh, dyh = X.float().numpy(), dy.float().numpy()
    Or, rr = ref.rmsnorm(Xh, gamma)
    O, rinv = block.rmsnorm_fwd(X.to(cuda), torch.from_numpy(gamma).to(cuda))
    tol = 1e-5 if dt == torch.float32 else 1e-2
    assert rel(rinv.cpu().numpy(), rr) < 1e-5
    assert rel(O.float().cpu().numpy(), Or) < tol
    dx0 = rng.standard_normal((N, D)).astype(np.float32)
    dg0 = rng.standard_normal(D).astype(np.float32)
    dxr, dgr = dx0.copy(), dg0.copy()
    ref.rmsnorm_bwd(Xh, gamma, rr, dyh, dxr, dgr)
    dx = torch.from_numpy(dx0.copy()).to(cuda); dg = torch.from_numpy(dg0.copy()).to(cuda)
    block.rmsnorm_bwd(dx, X.to(cuda), torch.from_numpy(gamma).to(cuda), torch.from_numpy(rr).to(cuda), dy.to(cuda), dgamma=dg)
    assert rel(dx.cpu().numpy(), dxr) < 1e-5
    assert rel(dg.cpu().numpy(), dgr) < 1e-5


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_rope(cuda, ref, dt):
    from cudalm_c_b200 import block
    rng = np.random.default_rng(2)
    B, T, nh, hd = 3, 100, 4, 64
    cosb, sinb = block.rope_tables(T, hd)
    buf = torch.from_numpy(rng.standard_normal((B * T, nh * hd)).astype(np.float32)).to(dt)
    for back in (0, 1):
        r = buf.float().numpy().copy()
        ref.rope(r, cosb.numpy(), sinb.numpy(), nh, hd, T, back)
        d = buf.clone().to(cuda)
        block.rope(d, cosb.to(cuda), sinb.to(cuda), nh, hd, T, back=bool(back))
        assert rel(d.float().cpu().numpy(), r) < (1e-6 if dt == torch.float32 else 1e-2)


def test_softmax_ce(cuda, ref):
    from cudalm_c_b200 import block
    rng = np.random.default_rng(3)
    rows, V = 64, 16384
    lg = (rng.standard_normal((rows, V)) * 3).astype(np.float32)
    tgt = rng.integers(0, V, rows).astype(np.int32); tgt[5] = -1
    lr, dr = ref.softmax_ce(lg, tgt, rows)
    loss, dl = block.softmax_ce(torch.from_numpy(lg).to(cuda), torch.from_numpy(tgt).to(cuda), rows)
    assert np.abs(loss.cpu().numpy() - lr).max() < 1e-5 * max(1.0, np.abs(lr).max())
    assert rel(dl.cpu().numpy(), dr) < 1e-5
    assert loss[5] == 0 and (dl[5] == 0).all()


def test_lm_head_ce_and_backward(cuda, ref):
    """gpu_head_bwd (cudalm.cu:5790-5872) composed from the library's GEMMs and softmax_ce against the
    reference's g_abt / k_softmax_ce / g_ab / g_atb on the same bf16-rounded operands; the gradient of
    the logits is rounded to bf16 before the two backward GEMMs, hence 1e-2."""
    from cudalm_c_b200 import block
    rng = np.random.default_rng(4)
    N, D, V = 512, 256, 1024
    fn = torch.from_numpy(rng.standard_normal((N, D)).astype(np.float32)).bfloat16()
    emb = torch.from_numpy((rng.standard_normal((V, D)) * 0.05).astype(np.float32)).bfloat16().float()   # bf16-exact values
    tgt = rng.integers(0, V, N).astype(np.int32); tgt[3] = -1
    G0 = (rng.standard_normal((V, D)) * 0.01).astype(np.float32)
    G = torch.from_numpy(G0.copy()).to(cuda)
    loss, dfn = block.head_bwd(fn.to(cuda), emb.to(cuda), torch.from_numpy(tgt).to(cuda), G, chunk_rows=256)
    fnh, embh = fn.float().numpy(), emb.numpy()
    logits = ref.g_abt(fnh, embh)
    lr, dl = ref.softmax_ce(logits, tgt, N)
    dfnr = ref.g_ab(dl, embh)
    Gr = ref.g_atb(dl, fnh, G0.copy())
    assert np.abs(loss.cpu().numpy() - lr).max() < 2e-3
    a, b = dfn.float().cpu().numpy().astype(np.float64), dfnr.astype(np.float64)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 1e-2
    a, b = (G.cpu().numpy() - G0).astype(np.float64), (Gr - G0).astype(np.float64)
    assert np.linalg.norm(a - b) / np.linalg.norm(b) < 1e-2


def test_ngram_keys_and_gather(cuda, ref):
    """k_ngram_key / k_ngram_gather (cudalm.cu:4438-4451) against the reference's CPU kernels: keys bit-exact, the
    gathered sums bit-exact (same order); k_dec_ngkey gives the key the training kernel gives at the same position."""
    import cudalm_c_b200 as q
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    rng = np.random.default_rng(5)
    B, T, V, R, De = 3, 50, 500, 300, 32
    N = B * T
    tok = rng.integers(0, V, N).astype(np.int32)
    L = lib()
    d_tok = torch.from_numpy(tok).to(cuda)
    keys = []
    for order, base in ((2, 0), (3, R)):
        k = torch.zeros(N, dtype=torch.int32, device=cuda)
        check(L.qlmb_ngram_key(ptr(k), ptr(d_tok), N, T, R, order, base, stream_ptr()))
        kr = ref.ngram_key(tok, T, R, order, base)
        assert (k.cpu().numpy() == kr).all()
        keys.append(kr)
    key2 = np.concatenate(keys)                                     # two key sets, as with the trigram half on
    tbl = rng.standard_normal((2 * R, De)).astype(np.float32)
    buf = torch.zeros(N, De, device=cuda)
    d_tbl, d_key2 = torch.from_numpy(tbl).to(cuda), torch.from_numpy(key2).to(cuda)      # kept alive across the call
    check(L.qlmb_ngram_gather(ptr(buf), ptr(d_tbl), ptr(d_key2), N, De, 2, stream_ptr()))
    assert (buf.cpu().numpy() == ref.ngram_gather(tbl, key2, N, De, 2)).all()
    # decoder: slot b sits at position p of sequence b; its window holds the last four tokens
    p = 17
    tokw = np.stack([tok[b * T + p - 3:b * T + p + 1] for b in range(B)]).astype(np.int32)
    dk = torch.zeros(B, dtype=torch.int32, device=cuda)
    d_tokw, d_pos = torch.from_numpy(tokw).to(cuda), torch.full((B,), p, dtype=torch.int32, device=cuda)
    check(L.qlmb_dec_ngkey(ptr(dk), ptr(d_tokw), ptr(d_pos), B, R, 3, R, stream_ptr()))
    assert (dk.cpu().numpy() == keys[1].reshape(B, T)[:, p]).all()
    q.check(q.lib().qlmb_check_device(None))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ngram_context_gate(cuda, ref, dtype):
    """k_nggate_f / k_nggate_b (cudalm.cu:3362-3378) against the reference's CPU kernels.  fp32: 1e-5 relative (the
    row sums are taken in another order); bf16 storage: 1e-2, inputs rounded to bf16 on both sides."""
    from cudalm_c_b200 import block
    rng = np.random.default_rng(9)
    N, D = 203, 768
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    rnd = lambda a: torch.from_numpy(a).to(dtype).float().numpy()
    h, v, k, dy = [rnd(rng.standard_normal((N, D)).astype(np.float32)) for _ in range(4)]
    k *= 3.0; k = rnd(k)
    k[:, :64] += h[:, :64]                                   # correlated rows: gates away from 1/2
    k = rnd(k)
    d = lambda a: torch.from_numpy(a).to(cuda).to(dtype)
    dh, dv_, dk_, ddy = d(h), d(v), d(k), d(dy)
    hn, g, rh, rk = block.nggate_fwd(dh, dv_, dk_)
    h2, k2 = h.copy(), k.copy()
    hn_r, g_r, rh_r, rk_r = ref.nggate_f(h2, v, k2)
    rel = lambda a, b: float(np.abs(a.float().cpu().numpy() - b).max() / np.abs(b).max())
    assert g_r.std() > 0.02
    assert rel(g, g_r) < tol and rel(rh, rh_r) < 1e-5 and rel(rk, rk_r) < 1e-5
    assert rel(hn, hn_r) < tol and rel(dk_, k2) < tol and rel(dh, h2) < tol
    # backward from the reference's own forward state, so that both sides start from the same numbers
    st = [rnd(a) for a in (hn_r, k2)]
    gd, rhd, rkd = [torch.from_numpy(a).to(cuda) for a in (g_r, rh_r, rk_r)]
    dvo, dko = block.nggate_bwd(ddy, dv_, d(st[0]), d(st[1]), gd, rhd, rkd)
    dy2 = dy.copy()
    dv_r, dk_r = ref.nggate_b(dy2, v, st[0], st[1], g_r, rh_r, rk_r)
    assert rel(dvo, dv_r) < tol and rel(dko, dk_r) < 5 * tol and rel(ddy, dy2) < tol


def test_ngram_context_gate_fixture(cuda):
    """The gate kernels against the committed vectors of the reference's CPU kernels (fp32, 1e-5 relative)."""
    from conftest import golden
    from cudalm_c_b200 import block
    g = golden("nggate")
    d = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(cuda)
    rel = lambda a, b: float(np.abs(a.cpu().numpy() - b).max() / np.abs(b).max())
    h, k, dy = d(g["h0"]), d(g["k0"]), d(g["dy0"])
    hn, gg, rh, rk = block.nggate_fwd(h, d(g["v"]), k)
    for a, b in ((gg, g["g"]), (rh, g["rh"]), (rk, g["rk"]), (hn, g["hn"]), (k, g["k"]), (h, g["h"])):
        assert rel(a, b) < 1e-5
    dv, dk = block.nggate_bwd(dy, d(g["v"]), d(g["hn"]), d(g["k"]), d(g["g"]), d(g["rh"]), d(g["rk"]))
    for a, b in ((dv, g["dv"]), (dk, g["dk"]), (dy, g["dy"])):
        assert rel(a, b) < 1e-5
