"""The decoder (Dec / dec_prefill / dec_step, cudalm.cu:7020-7212) checked the way the reference's own
`decheck` does (cudalm.cu:7233-7285): logits of the cached one-token steps against the full forward over the
same tokens (teacher forcing), two slots with different prefixes; bar as there: worst |dlogit| < 5e-2 and
the same arg-max at every position."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_decoder_matches_full_forward(cuda):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import block, model
    cfg = model.Config(L=2, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=128, B=2)
    m = model.QlmModel(cfg, cuda, seed=5)
    g = torch.Generator(device="cpu"); g.manual_seed(1)
    B, n, k = 2, 40, 8
    ids = torch.randint(0, cfg.V, (B, n + k), generator=g, dtype=torch.int32).to(cuda)
    # reference: the full forward over prompt + continuation
    full = model.Decoder(m, B, 64)
    moes = [full._moe(l, B * (n + k)) for l in range(cfg.L)]
    fn = m.forward(ids.reshape(-1).contiguous(), B=B, T=n + k, moes=moes)
    emb_bf, _ = block.cast_bf16(m.emb)
    ref = block.gemm_nt(fn, emb_bf, torch.float32).view(B, n + k, cfg.V)
    dec = model.Decoder(m, B, 64)
    lg = dec.prefill(ids[:, :n].contiguous())
    worst, agree, tot = 0.0, 0, 0

    def cmp(got, want):
        nonlocal worst, agree, tot
        worst = max(worst, float((got - want).abs().max()))
        agree += int((got.argmax(-1) == want.argmax(-1)).sum()); tot += got.shape[0]

    cmp(lg, ref[:, n - 1])
    for j in range(k):
        dec.tok.copy_(ids[:, n + j])
        lg = dec.step(advance=False)
        dec.advance()
        cmp(lg, ref[:, n + j])
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert int(dec.pos[0]) == n + k
    assert worst < 5e-2 and agree == tot, (worst, agree, tot)
    # greedy continuation runs without host input and picks the arg-max
    dec.step()
    assert torch.equal(dec.otok.long(), dec.logits.argmax(-1))


def test_slot_past_its_cache_is_reported_not_written(cuda):
    """Positions live on the device: a slot whose position equals the cache length must not touch the cache, the
    score buffer or the rotation tables.  The kernels skip it and leave error 201 in the device error word."""
    import cudalm_c_b200 as q
    from cudalm_c_b200 import model
    cfg = model.Config(L=1, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=64, B=2)
    m = model.QlmModel(cfg, cuda, seed=6)
    dec = model.Decoder(m, 2, 32)
    g = torch.Generator(device="cpu"); g.manual_seed(2)
    ids = torch.randint(0, cfg.V, (2, 8), generator=g, dtype=torch.int32).to(cuda)
    dec.prefill(ids)
    dec.step()
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    K0, V0 = dec.K[0].clone(), dec.V[0].clone()
    dec.pos2.fill_(32)                                   # one past the last cache position
    dec.step(advance=False)
    torch.cuda.synchronize()
    assert q.lib().qlmb_check_device(None) == 4          # QLMB_E_DEVICE
    assert b"error code 201" in q.lib().qlmb_last_error()
    assert torch.equal(K0, dec.K[0]) and torch.equal(V0, dec.V[0])
    dec.pos2.fill_(9)
    dec.step()                                           # the context is intact: the next step runs
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    # the stand-alone rotation has the same guard: a position outside its tables leaves the row alone and is reported
    from cudalm_c_b200._lib import ptr, stream_ptr
    row = torch.randn(2, cfg.D, device=cuda).to(torch.bfloat16); keep = row.clone()
    pos = torch.tensor([3, 32], dtype=torch.int32, device=cuda)
    q.check(q.lib().qlmb_dec_rope(ptr(row), 1, ptr(dec.cosb), ptr(dec.sinb), ptr(pos), 2, cfg.H, cfg.hd, 32, stream_ptr()))
    torch.cuda.synchronize()
    assert q.lib().qlmb_check_device(None) == 4 and b"error code 201" in q.lib().qlmb_last_error()
    assert torch.equal(row[1], keep[1]) and not torch.equal(row[0], keep[0])


def test_sampler_topk_topp_temperature(cuda):
    """k_dec_sample (cudalm.cu:7048-7108) against a float64 restatement of its algorithm: arg-max and
    log-probability, the top-k / top-p cut, and the pick that the (seed, step) hash selects from the tempered
    distribution.  The device adds float32 exponentials, so the pick is accepted when the hashed number falls
    within 1e-4 of the pick's interval of the cumulative distribution."""
    import numpy as np
    import cudalm_c_b200 as q
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    rng = np.random.default_rng(0)
    V, B = 16384, 12
    lg = (rng.standard_normal((B, V)) * 2.5).astype(np.float32)
    lg[3, 100] = lg[3].max() + 3.0                               # a dominant token
    dt = np.dtype(dict(names=["temp", "top_p", "top_k", "seed", "step"], formats=["<f4", "<f4", "<i4", "<u8", "<i4"],
                       offsets=[0, 4, 8, 16, 24], itemsize=32))
    prm = np.zeros(B, dt)
    cases = [(0.0, 1.0, 0), (1.0, 1.0, 1), (1.0, 1.0, 0), (0.7, 0.9, 40), (1.3, 0.5, 0), (0.5, 1.0, 5),
             (1.0, 0.95, 200), (2.0, 0.99, 0), (0.9, 0.8, 3), (1.0, 0.3, 0), (0.8, 1.0, 1000), (1.5, 0.7, 64)]
    for b, (temp, top_p, top_k) in enumerate(cases):
        prm[b] = (temp, top_p, top_k, 1234 + 77 * b, 5 + b)
    d_lg = torch.from_numpy(lg).to(cuda)
    d_prm = torch.from_numpy(prm.view(np.uint8).reshape(B, 32).copy()).to(cuda)
    out = torch.zeros(B, dtype=torch.int32, device=cuda); lp = torch.zeros(B, device=cuda)
    check(lib().qlmb_dec_sample(ptr(out), ptr(lp), ptr(d_lg), ptr(d_prm), B, V, stream_ptr()))
    torch.cuda.synchronize()
    out, lp = out.cpu().numpy(), lp.cpu().numpy()
    M64 = (1 << 64) - 1
    for b, (temp, top_p, top_k) in enumerate(cases):
        l = lg[b].astype(np.float64)
        ls = l.max() + np.log(np.exp(l - l.max()).sum())
        assert abs(lp[b] - (l[out[b]] - ls)) < 1e-3
        if temp <= 0 or top_k == 1:
            assert out[b] == int(np.argmax(l))
            continue
        th = l.max() - 30.0
        while (lg[b] >= np.float32(th)).sum() > 2048:
            th = 0.5 * (th + l.max())
        idx = np.nonzero(lg[b] >= np.float32(th))[0]
        order = idx[np.lexsort((idx, -l[idx]))]                   # value descending, index ascending
        sv = l[order]
        k = min(top_k, len(order)) if top_k > 0 else len(order)
        e = np.exp(sv[:k] - sv[0])
        if top_p < 1.0:
            c = np.cumsum(e / e.sum())
            hit = np.nonzero(c >= top_p - 1e-6)[0]
            k_lo = int(np.nonzero(c >= top_p + 1e-6)[0][0]) + 1 if (c >= top_p + 1e-6).any() else k
            k = int(hit[0]) + 1 if len(hit) else k
        else:
            k_lo = k
        h = ((1234 + 77 * b) * 0x9E3779B97F4A7C15 + (5 + b + 1) * 0xD1B54A32D192ED03) & M64
        h ^= h >> 30; h = (h * 0xBF58476D1CE4E5B9) & M64; h ^= h >> 27; h = (h * 0x94D049BB133111EB) & M64; h ^= h >> 31
        u01 = (h >> 40) / 16777216.0
        ok = False
        for kk in {k, k_lo}:                                      # a cumulative sum within rounding of top_p may cut one later
            w = np.exp((sv[:kk] - sv[0]) / temp)
            cum = np.cumsum(w) / w.sum()
            pos = np.nonzero(order[:kk] == out[b])[0]
            if len(pos):
                i = int(pos[0])
                lo = cum[i - 1] if i else 0.0
                ok |= lo - 1e-4 <= u01 <= cum[i] + 1e-4
        assert ok, (b, cases[b], int(out[b]))
    q.check(q.lib().qlmb_check_device(None))
