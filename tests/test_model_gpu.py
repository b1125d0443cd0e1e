"""The composed training step (cudalm_c_b200/model.py = gpu_forward + gpu_head_bwd + gpu_backward +
gpu_adam of the reference, cudalm.cu:5736-6002, 6438-6465) against a plain fp32 PyTorch model of the
same architecture with autograd, on the dequantised weights and the same expert assignment.  Every
operator is checked against the reference on its own in the other test files; this one checks the
composition: loss within 1e-2, every gradient tensor within 5e-2 relative (activations are bf16)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F_

pytestmark = pytest.mark.gpu


def torch_model(m, tok, tgt):
    c, o = m.c, m.o
    P = torch.zeros(o.total, device=m.dev)
    m.q.render(P)
    for (off, n, _), t in zip(m.q.fs, m.fp):
        P[off:off + n] = t
    P.requires_grad_(True)
    N = c.B * c.T
    x = P[o.emb:o.emb + c.V * c.D].view(c.V, c.D)[tok.long()]
    cosb, sinb = m.cosb, m.sinb

    def rms(x, g):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * g

    def rope(v, nh):
        v = v.view(c.B, c.T, nh, c.hd)
        a, b = v[..., :c.hd // 2], v[..., c.hd // 2:]
        cs, sn = cosb[None, :, None, :], sinb[None, :, None, :]
        return torch.cat([a * cs - b * sn, b * cs + a * sn], -1).reshape(N, nh * c.hd)

    for l, lo in enumerate(o.layers):
        W = lambda nm, *shape: P[lo[nm][0]:lo[nm][0] + lo[nm][1]].view(*shape)
        a_norm = rms(x, W("an1", c.D))
        q = rope(a_norm @ W("wq", c.D, c.D), c.H); k = rope(a_norm @ W("wk", c.D, c.KD), c.KV); v = a_norm @ W("wv", c.D, c.KD)
        qh = q.view(c.B, c.T, c.H, c.hd).transpose(1, 2)
        kh = k.view(c.B, c.T, c.KV, c.hd).transpose(1, 2).repeat_interleave(c.H // c.KV, 1)
        vh = v.view(c.B, c.T, c.KV, c.hd).transpose(1, 2).repeat_interleave(c.H // c.KV, 1)
        att = F_.scaled_dot_product_attention(qh, kh, vh, is_causal=True).transpose(1, 2).reshape(N, c.D)
        f_in = att @ W("wo", c.D, c.D) + x
        f_norm = rms(f_in, W("an2", c.D))
        probs = torch.softmax(f_norm @ W("wr", c.D, c.E), -1)
        assign = m.layers[l]["moe"].member("assign", (c.K, N), torch.int32).long()
        W1, W3, W2 = W("w1", c.E, c.D, c.F), W("w3", c.E, c.D, c.F), W("w2", c.E, c.F, c.D)
        out = f_in
        for kk in range(c.K):
            e = assign[kk]
            gate = probs.gather(1, e[:, None])
            y = torch.zeros_like(f_in)
            for ex in range(c.E):
                sel = (e == ex).nonzero()[:, 0]
                if sel.numel():
                    xs = f_norm[sel]
                    y = y.index_add(0, sel, (F_.silu(xs @ W1[ex]) * (xs @ W3[ex])) @ W2[ex])
            out = out + gate * y
        x = out
    fn = rms(x, P[o.nf:o.nf + c.D])
    logits = fn @ P[o.emb:o.emb + c.V * c.D].view(c.V, c.D).t()
    loss = F_.cross_entropy(logits, tgt.long(), reduction="none")
    loss.mean().backward()
    return loss.detach(), P.grad


def test_training_step_matches_fp32_autograd(cuda):
    from cudalm_c_b200 import model
    import cudalm_c_b200 as q
    cfg = model.Config(L=2, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=128, B=2)
    m = model.QlmModel(cfg, cuda, seed=3)
    g = torch.Generator(device="cpu"); g.manual_seed(0)
    N = cfg.B * cfg.T
    tok = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).to(cuda)
    tgt = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).to(cuda)
    m.forward(tok)
    loss = m.backward(tok, tgt)
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    lr, Gr = torch_model(m, tok, tgt)
    assert abs(float(loss.mean()) - float(lr.mean())) < 1e-2 * float(lr.mean())
    o = m.o
    names = [("emb", o.emb, cfg.V * cfg.D), ("nf", o.nf, cfg.D)]
    for l, lo in enumerate(o.layers):
        names += [("%s[%d]" % (nm, l), lo[nm][0], lo[nm][1]) for nm in lo]
    worst = 0.0
    for nm, a, n in names:
        mine, ref = m.G[a:a + n].double(), Gr[a:a + n].double()
        r = float((mine - ref).norm() / ref.norm())
        worst = max(worst, r)
        assert r < 5e-2, (nm, r)
    # one optimizer step runs and changes the state
    d0 = m.q.r.clone()
    m.update()
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert not torch.equal(d0, m.q.r)
    print("worst relative gradient error", worst)


def test_model_file_is_loadable_by_the_reference(cuda, tmp_path):
    """QlmModel.save_model writes the rendered weights as a TLM4 file; the reference's model_load_full returns them."""
    from cudalm_c_b200 import model
    from oracle import loader
    ref = loader.reference()
    if ref is None:
        pytest.skip("compiled reference not present (make -C oracle ref)")
    cfg = model.Config(L=2, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=128, B=2)
    m = model.QlmModel(cfg, cuda, seed=4)
    path = str(tmp_path / "m.bin")
    m.save_model(path, eot=7)
    hdr, P = ref.model_load(path, m.o.total)
    assert list(hdr[:11]) == [256, 128, 2, 2, 2, 128, 128, 7, 0, 0, 4]
    assert (P == m.params().cpu().numpy()).all()


def test_fused_per_layer_update_equals_the_separate_update(cuda):
    """The fused per-layer update inside backward (CUDALM_QLM_FUSED: qlm_fused_layer / qlm_fused_tail, cudalm.cu:6105-6187;
    one gradient block shared by all layers) against the separate update on the same model, tokens and clip multiplier:
    every state array and every float parameter bit for bit.  (Given the multiplier: the fused form clips with the
    PREVIOUS step's norm, so the test hands it the norm the separate update computed.)  Then a second step runs on the
    multiplier the fused tail closed on the device."""
    from cudalm_c_b200 import model, qlm
    import cudalm_c_b200 as q
    cfg = model.Config(L=3, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=128, B=2)
    a = model.QlmModel(cfg, cuda, seed=5)
    b = model.QlmModel(cfg, cuda, seed=5, fused=True)
    assert b.G.numel() == cfg.V * cfg.D + b.layer_n + cfg.D and b.G.numel() < a.G.numel()
    g = torch.Generator(device="cpu"); g.manual_seed(1)
    N = cfg.B * cfg.T
    tok = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).to(cuda)
    tgt = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).to(cuda)
    a.forward(tok); la = a.backward(tok, tgt); a.update(3e-4, wdf=0.0)
    b.fgs.copy_(a.gs)                                     # this step's multiplier and norm, as if from the step before
    b.fused_lr = 3e-4
    b.forward(tok); lb = b.backward(tok, tgt); b.update(3e-4)
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert torch.equal(la, lb) and a.t == b.t == 1
    for k in ("d", "r", "s", "m8", "v8", "m8s", "v8s", "Mc", "Vc"):
        assert torch.equal(getattr(a.q, k), getattr(b.q, k)), k
    for ta, tb in zip(a.fp, b.fp):
        assert torch.equal(ta, tb)
    # the norm the fused tail closed is this step's norm (slices of 64 partial sums per layer instead of 64 chunks of G)
    assert abs(float(b.fgs[1]) - float(a.gs[1])) <= 1e-5 * float(a.gs[1])
    assert abs(float(b.fgs[0]) - float(a.gs[0])) <= 1e-5 * float(a.gs[0])
    r1 = b.q.r.clone()
    b.train_step(tok, tgt, lr=3e-4)
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert b.t == 2 and not torch.equal(r1, b.q.r)
