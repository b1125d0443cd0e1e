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
        dec.pos += 1
        cmp(lg, ref[:, n + j])
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert int(dec.pos[0]) == n + k
    assert worst < 5e-2 and agree == tot, (worst, agree, tot)
    # greedy continuation runs without host input and picks the arg-max
    dec.step()
    assert torch.equal(dec.otok.long(), dec.logits.argmax(-1))
