"""Flash attention (tcgen05, head dimension 64) through the C ABI against the reference's CPU
attention (cpu_kern.h:166-312, compiled from the reference's sources) on the same bf16-rounded inputs.
Bar: 1e-2 relative on outputs and gradients (P and dS are rounded to bf16 for the tensor core),
1e-3 absolute on the log-sum-exp."""
import numpy as np
import pytest
import torch

from oracle import loader

pytestmark = pytest.mark.gpu

SHAPES = [  # B, T, H, KV, win
    (2, 256, 4, 4, 0),
    (1, 200, 2, 1, 0),        # ragged sequence length, grouped-query heads
    (2, 384, 2, 2, 100),      # windowed
    (1, 1024, 2, 2, 0),
]


def rel(a, b):
    a, b = a.astype(np.float64), b.astype(np.float64)
    return max(np.linalg.norm(a - b) / np.linalg.norm(b), np.abs(a - b).max() / np.abs(b).max())


def torch_attention(Q, K, V, B, T, H, KV, win, dA=None):
    """Plain fp64 attention with autograd: the stand-in when the compiled reference is not on the box."""
    Q, K, V = [torch.from_numpy(x).double().requires_grad_(True) for x in (Q, K, V)]
    q = Q.view(B, T, H, 64).transpose(1, 2)
    k = K.view(B, T, KV, 64).transpose(1, 2).repeat_interleave(H // KV, 1)
    v = V.view(B, T, KV, 64).transpose(1, 2).repeat_interleave(H // KV, 1)
    s = q @ k.transpose(-1, -2) / 8.0
    i = torch.arange(T)[:, None]; j = torch.arange(T)[None, :]
    mask = (j <= i) & ((j > i - win) if win > 0 else torch.ones_like(j <= i))
    s = s.masked_fill(~mask, float("-inf"))
    lse = torch.logsumexp(s, -1)
    O = (torch.softmax(s, -1) @ v).transpose(1, 2).reshape(B * T, H * 64)
    if dA is None:
        return O.detach().numpy(), lse.detach().numpy()
    O.backward(torch.from_numpy(dA).double())
    return O.detach().numpy(), lse.detach().numpy(), Q.grad.numpy(), K.grad.numpy(), V.grad.numpy()


def inputs(B, T, H, KV, seed, cuda):
    g = torch.Generator(device="cpu"); g.manual_seed(seed)
    mk = lambda c: torch.randn(B * T, c * 64, generator=g).to(torch.bfloat16)
    Q, K, V = mk(H), mk(KV), mk(KV)
    return [x.to(cuda) for x in (Q, K, V)], [x.float().numpy() for x in (Q, K, V)]


@pytest.mark.parametrize("B,T,H,KV,win", SHAPES)
def test_attn_forward(cuda, B, T, H, KV, win):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import attn
    ref = loader.reference()
    (Qd, Kd, Vd), (Qh, Kh, Vh) = inputs(B, T, H, KV, 3, cuda)
    O, lse = attn.attn_fwd(Qd, Kd, Vd, B, T, H, KV, win)
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    if ref is not None:
        Or, lr = ref.attn_fwd(Qh, Kh, Vh, B, T, H, KV, 64, win)
    else:
        Or, lr = torch_attention(Qh, Kh, Vh, B, T, H, KV, win)
    assert rel(O.float().cpu().numpy(), Or) < 1e-2
    assert np.abs(lse.cpu().numpy() - lr).max() < 1e-3


@pytest.mark.parametrize("B,T,H,KV,win", SHAPES)
def test_attn_backward(cuda, B, T, H, KV, win):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import attn
    ref = loader.reference()
    (Qd, Kd, Vd), (Qh, Kh, Vh) = inputs(B, T, H, KV, 5, cuda)
    g = torch.Generator(device="cpu"); g.manual_seed(9)
    dA = torch.randn(B * T, H * 64, generator=g).to(torch.bfloat16)
    dAh = dA.float().numpy()
    if ref is not None:
        Or, lr = ref.attn_fwd(Qh, Kh, Vh, B, T, H, KV, 64, win)
        Ob = torch.from_numpy(Or).to(torch.bfloat16)
        dQr, dKr, dVr, drr = ref.attn_bwd(Qh, Kh, Vh, Ob.float().numpy(), dAh, lr, B, T, H, KV, 64, win)
    else:
        Or, lr, dQr, dKr, dVr = torch_attention(Qh, Kh, Vh, B, T, H, KV, win, dAh)
        Ob = torch.from_numpy(Or).to(torch.bfloat16)
        drr = None
    dQ, dK, dV, drow = attn.attn_bwd(Qd, Kd, Vd, Ob.to(cuda), dA.to(cuda), torch.from_numpy(lr.astype(np.float32)).to(cuda),
                                     B, T, H, KV, win)
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    if drr is not None:
        assert np.abs(drow.cpu().numpy() - drr).max() < 1e-3 * max(1.0, np.abs(drr).max())
    assert rel(dV.float().cpu().numpy(), dVr) < 1e-2
    assert rel(dK.float().cpu().numpy(), dKr) < 1e-2
    assert rel(dQ.float().cpu().numpy(), dQr) < 1e-2
