"""Dequant-fused linears (tcgen05) through the C ABI.
Tolerance (stated by the task): <= 1e-2 relative for bf16 tensor-core operands
against fp32 results, measured both as ||a-b||_F/||b||_F and max|a-b|/max|b|."""
import ctypes as C

import numpy as np
import pytest
import torch

from conftest import golden

pytestmark = pytest.mark.gpu
TOL = 1e-2
f32 = np.float32


def dev(a, cuda):
    return torch.from_numpy(np.ascontiguousarray(a)).to(cuda)


def rel(a, b):
    a, b = a.float(), b.float()
    return max(float((a - b).norm() / b.norm()), float((a - b).abs().max() / b.abs().max()))


def test_engine_plain_bf16(cuda):
    """TMA + tcgen05 + TMEM pipeline without the dequant warps vs fp32 matmul."""
    import cudalm_c_b200 as q
    from cudalm_c_b200._lib import ptr, stream_ptr
    L = q.lib()
    L.qlmb_selftest_gemm_bf16.argtypes = [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p]
    torch.manual_seed(1)
    for M, K, N in ((128, 64, 256), (1000, 512, 512), (4096, 1024, 1024)):
        A = torch.randn(M, K, device=cuda).bfloat16(); B = torch.randn(N, K, device=cuda).bfloat16()
        Cc = torch.zeros(M, N, device=cuda)
        q.check(L.qlmb_selftest_gemm_bf16(ptr(Cc), ptr(A), ptr(B), M, K, N, stream_ptr()))
        assert rel(Cc, A.float() @ B.float().T) < 1e-5
    q.check(L.qlmb_check_device(None))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_linear_matches_reference_vectors(cuda, dtype):
    """g_ab / g_abt / g_atb of the reference on its rendered weights (fixture)."""
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN, NK
    g = golden("linear")
    X, dY = dev(g["X"], cuda).to(dtype), dev(g["dY"], cuda).to(dtype)
    d, s = dev(g["d"], cuda), dev(g["s"], cuda)
    M, K = X.shape
    N = dY.shape[1]
    for lay, tag in ((KN, "kn"), (NK, "nk")):
        assert rel(linear.linear_fwd(X, d, s, lay, N), dev(g["Y_" + tag], cuda)) < TOL
        assert rel(linear.linear_dgrad(dY, d, s, lay, K), dev(g["dX_" + tag], cuda)) < TOL
        shape = (K, N) if lay == KN else (N, K)
        dW = torch.zeros(shape, device=cuda)
        linear.linear_wgrad(dW, dY, X, lay, beta=1.0)
        assert rel(dW, dev(g["dW_" + tag], cuda)) < TOL


def quantise(cuda, rows, cols, seed):
    from cudalm_c_b200 import qlm
    n = rows * cols
    Q = qlm.Qlm([(0, n)], n, cuda)
    gen = torch.Generator(device=cuda); gen.manual_seed(seed)
    P = torch.randn(n, device=cuda, generator=gen) * 0.02
    Q.init_from(P)                       # P now holds the rendered view s*d
    return Q, P.view(rows, cols)


@pytest.mark.parametrize("layout_name", ["KN", "NK"])
def test_config1_shape(cuda, oracle, layout_name):
    """BASELINE config 1: X[8192,512], W[2048,512] (NK) resp. [512,2048] (KN),
    fwd + dgrad + wgrad with fp32 I/O; full result vs fp32 matmul on the rendered
    view, 32 rows vs the oracle, plus linearity and run-to-run determinism."""
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN, NK
    lay = KN if layout_name == "KN" else NK
    M, K, N = 8192, 512, 2048
    Q, W = quantise(cuda, K, N, 3) if lay == KN else quantise(cuda, N, K, 3)
    Wm = W if lay == KN else W.T
    gen = torch.Generator(device=cuda); gen.manual_seed(4)
    X = torch.randn(M, K, device=cuda, generator=gen); dY = torch.randn(M, N, device=cuda, generator=gen)
    Y = linear.linear_fwd(X, Q.d, Q.s, lay, N)
    assert rel(Y, X @ Wm) < TOL
    dX = linear.linear_dgrad(dY, Q.d, Q.s, lay, K)
    assert rel(dX, dY @ Wm.T) < TOL
    dW = torch.zeros_like(W)
    linear.linear_wgrad(dW, dY, X, lay, beta=0.0)
    assert rel(dW, X.T @ dY if lay == KN else dY.T @ X) < TOL
    # oracle on a slice of rows
    dn, sn = Q.d.cpu().numpy(), Q.s.cpu().numpy()
    Yo = oracle.linear_fwd(X[:32].cpu().numpy(), dn, sn, lay, N)
    assert rel(Y[:32], dev(Yo, cuda)) < TOL
    dXo = oracle.linear_dgrad(dY[:32].cpu().numpy(), dn, sn, lay, K)
    assert rel(dX[:32], dev(dXo, cuda)) < TOL
    # size-independent properties: determinism, and linearity in the bf16-exact factor 2
    assert torch.equal(Y, linear.linear_fwd(X, Q.d, Q.s, lay, N))
    assert torch.equal(linear.linear_fwd(2 * X, Q.d, Q.s, lay, N), 2 * Y)
    # residual epilogue and accumulate modes
    R = torch.randn(M, N, device=cuda, generator=gen)
    assert rel(linear.linear_fwd(X, Q.d, Q.s, lay, N, R=R) - R, Y) < 1e-5
    acc = dX.clone()
    linear.linear_dgrad(dY, Q.d, Q.s, lay, K, beta=1.0, out=acc)
    assert rel(acc, 2 * dX) < 1e-6
    dW2 = dW.clone()
    linear.linear_wgrad(dW2, dY, X, lay, beta=1.0)
    assert rel(dW2, 2 * dW) < 1e-6


@pytest.mark.parametrize("M", [1, 127, 129, 300])
def test_ragged_row_counts(cuda, M):
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN, NK
    K, N = 256, 384
    for lay in (KN, NK):
        Q, W = quantise(cuda, K, N, 7) if lay == KN else quantise(cuda, N, K, 7)
        Wm = W if lay == KN else W.T
        X = torch.randn(M, K, device=cuda).bfloat16(); dY = torch.randn(M, N, device=cuda).bfloat16()
        guard = torch.full((M + 1, N), 7.0, device=cuda, dtype=torch.bfloat16)
        linear.linear_fwd(X, Q.d, Q.s, lay, N, out=guard[:M])
        assert rel(guard[:M], X.float() @ Wm) < TOL
        assert (guard[M] == 7.0).all()            # rows past M are never written
        assert rel(linear.linear_dgrad(dY, Q.d, Q.s, lay, K), dY.float() @ Wm.T) < TOL
        dW = torch.zeros_like(W)
        linear.linear_wgrad(dW, dY, X, lay, beta=0.0)
        assert rel(dW, X.float().T @ dY.float() if lay == KN else dY.float().T @ X.float()) < TOL


def test_empty_and_unsupported(cuda):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN
    Q, W = quantise(cuda, 128, 128, 9)
    assert linear.linear_fwd(torch.zeros(0, 128, device=cuda), Q.d, Q.s, KN, 128).shape == (0, 128)
    dW = torch.ones(128, 128, device=cuda)
    linear.linear_wgrad(dW, torch.zeros(0, 128, device=cuda), torch.zeros(0, 128, device=cuda), KN, beta=0.0)
    assert (dW == 0).all()
    with pytest.raises(q.QlmbError):               # K not a multiple of the scale group
        linear.linear_fwd(torch.zeros(4, 96, device=cuda), Q.d, Q.s, KN, 128)
    q.check(q.lib().qlmb_check_device(None))


@pytest.mark.parametrize("B", [1, 8, 64])
def test_gemv_decode(cuda, oracle, B):
    """Decode path (M = live slots <= 64).  fp32 activations: fp32 accumulation of exact dequantised weights (the
    digits are multiplied as 136 + d and the constant is taken out of the finished sums, which costs about five of
    the 24 mantissa bits), so the result agrees with the fp32 reference to round-off (3e-5).  bf16 activations with
    more than four slots run on warp-level MMAs with bf16(x * scale) operands: 8e-3."""
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN, NK
    for K, N in ((768, 1536), (1536, 768), (768, 16384), (2048, 4096)):
        for lay in (KN, NK):
            Q, W = quantise(cuda, K, N, 5) if lay == KN else quantise(cuda, N, K, 5)
            Wm = W if lay == KN else W.T
            for dt in (torch.float32, torch.bfloat16):
                X = torch.randn(B, K, device=cuda).to(dt)
                Y = linear.gemv_decode(X, Q.d, Q.s, lay, N)
                ref = X.float() @ Wm
                assert rel(Y, ref) < (3e-5 if dt == torch.float32 else 8e-3), (K, N, lay, dt)
                assert torch.equal(Y, linear.gemv_decode(X, Q.d, Q.s, lay, N))      # deterministic
    # oracle on one case
    Q, W = quantise(cuda, 256, 384, 6)
    X = torch.randn(B, 256, device=cuda)
    Yo = oracle.linear_fwd(X.cpu().numpy(), Q.d.cpu().numpy(), Q.s.cpu().numpy(), 0, 384)
    assert rel(linear.gemv_decode(X, Q.d, Q.s, KN, 384), dev(Yo, cuda)) < 1e-5


def test_gemv_rejects_more_than_64_slots(cuda):
    import cudalm_c_b200 as q
    from cudalm_c_b200 import linear
    from cudalm_c_b200._lib import KN
    Q, W = quantise(cuda, 128, 128, 9)
    with pytest.raises(q.QlmbError):
        linear.gemv_decode(torch.zeros(65, 128, device=cuda), Q.d, Q.s, KN, 128)


@pytest.mark.parametrize("B", [1, 3, 8, 64])
def test_gemv_decode_res_norm_equals_the_separate_kernels(cuda, B):
    """wo + residual + norm of a decode step in one launch pair (dec_step, cudalm.cu:7188-7190): F is the same bf16
    values as the GEMV followed by the bf16 add; Fn agrees with the separate norm kernel to one bf16 rounding."""
    from cudalm_c_b200 import block, linear
    from cudalm_c_b200._lib import KN, check, lib, ptr, stream_ptr
    for K, N in ((768, 768), (1536, 2048)):
        Q, W = quantise(cuda, K, N, 12)
        X = torch.randn(B, K, device=cuda).to(torch.bfloat16)
        res = torch.randn(B, N, device=cuda).to(torch.bfloat16)
        gamma = 1.0 + 0.1 * torch.randn(N, device=cuda)
        F = torch.empty(B, N, dtype=torch.bfloat16, device=cuda); Fn = torch.empty_like(F)
        check(lib().qlmb_gemv_decode_res_norm(ptr(F), ptr(Fn), ptr(X), ptr(Q.d), ptr(Q.s), ptr(res), ptr(gamma), B, K, N,
                                              stream_ptr()))
        # the separate kernels of the same family (the plain qlmb_gemv_decode sums in another order for few rows)
        Y = torch.empty(B, N, dtype=torch.bfloat16, device=cuda)
        check(lib().qlmb_gemv_decode_stack(ptr(Y), ptr(X), ptr(Q.d), ptr(Q.s), 1, B, K, N, 1, stream_ptr()))
        Y += res
        assert torch.equal(F, Y)
        Yn, _ = block.rmsnorm_fwd(Y, gamma)
        assert rel(Fn, Yn) < 8e-3
        assert (Fn.float() - Yn.float()).abs().max() <= 2.0 ** -7 * Yn.float().abs().max()
        assert rel(F, X.float() @ W + res.float()) < 8e-3


@pytest.mark.parametrize("B", [1, 8, 64])
def test_gemv_decode_norm_stack(cuda, B):
    """The norm in front of the q, k, v projections applied while the rows are staged (e_rmsf + three g_ab,
    cudalm.cu:7176-7180): the same numbers as the norm kernel followed by the stacked GEMV, up to one bf16 rounding
    of a normalised input where the two row sums differ in their last bit."""
    from cudalm_c_b200 import block
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    K = N = 768
    Q, W = quantise(cuda, 3 * K, N, 14)                       # three [K, N] matrices one after the other
    X = torch.randn(B, K, device=cuda).to(torch.bfloat16)
    gamma = 1.0 + 0.1 * torch.randn(K, device=cuda)
    Y = torch.empty(3 * B, N, dtype=torch.bfloat16, device=cuda); Y2 = torch.empty_like(Y)
    check(lib().qlmb_gemv_decode_norm_stack(ptr(Y), ptr(X), ptr(gamma), ptr(Q.d), ptr(Q.s), 3, B, K, N, 1, stream_ptr()))
    Xn, _ = block.rmsnorm_fwd(X, gamma)
    check(lib().qlmb_gemv_decode_stack(ptr(Y2), ptr(Xn), ptr(Q.d), ptr(Q.s), 3, B, K, N, 1, stream_ptr()))
    assert rel(Y, Y2) < 2e-3
    assert (Y == Y2).float().mean() > 0.99
    ref = torch.cat([Xn.float() @ W[m * K:(m + 1) * K] for m in range(3)])
    assert rel(Y, ref) < 8e-3


@pytest.mark.parametrize("B", [1, 5, 64])
def test_dec_qkv_equals_the_separate_kernels(cuda, B):
    """Norm, q / k / v projections, rotation and cache append of a decode step in one launch pair (dec_step,
    cudalm.cu:7176-7183) against the chain of separate kernels: same rows, same cache contents, nothing else touched."""
    from cudalm_c_b200 import block
    from cudalm_c_b200._lib import check, lib, ptr, stream_ptr
    D, hd, Tm = 768, 64, 96
    H = D // hd
    Q, W = quantise(cuda, 3 * D, D, 21)
    X = torch.randn(B, D, device=cuda).to(torch.bfloat16)
    gamma = 1.0 + 0.1 * torch.randn(D, device=cuda)
    cosb, sinb = block.rope_tables(Tm, hd, device=cuda)
    pos = torch.randint(0, Tm, (B,), device=cuda, dtype=torch.int32)
    Kc = torch.full((B, Tm, D), 7.0, dtype=torch.bfloat16, device=cuda); Vc = Kc.clone()
    Y = torch.empty(3 * B, D, dtype=torch.bfloat16, device=cuda)
    check(lib().qlmb_dec_qkv(ptr(Y), ptr(Kc), ptr(Vc), ptr(X), ptr(gamma), ptr(Q.d), ptr(Q.s), ptr(cosb), ptr(sinb), ptr(pos),
                             B, D, hd, Tm, stream_ptr()))
    Y2 = torch.empty_like(Y)
    check(lib().qlmb_gemv_decode_norm_stack(ptr(Y2), ptr(X), ptr(gamma), ptr(Q.d), ptr(Q.s), 3, B, D, D, 1, stream_ptr()))
    pos2 = torch.cat([pos, pos])
    check(lib().qlmb_dec_rope(ptr(Y2), 1, ptr(cosb), ptr(sinb), ptr(pos2), 2 * B, H, hd, Tm, stream_ptr()))
    Kc2 = torch.full((B, Tm, D), 7.0, dtype=torch.bfloat16, device=cuda); Vc2 = Kc2.clone()
    check(lib().qlmb_dec_kv(ptr(Kc2), ptr(Vc2), ptr(Y2[B:2 * B]), ptr(Y2[2 * B:]), ptr(pos), B, Tm, D, stream_ptr()))
    assert rel(Y, Y2) < 1e-3 and (Y == Y2).float().mean() > 0.999
    assert torch.equal(Kc[torch.arange(B), pos.long()], Y[B:2 * B]) and torch.equal(Vc[torch.arange(B), pos.long()], Y[2 * B:])
    assert rel(Kc, Kc2) < 1e-3 and rel(Vc, Vc2) < 1e-3
    assert int((Kc != 7.0).sum()) <= B * D and int((Vc != 7.0).sum()) <= B * D
