"""Host-side mirror of the reference's GEMM wrappers on quantised weights
(g_ab / g_abt / g_ab_res / g_abt_b / g_atb, cudalm.cu:3133-3202) and the decode GEMV.

`layout` says how the 4-bit codes are stored relative to Y = X W:
KN = codes of W[K,N] (the reference's own [in,out] storage, applied with g_ab),
NK = codes of W[N,K] (applied with g_abt)."""
import torch

from ._lib import BF16, F32, KN, NK, check, lib, ptr, stream_ptr  # noqa: F401


def _dt(t):
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise TypeError("activations must be float32 or bfloat16")


def linear_fwd(X, codes, scales, layout, N, R=None, out=None):
    """Y[M,N] = X[M,K] @ deq(W) (+ R)   -- g_ab / g_abt / g_ab_res."""
    M, K = X.shape
    Y = out if out is not None else torch.empty((M, N), dtype=X.dtype, device=X.device)
    check(lib().qlmb_linear_fwd(ptr(Y), ptr(X), ptr(codes), ptr(scales), layout, M, K, N, ptr(R), _dt(X), stream_ptr()))
    return Y


def linear_dgrad(dY, codes, scales, layout, K, beta=0.0, out=None):
    """dX[M,K] = beta*dX + dY[M,N] @ deq(W)^T   -- g_abt_b / g_ab."""
    M, N = dY.shape
    dX = out if out is not None else torch.empty((M, K), dtype=dY.dtype, device=dY.device)
    check(lib().qlmb_linear_dgrad(ptr(dX), ptr(dY), ptr(codes), ptr(scales), layout, M, K, N, beta, _dt(dY), stream_ptr()))
    return dX


def linear_wgrad(dW, dY, X, layout, beta=1.0):
    """dW (fp32, shape of W) = beta*dW + X^T dY (KN) or dY^T X (NK)   -- g_atb."""
    M, K = X.shape
    N = dY.shape[1]
    check(lib().qlmb_linear_wgrad(ptr(dW), ptr(dY), ptr(X), layout, M, K, N, beta, _dt(X), stream_ptr()))
    return dW


def gemv_decode(X, codes, scales, layout, N, out=None):
    """Y[B,N] = X[B,K] @ deq(W) for B <= 64 live decode slots."""
    B, K = X.shape
    Y = out if out is not None else torch.empty((B, N), dtype=X.dtype, device=X.device)
    check(lib().qlmb_gemv_decode(ptr(Y), ptr(X), ptr(codes), ptr(scales), layout, B, K, N, _dt(X), stream_ptr()))
    return Y
