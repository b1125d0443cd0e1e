"""Host-side mirror of the reference's operators around the GEMMs of a block (e_rmsf, e_rmsb, e_rope,
k_embed, k_embed_bwd, k_softmax_ce; cudalm.cu:3630-3645, 5740, 5838, 6000) over the C ABI."""
import torch

from ._lib import BF16, F32, check, lib, ptr, stream_ptr


def _dt(t):
    if t.dtype == torch.bfloat16:
        return BF16
    if t.dtype == torch.float32:
        return F32
    raise TypeError("activations are float32 or bfloat16, got %s" % t.dtype)


def embed(emb, tok, dtype=torch.float32):
    N, D = tok.numel(), emb.shape[1]
    X = torch.empty(N, D, dtype=dtype, device=emb.device)
    check(lib().qlmb_embed(ptr(X), _dt(X), ptr(emb), ptr(tok), N, D, stream_ptr()))
    return X


def embed_bwd(G, dout, tok):
    """G[V, D] += scatter of dout rows by token, rows of one token added in ascending position."""
    check(lib().qlmb_embed_bwd(ptr(G), ptr(dout), _dt(dout), ptr(tok), tok.numel(), G.shape[1], G.shape[0], stream_ptr()))


def rmsnorm_fwd(X, gamma, out_dtype=None, out=None):
    N, D = X.shape
    O = out if out is not None else torch.empty(N, D, dtype=out_dtype or X.dtype, device=X.device)
    rinv = torch.empty(N, dtype=torch.float32, device=X.device)
    check(lib().qlmb_rmsnorm_fwd(ptr(O), _dt(O), ptr(rinv), ptr(X), _dt(X), ptr(gamma), N, D, stream_ptr()))
    return O, rinv


def rmsnorm_bwd(dx, X, gamma, rinv, dy, dgamma=None, accumulate=True):
    """dx (+)= the input gradient; dgamma += the gain gradient (e_rmsb accumulates into both)."""
    N, D = X.shape
    part = torch.empty(128 * D, dtype=torch.float32, device=X.device) if dgamma is not None else None
    check(lib().qlmb_rmsnorm_bwd(ptr(dx), _dt(dx), 1 if accumulate else 0, ptr(dgamma), ptr(part), ptr(X), _dt(X), ptr(gamma),
                                 ptr(rinv), ptr(dy), _dt(dy), N, D, stream_ptr()))


def rope_tables(T, hd, base=10000.0, device="cpu"):
    """cos / sin tables [T, hd/2] (angle t * base^(-2i/hd))."""
    hf = hd // 2
    inv = base ** (-torch.arange(hf, dtype=torch.float64) * 2.0 / hd)
    ang = torch.arange(T, dtype=torch.float64)[:, None] * inv[None, :]
    return ang.cos().float().to(device), ang.sin().float().to(device)


def rope(buf, cosb, sinb, nh, hd, T, back=False):
    """In place on buf[N, nh*hd]."""
    check(lib().qlmb_rope(ptr(buf), _dt(buf), ptr(cosb), ptr(sinb), buf.shape[0], nh, hd, T, 1 if back else 0, stream_ptr()))


def softmax_ce(logits, tgt, n_all, dl_dtype=None):
    rows, V = logits.shape
    loss = torch.empty(rows, dtype=torch.float32, device=logits.device)
    dl = torch.empty(rows, V, dtype=dl_dtype or logits.dtype, device=logits.device)
    check(lib().qlmb_softmax_ce(ptr(logits), _dt(logits), ptr(tgt), ptr(loss), ptr(dl), _dt(dl), rows, V, n_all, stream_ptr()))
    return loss, dl


def gemm_nt(A, B, out_dtype=torch.float32, out=None, beta=0.0):
    """C[M,N] = A[M,K] B[N,K]^T (+ C); A, B bf16."""
    M, K = A.shape
    N = B.shape[0]
    C_ = out if out is not None else torch.empty(M, N, dtype=out_dtype, device=A.device)
    check(lib().qlmb_gemm_nt(ptr(C_), _dt(C_), ptr(A), ptr(B), M, K, N, beta, stream_ptr()))
    return C_


def cast_bf16(src, plain=True, transposed=False):
    R, Cc = src.shape
    d = torch.empty(R, Cc, dtype=torch.bfloat16, device=src.device) if plain else None
    dt_ = torch.empty(Cc, R, dtype=torch.bfloat16, device=src.device) if transposed else None
    check(lib().qlmb_cast_bf16(ptr(d), ptr(dt_), ptr(src), R, Cc, stream_ptr()))
    return d, dt_


def head_bwd(fn, emb, tgt, G_emb, chunk_rows=2048, denom=None):
    """gpu_head_bwd (cudalm.cu:5790-5872): chunked lm_head over the tied embedding + softmax cross-entropy
    + its backward.  fn [N, D] bf16 (the final norm's output), emb [V, D] fp32, tgt [N] int32.
    Returns (loss per row, dfn bf16) and adds dlogits^T fn into G_emb [V, D] (fp32)."""
    from . import linear
    from ._lib import NK
    N, D = fn.shape
    V = emb.shape[0]
    denom = denom or N
    eb, ebt = cast_bf16(emb, plain=True, transposed=True)
    loss = torch.empty(N, dtype=torch.float32, device=fn.device)
    dfn = torch.empty(N, D, dtype=torch.bfloat16, device=fn.device)
    for r0 in range(0, N, chunk_rows):
        r1 = min(N, r0 + chunk_rows)
        logits = gemm_nt(fn[r0:r1], eb, torch.float32)
        ls, dl = softmax_ce(logits, tgt[r0:r1], denom, dl_dtype=torch.bfloat16)
        loss[r0:r1] = ls
        gemm_nt(dl, ebt, out=dfn[r0:r1])
        linear.linear_wgrad(G_emb, dl, fn[r0:r1], NK, beta=1.0)
    return loss, dfn


def ngram_key(tok, T, R, order, base=0):
    """k_ngram_key (cudalm.cu:4438-4445): table row of every position's last `order` tokens; -1 where masked."""
    key = torch.empty(tok.numel(), dtype=torch.int32, device=tok.device)
    check(lib().qlmb_ngram_key(ptr(key), ptr(tok), tok.numel(), T, R, order, base, stream_ptr()))
    return key


def ngram_gather(tbl, key, N, nk=1):
    """k_ngram_gather (cudalm.cu:4446-4451): buf[n] = sum of the nk table rows key[j * N + n]."""
    buf = torch.empty((N, tbl.shape[1]), dtype=torch.float32, device=tbl.device)
    check(lib().qlmb_ngram_gather(ptr(buf), ptr(tbl), ptr(key), N, tbl.shape[1], nk, stream_ptr()))
    return buf


def nggate_fwd(h, v, k):
    """k_nggate_f (cudalm.cu:3362-3368): h += g * v in place, k -> rms(k) in place; returns (hn, g, rh, rk)."""
    N, D = h.shape
    hn = torch.empty_like(h)
    g, rh, rk = (torch.empty(N, dtype=torch.float32, device=h.device) for _ in range(3))
    check(lib().qlmb_nggate_fwd(ptr(h), ptr(v), ptr(k), ptr(hn), _dt(h), ptr(g), ptr(rh), ptr(rk), N, D, stream_ptr()))
    return hn, g, rh, rk


def nggate_bwd(dy, v, hn, kn, g, rh, rk):
    """k_nggate_b (cudalm.cu:3370-3378): dy += the gate's share of dh in place; returns (dv, dk)."""
    N, D = dy.shape
    dv, dk = torch.empty_like(dy), torch.empty_like(dy)
    check(lib().qlmb_nggate_bwd(ptr(dy), ptr(v), ptr(hn), ptr(kn), _dt(dy), ptr(g), ptr(rh), ptr(rk), ptr(dv), ptr(dk), N, D,
                                stream_ptr()))
    return dv, dk
