"""Host-side mirror of the reference's attention operators (e_attn, cudalm.cu:3705-3730, and the
attention part of gpu_backward, cudalm.cu:5918-5960) over the C ABI."""
import torch

from ._lib import check, lib, ptr, stream_ptr


def attn_fwd(Q, K, V, B, T, H, KV, win=0):
    """Causal attention: Q [B*T, H*64], K, V [B*T, KV*64] bf16 -> O bf16, lse [B, H, T] fp32."""
    O = torch.empty_like(Q)
    lse = torch.empty(B, H, T, dtype=torch.float32, device=Q.device)
    check(lib().qlmb_attn_fwd(ptr(O), ptr(lse), ptr(Q), ptr(K), ptr(V), B, T, H, KV, 64, win, stream_ptr()))
    return O, lse


def attn_bwd(Q, K, V, O, dA, lse, B, T, H, KV, win=0):
    """Gradients of attn_fwd's inputs: dQ, dK, dV (bf16) and drow = rowsum(dA * O) [B, H, T]."""
    dQ, dK, dV = torch.empty_like(Q), torch.empty_like(K), torch.empty_like(V)
    drow = torch.empty(B, H, T, dtype=torch.float32, device=Q.device)
    check(lib().qlmb_attn_bwd(ptr(dQ), ptr(dK), ptr(dV), ptr(drow), ptr(Q), ptr(K), ptr(V), ptr(O), ptr(dA), ptr(lse),
                              B, T, H, KV, 64, win, stream_ptr()))
    return dQ, dK, dV, drow
