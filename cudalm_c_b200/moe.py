"""Host-side mirror of the reference's MoE operators (cudalm.cu:2515-2534,
3537-3602, 4151-4393): router_topk, moe_perm_all, moe_forward, moe_backward."""
import torch

from ._lib import BF16, F32, MoeLayer, check, lib, ptr, stream_ptr


def _dt(t):
    return BF16 if t.dtype == torch.bfloat16 else F32


def router_topk(rt=None, X=None, Wr=None, K=2, bias=None, bias_stride=0):
    """k_router_topk on given logits `rt` [N,E], or on X[N,D] @ Wr[D,E] computed
    on the device.  Returns (rt, rprobs, assign[K,N], gate[K,N])."""
    if rt is not None:
        N, E = rt.shape
        dev, D = rt.device, 0
    else:
        N, D = X.shape
        E = Wr.shape[1]
        dev = X.device
    rprobs = torch.empty((N, E), dtype=torch.float32, device=dev)
    assign = torch.empty((K, N), dtype=torch.int32, device=dev)
    gate = torch.empty((K, N), dtype=torch.float32, device=dev)
    rt_out = None if rt is not None else torch.empty((N, E), dtype=torch.float32, device=dev)
    check(lib().qlmb_router_topk(ptr(rt), ptr(rt_out), ptr(X), _dt(X) if X is not None else F32, ptr(Wr),
                                 ptr(bias), bias_stride, ptr(rprobs), ptr(assign), ptr(gate), N, D, E, K,
                                 stream_ptr()))
    return (rt if rt is not None else rt_out), rprobs, assign, gate


def moe_perm_all(assign, E, merged=False, pad=1):
    """Stable grouping of token slots by expert.  Returns (perm, inv, off, counts, bad)."""
    K, N = assign.shape
    sorts, length = (1, K * N) if merged else (K, N)
    dev = assign.device
    plen = length + E * (pad - 1)
    perm = torch.full((sorts, plen), -2, dtype=torch.int32, device=dev)
    inv = torch.empty((sorts, length), dtype=torch.int32, device=dev)
    off = torch.empty((sorts, E + 1), dtype=torch.int32, device=dev)
    counts = torch.empty((sorts, E), dtype=torch.int32, device=dev)
    bad = torch.zeros(1, dtype=torch.int32, device=dev)
    check(lib().qlmb_perm_build(ptr(assign), N, E, K, 1 if merged else 0, pad, ptr(perm), ptr(inv), ptr(off),
                                ptr(counts), ptr(bad), stream_ptr()))
    return perm, inv, off, counts, bad
