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


def router_bias_update(bias, assign, E, per_slot=True, u=0.001, proportional=True):
    """mbias_upd (cudalm.cu:3791-3802) on the device: bias [K, E] (per_slot) or [E]; assign [K, N]."""
    K, N = assign.shape
    check(lib().qlmb_router_bias_update(ptr(bias), ptr(assign), N, E, K, 1 if per_slot else 0, u, 1 if proportional else 0,
                                        stream_ptr()))


class MoeLayerState:
    """One MoE layer's 4-bit expert weights, router and activation arena: the
    slice of the reference's GA / P that moe_forward and moe_backward touch."""

    def __init__(self, N, D, F, E, K, q1, q3, q2, wr, dtype=torch.bfloat16, aux=0.03, bias=None, bias_stride=0):
        self.N, self.D, self.F, self.E, self.K = N, D, F, E, K
        self.q1, self.q3, self.q2, self.wr, self.bias = q1, q3, q2, wr, bias   # (codes, scales) pairs
        self.dtype = dtype
        dev = wr.device
        nbytes = lib().qlmb_moe_arena_bytes(N, D, F, E, K)
        self.arena = torch.zeros(nbytes + 256, dtype=torch.uint8, device=dev)
        self.arena_ptr = (self.arena.data_ptr() + 255) // 256 * 256
        self.c = MoeLayer(N, D, F, E, K, BF16 if dtype == torch.bfloat16 else F32,
                          ptr(q1[0]), ptr(q3[0]), ptr(q2[0]), ptr(q1[1]), ptr(q3[1]), ptr(q2[1]),
                          ptr(wr), ptr(bias), bias_stride, aux)
        self.rows_cap = (K * N + E * 127 + 127) // 128 * 128

    def member(self, name, shape, dtype):
        """A named arena member viewed as a tensor (no copy)."""
        p = lib().qlmb_moe_arena_member(self.arena_ptr, self.N, self.D, self.F, self.E, self.K, name.encode())
        if not p:
            raise KeyError(name)
        off = p - self.arena.data_ptr()
        n = 1
        for s in shape:
            n *= s
        esz = torch.empty(0, dtype=dtype).element_size()
        return self.arena[off:off + n * esz].view(dtype).view(*shape)

    def update_bias(self, u=0.001, proportional=True):
        """After a training forward: move the selection bias towards balanced load (mbias_upd, cudalm.cu:4385).
        bias_stride = E means one bias row per top-k pass, 0 one shared row."""
        if self.bias is None:
            raise ValueError("update_bias: the layer has no selection bias")
        router_bias_update(self.bias, self.member("assign", (self.K, self.N), torch.int32), self.E,
                           per_slot=self.c.bias_stride != 0, u=u, proportional=proportional)

    def forward(self, f_in, f_norm, out=None, rt=None):
        """moe_forward; with rt [N, E] the router's logits are taken from it (parity runs on identical routing)."""
        out = out if out is not None else torch.empty_like(f_in)
        if rt is not None:
            check(lib().qlmb_moe_forward_routed(self.c, self.arena_ptr, ptr(out), ptr(f_in), ptr(f_norm), ptr(rt), stream_ptr()))
        else:
            check(lib().qlmb_moe_forward(self.c, self.arena_ptr, ptr(out), ptr(f_in), ptr(f_norm), stream_ptr()))
        return out

    def decode(self, f_in, f_norm, out=None):
        """The forward of a decode step: no stash; routed GEMVs when K*N <= 128."""
        out = out if out is not None else torch.empty_like(f_in)
        check(lib().qlmb_moe_decode(self.c, self.arena_ptr, ptr(out), ptr(f_in), ptr(f_norm), stream_ptr()))
        return out

    def backward(self, dout, f_norm, dW1, dW3, dW2, dWr, beta=1.0, dfnorm=None):
        dfnorm = dfnorm if dfnorm is not None else torch.empty_like(dout)
        check(lib().qlmb_moe_backward(self.c, self.arena_ptr, ptr(dfnorm), ptr(dout), ptr(f_norm), ptr(dW1),
                                      ptr(dW3), ptr(dW2), ptr(dWr), beta, stream_ptr()))
        return dfnorm
