"""Expert-parallel MoE layer: experts sharded over the ranks of a torch.distributed
group, tokens stay on their home rank, routed rows travel by all-to-all.

The reference is single-GPU; this is its moe_forward / moe_backward
(cudalm.cu:4151-4393) cut at the two exchange points.  Rank r owns the global
experts [r*E/W, (r+1)*E/W).  Per step and layer there is ONE host round trip (the
[W, E] matrix of routed-row counts, which the variable-size all-to-all needs as
split sizes -- the reference reads its expert offsets back once per layer too,
cudalm.cu:3554-3559); everything else is device work on the current stream.

torch.distributed is plumbing only: all arithmetic is in libqlm_b200.so.
"""
import numpy as np
import torch
import torch.distributed as dist

from ._lib import BF16, MoeLayer, check, lib, ptr, stream_ptr


def exchange_plan(counts_all, rank, world):
    """Split sizes and row tags for the dispatch all-to-all.

    counts_all[s][e] = rows that source rank s routed to global expert e.
    Returns (send_splits[W], recv_splits[W], expert_of_row[R]): rows arrive
    grouped by source rank, inside a source by local expert, which is the order
    they were packed in (expert-sorted), so expert_of_row is a run-length list."""
    counts_all = np.asarray(counts_all, dtype=np.int64)
    W, E = counts_all.shape
    assert W == world and E % world == 0
    el = E // world
    send = counts_all[rank].reshape(world, el).sum(1)
    mine = counts_all[:, rank * el:(rank + 1) * el]            # [W][el]
    recv = mine.sum(1)
    tags = np.repeat(np.tile(np.arange(el, dtype=np.int32), world), mine.reshape(-1))
    return [int(x) for x in send], [int(x) for x in recv], tags


def all_to_all_rows(out, inp, out_splits, in_splits, group=None):
    """Variable-size row exchange.  NCCL: one all_to_all_single.  Backends without
    all-to-all (gloo on CPU, used by the host-logic tests): all_gather + slicing."""
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(out, inp, out_splits, in_splits, group=group)
        return
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    bufs = [None] * world
    dist.all_gather_object(bufs, (inp.cpu().numpy() if inp.dtype != torch.bfloat16 else inp.float().cpu().numpy(), in_splits), group=group)
    pos = 0
    for s in range(world):
        data, splits = bufs[s]
        lo = int(np.sum(splits[:rank]))
        n = int(splits[rank])
        out[pos:pos + n] = torch.from_numpy(data[lo:lo + n]).to(out.dtype)
        pos += n


class ExpertParallelLayer:
    """One MoE layer with E/W local experts per rank (weak scaling: N tokens per rank)."""

    launches_per_step = 27          # library kernels per forward+backward on a rank

    def __init__(self, cfg, dev, rank, world, seed=1234, aux=0.03, group=None, weights=None, row_capacity=None):
        from . import qlm
        self.N, self.D, self.F, self.E, self.K = cfg["N"], cfg["D"], cfg["F"], cfg["E"], cfg["K"]
        N, D, F, E, K = self.N, self.D, self.F, self.E, self.K
        assert E % world == 0
        self.rank, self.world, self.group, self.dev = rank, world, group, dev
        self.el = E // world
        el = self.el
        gen = torch.Generator(device=dev); gen.manual_seed(seed)
        # identical full synthetic weights on every rank (same seed), of which the local slice is kept
        self.q = []
        for wi, (rows, cols) in enumerate(((D, F), (D, F), (F, D))):
            if weights is not None:
                full = weights[wi]
            else:
                full = torch.randn(E * rows * cols, device=dev, generator=gen) * 0.02
            n = el * rows * cols
            Q = qlm.Qlm([(0, n)], n, dev)
            Q.init_from(full[rank * n:(rank + 1) * n].clone(), render=False)
            self.q.append((Q.d, Q.s))
            del full
        self.wr = weights[3] if weights is not None else torch.randn(D, E, device=dev, generator=gen) * 0.02
        L = lib()
        # home side: routing state for N tokens over all E experts
        hb = L.qlmb_moe_arena_bytes(N, D, F, E, K)
        self.harena = torch.zeros(hb + 256, dtype=torch.uint8, device=dev)
        self.hptr = (self.harena.data_ptr() + 255) // 256 * 256
        self.home = MoeLayer(N, D, F, E, K, BF16, None, None, None, None, None, None, ptr(self.wr), None, 0, aux)
        # expert side: up to `cap` received rows over the local experts
        self.cap = row_capacity or 2 * K * N
        eb = L.qlmb_moe_arena_bytes(self.cap, D, F, el, 1)
        self.earena = torch.zeros(eb + 256, dtype=torch.uint8, device=dev)
        self.eptr = (self.earena.data_ptr() + 255) // 256 * 256
        self.loc = MoeLayer(self.cap, D, F, el, 1, BF16, ptr(self.q[0][0]), ptr(self.q[1][0]), ptr(self.q[2][0]),
                            ptr(self.q[0][1]), ptr(self.q[1][1]), ptr(self.q[2][1]), None, None, 0, aux)
        bf = dict(dtype=torch.bfloat16, device=dev)
        self.Xs, self.Ys, self.dYs, self.dXs = [torch.empty(K * N, D, **bf) for _ in range(4)]
        self.Xr, self.Yr, self.dYr, self.dXr = [torch.empty(self.cap, D, **bf) for _ in range(4)]
        self.counts_all = torch.empty(world, E, dtype=torch.int32, device=dev)
        self.dW = [torch.zeros(el, D, F, device=dev), torch.zeros(el, D, F, device=dev), torch.zeros(el, F, D, device=dev)]
        self.dWr = torch.zeros(D, E, device=dev)
        g2 = torch.Generator(device=dev); g2.manual_seed(seed + 1000 + rank)
        self.fn, self.fi, self.dout = [torch.randn(N, D, device=dev, generator=g2).bfloat16() for _ in range(3)]
        self.out = torch.empty_like(self.fi); self.dfn = torch.empty_like(self.fi)
        self.R = 0

    def member(self, name, shape, dtype):
        p = lib().qlmb_moe_arena_member(self.hptr, self.N, self.D, self.F, self.E, self.K, name.encode())
        off = p - self.harena.data_ptr()
        n = int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()
        return self.harena[off:off + n].view(dtype).view(*shape)

    def forward(self, fi=None, fn=None, out=None):
        fi = self.fi if fi is None else fi
        fn = self.fn if fn is None else fn
        out = self.out if out is None else out
        L, st = lib(), stream_ptr()
        check(L.qlmb_moe_route(self.home, self.hptr, ptr(self.Xs), ptr(fn), st))
        counts = self.member("counts", (self.E,), torch.int32)
        dist.all_gather_into_tensor(self.counts_all.view(-1), counts, group=self.group)
        plan = exchange_plan(self.counts_all.cpu().numpy(), self.rank, self.world)   # the one host round trip
        self.send, self.recv, tags = plan
        self.R = int(sum(self.recv))
        if self.R > self.cap:
            raise RuntimeError("expert-parallel layer: %d rows arrived, capacity is %d" % (self.R, self.cap))
        self.tags = torch.from_numpy(tags).to(self.dev, non_blocking=True)
        all_to_all_rows(self.Xr[:self.R], self.Xs, self.recv, self.send, self.group)
        check(L.qlmb_moe_experts_forward(self.loc, self.eptr, ptr(self.Yr), ptr(self.Xr), ptr(self.tags), self.R, st))
        all_to_all_rows(self.Ys, self.Yr[:self.R], self.send, self.recv, self.group)
        check(L.qlmb_moe_combine(self.home, self.hptr, ptr(out), ptr(fi), ptr(self.Ys), st))
        return out

    def backward(self, dout=None, fn=None, beta=0.0, dfn=None):
        dout = self.dout if dout is None else dout
        fn = self.fn if fn is None else fn
        dfn = self.dfn if dfn is None else dfn
        L, st = lib(), stream_ptr()
        check(L.qlmb_moe_dgate(self.home, self.hptr, ptr(self.dYs), ptr(dout), ptr(self.Ys), st))
        all_to_all_rows(self.dYr[:self.R], self.dYs, self.recv, self.send, self.group)
        check(L.qlmb_moe_experts_backward(self.loc, self.eptr, ptr(self.dXr), ptr(self.dYr), self.R, ptr(self.dW[0]),
                                          ptr(self.dW[1]), ptr(self.dW[2]), beta, st))
        all_to_all_rows(self.dXs, self.dXr[:self.R], self.send, self.recv, self.group)
        check(L.qlmb_moe_route_backward(self.home, self.hptr, ptr(dfn), ptr(self.dXs), ptr(fn), ptr(self.dWr), beta, st))
        return dfn

    def step(self):
        self.forward()
        self.backward()


class _DeviceWindow:
    """A raw device allocation exposed to torch without a copy."""

    def __init__(self, address, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (address, False), "version": 2}


class PeerExpertParallelLayer:
    """The same layer with no exchange step: rows cross NVLink inside kernels that exist anyway -- the
    expert side's gathers read foreign rows through peer-mapped pointers, the epilogues of its down
    and dX GEMMs store result rows straight into their home rank's buffers (include/qlm_b200.h, qlmb_ep_*).  Every rank owns one window
    of device memory (token inputs, router-side arena, expert-side arena) with the same layout;
    the ranks of the node map each other's windows once at construction.  Per step the ranks
    exchange only the routing table (one fixed-size all-gather) and two one-element all-reduces
    that act as stream-ordered barriers; nothing waits on the host."""

    launches_per_step = 22          # library kernels per forward+backward on a rank

    def __init__(self, cfg, dev, rank, world, seed=1234, aux=0.03, group=None, weights=None, ext=None):
        """ext (a model's own storage instead of the synthetic weights and inputs of the bench):
        dict(q=[(codes, scales) of the local experts' W1, W3, W2], wr=router [D, E], dW=[three fp32 gradient
        tensors of the local experts], dWr=[D, E])."""
        import ctypes as C
        from . import qlm
        from ._lib import EpPeers
        self.N, self.D, self.F, self.E, self.K = cfg["N"], cfg["D"], cfg["F"], cfg["E"], cfg["K"]
        N, D, F, E, K = self.N, self.D, self.F, self.E, self.K
        assert E % world == 0 and world <= 8
        self.rank, self.world, self.group, self.dev = rank, world, group, dev
        self.el = el = E // world
        L = lib()
        gen = torch.Generator(device=dev); gen.manual_seed(seed)
        self.q = list(ext["q"]) if ext is not None else []
        for wi, (rows, cols) in enumerate(((D, F), (D, F), (F, D)) if ext is None else ()):
            full = weights[wi] if weights is not None else torch.randn(E * rows * cols, device=dev, generator=gen) * 0.02
            n = el * rows * cols
            Q = qlm.Qlm([(0, n)], n, dev)
            Q.init_from(full[rank * n:(rank + 1) * n].clone(), render=False)
            self.q.append((Q.d, Q.s))
            del full
        if ext is not None:
            self.wr = ext["wr"]
        else:
            self.wr = weights[3] if weights is not None else torch.randn(D, E, device=dev, generator=gen) * 0.02
        # window layout (identical on every rank)
        self.slots = world * K * N
        hb = L.qlmb_moe_arena_bytes(N, D, F, E, K)
        eb = L.qlmb_moe_arena_bytes(self.slots, D, F, el, 1)
        al = lambda x: (x + 255) // 256 * 256
        row_bytes = al(N * D * 2)
        self.off_fn = [0, row_bytes]
        self.off_dout = [2 * row_bytes, 3 * row_bytes]
        slot_bytes = al(K * N * D * 2)
        self.off_ys = 4 * row_bytes
        self.off_dxs = self.off_ys + slot_bytes
        self.off_h = self.off_dxs + slot_bytes
        self.off_e = self.off_h + al(hb)
        self.win_bytes = self.off_e + al(eb)
        p = C.c_void_p()
        check(L.qlmb_peer_alloc(self.win_bytes, C.byref(p)))
        self.win_ptr = p.value
        self.win = torch.as_tensor(_DeviceWindow(self.win_ptr, self.win_bytes), device=dev)
        self.win.zero_()
        self.peers = EpPeers()
        self.peers.rank, self.peers.world = rank, world
        self._opened = []
        if world > 1:
            hbuf = (C.c_ubyte * 64)()
            check(L.qlmb_peer_export(self.win_ptr, hbuf))
            mine = torch.tensor(list(hbuf), dtype=torch.uint8, device=dev)
            allh = torch.empty(world, 64, dtype=torch.uint8, device=dev)
            dist.all_gather_into_tensor(allh.view(-1), mine, group=group)
            allh = allh.cpu().numpy()
            for r in range(world):
                if r == rank:
                    self.peers.base[r] = self.win_ptr
                    continue
                hb_r = (C.c_ubyte * 64)(*[int(x) for x in allh[r]])
                q = C.c_void_p()
                check(L.qlmb_peer_open(hb_r, C.byref(q)))
                self.peers.base[r] = q.value
                self._opened.append(q.value)
        else:
            self.peers.base[0] = self.win_ptr
        self.hptr = self.win_ptr + self.off_h
        self.eptr = self.win_ptr + self.off_e
        bf = torch.bfloat16

        def view(off, shape, dtype):
            n = int(np.prod(shape)) * torch.empty(0, dtype=dtype).element_size()
            return self.win[off:off + n].view(dtype).view(*shape)
        self.Ys = view(self.off_ys, (K * N, D), bf)
        self.dXs = view(self.off_dxs, (K * N, D), bf)
        self.fn_set = [view(o, (N, D), bf) for o in self.off_fn]
        self.dout_set = [view(o, (N, D), bf) for o in self.off_dout]
        self.home = MoeLayer(N, D, F, E, K, BF16, None, None, None, None, None, None, ptr(self.wr), None, 0, aux)
        self.loc = MoeLayer(self.slots, D, F, el, 1, BF16, ptr(self.q[0][0]), ptr(self.q[1][0]), ptr(self.q[2][0]),
                            ptr(self.q[0][1]), ptr(self.q[1][1]), ptr(self.q[2][1]), None, None, 0, aux)
        ap = L.qlmb_moe_arena_member(self.hptr, N, D, F, E, K, b"assign")
        self.assign = view(ap - self.win_ptr, (K * N,), torch.int32)
        self.assign_all = torch.empty(world, K * N, dtype=torch.int32, device=dev)
        self.flag = torch.zeros(1, dtype=torch.int32, device=dev)
        self.fn, self.dout = self.fn_set[0], self.dout_set[0]
        # inside a model the gradient arrives in the window just before backward(): the ranks then meet once more
        # before the expert side pulls it (in forward the all-gather of the routing table already orders f_norm)
        self.dynamic_inputs = ext is not None
        if ext is not None:
            self.dW, self.dWr = list(ext["dW"]), ext["dWr"]
        else:
            self.dW = [torch.zeros(el, D, F, device=dev), torch.zeros(el, D, F, device=dev), torch.zeros(el, F, D, device=dev)]
            self.dWr = torch.zeros(D, E, device=dev)
            g2 = torch.Generator(device=dev); g2.manual_seed(seed + 1000 + rank)
            self.fn.copy_(torch.randn(N, D, device=dev, generator=g2).bfloat16())
            self.fi = torch.randn(N, D, device=dev, generator=g2).bfloat16()
            self.dout.copy_(torch.randn(N, D, device=dev, generator=g2).bfloat16())
            self.out = torch.empty_like(self.fi); self.dfn = torch.empty_like(self.fi)
        if world > 1:
            dist.barrier(group=group)           # every window is mapped before the first step reads one

    def _barrier(self):
        if self.world > 1:
            dist.all_reduce(self.flag, group=self.group)

    def forward(self, fi=None, fn=None, out=None):
        """fn must be one of fn_set (it is read by the other ranks)."""
        fi = self.fi if fi is None else fi
        fn = self.fn if fn is None else fn
        out = self.out if out is None else out
        L, st = lib(), stream_ptr()
        check(L.qlmb_ep_route(self.home, self.hptr, ptr(fn), st))
        if self.world > 1:
            dist.all_gather_into_tensor(self.assign_all.view(-1), self.assign, group=self.group)
        else:
            self.assign_all.view(-1).copy_(self.assign)
        check(L.qlmb_ep_experts_forward(self.loc, self.eptr, self.peers, ptr(self.assign_all), ptr(fn), BF16, self.N, self.K,
                                        ptr(self.Ys), st))
        self._barrier()
        check(L.qlmb_ep_combine(self.home, self.hptr, ptr(self.Ys), ptr(out), ptr(fi), st))
        return out

    def backward(self, dout=None, fn=None, beta=0.0, dfn=None):
        """dout must be one of dout_set (it is read by the other ranks)."""
        dout = self.dout if dout is None else dout
        fn = self.fn if fn is None else fn
        dfn = self.dfn if dfn is None else dfn
        L, st = lib(), stream_ptr()
        check(L.qlmb_ep_dgate(self.home, self.hptr, ptr(self.Ys), ptr(dout), st))
        if self.dynamic_inputs:
            self._barrier()         # every rank's dout is in its window before another rank's expert side reads it
        check(L.qlmb_ep_experts_backward(self.loc, self.eptr, self.home, self.hptr, self.peers, ptr(dout), self.N, self.K,
                                         ptr(self.dXs), ptr(self.dW[0]), ptr(self.dW[1]), ptr(self.dW[2]), beta, st))
        self._barrier()
        check(L.qlmb_ep_route_backward(self.home, self.hptr, ptr(self.dXs), ptr(dfn), ptr(fn), ptr(self.dWr), beta, st))
        return dfn

    def step(self):
        self.forward()
        self.backward()

    def close(self):
        L = lib()
        torch.cuda.synchronize()
        if self.world > 1:
            dist.barrier(group=self.group)      # nobody reads a window that is about to go away
        for q in self._opened:
            L.qlmb_peer_close(q)
        self._opened = []
        self.win = None
        if self.win_ptr:
            L.qlmb_peer_free(self.win_ptr)
            self.win_ptr = 0
