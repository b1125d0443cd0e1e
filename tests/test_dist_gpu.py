"""Expert-parallel layer, in both forms (split C-ABI calls + NCCL all-to-all; peer loads
inside the row kernels, no exchange step), against the
single-call layer with the same weights and tokens; the data-parallel training step against
the single-GPU step on the concatenated batch; the sharded (ZeRO-1) integer AdamW against the
whole-state step.  These need two GPUs and are SKIPPED on a one-GPU box (a run with one rank
would compare the single-GPU code with itself); `*_one_rank` keeps a smoke run of the
multi-rank code paths with world = 1.  Rows of an expert GEMM are independent, so the
layer output and the input gradient must be bit-identical to the single-GPU
result; weight gradients are sums over rows in another order (1e-2)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
CFG = dict(N=1024, D=256, F=512, E=8, K=2)


def two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs: %d visible (not run, which is not a pass)" % torch.cuda.device_count())
    return 2


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def rel(a, b):
    a, b = a.float(), b.float()
    return max(float((a - b).norm() / b.norm()), float((a - b).abs().max() / b.abs().max()))


def worker(rank, world, port, ret, mode, cfg=None):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cudalm_c_b200 as q
    from cudalm_c_b200 import dist_moe, moe, qlm
    c = cfg or CFG
    N, D, F, E, K = c["N"], c["D"], c["F"], c["E"], c["K"]
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    full = [torch.randn(E * D * F, device=dev, generator=gen) * 0.02 for _ in range(3)]
    wr = torch.randn(D, E, device=dev, generator=gen) * 0.02
    if mode == "peer":
        ep = dist_moe.PeerExpertParallelLayer(c, dev, rank, world, seed=7, weights=full + [wr])
    else:
        ep = dist_moe.ExpertParallelLayer(c, dev, rank, world, seed=7, weights=full + [wr])
    # single-call reference with all experts local, on this rank's tokens
    qs = []
    for w in full:
        Q = qlm.Qlm([(0, w.numel())], w.numel(), dev); Q.init_from(w.clone(), render=False); qs.append((Q.d, Q.s))
    ref = moe.MoeLayerState(N, D, F, E, K, qs[0], qs[1], qs[2], wr)
    out_ref = ref.forward(ep.fi, ep.fn)
    dW = [torch.zeros(E, D, F, device=dev), torch.zeros(E, D, F, device=dev), torch.zeros(E, F, D, device=dev)]
    dWr = torch.zeros(D, E, device=dev)
    dfn_ref = ref.backward(ep.dout, ep.fn, dW[0], dW[1], dW[2], dWr, beta=0.0)
    for _ in range(2):                       # twice: buffers and arenas are reused
        out = ep.forward(); dfn = ep.backward()
    torch.cuda.synchronize()
    mine = ep.assign.view(K, N) if mode == "peer" else ep.member("assign", (K, N), torch.int32)
    assert torch.equal(mine, ref.member("assign", (K, N), torch.int32))
    assert torch.equal(out, out_ref)
    assert torch.equal(dfn, dfn_ref)
    assert rel(ep.dWr, dWr) < 1e-5
    el = E // world
    for i in range(3):
        tot = dW[i].clone()
        dist.all_reduce(tot)                 # weight gradients over all ranks' tokens
        assert rel(ep.dW[i], tot[rank * el:(rank + 1) * el]) < 1e-2, i
    q.check(q.lib().qlmb_check_device(None))
    if mode == "peer":
        ep.close()
    ret[rank] = True
    dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_one_rank(cuda, mode):
    """World = 1: the split calls and the window code run, nothing crosses a GPU."""
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(1, free_port(), ret, mode, dict(N=256, D=128, F=128, E=4, K=2)), nprocs=1, join=True)
        assert ret.get(0)


@pytest.mark.parametrize("mode", ["nccl", "peer"])
def test_expert_parallel_matches_single_call(cuda, mode):
    world = two_gpus()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(world, free_port(), ret, mode), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_expert_parallel_small_layer(cuda):
    """The peer form on the smallest layer the training-step test uses (256 tokens, 4 experts of 128 x 128)."""
    world = two_gpus()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(world, free_port(), ret, "peer", dict(N=256, D=128, F=128, E=4, K=2)), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def worker_dp(rank, world, port, ret):
    """Data-parallel training step with sharded experts (cudalm_c_b200/model.py, world > 1) against the
    single-GPU step on the concatenated batch: same losses, same gradients (replicated tensors after the
    all-reduce, this rank's experts), same clip norm."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cudalm_c_b200 as q
    from cudalm_c_b200 import model
    kw = dict(L=2, D=128, H=2, KV=2, hd=64, E=4, K=2, F=128, V=256, T=128)
    Bl = 2
    g = torch.Generator(device="cpu"); g.manual_seed(0)
    Nall = world * Bl * kw["T"]
    tok_all = torch.randint(0, kw["V"], (Nall,), generator=g, dtype=torch.int32).to(dev)
    tgt_all = torch.randint(0, kw["V"], (Nall,), generator=g, dtype=torch.int32).to(dev)
    N = Bl * kw["T"]
    sl = slice(rank * N, (rank + 1) * N)
    m = model.QlmModel(model.Config(B=Bl, **kw), dev, seed=3, rank=rank, world=world, init_blocks=world)
    m.forward(tok_all[sl].contiguous())
    loss = m.backward(tok_all[sl].contiguous(), tgt_all[sl].contiguous())
    m.update()
    torch.cuda.synchronize()
    ref = model.QlmModel(model.Config(B=world * Bl, **kw), dev, seed=3, init_blocks=world)
    ref.forward(tok_all)
    loss_ref = ref.backward(tok_all, tgt_all)
    ref.update()
    torch.cuda.synchronize()
    q.check(q.lib().qlmb_check_device(None))
    assert float((loss - loss_ref[sl]).abs().max()) < 2e-3
    c, el = m.c, m.el

    def rel(a, b):
        return float((a.double() - b.double()).norm() / b.double().norm())
    errs = {}
    for l in range(c.L):
        for nm in ("an1", "wq", "wk", "wv", "wo", "an2", "wr"):
            errs[(l, nm)] = rel(m._g(l, nm), ref._g(l, nm))
        for nm in ("w1", "w3", "w2"):
            n = m.o.layers[l][nm][1]
            errs[(l, nm)] = rel(m._g(l, nm), ref._g(l, nm)[rank * n:(rank + 1) * n])
    errs["emb"] = rel(m.G[:c.V * c.D], ref.G[:c.V * c.D])
    bad = {k: round(v, 4) for k, v in errs.items() if not v < 2e-2}
    assert not bad, (bad, {k: round(v, 5) for k, v in errs.items()})
    assert abs(float(m.gs[1]) - float(ref.gs[1])) < 1e-2 * float(ref.gs[1])
    if world > 1:
        for ly in m.layers:
            ly["moe"].close()
    ret[rank] = True
    dist.destroy_process_group()


def test_data_parallel_training_step(cuda):
    world = two_gpus()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker_dp, args=(world, free_port(), ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def worker_zero1(rank, world, port, ret):
    """ZeRO-1 form of the integer AdamW: rank r steps its share of the groups of one span and the state is
    all-gathered; every gathered array must equal the whole-span step's bytes (the rounding hash uses global
    element indices, so the split cannot show)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    from cudalm_c_b200 import qlm
    n = 128 * 65536
    ngrp = n // 128
    per = ngrp // world
    gen = torch.Generator(device=dev); gen.manual_seed(5)          # same seed: every rank holds the same P and G
    P = torch.randn(n, device=dev, generator=gen) * 0.02
    whole = qlm.Qlm([(0, n)], n, dev); whole.init_from(P.clone(), render=False)
    shard = qlm.Qlm([(0, n)], n, dev); shard.init_from(P.clone(), render=False)
    gi0 = rank * per
    for t in range(1, 4):
        G = torch.randn(n, device=dev, generator=gen) * 1e-3
        whole.step(None, G, 3e-4, 0.9, 0.95, 0.1, t)
        shard.step(None, G, 3e-4, 0.9, 0.95, 0.1, t, gi_base=gi0, ng=per)
        e0, e1 = gi0 * 128, (gi0 + per) * 128
        dist.all_gather_into_tensor(shard.d[:n // 2], shard.d[e0 // 2:e1 // 2].clone())
        for a in (shard.r, shard.m8, shard.v8):
            dist.all_gather_into_tensor(a[:n], a[e0:e1].clone())
        for a in (shard.m8s, shard.v8s):
            dist.all_gather_into_tensor(a, a[gi0:gi0 + per].clone())
        torch.cuda.synchronize()
        for k in ("d", "r", "m8", "v8", "m8s", "v8s"):
            assert torch.equal(getattr(whole, k), getattr(shard, k)), (k, t)
    ret[rank] = True
    dist.destroy_process_group()


def test_zero1_sharded_state_equals_whole(cuda):
    world = two_gpus()
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker_zero1, args=(world, free_port(), ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def worker_native(rank, world, port, ret):
    """The library's own communicator (NCCL bound inside the shared library; torch.distributed only hands the id
    over): collectives, the ZeRO-1 step against the whole-span step, and one expert-parallel layer driven by
    qlmb_ep_layer_forward / _backward against the Python-orchestrated layer (same kernels, same order: bit-equal)."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import ctypes as C
    from cudalm_c_b200 import comm, dist_moe, qlm
    from cudalm_c_b200._lib import BF16, EpPeers, check, lib, ptr, stream_ptr
    box = [comm.unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0)
    cm = comm.Comm(box[0], rank, world)
    # collectives
    a = torch.full((1000,), float(rank + 1), device=dev)
    cm.allreduce(a); assert float(a[0]) == sum(range(1, world + 1))
    cm.allreduce(a, avg=True); assert float(a[0]) == sum(range(1, world + 1))
    g = torch.zeros(world, 256, dtype=torch.int32, device=dev); g[rank] = rank + 7
    cm.allgather_inplace(g); cm.barrier(); torch.cuda.synchronize()
    assert all(int(g[r, 0]) == r + 7 and int(g[r, 255]) == r + 7 for r in range(world))
    # ZeRO-1: codes equal the whole-span step's on every rank; the share's other state equals the whole's share
    n = 128 * 16384
    ngrp = n // 128; per = ngrp // world; e0, e1 = rank * per * 128, (rank + 1) * per * 128
    gen = torch.Generator(device=dev); gen.manual_seed(5)
    P = torch.randn(n, device=dev, generator=gen) * 0.02
    whole = qlm.Qlm([(0, n)], n, dev); whole.init_from(P.clone(), render=False)
    shard = qlm.Qlm([(0, n)], n, dev); shard.init_from(P.clone(), render=False)
    for t in range(1, 4):
        G = torch.randn(n, device=dev, generator=gen) * 1e-3
        whole.step(None, G, 3e-4, 0.9, 0.95, 0.1, t)
        cm.zero1_step(shard, None, G, 3e-4, 0.9, 0.95, 0.1, t)
    torch.cuda.synchronize()
    assert torch.equal(whole.d, shard.d)
    for k in ("r", "m8", "v8"):
        assert torch.equal(getattr(whole, k)[e0:e1], getattr(shard, k)[e0:e1]), k
    for k in ("m8s", "v8s"):
        assert torch.equal(getattr(whole, k)[rank * per:(rank + 1) * per], getattr(shard, k)[rank * per:(rank + 1) * per]), k
    # expert-parallel layer: the natively orchestrated calls on a second window against the Python-orchestrated layer
    if world > 1:
        dist.destroy_process_group()
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    c = CFG
    gen = torch.Generator(device=dev); gen.manual_seed(7)
    full = [torch.randn(c["E"] * c["D"] * c["F"], device=dev, generator=gen) * 0.02 for _ in range(3)]
    wr = torch.randn(c["D"], c["E"], device=dev, generator=gen) * 0.02
    ep = dist_moe.PeerExpertParallelLayer(c, dev, rank, world, seed=7, weights=full + [wr])
    out_py = ep.forward().clone(); dfn_py = ep.backward().clone()
    dW_py = [w.clone() for w in ep.dW]; dWr_py = ep.dWr.clone()
    torch.cuda.synchronize()
    L, st = lib(), stream_ptr()
    peers = EpPeers()
    check(L.qlmb_ep_window_open(cm.h, ep.win_ptr, C.byref(peers), st))
    for w in ep.dW:
        w.zero_()
    ep.dWr.zero_(); ep.Ys.zero_(); ep.dXs.zero_()
    out = torch.empty_like(ep.fi); dfn = torch.empty_like(ep.fi)
    cm.barrier()
    check(L.qlmb_ep_layer_forward(cm.h, ep.home, ep.hptr, ep.loc, ep.eptr, C.byref(peers), ptr(ep.assign_all), ptr(ep.fn), BF16,
                                  ptr(ep.fi), ptr(ep.Ys), ptr(out), st))
    check(L.qlmb_ep_layer_backward(cm.h, ep.home, ep.hptr, ep.loc, ep.eptr, C.byref(peers), ptr(ep.dout), ptr(ep.fn), ptr(ep.Ys),
                                   ptr(ep.dXs), ptr(dfn), ptr(ep.dW[0]), ptr(ep.dW[1]), ptr(ep.dW[2]), ptr(ep.dWr), 0.0, 1, st))
    torch.cuda.synchronize()
    assert torch.equal(out, out_py) and torch.equal(dfn, dfn_py)
    assert all(torch.equal(a_, b_) for a_, b_ in zip(ep.dW, dW_py)) and torch.equal(ep.dWr, dWr_py)
    check(L.qlmb_ep_window_close(cm.h, C.byref(peers), st))
    ep.close()
    cm.close()
    ret[rank] = True
    dist.destroy_process_group()


def _run_native(world):
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker_native, args=(world, free_port(), ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_native_comm_one_rank(cuda):
    _run_native(1)


def test_native_comm_two_ranks(cuda):
    _run_native(two_gpus())
