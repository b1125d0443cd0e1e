"""Expert-parallel layer, in both forms (split C-ABI calls + NCCL all-to-all; peer loads
inside the row kernels, no exchange step), against the
single-call layer with the same weights and tokens.  Runs on every visible GPU
(1, or 2 when the box has them): rows of an expert GEMM are independent, so the
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


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def rel(a, b):
    a, b = a.float(), b.float()
    return max(float((a - b).norm() / b.norm()), float((a - b).abs().max() / b.abs().max()))


def worker(rank, world, port, ret, mode):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    import cudalm_c_b200 as q
    from cudalm_c_b200 import dist_moe, moe, qlm
    c = CFG
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
def test_expert_parallel_matches_single_call(cuda, mode):
    world = min(torch.cuda.device_count(), 2)
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(world, free_port(), ret, mode), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))
