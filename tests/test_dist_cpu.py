"""Host-side logic of the expert-parallel path on two gloo ranks (no GPU):
split sizes, arrival order and row tags of the dispatch all-to-all, and that the
return exchange is its exact inverse."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import loader


def free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close(); return p


def worker(rank, world, port, E, K, N, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from cudalm_c_b200.dist_moe import all_to_all_rows, exchange_plan
    o = loader.restatement()
    el = E // world
    # every rank can rebuild every rank's routing (seeded), so the expected result is known everywhere
    asg = [np.random.default_rng(100 + r).integers(0, E, size=(K, N)).astype(np.int32) for r in range(world)]
    perms, counts = [], []
    for r in range(world):
        perm, inv, off, bad = o.perm_build(asg[r], E, merged=1)
        perms.append(perm); counts.append(np.diff(off))
    counts_all = np.stack(counts)
    send, recv, tags = exchange_plan(counts_all, rank, world)
    assert sum(send) == K * N and len(tags) == sum(recv)
    # rows carry (source rank, slot) so their origin can be checked after the exchange
    mine = torch.tensor([[rank, int(s)] for s in perms[rank]], dtype=torch.float32)
    got = torch.zeros(sum(recv), 2)
    all_to_all_rows(got, mine, recv, send)
    exp_rows, exp_tags = [], []
    for s in range(world):
        off = np.concatenate([[0], np.cumsum(counts[s])])
        for e in range(rank * el, (rank + 1) * el):
            for slot in perms[s][off[e]:off[e + 1]]:
                exp_rows.append([s, int(slot)]); exp_tags.append(e - rank * el)
    assert got.tolist() == [[float(a), float(b)] for a, b in exp_rows]
    assert tags.tolist() == exp_tags
    # every arrived row really belongs to the tagged local expert
    for (s, slot), t in zip(exp_rows, tags):
        assert asg[s].reshape(-1)[slot] == rank * el + t
    # the return trip restores the packed order
    back = torch.zeros(K * N, 2)
    all_to_all_rows(back, got, send, recv)
    assert torch.equal(back, mine)
    ret[rank] = True
    dist.destroy_process_group()


def test_exchange_plan_two_ranks():
    world, E, K, N = 2, 8, 2, 257
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(worker, args=(world, free_port(), E, K, N, ret), nprocs=world, join=True)
        assert all(ret.get(r) for r in range(world))


def test_exchange_plan_shapes():
    from cudalm_c_b200.dist_moe import exchange_plan
    counts = np.array([[3, 0, 2, 1], [1, 1, 0, 4]])
    send, recv, tags = exchange_plan(counts, 1, 2)
    assert send == [2, 4] and recv == [3, 4]
    assert tags.tolist() == [0, 0, 1, 1, 1, 1, 1]
    send, recv, tags = exchange_plan(counts, 0, 2)
    assert send == [3, 3] and recv == [3, 2] and tags.tolist() == [0, 0, 0, 0, 1]
