"""The allocation-free grad-norm entry point, through the C ABI.

qlmb_gnorm_noalloc exists for hosts that cannot let the library call cudaMalloc
(their own pool owns all device memory, or an allocation's device-wide
synchronisation is unacceptable mid-step).  It must give exactly what qlmb_gnorm
gives -- both run the same kernels, only the scratch differs -- also on a second
call that finds the previous call's partial sums still in the fixed array.
This file is named so that pytest collects it last."""
import ctypes as C

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def call(fn, G, sides, clip_side, gs):
    import cudalm_c_b200 as q
    from cudalm_c_b200._lib import ptr, stream_ptr
    ns = len(sides)
    ptrs = (C.c_void_p * max(ns, 1))(*[x.data_ptr() for x in sides])
    lens = (C.c_size_t * max(ns, 1))(*[x.numel() for x in sides])
    return fn(ptr(G), G.numel(), C.cast(ptrs, C.c_void_p), C.cast(lens, C.c_void_p), ns, clip_side, ptr(gs), stream_ptr())


def test_noalloc_matches_gnorm_twice_in_a_row(cuda):
    import cudalm_c_b200 as q
    L = q.lib()
    gen = torch.Generator(device=cuda); gen.manual_seed(99)
    # first call: a large gradient with three side buffers; second call: different,
    # smaller inputs, so stale partial sums of call one would show if they were read
    cases = [
        (torch.randn(5_000_003, device=cuda, generator=gen) * 3e-3,
         [torch.randn(n, device=cuda, generator=gen) * 0.1 for n in (1234, 77, 40_000)], 1),
        (torch.randn(70_001, device=cuda, generator=gen) * 1e-3, [], 0),
    ]
    for G, sides, clip in cases:
        want = torch.zeros(2, device=cuda); got = torch.full((2,), -1.0, device=cuda)
        q.check(call(L.qlmb_gnorm, G, sides, clip, want))
        q.check(call(L.qlmb_gnorm_noalloc, G, sides, clip, got))
        torch.cuda.synchronize()
        assert torch.equal(got, want)                 # same kernels, same order: bit-identical
        ref = float(torch.sqrt(sum((x.double() ** 2).sum() for x in [G] + (sides if clip else []))))
        assert abs(float(got[1]) - ref) <= 1e-6 * ref


def test_noalloc_rejects_more_sides_than_its_scratch_holds(cuda):
    import cudalm_c_b200 as q
    L = q.lib()
    G = torch.ones(1000, device=cuda)
    sides = [torch.ones(10, device=cuda) for _ in range(8)]
    gs = torch.zeros(2, device=cuda)
    rc = call(L.qlmb_gnorm_noalloc, G, sides, 1, gs)
    assert rc == 1 and b"exceed the fixed scratch" in L.qlmb_last_error()
    q.check(call(L.qlmb_gnorm_noalloc, G, sides[:7], 1, gs))      # the stated maximum is accepted
    torch.cuda.synchronize()
    assert abs(float(gs[1]) - np.sqrt(1000 + 70)) < 1e-4
