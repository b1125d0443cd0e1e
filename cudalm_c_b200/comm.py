"""Host mirror of the library's native multi-GPU layer (qlmb_comm_*, qlmb_zero1_*, qlmb_ep_layer_*): the calls a C or
C++ trainer makes, reachable from Python for tests and the bench.  The communicator is the library's own (NCCL bound
inside libqlm_b200.so); torch.distributed is not involved beyond handing the 128-byte id to the other ranks."""
import ctypes as C

import numpy as np

from ._lib import check, lib, ptr, stream_ptr


def unique_id():
    """bytes(128) made on one rank; hand it to the others by any host channel."""
    buf = (C.c_ubyte * 128)()
    check(lib().qlmb_comm_unique_id(buf))
    return bytes(buf)


class Comm:
    def __init__(self, uid, rank, world):
        self.h = C.c_void_p()
        buf = (C.c_ubyte * 128)(*uid)
        check(lib().qlmb_comm_init(C.byref(self.h), buf, rank, world))
        self.rank, self.world = rank, world

    def close(self):
        if self.h:
            lib().qlmb_comm_destroy(self.h)
            self.h = C.c_void_p()

    def allreduce(self, t, avg=False):
        check(lib().qlmb_comm_allreduce_f32(self.h, ptr(t), t.numel(), int(avg), stream_ptr()))

    def allgather_inplace(self, t):
        """t holds world equal shares; this rank's share is already in place"""
        nb = t.numel() * t.element_size() // self.world
        check(lib().qlmb_comm_allgather(self.h, t.data_ptr() + self.rank * nb, ptr(t), nb, stream_ptr()))

    def barrier(self):
        check(lib().qlmb_comm_barrier(self.h, stream_ptr()))

    def zero1_step(self, Q, P, G, lr, b1, b2, wd, t, gscale=1.0, gsp=None):
        """qlmb_zero1_step on a cudalm_c_b200.qlm.Qlm state: this rank's share of the groups, codes all-gathered"""
        from .qlm import bias_corrections
        f = np.float32
        bc1, bc2 = bias_corrections(b1, b2, t)
        check(lib().qlmb_zero1_step(self.h, ptr(P), ptr(G), ptr(Q.d), ptr(Q.r), ptr(Q.s), ptr(Q.m8), ptr(Q.m8s), ptr(Q.v8),
                                    ptr(Q.v8s), ptr(Q.spanD), Q.nspan, Q.ngrp, Q.group, Q.dmax, lr, b1, b2, wd, gscale, ptr(gsp),
                                    float(f(1) / f(bc1)), float(f(1) / np.sqrt(f(bc2))), Q.lrmode, t, Q.adam, None, Q.packed,
                                    stream_ptr()))
