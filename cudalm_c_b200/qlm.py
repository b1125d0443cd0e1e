"""Host-side mirror of the reference's QLM state interface (qlm.cuh).

Function names follow the reference: k_qlm_encode -> qlm_encode, k_qlm_render
-> qlm_render, qlm_step_launch, k_qlm_servo -> qlm_servo, k_sqsum+k_gnorm ->
gnorm, k_adamw -> adamw; `Qlm` mirrors the reference's Qlm struct together with
qlm_gpu_init / qlm_gpu_update.  Tensors are torch CUDA tensors used purely as
device memory; every operation is one call into libqlm_b200.so.
"""
import ctypes as C
import math

import numpy as np
import torch

from ._lib import SPAN_DTYPE, check, lib, ptr, stream_ptr


def qd_bytes(nq, packed):
    """Bytes of the digit array (qlm.cuh:109-111)."""
    return (nq + 1) // 2 if packed else nq


def spans_to_device(spans, device):
    return torch.from_numpy(spans.view(np.uint8).reshape(-1)).to(device)


def qlm_encode(P, d, r, s, spans_dev, nspan, group=128, dmax=7, packed=1):
    check(lib().qlmb_encode(ptr(P), ptr(d), ptr(r), ptr(s), ptr(spans_dev), nspan, s.numel(), group, dmax,
                            packed, stream_ptr()))


def qlm_render(P, d, s, spans_dev, nspan, group=128, packed=1, gi_base=0, ng=None):
    ng = s.numel() if ng is None else ng
    check(lib().qlmb_render(ptr(P), ptr(d), ptr(s), ptr(spans_dev), nspan, group, packed, gi_base, ng,
                            stream_ptr()))


def qlm_step_launch(P, G, d, r, s, m8, m8s, v8, v8s, spans_dev, nspan, group, dmax, lr, b1, b2, wd, gscale,
                    gsp, inv_bc1, inv_sqrt_bc2, lrmode, t, adam, stat, packed, gi_base, ng):
    """Argument for argument the reference's qlm_step_launch (qlm.cuh:377-383)."""
    check(lib().qlmb_step(ptr(P), ptr(G), ptr(d), ptr(r), ptr(s), ptr(m8), ptr(m8s), ptr(v8), ptr(v8s),
                          ptr(spans_dev), nspan, group, dmax, lr, b1, b2, wd, gscale, ptr(gsp), inv_bc1,
                          inv_sqrt_bc2, lrmode, t, adam, ptr(stat), packed, gi_base, ng, stream_ptr()))


def qlm_servo(d, r, s, spans_dev, nspan, group, dmax, f_hi, f_lo, packed=1):
    check(lib().qlmb_servo(ptr(d), ptr(r), ptr(s), ptr(spans_dev), nspan, s.numel(), group, dmax, f_hi, f_lo,
                           packed, stream_ptr()))


def gnorm(G, sides=(), clip_side=0, out=None):
    """gs[0] = clip multiplier, gs[1] = norm (k_sqsum + k_gnorm, cudalm.cu:6442-6444)."""
    gs = out if out is not None else torch.empty(2, dtype=torch.float32, device=G.device)
    ns = len(sides)
    ptrs = (C.c_void_p * max(ns, 1))(*[x.data_ptr() for x in sides])
    lens = (C.c_size_t * max(ns, 1))(*[x.numel() for x in sides])
    check(lib().qlmb_gnorm(ptr(G), G.numel(), C.cast(ptrs, C.c_void_p), C.cast(lens, C.c_void_p), ns, clip_side,
                           ptr(gs), stream_ptr()))
    return gs


def adamw(P, G, M, V, lr, b1, b2, wd, bc1, bc2, gs=None):
    """k_adamw for float spans; M, V are bf16 bit patterns (int16/uint16 storage)."""
    check(lib().qlmb_adamw(ptr(P), ptr(G), ptr(M), ptr(V), P.numel(), lr, b1, b2, wd, bc1, bc2, ptr(gs),
                           stream_ptr()))


def sqsum(G, part64):
    """k_sqsum into a caller-owned slice of 64 floats (qlm_fused_layer, cudalm.cu:6122)."""
    check(lib().qlmb_sqsum(ptr(G), G.numel(), ptr(part64), stream_ptr()))


def gnorm_close(part, nslice, gs):
    """The norm of all slices -> gs[0] = next step's clip multiplier, gs[1] = norm (cudalm.cu:6182-6186)."""
    check(lib().qlmb_gnorm_close(ptr(part), nslice, ptr(gs), stream_ptr()))


def bias_corrections(b1, b2, t):
    """(bc1, bc2) in fp32 as gpu_adam derives them with powf (cudalm.cu:6454)."""
    f = np.float32
    return float(f(1) - f(np.power(f(b1), f(t)))), float(f(1) - f(np.power(f(b2), f(t))))


class Qlm:
    """The reference's Qlm state for a list of quantised spans (qlm.cuh:40-58).

    `matrices` is a list of (offset_in_P, n_elements) in ascending offset order,
    as qlm_gpu_init builds it from the model layout (qlm.cuh:479-489); the gaps
    between them are the float spans (qlm.cuh:493-502)."""

    def __init__(self, matrices, np_total, device, bits=4, group=128, lrmode=0, servo_every=100, adam=1):
        self.dmax = 1 if bits <= 2 else 3 if bits == 3 else 7 if bits == 4 else 127
        self.group = max(32, min(256, group))
        self.lrmode, self.servo_every, self.adam = lrmode, servo_every, adam
        self.fstar = 0.60 if self.dmax == 1 else 1.5 / self.group
        self.f_hi, self.f_lo = self.fstar * 1.5, self.fstar * 0.5
        self.packed = 1 if self.dmax <= 7 else 0
        self.np = np_total
        self.device = device
        sp = np.zeros(len(matrices), SPAN_DTYPE)
        nq = ngrp = 0
        for i, (pof, n) in enumerate(matrices):
            g = (n + self.group - 1) // self.group
            sp[i] = (pof, pof, nq, n, ngrp, g, 1.0, 0)
            nq += n
            ngrp += g
        self.spanH, self.nspan, self.nq, self.ngrp = sp, len(matrices), nq, ngrp
        self.fs = []                       # (offset, n, compact offset) of the float spans
        cur = acc = 0
        for pof, n in matrices:
            if pof > cur:
                self.fs.append((cur, pof - cur, acc)); acc += pof - cur
            cur = pof + n
        if cur < np_total:
            self.fs.append((cur, np_total - cur, acc)); acc += np_total - cur
        self.nfloat = acc
        z = lambda n, dt: torch.zeros(max(n, 1), dtype=dt, device=device)
        self.d = z(qd_bytes(nq, self.packed), torch.int8)
        self.r = z(nq, torch.int8)
        self.m8 = z(nq, torch.int8)
        self.v8 = z(nq, torch.uint8)
        self.s = z(ngrp, torch.float32)[:ngrp]
        self.m8s = z(ngrp, torch.float32)[:ngrp]
        self.v8s = z(ngrp, torch.float32)[:ngrp]
        self.Mc = z(self.nfloat, torch.int16)
        self.Vc = z(self.nfloat, torch.int16)
        self.spanD = spans_to_device(sp, device)

    def init_from(self, P, render=True):
        """qlm_gpu_init's device part: encode, freeze sref = mean group scale of
        each span (double mean -> float, qlm.cuh:528-533), render."""
        qlm_encode(P, self.d, self.r, self.s, self.spanD, self.nspan, self.group, self.dmax, self.packed)
        sh = self.s.cpu().numpy()
        for i in range(self.nspan):
            g0, g = int(self.spanH[i]["gi0"]), int(self.spanH[i]["ngrp"])
            self.spanH[i]["sref"] = np.float32(np.cumsum(sh[g0:g0 + g].astype(np.float64))[-1] / float(g))
        self.spanD = spans_to_device(self.spanH, self.device)
        if render:
            self.render(P)

    def render(self, P, gi_base=0, ng=None):
        qlm_render(P, self.d, self.s, self.spanD, self.nspan, self.group, self.packed, gi_base, ng)

    def step(self, P, G, lr, b1, b2, wd, t, gscale=1.0, gsp=None, stat=None, gi_base=0, ng=None):
        bc1, bc2 = bias_corrections(b1, b2, t)
        f = np.float32
        inv_bc1 = float(f(1) / f(bc1))
        inv_sqrt_bc2 = float(f(1) / np.sqrt(f(bc2)))
        ng = self.ngrp if ng is None else ng
        qlm_step_launch(P, G, self.d, self.r, self.s, self.m8, self.m8s, self.v8, self.v8s, self.spanD,
                        self.nspan, self.group, self.dmax, lr, b1, b2, wd, gscale, gsp, inv_bc1, inv_sqrt_bc2,
                        self.lrmode, t, self.adam, stat, self.packed, gi_base, ng)

    def servo(self):
        qlm_servo(self.d, self.r, self.s, self.spanD, self.nspan, self.group, self.dmax, self.f_hi, self.f_lo,
                  self.packed)

    def update(self, P, G, lr, b1, b2, wd, t, gs=None, wdf=None):
        """qlm_gpu_update (cudalm.cu:6082-6103): integer AdamW over every group,
        bf16-moment AdamW over the float spans, servo tick every servo_every steps."""
        self.step(P, G, lr, b1, b2, wd, t, gscale=1.0, gsp=gs)
        bc1, bc2 = bias_corrections(b1, b2, t)
        for off, n, cs in self.fs:
            adamw(P[off:off + n], G[off:off + n], self.Mc[cs:cs + n], self.Vc[cs:cs + n], lr, b1, b2,
                  wd if wdf is None else wdf, bc1, bc2, gs)
        if self.servo_every > 0 and t % self.servo_every == 0:
            self.servo()

    # ---- QLMH state file (qlm_save / qlm_load, qlm.cuh:703-788) ----
    def _statefile(self, arrays):
        from ._lib import StateFile
        v = StateFile()
        v.dmax, v.group, v.adam, v.nspan, v.packed = self.dmax, self.group, self.adam, self.nspan, self.packed
        v.nq, v.ngrp, v.nfloat = self.nq, self.ngrp, self.nfloat
        for k, a in arrays.items():
            setattr(v, k, a.ctypes.data if a is not None and a.size else None)
        return v

    def save(self, path, iteration, prev_gn=1.0):
        """Write the integer state as the reference's .opt.q file (device -> host -> file, atomic replace)."""
        h = lambda t, n: np.ascontiguousarray(t[:n].cpu().numpy())
        arr = dict(Mc=h(self.Mc, self.nfloat).view(np.uint16), Vc=h(self.Vc, self.nfloat).view(np.uint16),
                   d=h(self.d, qd_bytes(self.nq, self.packed)), r=h(self.r, self.nq), m8=h(self.m8, self.nq),
                   v8=h(self.v8, self.nq) if self.adam else None, s=h(self.s, self.ngrp), m8s=h(self.m8s, self.ngrp),
                   v8s=h(self.v8s, self.ngrp) if self.adam else None,
                   sref=np.ascontiguousarray(self.spanH["sref"].astype(np.float32)))
        v = self._statefile(arr)
        v.iter, v.prev_gn = int(iteration), float(prev_gn)
        check(lib().qlmb_statefile_write(str(path).encode(), v))

    def load(self, path):
        """Read a .opt.q file written by this library or by the reference into this state.
        Returns (iteration, prev_gn or None).  A file of another shape raises QlmbError; without the
        SREF trailer the spans keep their current reference scales, as in the reference."""
        z = lambda n, dt: np.zeros(max(int(n), 1), dt)
        arr = dict(Mc=z(self.nfloat, np.uint16), Vc=z(self.nfloat, np.uint16), d=z(qd_bytes(self.nq, self.packed), np.int8),
                   r=z(self.nq, np.int8), m8=z(self.nq, np.int8), v8=z(self.nq, np.uint8) if self.adam else None,
                   s=z(self.ngrp, np.float32), m8s=z(self.ngrp, np.float32),
                   v8s=z(self.ngrp, np.float32) if self.adam else None, sref=z(self.nspan, np.float32))
        v = self._statefile(arr)
        for k in ("Mc", "Vc", "d", "r", "m8", "s", "m8s", "sref"):
            setattr(v, k, arr[k].ctypes.data)
        check(lib().qlmb_statefile_read(str(path).encode(), v))
        nf = int(v.nfloat)
        up = lambda t, a, n: t[:n].copy_(torch.from_numpy(a[:n].copy()).to(t.device)) if n else None
        up(self.Mc, arr["Mc"].view(np.int16), nf); up(self.Vc, arr["Vc"].view(np.int16), nf)
        up(self.d, arr["d"], qd_bytes(self.nq, self.packed)); up(self.r, arr["r"], self.nq); up(self.m8, arr["m8"], self.nq)
        up(self.s, arr["s"], self.ngrp); up(self.m8s, arr["m8s"], self.ngrp)
        if self.adam:
            up(self.v8, arr["v8"], self.nq); up(self.v8s, arr["v8s"], self.ngrp)
        if v.have_sref:
            self.spanH["sref"] = arr["sref"][:self.nspan]
            self.spanD = spans_to_device(self.spanH, self.device)
        return int(v.iter), (float(v.prev_gn) if v.have_prev_gn else None)

    def persist_bytes(self):
        """qlm_persist_bytes (qlm.cuh:678-683)."""
        return (qd_bytes(self.nq, self.packed) + self.nq + self.nq * (2 if self.adam else 1)
                + self.ngrp * 4 * (3 if self.adam else 2))


class FusedUpdate:
    """The fused per-layer update (qlm_fused_layer / qlm_fused_tail, cudalm.cu:6105-6187).

    Backward calls layer(l) as soon as layer l's gradients are complete, so all layers can share one
    gradient block (calc_goffsets, cudalm.cu:6008-6040; the spans' gof then differ from pof, set with
    set_gof as qlm_set_gof does, qlm.cuh:555-575); tail() updates what keeps private gradient slots
    and closes the step's norm, which clips the NEXT step.  `gs` (device: multiplier, norm) plays
    g_prev_gn / g_fgs and never visits the host.

    layer_float[l] and tail_float are lists of (p_off, g_off, n, wd) float spans; a layer owns
    `spans_per_layer` consecutive quantised spans (7 in the reference's models)."""

    def __init__(self, q, n_layers, layer_g0, layer_gn, layer_float, tail_float, spans_per_layer=7):
        self.q, self.L, self.spl = q, n_layers, spans_per_layer
        self.layer_g0, self.layer_gn = layer_g0, layer_gn
        self.layer_float, self.tail_float = layer_float, tail_float
        dev = q.device
        self.gnpart = torch.zeros(64 * (n_layers + len(tail_float)), dtype=torch.float32, device=dev)
        self.gs = torch.ones(2, dtype=torch.float32, device=dev)          # g_prev_gn = 1 before the first step

    def set_gof(self, gofs):
        """Point each quantised span's gradient read at the compact map (qlm_set_gof)."""
        for i, g in enumerate(gofs):
            self.q.spanH[i]["gof"] = g
        self.q.spanD = spans_to_device(self.q.spanH, self.q.device)

    def _cs(self, p_off):
        for off, n, cs in self.q.fs:
            if off <= p_off < off + n:
                return cs + (p_off - off)
        raise ValueError("offset %d is not in a float span" % p_off)

    def _float(self, P, G, spans, lr, b1, b2, t):
        bc1, bc2 = bias_corrections(b1, b2, t)
        q = self.q
        for p_off, g_off, n, wd in spans:
            cs = self._cs(p_off)
            adamw(P[p_off:p_off + n], G[g_off:g_off + n], q.Mc[cs:cs + n], q.Vc[cs:cs + n], lr, b1, b2, wd,
                  bc1, bc2, self.gs)

    def layer(self, P, G, l, lr, t, b1=0.9, b2=0.95, wd=0.1):
        q = self.q
        sqsum(G[self.layer_g0:self.layer_g0 + self.layer_gn], self.gnpart[64 * l:64 * l + 64])
        s0 = self.spl * l
        gi0 = int(q.spanH[s0]["gi0"])
        ng = int(sum(int(q.spanH[i]["ngrp"]) for i in range(s0, s0 + self.spl)))
        q.step(P, G, lr, b1, b2, wd, t, gscale=1.0, gsp=self.gs, gi_base=gi0, ng=ng)
        self._float(P, G, self.layer_float[l], lr, b1, b2, t)

    def tail(self, P, G, lr, t, b1=0.9, b2=0.95):
        self._float(P, G, self.tail_float, lr, b1, b2, t)
        for i, (p_off, g_off, n, wd) in enumerate(self.tail_float):
            k = self.L + i
            sqsum(G[g_off:g_off + n], self.gnpart[64 * k:64 * k + 64])
        gnorm_close(self.gnpart, self.L + len(self.tail_float), self.gs)
