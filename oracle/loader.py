"""ctypes loaders for the two CPU checkers.  TEST INFRASTRUCTURE ONLY.

`restatement()` loads oracle/_build/libqlm_oracle.so (the C restatement in
qlm_oracle.c).  `reference(exact=True)` loads oracle/_ref/libcudalm_ref_*.so
(the unmodified reference compiled by the Makefile) or returns None when it was
never built.  Both are used only by tests/, by __graft_entry__.smoke() and by
bench.py's CPU-baseline legs; the shipped package never imports this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

SPAN_DTYPE = np.dtype(
    [("pof", "<u8"), ("gof", "<u8"), ("qi0", "<u8"), ("n", "<u8"),
     ("gi0", "<i4"), ("ngrp", "<i4"), ("sref", "<f4"), ("_pad", "<i4")])
assert SPAN_DTYPE.itemsize == 48


def make_spans(sizes, group=128, pofs=None):
    """Span table for consecutive matrices of the given element counts
    (the reference's qlm_add_span, qlm.cuh:448-455)."""
    sp = np.zeros(len(sizes), SPAN_DTYPE)
    nq = 0
    ngrp = 0
    pof = 0
    for i, n in enumerate(sizes):
        sp[i]["pof"] = pofs[i] if pofs is not None else pof
        sp[i]["gof"] = sp[i]["pof"]
        sp[i]["qi0"] = nq
        sp[i]["n"] = n
        sp[i]["gi0"] = ngrp
        sp[i]["ngrp"] = (n + group - 1) // group
        sp[i]["sref"] = 1.0
        nq += n
        ngrp += int(sp[i]["ngrp"])
        pof += n
    return sp, nq, ngrp


def _p(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def build(target="oracle"):
    subprocess.check_call(["make", "-s", "-C", HERE, target])


class Restatement:
    def __init__(self, path):
        L = self.lib = C.CDLL(path)
        L.qo_hash.restype = C.c_uint32
        L.qo_hash.argtypes = [C.c_uint64]
        L.qo_sround.restype = C.c_int
        L.qo_sround.argtypes = [C.c_float, C.c_uint64, C.c_uint64]
        L.qo_fexp.restype = C.c_float
        L.qo_fexp.argtypes = [C.c_float]
        L.qo_perm_build.restype = C.c_int
        self.threads = os.cpu_count()

    def hash(self, x):
        return self.lib.qo_hash(x)

    def sround(self, v, i, t):
        return self.lib.qo_sround(v, i, t)

    def fexp(self, x):
        return self.lib.qo_fexp(x)

    def encode(self, P, d, r, s, sp, group=128, dmax=7, packed=1):
        self.lib.qo_encode(_p(P), _p(d), _p(r), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(len(s)),
                           C.c_int(group), C.c_int(dmax), C.c_int(packed))

    def render(self, P, d, s, sp, group=128, packed=1, gi_base=0, ng=None):
        ng = len(s) if ng is None else ng
        self.lib.qo_render(_p(P), _p(d), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(group),
                           C.c_int(packed), C.c_int(gi_base), C.c_int(ng))

    def step(self, P, G, d, r, s, m8, m8s, v8, v8s, sp, *, group=128, dmax=7, lr, b1, b2, wd,
             gscale=1.0, inv_bc1, inv_sqrt_bc2, lrmode=0, t, adam=1, stat=None, packed=1,
             gi_base=0, ng=None):
        ng = len(s) if ng is None else ng
        f = C.c_float
        self.lib.qo_step(_p(P), _p(G), _p(d), _p(r), _p(s), _p(m8), _p(m8s), _p(v8), _p(v8s), _p(sp),
                         C.c_int(len(sp)), C.c_int(group), C.c_int(dmax), f(lr), f(b1), f(b2), f(wd),
                         f(gscale), f(inv_bc1), f(inv_sqrt_bc2), C.c_int(lrmode), C.c_uint64(t),
                         C.c_int(adam), _p(stat), C.c_int(packed), C.c_int(gi_base), C.c_int(ng))

    def set_v4(self, on):
        self.lib.qo_set_v4(C.c_int(1 if on else 0))

    def servo(self, d, r, s, sp, group=128, dmax=7, f_hi=0.0, f_lo=0.0, packed=1):
        self.lib.qo_servo(_p(d), _p(r), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(len(s)),
                          C.c_int(group), C.c_int(dmax), C.c_float(f_hi), C.c_float(f_lo),
                          C.c_int(packed))

    def gnorm(self, G, sides=(), clip_side=0):
        gs = np.zeros(2, np.float32)
        ns = len(sides)
        ptrs = (C.c_void_p * max(ns, 1))(*[x.ctypes.data for x in sides])
        lens = (C.c_size_t * max(ns, 1))(*[x.size for x in sides])
        self.lib.qo_gnorm(_p(G), C.c_size_t(G.size), ptrs, lens, C.c_int(ns), C.c_int(clip_side), _p(gs))
        return gs

    def bias_update(self, b, counts, m, u, prop):
        ns, E = counts.shape
        self.lib.qo_bias_update(_p(b), _p(counts), C.c_int(ns), C.c_int(E), C.c_float(m), C.c_float(u), C.c_int(prop))

    def nggate_f(self, h, v, k):
        N, D = h.shape
        hn = np.zeros_like(h); g, rh, rk = (np.zeros(N, np.float32) for _ in range(3))
        self.lib.qo_nggate_f(_p(h), _p(v), _p(k), _p(hn), _p(g), _p(rh), _p(rk), C.c_int(N), C.c_int(D))
        return hn, g, rh, rk

    def nggate_b(self, dy, v, hn, kn, g, rh, rk):
        N, D = dy.shape
        dv, dk = np.zeros_like(dy), np.zeros_like(dy)
        self.lib.qo_nggate_b(_p(dy), _p(v), _p(hn), _p(kn), _p(g), _p(rh), _p(rk), _p(dv), _p(dk), C.c_int(N), C.c_int(D))
        return dv, dk

    def sqsum(self, G):
        part = np.zeros(64, np.float32)
        self.lib.qo_sqsum(_p(G), C.c_size_t(G.size), _p(part))
        return part

    def adamw(self, P, G, M, V, lr, b1, b2, wd, bc1, bc2, gs=None):
        f = C.c_float
        self.lib.qo_adamw(_p(P), _p(G), _p(M), _p(V), C.c_size_t(P.size), f(lr), f(b1), f(b2), f(wd),
                          f(bc1), f(bc2), _p(gs))

    def router_topk(self, rt, K, bias=None, bs=0):
        N, E = rt.shape
        rprobs = np.zeros((N, E), np.float32)
        assign = np.zeros((K, N), np.int32)
        gate = np.zeros((K, N), np.float32)
        self.lib.qo_router_topk(_p(rt), _p(rprobs), _p(assign), _p(gate), C.c_int(N), C.c_int(E),
                                C.c_int(K), _p(bias), C.c_int(bs))
        return rprobs, assign, gate

    def perm_build(self, assign, E, merged):
        K, N = assign.shape
        perm = np.zeros(K * N, np.int32)
        inv = np.zeros(K * N, np.int32)
        off = np.zeros((1 if merged else K) * (E + 1), np.int32)
        bad = self.lib.qo_perm_build(_p(assign), C.c_int(N), C.c_int(E), C.c_int(K), C.c_int(merged),
                                     _p(perm), _p(inv), _p(off))
        return perm, inv, off, bad

    def linear_fwd(self, X, d, s, layout, N, group=128):
        M, K = X.shape
        Y = np.zeros((M, N), np.float32)
        self.lib.qo_linear_fwd(_p(Y), _p(X), _p(d), _p(s), C.c_int(layout), C.c_int(M), C.c_int(K),
                               C.c_int(N), C.c_int(group))
        return Y

    def linear_dgrad(self, dY, d, s, layout, K, group=128):
        M, N = dY.shape
        dX = np.zeros((M, K), np.float32)
        self.lib.qo_linear_dgrad(_p(dX), _p(dY), _p(d), _p(s), C.c_int(layout), C.c_int(M), C.c_int(K),
                                 C.c_int(N), C.c_int(group))
        return dX

    def linear_wgrad(self, dW, dY, X, layout):
        M, K = X.shape
        N = dY.shape[1]
        self.lib.qo_linear_wgrad(_p(dW), _p(dY), _p(X), C.c_int(layout), C.c_int(M), C.c_int(K), C.c_int(N))
        return dW

    def moe_fwd(self, f_in, fnorm, Wr, q1, q3, q2, F, K, group=128):
        """q1/q3/q2 = (codes, scales) of W1,W3 [E,D,F] and W2 [E,F,D]."""
        N, D = fnorm.shape
        E = Wr.shape[1]
        o = dict(out=np.zeros((N, D), np.float32), rt=np.zeros((N, E), np.float32),
                 rprobs=np.zeros((N, E), np.float32), assign=np.zeros((K, N), np.int32),
                 gate=np.zeros((K, N), np.float32), g=np.zeros((K * N, F), np.float32),
                 u=np.zeros((K * N, F), np.float32), y=np.zeros((K * N, D), np.float32))
        self.lib.qo_moe_fwd(_p(o["out"]), _p(f_in), _p(fnorm), _p(Wr), _p(q1[0]), _p(q1[1]), _p(q3[0]),
                            _p(q3[1]), _p(q2[0]), _p(q2[1]), C.c_int(N), C.c_int(D), C.c_int(F),
                            C.c_int(E), C.c_int(K), _p(o["rt"]), _p(o["rprobs"]), _p(o["assign"]),
                            _p(o["gate"]), _p(o["g"]), _p(o["u"]), _p(o["y"]), C.c_int(group))
        return o

    def moe_bwd(self, dout, fnorm, Wr, q1, q3, q2, F, K, fw, aux=0.03, group=128):
        N, D = fnorm.shape
        E = Wr.shape[1]
        o = dict(dfnorm=np.zeros((N, D), np.float32), dW1=np.zeros((E, D, F), np.float32),
                 dW3=np.zeros((E, D, F), np.float32), dW2=np.zeros((E, F, D), np.float32),
                 dWr=np.zeros((D, E), np.float32), d_gate=np.zeros((K, N), np.float32))
        self.lib.qo_moe_bwd(_p(o["dfnorm"]), _p(o["dW1"]), _p(o["dW3"]), _p(o["dW2"]), _p(o["dWr"]),
                            _p(o["d_gate"]), _p(dout), _p(fnorm), _p(Wr), _p(q1[0]), _p(q1[1]),
                            _p(q3[0]), _p(q3[1]), _p(q2[0]), _p(q2[1]), C.c_int(N), C.c_int(D),
                            C.c_int(F), C.c_int(E), C.c_int(K), _p(fw["rprobs"]), _p(fw["assign"]),
                            _p(fw["gate"]), _p(fw["g"]), _p(fw["u"]), _p(fw["y"]), C.c_float(aux),
                            C.c_int(group))
        return o


class Reference:
    """The unmodified reference's CPU build behind ref_harness.cpp."""

    def __init__(self, path):
        L = self.lib = C.CDLL(path)
        L.ref_hash.restype = C.c_uint32
        L.ref_hash.argtypes = [C.c_uint64]
        L.ref_sround.restype = C.c_int
        L.ref_sround.argtypes = [C.c_float, C.c_uint64, C.c_uint64]
        L.ref_threads.restype = C.c_int
        L.ref_moe_new.restype = C.c_void_p
        L.ref_moe_buf.restype = C.c_void_p
        L.ref_moe_buf.argtypes = [C.c_void_p, C.c_char_p]
        L.ref_moe_off.restype = C.c_longlong
        L.ref_moe_off.argtypes = [C.c_void_p, C.c_char_p]
        L.ref_moe_forward.argtypes = [C.c_void_p]
        L.ref_moe_backward.argtypes = [C.c_void_p]
        self.threads = L.ref_threads()

    def set_threads(self, n):
        """omp_set_num_threads for the compiled reference (a launcher may have forced OMP_NUM_THREADS=1)."""
        self.lib.ref_set_threads(C.c_int(int(n)))
        self.threads = self.lib.ref_threads()
        return self.threads

    def hash(self, x):
        return self.lib.ref_hash(x)

    def sround(self, v, i, t):
        return self.lib.ref_sround(v, i, t)

    def encode(self, P, d, r, s, sp, group=128, dmax=7, packed=1):
        self.lib.ref_encode(_p(P), _p(d), _p(r), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(len(s)),
                            C.c_int(group), C.c_int(dmax), C.c_int(packed))

    def render(self, P, d, s, sp, group=128, packed=1, gi_base=0, ng=None):
        ng = len(s) if ng is None else ng
        self.lib.ref_render(_p(P), _p(d), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(group),
                            C.c_int(packed), C.c_int(gi_base), C.c_int(ng))

    def step(self, P, G, d, r, s, m8, m8s, v8, v8s, sp, *, group=128, dmax=7, lr, b1, b2, wd,
             gscale=1.0, inv_bc1, inv_sqrt_bc2, lrmode=0, t, adam=1, stat=None, packed=1,
             gi_base=0, ng=None):
        ng = len(s) if ng is None else ng
        f = C.c_float
        self.lib.ref_step(_p(P), _p(G), _p(d), _p(r), _p(s), _p(m8), _p(m8s), _p(v8), _p(v8s), _p(sp),
                          C.c_int(len(sp)), C.c_int(group), C.c_int(dmax), f(lr), f(b1), f(b2), f(wd),
                          f(gscale), None, f(inv_bc1), f(inv_sqrt_bc2), C.c_int(lrmode), C.c_uint64(t),
                          C.c_int(adam), _p(stat), C.c_int(packed), C.c_int(gi_base), C.c_int(ng))

    def set_v4(self, on):
        self.lib.ref_set_v4(C.c_int(1 if on else 0))

    def servo(self, d, r, s, sp, group=128, dmax=7, f_hi=0.0, f_lo=0.0, packed=1):
        self.lib.ref_servo(_p(d), _p(r), _p(s), _p(sp), C.c_int(len(sp)), C.c_int(len(s)),
                           C.c_int(group), C.c_int(dmax), C.c_float(f_hi), C.c_float(f_lo),
                           C.c_int(packed))

    def gnorm(self, G, sides=(), clip_side=0):
        gs = np.zeros(2, np.float32)
        ns = len(sides)
        ptrs = (C.c_void_p * max(ns, 1))(*[x.ctypes.data for x in sides])
        lens = (C.c_size_t * max(ns, 1))(*[x.size for x in sides])
        self.lib.ref_gnorm(_p(G), C.c_size_t(G.size), ptrs, lens, C.c_int(ns), C.c_int(clip_side), _p(gs))
        return gs

    # ---- model file (cudalm.cu:431-466, 554-565) ----
    def param_count(self, hdr13):
        self.lib.ref_param_count.restype = C.c_ulonglong
        return int(self.lib.ref_param_count(_p(hdr13)))

    def model_save(self, path, hdr13, P):
        self.lib.ref_model_save(path.encode(), _p(hdr13), _p(P), C.c_ulonglong(P.size))

    def model_load(self, path, cap):
        self.lib.ref_model_load.restype = C.c_ulonglong
        hdr = np.zeros(13, np.int32); P = np.zeros(cap, np.float32)
        n = int(self.lib.ref_model_load(path.encode(), _p(hdr), _p(P), C.c_ulonglong(cap)))
        return hdr, P[:n]

    # ---- n-gram table forward (cpu_kern.h:598-610) ----
    def ngram_key(self, tok, T, R, order, base):
        key = np.zeros(tok.size, np.int32)
        self.lib.ref_ngram_key(_p(tok), _p(key), C.c_int(tok.size), C.c_int(T), C.c_int(R), C.c_int(order), C.c_int(base))
        return key

    def ngram_gather(self, tbl, key, N, De, nk):
        buf = np.zeros((N, De), np.float32)
        self.lib.ref_ngram_gather(_p(tbl), _p(key), _p(buf), C.c_int(N), C.c_int(De), C.c_int(nk))
        return buf

    # ---- sparse engram (engram_setup cudalm.cu:5030-5047; kernels cpu_kern.h:665-688) ----
    def eg_tables(self, Rraw, ord_of_sub):
        """primes below Rraw + 1 (descending) and the splitmix64 multipliers of S sub-tables; loads the kernels' constants"""
        ords = np.ascontiguousarray(ord_of_sub, np.int32); S = ords.size
        prime = np.zeros(S, np.int32); mult = np.zeros(S * 4, np.uint64)
        self.lib.ref_eg_tables(C.c_int(Rraw), C.c_int(S), _p(ords), _p(prime), _p(mult))
        return prime, mult

    def eg_key(self, tok, canon, T, S, Rp):
        key = np.zeros(S * tok.size, np.int32)
        self.lib.ref_eg_key(_p(tok), _p(canon), _p(key), C.c_int(tok.size), C.c_int(T), C.c_int(S), C.c_int(Rp))
        return key

    def eg_gather(self, tbl, key, N, S, De):
        buf = np.zeros((N, S * De), np.float32)
        self.lib.ref_eg_gather(_p(tbl), _p(key), _p(buf), C.c_int(N), C.c_int(S), C.c_int(De))
        return buf

    def eg_scatter_c(self, Gc, key, cidx, db, N, S, De, grp):
        self.lib.ref_eg_scatter_c(_p(Gc), _p(key), _p(cidx), _p(db), C.c_int(N), C.c_int(S), C.c_int(De), C.c_int(grp))

    # ---- exact 4-bit export (quantize_params / dequantize_params qtype 3, cudalm.cu:639-656, 688-695) ----
    def q4n_export(self, P, group=128):
        P = np.ascontiguousarray(P, np.float32)
        cap = (P.size + group - 1) // group * 4 + P.size * 4 + 8
        out = np.zeros(cap, np.uint8)
        self.lib.ref_q4n_export.restype = C.c_ulonglong
        n = int(self.lib.ref_q4n_export(_p(P), C.c_ulonglong(P.size), C.c_int(group), _p(out), C.c_ulonglong(cap)))
        return out[:n].copy()

    def q4n_decode(self, stream, n, group=128):
        stream = np.ascontiguousarray(stream, np.uint8)
        P = np.zeros(n, np.float32)
        ok = self.lib.ref_q4n_decode(_p(stream), C.c_ulonglong(stream.size), _p(P), C.c_ulonglong(n), C.c_int(group))
        return P if ok else None

    # ---- selection bias update (mbias_upd, cudalm.cu:3793-3802); b [ns, E] is updated in place ----
    def mbias_upd(self, b, counts, m, u, lmul, prop):
        ns, E = counts.shape
        self.lib.ref_mbias_upd(_p(b), _p(counts), C.c_int(ns), C.c_int(E), C.c_float(m), C.c_float(u), C.c_float(lmul), C.c_int(prop))

    # ---- the table's context gate (cpu_kern.h:573-589); h, k and dy are updated in place ----
    def nggate_f(self, h, v, k):
        N, D = h.shape
        hn = np.zeros_like(h); g, rh, rk = (np.zeros(N, np.float32) for _ in range(3))
        self.lib.ref_nggate_f(_p(h), _p(v), _p(k), _p(hn), _p(g), _p(rh), _p(rk), C.c_int(N), C.c_int(D))
        return hn, g, rh, rk

    def nggate_b(self, dy, v, hn, kn, g, rh, rk):
        N, D = dy.shape
        dv, dk = np.zeros_like(dy), np.zeros_like(dy)
        self.lib.ref_nggate_b(_p(dy), _p(v), _p(hn), _p(kn), _p(g), _p(rh), _p(rk), _p(dv), _p(dk), C.c_int(N), C.c_int(D))
        return dv, dk

    # ---- 4-bit n-gram table update (cpu_kern.h:615-660) ----
    def ng_touched(self, key, De, group, ngrp):
        slot = np.full(ngrp, -1, np.int32); tgi = np.zeros(key.size, np.int32); cidx = np.zeros(key.size, np.int32)
        cnt = self.lib.ref_ng_touched(_p(key), _p(slot), _p(tgi), _p(cidx), C.c_int(key.size), C.c_int(De), C.c_int(group))
        return tgi[:cnt].copy(), cidx

    def ng_scatter_compact(self, Gc, key, cidx, dbuf, De, group, Nd):
        self.lib.ref_ng_scatter_compact(_p(Gc), _p(key), _p(cidx), _p(dbuf), C.c_int(key.size), C.c_int(De), C.c_int(group), C.c_int(Nd))

    def ng_step(self, P, Gc, d, r, s, m8, m8s, v8, v8s, tgi, group, dmax, lr, b1, b2, wd, sref, inv_bc1, inv_sqrt_bc2, t, nt, gs=None):
        f = C.c_float
        self.lib.ref_ng_step(_p(P), _p(Gc), _p(d), _p(r), _p(s), _p(m8), _p(m8s), _p(v8), _p(v8s), _p(tgi), C.c_int(tgi.size),
                             C.c_int(group), C.c_int(dmax), f(lr), f(b1), f(b2), f(wd), f(sref), f(inv_bc1), f(inv_sqrt_bc2),
                             C.c_ulonglong(t), C.c_ulonglong(nt), _p(gs))

    # ---- block operators (cpu_kern.h:87-152, 489-503) ----
    def embed(self, emb, tok):
        X = np.zeros((tok.size, emb.shape[1]), np.float32)
        self.lib.ref_embed(_p(emb), _p(tok), _p(X), C.c_int(tok.size), C.c_int(emb.shape[1]))
        return X

    def embed_bwd(self, G, dout, tok):
        self.lib.ref_embed_bwd(_p(tok), _p(dout), _p(G), C.c_int(tok.size), C.c_int(G.shape[1]))

    def rmsnorm(self, X, gamma):
        O = np.zeros_like(X); rinv = np.zeros(X.shape[0], np.float32)
        self.lib.ref_rmsnorm(_p(X), _p(gamma), _p(O), _p(rinv), C.c_int(X.shape[0]), C.c_int(X.shape[1]))
        return O, rinv

    def rmsnorm_bwd(self, X, gamma, rinv, dy, dx, dgamma):
        self.lib.ref_rmsnorm_bwd(_p(X), _p(gamma), _p(rinv), _p(dy), _p(dx), _p(dgamma), C.c_int(X.shape[0]), C.c_int(X.shape[1]))

    def rope(self, buf, cosb, sinb, nh, hd, T, back=0):
        self.lib.ref_rope(_p(buf), _p(cosb), _p(sinb), C.c_int(buf.shape[0]), C.c_int(nh), C.c_int(hd), C.c_int(T), C.c_int(back))

    def softmax_ce(self, lg, tgt, n_all):
        loss = np.zeros(lg.shape[0], np.float32); dl = np.zeros_like(lg)
        self.lib.ref_softmax_ce(_p(lg), _p(tgt), _p(loss), _p(dl), C.c_int(lg.shape[0]), C.c_int(lg.shape[1]), C.c_int(n_all))
        return loss, dl

    def attn_fwd(self, Q, K, V, B, T, H, KV, hd, win=0):
        """k_attn_fwd's CPU twin: Q [B*T, H*hd], K, V [B*T, KV*hd] fp32 -> O, lse [B, H, T]."""
        O = np.zeros((B * T, H * hd), np.float32)
        lse = np.zeros((B, H, T), np.float32)
        self.lib.ref_attn_fwd(_p(Q), _p(K), _p(V), _p(O), _p(lse), C.c_int(win), C.c_int(B), C.c_int(T), C.c_int(H),
                              C.c_int(KV), C.c_int(hd))
        return O, lse

    def attn_bwd(self, Q, K, V, O, dA, lse, B, T, H, KV, hd, win=0):
        """k_attn_drow + cpu_attn_bwd: gradients of Q, K, V (into zeroed buffers)."""
        dQ = np.zeros_like(Q); dK = np.zeros_like(K); dV = np.zeros_like(V)
        drow = np.zeros((B, H, T), np.float32)
        self.lib.ref_attn_bwd(_p(Q), _p(K), _p(V), _p(O), _p(dA), _p(lse), _p(drow), _p(dQ), _p(dK), _p(dV),
                              C.c_int(win), C.c_int(B), C.c_int(T), C.c_int(H), C.c_int(KV), C.c_int(hd))
        return dQ, dK, dV, drow

    def sqsum(self, G):
        part = np.zeros(64, np.float32)
        self.lib.ref_sqsum(_p(G), C.c_size_t(G.size), _p(part))
        return part

    def adamw(self, P, G, M, V, lr, b1, b2, wd, bc1, bc2, gs=None):
        f = C.c_float
        self.lib.ref_adamw(_p(P), _p(G), _p(M), _p(V), C.c_size_t(P.size), f(lr), f(b1), f(b2), f(wd),
                           f(bc1), f(bc2), _p(gs))

    def router_topk(self, rt, K, bias=None, bs=0):
        N, E = rt.shape
        rprobs = np.zeros((N, E), np.float32)
        assign = np.zeros((K, N), np.int32)
        gate = np.zeros((K, N), np.float32)
        self.lib.ref_router_topk(_p(rt), _p(rprobs), _p(assign), _p(gate), C.c_int(N), C.c_int(E),
                                 C.c_int(K), _p(bias), C.c_int(bs))
        return rprobs, assign, gate

    def g_ab(self, A, B):
        M, K = A.shape
        N = B.shape[1]
        Cc = np.zeros((M, N), np.float32)
        self.lib.ref_g_ab(_p(A), _p(B), _p(Cc), C.c_int(M), C.c_int(K), C.c_int(N))
        return Cc

    def g_abt(self, A, B):
        M, K = A.shape
        N = B.shape[0]
        Cc = np.zeros((M, N), np.float32)
        self.lib.ref_g_abt(_p(A), _p(B), _p(Cc), C.c_int(M), C.c_int(K), C.c_int(N))
        return Cc

    def g_atb(self, A, B, Cc):
        """Cc[K,N] += A[M,K]^T @ B[M,N]"""
        M, K = A.shape
        N = B.shape[1]
        self.lib.ref_g_atb(_p(A), _p(B), _p(Cc), C.c_int(M), C.c_int(K), C.c_int(N))
        return Cc

    # QLMH state file (qlm_save / qlm_load) on host arrays
    def _state_args(self, st, sp):
        ull = C.c_ulonglong
        return [C.c_int(st["dmax"]), C.c_int(st["group"]), C.c_int(st["adam"]), C.c_int(st["packed"]), _p(sp),
                C.c_int(len(sp)), ull(st["r"].size), ull(st["s"].size), ull(st["Mc"].size), _p(st["d"]), _p(st["r"]),
                _p(st["m8"]), _p(st.get("v8")), _p(st["s"]), _p(st["m8s"]), _p(st.get("v8s")), _p(st["Mc"]), _p(st["Vc"])]

    def qlm_save(self, path, st, sp, iter_, prev_gn):
        """st: dict of numpy arrays d, r, m8, v8, s, m8s, v8s, Mc, Vc (uint16) + ints dmax, group, adam, packed."""
        self.lib.ref_qlm_save.restype = C.c_int
        return self.lib.ref_qlm_save(path.encode(), C.c_int(iter_), C.c_float(prev_gn), *self._state_args(st, sp))

    def qlm_load(self, path, st, sp):
        it = C.c_int(-1); pg = C.c_float(0.0)
        self.lib.ref_qlm_load.restype = C.c_int
        ok = self.lib.ref_qlm_load(path.encode(), C.byref(it), C.byref(pg), *self._state_args(st, sp))
        return ok, it.value, pg.value

    # one MoE layer
    def moe_new(self, N, D, F, E, K, aux=0.03):
        h = self.lib.ref_moe_new(C.c_int(N), C.c_int(D), C.c_int(F), C.c_int(E), C.c_int(K), C.c_float(aux))
        return RefMoeLayer(self, h, N, D, F, E, K)

    # the whole model (gpu_forward / gpu_loss / gpu_backward / gpu_adam with QLM on)
    def model_new(self, V, D, L, H, KV, F, T, E, K, B, aux=0.0):
        self.lib.ref_model_new.restype = C.c_void_p
        h = self.lib.ref_model_new(*[C.c_int(x) for x in (V, D, L, H, KV, F, T, E, K, B)], C.c_float(aux))
        return RefModel(self, h, B * T, D, V)


class RefModel:
    """One model inside the compiled reference (it keeps configuration and Qlm in globals: one at a time)."""

    def __init__(self, ref, h, N, D, V):
        L = ref.lib
        self.ref, self.h, self.N, self.D, self.V = ref, C.c_void_p(h), N, D, V
        L.ref_model_np.restype = C.c_ulonglong
        L.ref_model_np.argtypes = [C.c_void_p]
        L.ref_model_buf.restype = C.c_void_p
        L.ref_model_buf.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.ref_model_loss.restype = C.c_double
        L.ref_model_backward.restype = C.c_double
        L.ref_model_adam.restype = C.c_int
        self.np = int(L.ref_model_np(self.h))
        self.P = self.buf("P", (self.np,))
        self.G = self.buf("G", (self.np,))

    def buf(self, name, shape, dtype=np.float32, l=0):
        ptr = self.ref.lib.ref_model_buf(self.h, name.encode(), l)
        assert ptr, name
        n = int(np.prod(shape))
        ct = {np.float32: C.c_float, np.int32: C.c_int32, np.int8: C.c_int8, np.uint8: C.c_uint8, np.uint16: C.c_uint16}[dtype]
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ct)), shape=(n,)).reshape(shape)

    def qlm_init(self):
        """qlm_gpu_init: quantise the matrices of P in place; returns the state arrays as numpy views."""
        self.ref.lib.ref_model_qlm_init(self.h)
        dims = (C.c_ulonglong * 4)()
        self.ref.lib.ref_model_qlm_dims(dims)
        nq, ngrp, nspan, nfloat = (int(x) for x in dims)
        ptr = self.ref.lib.ref_model_buf(self.h, b"q.span", 0)
        sp = np.frombuffer((C.c_char * (48 * nspan)).from_address(ptr), dtype=SPAN_DTYPE)
        self.q = dict(nq=nq, ngrp=ngrp, nfloat=nfloat, sp=sp,
                      d=self.buf("q.d", (nq // 2,), np.int8), r=self.buf("q.r", (nq,), np.int8),
                      m8=self.buf("q.m8", (nq,), np.int8), v8=self.buf("q.v8", (nq,), np.uint8),
                      s=self.buf("q.s", (ngrp,)), m8s=self.buf("q.m8s", (ngrp,)), v8s=self.buf("q.v8s", (ngrp,)),
                      Mc=self.buf("q.Mc", (nfloat,), np.uint16), Vc=self.buf("q.Vc", (nfloat,), np.uint16))
        return self.q

    def forward(self, tok):
        tok = np.ascontiguousarray(tok, np.int32)
        assert tok.size == self.N
        self.ref.lib.ref_model_forward(self.h, _p(tok))
        return self.buf("fn", (self.N, self.D))

    def loss(self, tgt, perpos=None):
        tgt = np.ascontiguousarray(tgt, np.int32)
        return float(self.ref.lib.ref_model_loss(self.h, _p(tgt), _p(perpos)))

    def backward(self, tgt):
        tgt = np.ascontiguousarray(tgt, np.int32)
        return float(self.ref.lib.ref_model_backward(self.h, _p(tgt)))

    def adam(self, lr, t):
        gn = C.c_float(0.0)
        ok = self.ref.lib.ref_model_adam(self.h, C.c_float(lr), C.c_int(t), C.byref(gn))
        return ok, gn.value


class RefMoeLayer:
    def __init__(self, ref, h, N, D, F, E, K):
        self.ref, self.h = ref, h
        self.N, self.D, self.F, self.E, self.K = N, D, F, E, K
        self.np = ref.lib.ref_moe_off(h, b"np")

    def buf(self, name, shape, dtype=np.float32):
        ptr = self.ref.lib.ref_moe_buf(self.h, name.encode())
        assert ptr, name
        n = int(np.prod(shape))
        ct = {np.float32: C.c_float, np.int32: C.c_int32}[dtype]
        arr = np.ctypeslib.as_array(C.cast(ptr, C.POINTER(ct)), shape=(n,))
        return arr.reshape(shape)

    def off(self, name):
        return int(self.ref.lib.ref_moe_off(self.h, name.encode()))

    def forward(self):
        self.ref.lib.ref_moe_forward(self.h)

    def backward(self):
        self.ref.lib.ref_moe_backward(self.h)


_cache = {}


def bias_update_np(b, assign, E, per_slot, u, prop):
    """numpy float32 restatement of mbias_upd and its two call forms (cudalm.cu:3793-3798, 4385): b [K, E] with one
    count row per top-k pass and target N/E, or b [1, E] with the combined counts and target K*N/E.  Returns the new b."""
    f32 = np.float32
    K, N = assign.shape
    u = f32(u)
    m = f32(N) / f32(E) if per_slot else f32(K) * f32(N) / f32(E)
    rows = [assign[k] for k in range(K)] if per_slot else [assign.ravel()]
    out = b.astype(f32).copy()
    for s, a in enumerate(rows):
        c = np.bincount(a, minlength=E).astype(f32)
        d = (m - c) / m if prop else np.where(c < m, f32(1), np.where(c > m, f32(-1), f32(0))).astype(f32)
        out[s] = out[s] + (u * d.astype(f32)).astype(f32)
    return out


def restatement():
    if "o" not in _cache:
        path = os.path.join(HERE, "_build", "libqlm_oracle.so")
        if not os.path.exists(path):
            build("oracle")
        _cache["o"] = Restatement(path)
    return _cache["o"]


def reference(exact=True):
    key = "exact" if exact else "fast"
    if key not in _cache:
        path = os.path.join(HERE, "_ref", "libcudalm_ref_%s.so" % key)
        _cache[key] = Reference(path) if os.path.exists(path) else None
    return _cache[key]


# ---- the fused per-layer update, composed from an implementation's primitives ----
def fused_layout(L, D, E, F, V, group=128):
    """Offsets of a small model in the reference's parameter order (emb, per layer an1 wq wk wv wo an2
    wr w1 w3 w2, then nf) and its compact gradient map: emb and nf keep private slots, all layers
    share one block (calc_goffsets, cudalm.cu:6008-6040)."""
    names = ["an1", "wq", "wk", "wv", "wo", "an2", "wr", "w1", "w3", "w2"]
    size = dict(an1=D, wq=D * D, wk=D * D, wv=D * D, wo=D * D, an2=D, wr=D * E, w1=E * D * F, w3=E * D * F,
                w2=E * F * D)
    quant = ("wq", "wk", "wv", "wo", "w1", "w3", "w2")
    p = V * D
    rel = {}
    b = 0
    for n in names:
        rel[n] = b; b += size[n]
    per = b
    g_emb, g_nf, g_layer = 0, V * D, V * D + D
    lay = dict(L=L, per=per, layer_g0=g_layer, layer_gn=per, np=V * D + L * per + D, ng_total=g_layer + per,
               q_sizes=[], q_pofs=[], q_gofs=[], layer_float=[], tail_float=[])
    for l in range(L):
        base = p + l * per
        for n in quant:
            lay["q_sizes"].append(size[n]); lay["q_pofs"].append(base + rel[n]); lay["q_gofs"].append(g_layer + rel[n])
        lay["layer_float"].append([(base + rel[n], g_layer + rel[n], size[n]) for n in ("an1", "an2", "wr")])
    lay["tail_float"] = [(0, g_emb, V * D), (p + L * per, g_nf, D)]
    return lay


def fused_steps(impl, lay, P, state, Mc, Vc, cs_of, grads, *, group=128, dmax=7, lr=3e-4, b1=0.9, b2=0.95,
                wd=0.1, wdf=0.0, prev_gn=1.0):
    """qlm_fused_layer for l = L-1 .. 0 and qlm_fused_tail per step (cudalm.cu:6105-6187), from
    impl.sqsum / impl.step / impl.adamw.  grads[t] = (list of per-layer blocks, emb, nf).
    Returns the norms that closed each step."""
    f32 = np.float32
    sp = state["sp"]
    L = lay["L"]
    G = np.zeros(lay["ng_total"], f32)
    part = np.zeros(64 * (L + 2), f32)
    norms = []
    prev = f32(prev_gn)
    for t, (blocks, g_emb, g_nf) in enumerate(grads, start=1):
        gscale = f32(1) / prev if prev > f32(1) else f32(1)
        gs = np.array([gscale, prev], f32)
        bc1 = f32(1) - f32(np.power(f32(b1), f32(t))); bc2 = f32(1) - f32(np.power(f32(b2), f32(t)))
        for l in range(L - 1, -1, -1):
            g0, gn = lay["layer_g0"], lay["layer_gn"]
            G[g0:g0 + gn] = blocks[l]
            part[64 * l:64 * l + 64] = impl.sqsum(G[g0:g0 + gn])
            gi0 = int(sp[7 * l]["gi0"]); ng = int(sp[7 * l:7 * l + 7]["ngrp"].sum())
            impl.step(P, G, state["d"], state["r"], state["s"], state["m8"], state["m8s"], state["v8"],
                      state["v8s"], sp, group=group, dmax=dmax, lr=lr, b1=b1, b2=b2, wd=wd, gscale=float(gscale),
                      inv_bc1=float(f32(1) / bc1), inv_sqrt_bc2=float(f32(1) / np.sqrt(bc2)), t=t, gi_base=gi0, ng=ng)
            for p_off, g_off, n in lay["layer_float"][l]:
                cs = cs_of(p_off)
                impl.adamw(P[p_off:p_off + n], G[g_off:g_off + n], Mc[cs:cs + n], Vc[cs:cs + n], lr, b1, b2, wdf,
                           float(bc1), float(bc2), gs)
        G[0:g_emb.size] = g_emb
        G[g_emb.size:g_emb.size + g_nf.size] = g_nf
        for i, (p_off, g_off, n) in enumerate(lay["tail_float"]):
            cs = cs_of(p_off)
            impl.adamw(P[p_off:p_off + n], G[g_off:g_off + n], Mc[cs:cs + n], Vc[cs:cs + n], lr, b1, b2, wdf,
                       float(bc1), float(bc2), gs)
            part[64 * (L + i):64 * (L + i) + 64] = impl.sqsum(G[g_off:g_off + n])
        ss = 0.0
        for v in part:
            ss += float(v)
        prev = f32(np.sqrt(ss))
        norms.append(prev)
    return np.array(norms, f32)
