"""The reference's training step on its MoE transformer, composed from the library's operators:
gpu_forward (cudalm.cu:5736-5788), gpu_head_bwd (5790-5872), gpu_backward (5874-6002) and gpu_adam
with QLM on (6438-6465, qlm_gpu_update 6082-6103).

Parameters follow the reference's layout (emb; per layer an1 wq wk wv wo an2 wr w1 w3 w2; nf): the seven
matrices of a layer are quantised spans of one Qlm (4-bit digits + residual + int8 moments), everything
else is a float span with bf16 moments.  No fp32 or bf16 copy of a quantised weight exists: the GEMMs
read the digits.  Activations and their gradients are bf16, weight gradients fp32 in the flat G."""
import math

import torch

from . import attn, block, linear, moe, qlm
from ._lib import KN


class Config:
    def __init__(self, L=12, D=768, H=12, KV=12, hd=64, E=32, K=2, F=1536, V=16384, T=1024, B=8):
        self.L, self.D, self.H, self.KV, self.hd, self.E, self.K, self.F, self.V, self.T, self.B = L, D, H, KV, hd, E, K, F, V, T, B
        self.KD = KV * hd
        assert H * hd == D


class Offsets:
    """Off (cudalm.cu:263-275): element offsets of every tensor in the flat parameter vector."""

    def __init__(self, c, experts=None):
        E_ = experts if experts is not None else c.E     # experts stored on this rank (expert parallelism)
        p = 0
        self.emb = p; p += c.V * c.D
        self.layers = []
        for _ in range(c.L):
            o = {}
            for name, n in (("an1", c.D), ("wq", c.D * c.D), ("wk", c.D * c.KD), ("wv", c.D * c.KD), ("wo", c.D * c.D),
                            ("an2", c.D), ("wr", c.D * c.E), ("w1", E_ * c.D * c.F), ("w3", E_ * c.D * c.F),
                            ("w2", E_ * c.F * c.D)):
                o[name] = (p, n); p += n
            self.layers.append(o)
        self.nf = p; p += c.D
        self.total = p


QUANT = ("wq", "wk", "wv", "wo", "w1", "w3", "w2")


class QlmModel:
    """With world > 1 (one process per GPU, torch.distributed): data parallel over the batch with the experts
    sharded (rank r owns experts r*E/W .. of every layer, PeerExpertParallelLayer), everything else replicated;
    the replicated gradients are all-reduced, the clip norm is global, every rank steps its own spans."""

    def __init__(self, cfg, device, seed=1, aux=0.0, rank=0, world=1, group=None, init_blocks=None, P_init=None, fused=False):
        """fused (one GPU): the fused per-layer update of the reference (CUDALM_QLM_FUSED; qlm_fused_layer / qlm_fused_tail,
        cudalm.cu:6105-6187, gradient layout calc_goffsets 6008-6040): all layers share ONE gradient block, which
        backward() consumes as soon as a layer's gradients are complete; the clip multiplier is the previous step's."""
        c = self.c = cfg
        self.dev = device
        self.rank, self.world, self.group = rank, world, group
        self.fused = bool(fused)
        assert not (fused and world > 1)
        assert c.E % world == 0
        self.el = el = c.E // world
        o = self.o = Offsets(c, el)
        # cmd_new's init (cudalm.cu:7349-7365): N(0, 0.02), wo and w2 scaled by 1/sqrt(2L), norm gains 1.
        # Every tensor has its own generator (seed, layer, tensor), and the expert weights one per block of
        # E / init_blocks experts, so that a rank of an expert-parallel run and a single-GPU run
        # (init_blocks = that run's world) hold the same values whatever the local layout is.
        P = torch.empty(o.total, dtype=torch.float32, device=device)

        def fill(dst, key):
            gb = torch.Generator(device=device); gb.manual_seed(seed * 1000003 + key)
            dst.normal_(0.0, 0.02, generator=gb)
        if P_init is not None:
            # a caller-made fp32 parameter vector in the reference's layout (what model_load_full returns): used as is
            assert world == 1 and P_init.numel() == o.total
            P.copy_(torch.as_tensor(P_init).reshape(-1))
        else:
            fill(P[o.emb:o.emb + c.V * c.D], 1)
        nb = init_blocks or world
        eb = c.E // nb                                    # experts per block
        for l, lo in enumerate(o.layers if P_init is None else []):
            for ti, nm in enumerate(("wq", "wk", "wv", "wo", "wr")):
                a, n = lo[nm]
                fill(P[a:a + n], 1000 + l * 16 + ti)
            for wi, nm in enumerate(("w1", "w3", "w2")):
                a, n = lo[nm]
                per = n // el
                blk = None
                for e in range(el):
                    ge = rank * el + e                    # global expert
                    if blk is None or ge % eb == 0:
                        blk = torch.empty(eb * per, dtype=torch.float32, device=device)
                        fill(blk, 100000 + ((l * 3 + wi) * 64 + ge // eb) * 7)
                    P[a + e * per:a + (e + 1) * per] = blk[(ge % eb) * per:(ge % eb + 1) * per]
        sc = 1.0 / math.sqrt(2.0 * c.L)
        for lo in (o.layers if P_init is None else []):
            for nm in ("wo", "w2"):
                a, n = lo[nm]; P[a:a + n] *= sc
            for nm in ("an1", "an2"):
                a, n = lo[nm]; P[a:a + n] = 1.0
        if P_init is None:
            P[o.nf:o.nf + c.D] = 1.0
        mats = [lo[nm] for lo in o.layers for nm in QUANT]
        self.q = qlm.Qlm(mats, o.total, device)
        self.q.init_from(P, render=False)
        # float spans (the gaps between the quantised spans, qlm.cuh:493-502) keep their fp32 values;
        # the quantised part of P is not kept
        self.fp = [P[off:off + n].clone() for off, n, _ in self.q.fs]
        self.emb = self._fview(o.emb, c.V * c.D).view(c.V, c.D)
        self.nf = self._fview(o.nf, c.D)
        self.fl = [{nm: self._fview(*lo[nm]) for nm in ("an1", "an2", "wr")} for lo in o.layers]
        del P
        # gradients: the reference's layout, or (fused) emb | one layer block shared by all layers | nf
        self.layer_n = o.layers[0]["w2"][0] + o.layers[0]["w2"][1] - o.layers[0]["an1"][0]
        self.g_layer0 = o.layers[0]["an1"][0]
        if self.fused:
            self.g_nf = self.g_layer0 + self.layer_n
            self.G = torch.zeros(self.g_nf + c.D, dtype=torch.float32, device=device)
            for i in range(self.q.nspan):                               # qlm_set_gof: gradients are read from the shared block
                self.q.spanH[i]["gof"] = int(self.q.spanH[i]["pof"]) - (i // 7) * self.layer_n
            self.q.spanD = qlm.spans_to_device(self.q.spanH, device)
            self.gnpart = torch.zeros(64 * (c.L + 2), dtype=torch.float32, device=device)
            self.fgs = torch.ones(2, dtype=torch.float32, device=device)       # g_prev_gn = 1 before the first step
            self.fused_lr = 3e-4
        else:
            self.g_nf = o.nf
            self.G = torch.zeros(o.total, dtype=torch.float32, device=device)
        self.cosb, self.sinb = block.rope_tables(c.T, c.hd, device=device)
        N = c.B * c.T
        self.N = N
        self.layers = []
        for l, lo in enumerate(o.layers):
            w = {nm: self._codes(7 * l + i) for i, nm in enumerate(QUANT)}
            if world > 1:
                from . import dist_moe
                gv = lambda nm, shape: self._g(l, nm).view(*shape)
                ext = dict(q=[w["w1"], w["w3"], w["w2"]], wr=self.fl[l]["wr"].view(c.D, c.E),
                           dW=[gv("w1", (el, c.D, c.F)), gv("w3", (el, c.D, c.F)), gv("w2", (el, c.F, c.D))], dWr=gv("wr", (c.D, c.E)))
                m = dist_moe.PeerExpertParallelLayer(dict(N=N, D=c.D, F=c.F, E=c.E, K=c.K), device, rank, world, aux=aux,
                                                     group=group, ext=ext)
            else:
                m = moe.MoeLayerState(N, c.D, c.F, c.E, c.K, w["w1"], w["w3"], w["w2"], self.fl[l]["wr"].view(c.D, c.E), aux=aux)
            self.layers.append(dict(w=w, moe=m))
        self.pending = []
        self.t = 0
        self.gs = torch.ones(2, dtype=torch.float32, device=device)

    def _fview(self, a, n):
        for (off, m, _), t in zip(self.q.fs, self.fp):
            if off <= a and a + n <= off + m:
                return t[a - off:a - off + n]
        raise ValueError("offset %d is not inside a float span" % a)

    def _codes(self, si):
        sp = self.q.spanH[si]
        q0, n, g0, ng = int(sp["qi0"]), int(sp["n"]), int(sp["gi0"]), int(sp["ngrp"])
        return self.q.d[q0 // 2:(q0 + n) // 2], self.q.s[g0:g0 + ng]

    def _g(self, l, nm):
        a, n = self.o.layers[l][nm]
        if self.fused:
            a -= l * self.layer_n                        # every layer's gradients live in the one shared block
        return self.G[a:a + n]

    def _fused_layer(self, l, b1=0.9, b2=0.95, wd=0.1, wdf=0.0):
        """qlm_fused_layer (cudalm.cu:6110-6140): layer l's gradients are complete and still in the shared block."""
        q, t, lr = self.q, self.t + 1, self.fused_lr
        qlm.sqsum(self.G[self.g_layer0:self.g_layer0 + self.layer_n], self.gnpart[64 * l:64 * l + 64])
        s0 = 7 * l
        gi0 = int(q.spanH[s0]["gi0"])
        ng = int(sum(int(q.spanH[i]["ngrp"]) for i in range(s0, s0 + 7)))
        q.step(None, self.G, lr, b1, b2, wd, t, gscale=1.0, gsp=self.fgs, gi_base=gi0, ng=ng)
        bc1, bc2 = qlm.bias_corrections(b1, b2, t)
        for nm in ("an1", "an2", "wr"):
            a, n = self.o.layers[l][nm]
            cs = self._cs(a)
            qlm.adamw(self.fl[l][nm], self._g(l, nm), q.Mc[cs:cs + n], q.Vc[cs:cs + n], lr, b1, b2, wdf, bc1, bc2, self.fgs)

    def _fused_tail(self, b1=0.9, b2=0.95, wd=0.1, wdf=0.0):
        """qlm_fused_tail (cudalm.cu:6148-6187): emb and nf keep private gradient slots; the step's norm is closed on the
        device and clips the NEXT step."""
        c, o, q, t, lr = self.c, self.o, self.q, self.t + 1, self.fused_lr
        bc1, bc2 = qlm.bias_corrections(b1, b2, t)
        tail = ((self.emb.view(-1), o.emb, 0, c.V * c.D), (self.nf, o.nf, self.g_nf, c.D))
        for pt, p_off, g_off, n in tail:
            cs = self._cs(p_off)
            qlm.adamw(pt, self.G[g_off:g_off + n], q.Mc[cs:cs + n], q.Vc[cs:cs + n], lr, b1, b2, wdf, bc1, bc2, self.fgs)
        for i, (pt, p_off, g_off, n) in enumerate(tail):
            qlm.sqsum(self.G[g_off:g_off + n], self.gnpart[64 * (c.L + i):64 * (c.L + i) + 64])
        qlm.gnorm_close(self.gnpart, c.L + 2, self.fgs)

    def _cs(self, p_off):
        for off, n, cs in self.q.fs:
            if off <= p_off < off + n:
                return cs + (p_off - off)
        raise ValueError("offset %d is not in a float span" % p_off)

    # ------------------------------------------------------------------ model file
    def params(self):
        """The fp32 parameter vector in the reference's layout: rendered digits (digit * scale) + the float spans."""
        P = torch.zeros(self.o.total, dtype=torch.float32, device=self.dev)
        self.q.render(P)
        for (off, n, _), t in zip(self.q.fs, self.fp):
            P[off:off + n] = t
        return P

    def save_model(self, path, eot=0):
        """model_save_bundle (cudalm.cu:554-565): a TLM4 file the reference loads (single-GPU layout only)."""
        import ctypes as C
        import numpy as np
        from ._lib import check, lib
        assert self.world == 1, "gather the experts first"
        c = self.c
        hdr = np.array([c.V, c.D, c.L, c.H, c.KV, c.F, c.T, eot, 0, 0, c.E, 0, 0], np.int32)
        P = self.params().cpu().numpy()
        check(lib().qlmb_modelfile_write(path.encode(), hdr.ctypes.data_as(C.c_void_p), P.ctypes.data_as(C.c_void_p), P.size, None, 0))

    def save_model_q4n(self, path, eot=0):
        """`quantize <model> <out> q4n` (cudalm.cu:9753-9793) straight from the device: the rendered 4-bit weights
        export without loss; the float spans (gains) are stored raw where they lie on no 4-bit grid."""
        import numpy as np
        from . import q4n
        assert self.world == 1, "gather the experts first"
        c = self.c
        hdr = np.array([c.V, c.D, c.L, c.H, c.KV, c.F, c.T, eot, 0, 0, c.E, 0, 0], np.int32)
        return q4n.save(path, hdr, self.params())

    # ------------------------------------------------------------------ forward
    def forward(self, tok, B=None, T=None, moes=None, route_logits=None):
        """gpu_forward over B sequences of T tokens (default: the training batch); `moes` replaces the
        layers' MoE states when the row count differs from the training batch (decoder prefill);
        route_logits[l] ([N, E] fp32) replaces layer l's router logits (parity runs on given routing)."""
        c = self.c
        B, T = B or c.B, T or c.T
        bf = torch.bfloat16
        x = block.embed(self.emb, tok, dtype=bf)
        self.saved = []
        for l, ly in enumerate(self.layers):
            w, f = ly["w"], self.fl[l]
            mo = moes[l] if moes is not None else ly["moe"]
            a_norm, r1 = block.rmsnorm_fwd(x, f["an1"])
            qh = linear.linear_fwd(a_norm, *w["wq"], KN, c.D)
            kh = linear.linear_fwd(a_norm, *w["wk"], KN, c.KD)
            vh = linear.linear_fwd(a_norm, *w["wv"], KN, c.KD)
            block.rope(qh, self.cosb, self.sinb, c.H, c.hd, T)
            block.rope(kh, self.cosb, self.sinb, c.KV, c.hd, T)
            att, lse = attn.attn_fwd(qh, kh, vh, B, T, c.H, c.KV)
            f_in = linear.linear_fwd(att, *w["wo"], KN, c.D, R=x)
            if self.world > 1 and moes is None:
                f_norm, r2 = block.rmsnorm_fwd(f_in, f["an2"], out=mo.fn_set[0])       # read by the other ranks
                out = mo.forward(fi=f_in, fn=f_norm, out=torch.empty_like(f_in))
            else:
                f_norm, r2 = block.rmsnorm_fwd(f_in, f["an2"])
                out = mo.forward(f_in, f_norm, rt=route_logits[l] if route_logits is not None else None)
            self.saved.append(dict(a_in=x, a_norm=a_norm, r1=r1, q=qh, k=kh, v=vh, att=att, lse=lse, f_in=f_in, f_norm=f_norm, r2=r2))
            x = out
        self.x_final = x
        self.fn, self.fnr = block.rmsnorm_fwd(x, self.nf)
        return self.fn

    # ------------------------------------------------------------------ head + backward
    def backward(self, tok, tgt):
        c, o, N = self.c, self.o, self.N
        G = self.G
        G_emb = G[o.emb:o.emb + c.V * c.D].view(c.V, c.D)
        G_emb.zero_()
        loss, dfn = block.head_bwd(self.fn, self.emb, tgt, G_emb, chunk_rows=2048, denom=N * self.world)
        g_nf = G[self.g_nf:self.g_nf + c.D]; g_nf.zero_()
        dout = torch.empty(N, c.D, dtype=torch.bfloat16, device=self.dev)
        block.rmsnorm_bwd(dout, self.x_final, self.nf, self.fnr, dfn, dgamma=g_nf, accumulate=False)
        for l in range(c.L - 1, -1, -1):
            ly, s, f, w = self.layers[l], self.saved[l], self.fl[l], self.layers[l]["w"]
            gv = lambda nm, shape: self._g(l, nm).view(*shape)
            if self.world > 1:
                mo = ly["moe"]
                mo.dout_set[0].copy_(dout)                                                   # read by the other ranks
                dfnorm = mo.backward(dout=mo.dout_set[0], fn=s["f_norm"], beta=0.0, dfn=torch.empty_like(dout))
            else:
                dfnorm = ly["moe"].backward(dout, s["f_norm"], gv("w1", (c.E, c.D, c.F)), gv("w3", (c.E, c.D, c.F)),
                                            gv("w2", (c.E, c.F, c.D)), gv("wr", (c.D, c.E)), beta=0.0)
            g = self._g(l, "an2"); g.zero_()
            block.rmsnorm_bwd(dout, s["f_in"], f["an2"], s["r2"], dfnorm, dgamma=g)          # dout now = d f_in
            d_att = linear.linear_dgrad(dout, *w["wo"], KN, c.D)
            linear.linear_wgrad(gv("wo", (c.D, c.D)), dout, s["att"], KN, beta=0.0)
            dq, dk, dv, _ = attn.attn_bwd(s["q"], s["k"], s["v"], s["att"], d_att, s["lse"], c.B, c.T, c.H, c.KV)
            block.rope(dq, self.cosb, self.sinb, c.H, c.hd, c.T, back=True)
            block.rope(dk, self.cosb, self.sinb, c.KV, c.hd, c.T, back=True)
            d_an = linear.linear_dgrad(dq, *w["wq"], KN, c.D)
            linear.linear_dgrad(dk, *w["wk"], KN, c.D, beta=1.0, out=d_an)
            linear.linear_dgrad(dv, *w["wv"], KN, c.D, beta=1.0, out=d_an)
            linear.linear_wgrad(gv("wq", (c.D, c.D)), dq, s["a_norm"], KN, beta=0.0)
            linear.linear_wgrad(gv("wk", (c.D, c.KD)), dk, s["a_norm"], KN, beta=0.0)
            linear.linear_wgrad(gv("wv", (c.D, c.KD)), dv, s["a_norm"], KN, beta=0.0)
            g = self._g(l, "an1"); g.zero_()
            block.rmsnorm_bwd(dout, s["a_in"], f["an1"], s["r1"], d_an, dgamma=g)             # dout now = d a_in
            if self.fused:
                self._fused_layer(l)
            if self.world > 1:      # an1 wq wk wv wo an2 wr are one contiguous range of G: sum over the ranks, overlapped
                a0, a1 = o.layers[l]["an1"][0], o.layers[l]["wr"][0] + o.layers[l]["wr"][1]
                self.pending.append(torch.distributed.all_reduce(G[a0:a1], group=self.group, async_op=True))
        block.embed_bwd(G_emb, dout, tok)
        if self.world > 1:
            self.pending.append(torch.distributed.all_reduce(G_emb, group=self.group, async_op=True))
            self.pending.append(torch.distributed.all_reduce(g_nf, group=self.group, async_op=True))
        if self.fused:
            self._fused_tail()
        self.saved = None
        return loss

    # ------------------------------------------------------------------ optimizer
    def update(self, lr=3e-4, b1=0.9, b2=0.95, wd=0.1, wdf=0.0):
        """gpu_adam with QLM on: global-norm clip (k_sqsum + k_gnorm), integer AdamW over the quantised
        spans, bf16-moment AdamW over the float spans, servo tick every 100 steps."""
        self.t += 1
        q = self.q
        if self.fused:                                   # backward() has updated everything already
            if q.servo_every > 0 and self.t % q.servo_every == 0:
                q.servo()
            return
        for w in self.pending:
            w.wait()
        self.pending = []
        if self.world > 1:
            # replicated ranges are identical on every rank after the all-reduce; the expert ranges are this rank's
            # share of the squared norm: their 64-float partial sums are added over the ranks, then the norm is closed
            c, o = self.c, self.o
            L_ = c.L
            if not hasattr(self, "gpart"):
                self.gpart = torch.zeros(64 * (2 * L_ + 2), dtype=torch.float32, device=self.dev)
            k = 0
            rep = [(o.emb, c.V * c.D), (o.nf, c.D)] + [(lo["an1"][0], lo["wr"][0] + lo["wr"][1] - lo["an1"][0]) for lo in o.layers]
            for a, n in rep:
                qlm.sqsum(self.G[a:a + n], self.gpart[64 * k:64 * k + 64]); k += 1
            for lo in o.layers:
                a, n = lo["w1"][0], lo["w2"][0] + lo["w2"][1] - lo["w1"][0]
                qlm.sqsum(self.G[a:a + n], self.gpart[64 * k:64 * k + 64]); k += 1
            torch.distributed.all_reduce(self.gpart[64 * (L_ + 2):], group=self.group)
            qlm.gnorm_close(self.gpart, 2 * L_ + 2, self.gs)
        else:
            qlm.gnorm(self.G, out=self.gs)
        q.step(None, self.G, lr, b1, b2, wd, self.t, gscale=1.0, gsp=self.gs)
        bc1, bc2 = qlm.bias_corrections(b1, b2, self.t)
        for (off, n, cs), pt in zip(q.fs, self.fp):
            qlm.adamw(pt, self.G[off:off + n], q.Mc[cs:cs + n], q.Vc[cs:cs + n], lr, b1, b2, wdf, bc1, bc2, self.gs)
        if q.servo_every > 0 and self.t % q.servo_every == 0:
            q.servo()

    def train_step(self, tok, tgt, lr=3e-4):
        if self.fused:
            self.fused_lr = lr                           # g_fused_lr: the layers are stepped inside backward()
        self.forward(tok)
        loss = self.backward(tok, tgt)
        self.update(lr)
        return loss


class Decoder:
    """Dec / dec_new / dec_prefill / dec_step (cudalm.cu:7020-7212): B live slots, a bf16 K/V cache of Tm
    positions per layer, one new token per slot and step.  All per-step state (token, position, pick) stays
    on the device, so a step has no host round trip and can be captured in a CUDA graph."""

    def __init__(self, model, B, Tm):
        c, dev = model.c, model.dev
        self.m, self.B, self.Tm = model, B, Tm
        # k_dec_attn keeps one score per cached position in shared memory (at most 4096); the rotation tables must
        # cover every position a slot can reach, so the decoder makes its own when the cache is longer than the
        # model's training context
        assert 1 <= Tm <= 4096, "cache length %d: 1..4096 positions" % Tm
        if Tm <= c.T:
            self.cosb, self.sinb = model.cosb, model.sinb
        else:
            self.cosb, self.sinb = block.rope_tables(Tm, c.hd, device=dev)
        bf = torch.bfloat16
        self.K = [torch.zeros(B, Tm, c.KD, dtype=bf, device=dev) for _ in range(c.L)]
        self.V = [torch.zeros(B, Tm, c.KD, dtype=bf, device=dev) for _ in range(c.L)]
        self.pos2 = torch.zeros(2 * B, dtype=torch.int32, device=dev)     # positions of the q rows and of the k rows
        self.pos = self.pos2[:B]
        self.tok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.otok = torch.zeros(B, dtype=torch.int32, device=dev)
        self.olp = torch.zeros(B, dtype=torch.float32, device=dev)
        self.moes = [self._moe(l, B) for l in range(c.L)]
        self.emb_bf, _ = block.cast_bf16(model.emb, plain=True, transposed=False)
        self.logits = None

    def _moe(self, l, N):
        c, m = self.m.c, self.m
        w = m.layers[l]["w"]
        return moe.MoeLayerState(N, c.D, c.F, c.E, c.K, w["w1"], w["w3"], w["w2"], m.fl[l]["wr"].view(c.D, c.E), aux=0.0)

    def prefill(self, ids):
        """dec_prefill for all slots at once: ids [B, n] (equal prompt lengths) through the full forward, keys and
        values of every layer into the cache, the last row's logits picked greedily as the first new token."""
        c, m = self.m.c, self.m
        B, n = ids.shape
        assert B == self.B and 1 <= n <= self.Tm and n <= c.T, "prompt of %d tokens: cache %d, model context %d" % (n, self.Tm, c.T)
        moes = [self._moe(l, B * n) for l in range(c.L)]
        fn = m.forward(ids.reshape(-1).contiguous(), B=B, T=n, moes=moes)
        for l in range(c.L):
            self.K[l][:, :n] = m.saved[l]["k"].view(B, n, c.KD)
            self.V[l][:, :n] = m.saved[l]["v"].view(B, n, c.KD)
        m.saved = None
        last = fn.view(B, n, c.D)[:, n - 1].contiguous()
        self.logits = block.gemm_nt(last, self.emb_bf, torch.float32, out=self.logits)   # same buffer every time: a captured step keeps writing to it
        self._pick()
        self.pos2.fill_(n)
        self.tok.copy_(self.otok)
        return self.logits

    def set_sampling(self, temp=0.0, top_p=1.0, top_k=0, seed=0):
        """Per-slot sampling parameters (the reference's DSP, cudalm.cu:7020); scalars or one value per slot.
        temp <= 0 keeps the greedy pick.  The step counter the draw is hashed from advances on the device."""
        import numpy as np
        dt = np.dtype(dict(names=["temp", "top_p", "top_k", "seed", "step"], formats=["<f4", "<f4", "<i4", "<u8", "<i4"],
                           offsets=[0, 4, 8, 16, 24], itemsize=32))
        a = np.zeros(self.B, dt)
        a["temp"], a["top_p"], a["top_k"], a["seed"] = temp, top_p, top_k, seed
        self.sp = torch.from_numpy(a.view(np.uint8).reshape(self.B, 32).copy()).to(self.m.dev)
        self.sp_step = self.sp.view(torch.int32)[:, 6]          # the `step` field of every slot

    def advance(self):
        """Move every slot to its next position (step(advance=True) does this itself)."""
        self.pos2 += 1

    def _pick(self):
        from ._lib import check, lib, ptr, stream_ptr
        if getattr(self, "sp", None) is not None:
            check(lib().qlmb_dec_sample(ptr(self.otok), ptr(self.olp), ptr(self.logits), ptr(self.sp), self.B, self.m.c.V,
                                        stream_ptr()))
            self.sp_step += 1
        else:
            check(lib().qlmb_dec_greedy(ptr(self.otok), ptr(self.olp), ptr(self.logits), self.B, self.m.c.V, stream_ptr()))

    def move(self, s, t):
        """dec_move (cudalm.cu:7222-7231): slot s's state into slot t (continuous batching keeps live slots first)."""
        n = int(self.pos[s])
        for l in range(self.m.c.L):
            self.K[l][t, :n] = self.K[l][s, :n]
            self.V[l][t, :n] = self.V[l][s, :n]
        self.pos2[t] = self.pos2[s]; self.pos2[self.B + t] = self.pos2[s]; self.tok[t] = self.tok[s]
        if getattr(self, "sp", None) is not None:
            self.sp[t] = self.sp[s]

    def step(self, advance=True):
        """dec_step: the token in self.tok at position self.pos for every slot; logits -> self.logits, greedy pick ->
        self.otok / self.olp; with advance the pick becomes the next step's token.  Positions live on the device
        only: a slot that has reached the end of its cache (pos == Tm) is not written or read by the kernels, which
        record error 201 in the device error word instead (qlmb_check_device); the caller bounds the step count."""
        from ._lib import check, lib, ptr, stream_ptr
        c, m, B = self.m.c, self.m, self.B
        L_ = lib()
        x = block.embed(m.emb, self.tok, dtype=torch.bfloat16)
        for l, ly in enumerate(m.layers):
            w, f = ly["w"], m.fl[l]
            if c.KD == c.D and 3 * B <= 256:
                # wq, wk, wv are consecutive spans of one shape: one GEMV launch pair for the three; the norm in front of
                # them is applied while the row is staged, the finish rotates q and k and appends k, v to the caches
                qkv = torch.empty(3 * B, c.D, dtype=torch.bfloat16, device=m.dev)
                check(L_.qlmb_dec_qkv(ptr(qkv), ptr(self.K[l]), ptr(self.V[l]), ptr(x), ptr(f["an1"]), ptr(w["wq"][0]),
                                      ptr(w["wq"][1]), ptr(self.cosb), ptr(self.sinb), ptr(self.pos), B, c.D, c.hd, self.Tm, stream_ptr()))
                qh = qkv[:B]
            else:
                a_norm, _ = block.rmsnorm_fwd(x, f["an1"])
                qh = linear.gemv_decode(a_norm, *w["wq"], KN, c.D)
                kh = linear.gemv_decode(a_norm, *w["wk"], KN, c.KD)
                vh = linear.gemv_decode(a_norm, *w["wv"], KN, c.KD)
                check(L_.qlmb_dec_rope(ptr(qh), 1, ptr(self.cosb), ptr(self.sinb), ptr(self.pos), B, c.H, c.hd, self.Tm, stream_ptr()))
                check(L_.qlmb_dec_rope(ptr(kh), 1, ptr(self.cosb), ptr(self.sinb), ptr(self.pos), B, c.KV, c.hd, self.Tm, stream_ptr()))
                check(L_.qlmb_dec_kv(ptr(self.K[l]), ptr(self.V[l]), ptr(kh), ptr(vh), ptr(self.pos), B, self.Tm, c.KD, stream_ptr()))
            att = torch.empty(B, c.D, dtype=torch.bfloat16, device=m.dev)
            check(L_.qlmb_dec_attn(ptr(att), ptr(qh), ptr(self.K[l]), ptr(self.V[l]), ptr(self.pos), 0, B, self.Tm, c.H, c.KV,
                                   c.hd, stream_ptr()))
            if B <= 256 and c.D <= 2048:
                # wo, the residual add and the FFN's input norm: one GEMV launch pair
                f_in = torch.empty(B, c.D, dtype=torch.bfloat16, device=m.dev)
                f_norm = torch.empty(B, c.D, dtype=torch.bfloat16, device=m.dev)
                check(L_.qlmb_gemv_decode_res_norm(ptr(f_in), ptr(f_norm), ptr(att), ptr(w["wo"][0]), ptr(w["wo"][1]), ptr(x),
                                                   ptr(f["an2"]), B, c.D, c.D, stream_ptr()))
            else:
                f_in = linear.gemv_decode(att, *w["wo"], KN, c.D)
                f_in += x
                f_norm, _ = block.rmsnorm_fwd(f_in, f["an2"])
            x = self.moes[l].decode(f_in, f_norm)
        fn, _ = block.rmsnorm_fwd(x, m.nf)
        self.logits = block.gemm_nt(fn, self.emb_bf, torch.float32, out=self.logits)
        self._pick()
        if advance:
            self.pos2 += 1
            self.tok.copy_(self.otok)
        return self.logits
