#!/usr/bin/env python
"""Headline benchmark: one MoE expert-FFN layer with 4-bit weights, forward +
backward (BASELINE config 2: 32 experts, top-2 softmax routing, d_model 768,
d_ff 1536, 8192 tokens of bf16 activations per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

A step is one qlmb_moe_forward + qlmb_moe_backward over one batch of synthetic
tokens.  Inputs are resident in HBM; batches of K steps run back to back (CUDA
events around every batch, max over ranks) until the timed region is at least
--min-seconds long: `value` / `ms_per_step` are the mean over that whole region,
`burst` is its first batch of exactly K steps.  `e2e` runs the same calls from
pinned HOST buffers with the H2D / D2H copies inside the timed region.  FLOPs are
counted on routed rows only (347.9 GFLOP per step and GPU), never on the zero
filler rows.  After the headline the same process measures the training step of
config 4 and the sharded integer AdamW of config 3 for a few iterations and puts
them into the line's `secondary` object (--no-secondary skips them).
--impl reference times the unmodified reference's CPU build (moe_forward +
moe_backward on the same shapes) on this machine's host cores.
"""
import argparse
import ctypes as C
import hashlib
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = dict(N=8192, D=768, F=1536, E=32, K=2)
METRIC = "moe_grouped_dequant_gemm_tflops"
UNIT = "TFLOP/s"


def flops_per_step(c, rows=None):
    rows = c["K"] * c["N"] if rows is None else rows
    fwd = 2.0 * rows * c["D"] * (2 * c["F"]) + 2.0 * rows * c["F"] * c["D"]
    return 3.0 * fwd


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return dict(hbm=d["hbm_gbs"], tf_burst=d["bf16_tflops"], tf_sustained=d["bf16_tflops_sustained"], src="measured")
    return dict(hbm=6650.0, tf_burst=1590.0, tf_sustained=1400.0, src="fallback")


def host_threads():
    """Host threads the CPU baseline may use: the cores this process may run on.  A launcher
    (torch.distributed.run) exports OMP_NUM_THREADS=1 for its workers; the baseline is not one of them."""
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def kernel_sources_digest():
    """sha256 over the sources of the GEMM engine and the MoE control flow: recorded DRAM traffic is only
    quoted while these files are the ones the capture was taken with."""
    h = hashlib.sha256()
    base = os.path.join(ROOT, "cudalm_c_b200", "csrc")
    for f in ("qlmb_gemm.cu", "qlmb_gemm.cuh", "qlmb_gemm_pair.cuh", "qlmb_tc.cuh", "qlmb_moe.cu"):
        with open(os.path.join(base, f), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def recorded_traffic():
    """DRAM bytes per launch from the committed ncu capture of this workload: lines `traffic <kernel> <bytes>` and
    `sources <digest>` of the summary file.  Returns {} when the kernels' sources changed since."""
    path = os.path.join(ROOT, "profiles", "k_gemm_pair_dram_traffic.md")
    out, digest = {}, None
    try:
        for ln in open(path):
            w = ln.split()
            if len(w) == 3 and w[0] == "traffic":
                out[w[1]] = float(w[2])
            elif len(w) == 2 and w[0] == "sources":
                digest = w[1]
    except OSError:
        return {}
    return out if digest == kernel_sources_digest() else {}


class ClockSampler(threading.Thread):
    """SM clock and throttle reasons while the timed region runs (NVML reads, ~1 ms apart;
    nvidia-smi as the fallback when the NVML binding is missing)."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.mhz, self.max_mhz, self.mask, self.stop_flag, self.active = index, [], None, 0, False, False
        self.stamp, self.watts = [], []
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        while not self.stop_flag:
            if not self.active:
                time.sleep(0.0005)
                continue
            try:
                if self.nv is not None:
                    self.mhz.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                    self.stamp.append(time.perf_counter())
                    self.mask |= int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                    self.watts.append(self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0)
                else:
                    out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=clocks.sm,clocks.max.sm",
                                          "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                    a, b = [int(x) for x in out.strip().split(",")]
                    self.mhz.append(a); self.max_mhz = b; self.stamp.append(time.perf_counter())
            except Exception:
                pass
            time.sleep(0.001)

    def median(self, t0=None, t1=None):
        m = sorted(v for v, t in zip(self.mhz, self.stamp) if (t0 is None or t >= t0) and (t1 is None or t <= t1))
        return m[len(m) // 2] if m else None

    def summary(self):
        if not self.mhz:
            return dict(sm_mhz=None, sm_max_mhz=self.max_mhz, reasons=["unsampled"])
        m = sorted(self.mhz)
        return dict(sm_mhz=m[len(m) // 2], sm_max_mhz=self.max_mhz, samples=len(m),
                    power_w_max=round(max(self.watts), 1) if self.watts else None,
                    reasons=[n for bit, n in self.REASONS.items() if self.mask & bit])


def make_layer(dev, seed, weights=None):
    """Synthetic layer of the config-2 shape: expert weights ~ N(0,0.02) quantised
    by the library's own encode kernel (bit-identical to the reference's, see the
    parity tests), router ~ N(0,0.02), activations ~ N(0,1) in bf16.  weights = [w1, w3, w2, wr]
    (fp32, flat) replaces the generated ones."""
    import torch
    from cudalm_c_b200 import moe, qlm
    c = CFG
    gen = torch.Generator(device=dev); gen.manual_seed(seed)
    qs = []
    for wi, (rows, cols) in enumerate(((c["E"] * c["D"], c["F"]), (c["E"] * c["D"], c["F"]), (c["E"] * c["F"], c["D"]))):
        n = rows * cols
        Q = qlm.Qlm([(0, n)], n, dev)
        P = weights[wi].clone() if weights is not None else torch.randn(n, device=dev, generator=gen) * 0.02
        Q.init_from(P, render=False)
        qs.append((Q.d, Q.s))
        del P
    wr = weights[3] if weights is not None else torch.randn(c["D"], c["E"], device=dev, generator=gen) * 0.02
    L = moe.MoeLayerState(c["N"], c["D"], c["F"], c["E"], c["K"], qs[0], qs[1], qs[2], wr, dtype=torch.bfloat16)
    acts = [torch.randn(c["N"], c["D"], device=dev, generator=gen).bfloat16() for _ in range(3)]
    grads = [torch.zeros(c["E"], c["D"], c["F"], device=dev), torch.zeros(c["E"], c["D"], c["F"], device=dev),
             torch.zeros(c["E"], c["F"], c["D"], device=dev), torch.zeros(c["D"], c["E"], device=dev)]
    return L, acts, grads


def run_ours(args):
    import gc
    import torch
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    line = _headline(args, dev, rank, world, local)          # its buffers are gone when it returns
    gc.collect(); torch.cuda.empty_cache()
    if not args.no_secondary:
        # secondary measurements in the same process, so that a scaling run records them at every N
        sec = run_secondary(args, dev, rank, world, peaks())
        if line is not None:
            line["secondary"] = sec
    if rank == 0:
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(steps=2)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def _headline(args, dev, rank, world, local):
    import torch
    import torch.distributed as dist
    import cudalm_c_b200 as q
    lib = q.lib()
    pk = peaks()
    c = CFG
    fn_dev = None
    parity = None
    if world > 1:
        from cudalm_c_b200 import dist_moe
        # the same full synthetic weights on every rank (same seed); every rank keeps its experts' slice
        gen = torch.Generator(device=dev); gen.manual_seed(1234)
        full = [torch.randn(c["E"] * c["D"] * c["F"], device=dev, generator=gen) * 0.02 for _ in range(3)]
        full.append(torch.randn(c["D"], c["E"], device=dev, generator=gen) * 0.02)
        if args.ep == "nccl":
            runner = dist_moe.ExpertParallelLayer(c, dev, rank, world, seed=1234, weights=full)
            parallelism = "ep%d (experts sharded, token all-to-all over NCCL)" % world
        else:
            runner = dist_moe.PeerExpertParallelLayer(c, dev, rank, world, seed=1234, weights=full)
            parallelism = "ep%d (experts sharded, foreign rows read by peer loads inside the row kernels)" % world
        step = runner.step
        fn, fi, dout, out, dfn = runner.fn, runner.fi, runner.dout, runner.out, runner.dfn
        launches_per_step = runner.launches_per_step
    else:
        L, (fn, fi, dout), grads = make_layer(dev, 1234)
        out = torch.empty_like(fi); dfn = torch.empty_like(fi)

        def step():
            L.forward(fi, fn, out=out)
            L.backward(dout, fn, grads[0], grads[1], grads[2], grads[3], beta=0.0, dfnorm=dfn)
        launches_per_step = 18
        parallelism = "single"

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    q.check(lib.qlmb_check_device(None))
    if world > 1:
        # correctness of the sharded run, once, before timing: this rank's layer output and input gradient against
        # the single-call layer that holds all experts on this GPU (rows of an expert GEMM are independent, so the
        # two must agree bit for bit); every rank checks its own tokens, the verdicts are combined
        Lr, _, gr = make_layer(dev, 1234, weights=full)
        o_ref = Lr.forward(fi, fn)
        d_ref = Lr.backward(dout, fn, gr[0], gr[1], gr[2], gr[3], beta=0.0)
        torch.cuda.synchronize()
        okv = torch.tensor([1 if (torch.equal(o_ref, out) and torch.equal(d_ref, dfn)) else 0], device=dev)
        dist.all_reduce(okv, op=dist.ReduceOp.MIN)
        parity = "ok: out and dfnorm of every rank bit-identical to the single-call layer with all experts" if int(okv.item()) == 1 \
            else "MISMATCH against the single-call layer"
        del Lr, gr, o_ref, d_ref, full
        torch.cuda.empty_cache()
        barrier()
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    # batch 0: exactly --steps steps (the burst figure); then as many more batches as fill --min-seconds
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
    barrier()
    sampler.active = True
    w_start = time.perf_counter()
    ev[0].record()
    for _ in range(args.steps):
        step()
    ev[1].record()
    torch.cuda.synchronize()
    w_burst = time.perf_counter()
    ms0 = ev[0].elapsed_time(ev[1]) / args.steps
    nb = int(min(2000, max(0, (args.min_seconds * 1e3 - ms0 * args.steps) / max(ms0 * args.steps, 1e-3) + 1)))
    if world > 1:
        tnb = torch.tensor([nb], device=dev)
        dist.all_reduce(tnb, op=dist.ReduceOp.MAX)
        nb = int(tnb.item())
    ev += [torch.cuda.Event(enable_timing=True) for _ in range(nb)]
    for b in range(nb):
        for _ in range(args.steps):
            step()
        ev[2 + b].record()
    barrier()
    w_end = time.perf_counter()
    sampler.active = False
    batch_ms = [ev[0].elapsed_time(ev[1])] + [ev[1 + b].elapsed_time(ev[2 + b]) for b in range(nb)]
    ms_burst = batch_ms[0] / args.steps
    ms = sum(batch_ms) / (len(batch_ms) * args.steps)
    t = torch.tensor([ms, ms_burst], device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, ms_burst = float(t[0].item()), float(t[1].item())
    value = world * flops_per_step(c) / (ms * 1e-3) / 1e12
    burst = dict(value=round(world * flops_per_step(c) / (ms_burst * 1e-3) / 1e12, 2), ms_per_step=round(ms_burst, 4), steps=args.steps,
                 sm_mhz=sampler.median(w_start, w_burst))
    region = dict(batches=len(batch_ms), steps_per_batch=args.steps, seconds=round(sum(batch_ms) * 1e-3, 3),
                  sm_mhz_steady=sampler.median(w_burst, w_end))

    # per-kernel durations (events inside the library) over a few extra steps
    roof, kern = None, {}
    if True:
        q.check(lib.qlmb_side_stream_enable(0))      # overlapped kernels would be timed with their waiting
        q.check(lib.qlmb_prof_enable(1))
        reps = 5
        for _ in range(reps):
            step()
        names = C.create_string_buffer(64 * 512); msb = (C.c_float * 512)()
        n = lib.qlmb_prof_read(names, msb, 512)
        lib.qlmb_prof_enable(0)
        q.check(lib.qlmb_side_stream_enable(1))
        for i in range(max(n, 0)):
            nm = names.raw[64 * i:64 * i + 64].split(b"\0")[0].decode()
            kern.setdefault(nm, []).append(msb[i])
        kern = {k: sum(v) / len(v) for k, v in kern.items()}
        rows = c["K"] * c["N"]
        fl = {"gemm_gate_up_swiglu": 2.0 * rows * c["D"] * 2 * c["F"], "gemm_down": 2.0 * rows * c["F"] * c["D"],
              "gemm_dact_swiglu_bwd": 2.0 * rows * c["D"] * c["F"], "gemm_dx": 2.0 * rows * 2 * c["F"] * c["D"],
              "gemm_wgrad_w1": 2.0 * rows * c["D"] * c["F"], "gemm_wgrad_w3": 2.0 * rows * c["D"] * c["F"],
              "gemm_wgrad_w2": 2.0 * rows * c["D"] * c["F"]}
        top = max((k for k in kern if k in fl), key=lambda k: kern[k])
        ach = fl[top] / (kern[top] * 1e-3) / 1e12
        # the kernels were timed right after a region of a second or more: the burst peak (a GEMM timed alone at the
        # maximum clock) is the comparator while the SM clock stayed near its maximum, else the sustained one
        clk, clk_max = sampler.median(w_burst, w_end), sampler.max_mhz
        held = clk is None or clk_max is None or clk >= 0.9 * clk_max
        peak = pk["tf_burst"] if held else pk["tf_sustained"]
        # DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the committed ncu capture of this
        # very workload; quoted only for the default configuration on one GPU and unchanged kernel sources
        traffic = recorded_traffic().get(top) if (world == 1 and c == dict(N=8192, D=768, F=1536, E=32, K=2)) else None
        roof = dict(bound="tensor", kernel=top, achieved=round(ach, 1), peak=peak, unit="TFLOP/s", frac=round(ach / peak, 4),
                    traffic=traffic, peak_kind=("burst" if held else "sustained") + " bf16 (SM clock %s of %s MHz over the timed region), of %s" % (clk, clk_max, pk["src"]),
                    kernel_ms={k: round(v, 4) for k, v in sorted(kern.items(), key=lambda kv: -kv[1])},
                    gemm_phase_tflops=round(sum(fl.values()) / (sum(kern[k] for k in fl) * 1e-3) / 1e12, 1))

    # End to end from pinned host buffers through the same calls.  Every step copies its three
    # inputs host->device and its two results device->host; the copies run on two copy streams
    # and device buffers alternate between two sets, so step i's compute overlaps the upload of
    # step i+1 and the download of step i-1 (what a training loop feeding this layer would do).
    e2e = None
    if True:
        hin = [torch.empty(c["N"], c["D"], dtype=torch.bfloat16).pin_memory() for _ in range(3)]
        for h, d in zip(hin, (fn, fi, dout)):
            h.copy_(d)
        hout = [torch.empty(c["N"], c["D"], dtype=torch.bfloat16).pin_memory() for _ in range(2)]
        peer_sets = world > 1 and hasattr(runner, "fn_set")      # inputs other ranks read live in the window
        sets = [dict(fn=fn, fi=fi, dout=dout, out=out, dfn=dfn),
                dict(fn=runner.fn_set[1] if peer_sets else torch.empty_like(fn), fi=torch.empty_like(fi),
                     dout=runner.dout_set[1] if peer_sets else torch.empty_like(dout),
                     out=torch.empty_like(out), dfn=torch.empty_like(dfn))]
        s_in, s_out, s_main = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.current_stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_comp = [torch.cuda.Event() for _ in range(2)]
        ev_out = [torch.cuda.Event() for _ in range(2)]
        for e in ev_comp + ev_out:
            e.record(s_main)

        def step_on(b):
            if world > 1:
                runner.forward(b["fi"], b["fn"], out=b["out"])
                runner.backward(b["dout"], b["fn"], dfn=b["dfn"])
            else:
                L.forward(b["fi"], b["fn"], out=b["out"])
                L.backward(b["dout"], b["fn"], grads[0], grads[1], grads[2], grads[3], beta=0.0, dfnorm=b["dfn"])

        def step_e2e(i):
            k = i & 1
            b = sets[k]
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_comp[k])              # the set's previous step no longer reads its inputs
                b["fn"].copy_(hin[0], non_blocking=True); b["fi"].copy_(hin[1], non_blocking=True)
                b["dout"].copy_(hin[2], non_blocking=True)
                ev_in[k].record(s_in)
            s_main.wait_event(ev_in[k])
            s_main.wait_event(ev_out[k])                 # the set's previous results have left
            step_on(b)
            ev_comp[k].record(s_main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_comp[k])
                hout[0].copy_(b["out"], non_blocking=True); hout[1].copy_(b["dfn"], non_blocking=True)
                ev_out[k].record(s_out)
        for i in range(4):
            step_e2e(i)
        barrier()
        w0 = time.perf_counter()
        for i in range(args.steps):
            step_e2e(i)
        s_main.wait_stream(s_out)
        barrier()
        ms_e = (time.perf_counter() - w0) * 1e3 / args.steps     # host clock around fully drained streams
        if world > 1:
            te = torch.tensor([ms_e], device=dev)
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
            ms_e = float(te.item())
        bi = 3 * c["N"] * c["D"] * 2
        bo = 2 * c["N"] * c["D"] * 2
        e2e = dict(value=round(world * flops_per_step(c) / (ms_e * 1e-3) / 1e12, 2), unit=UNIT, h2d_bytes_per_step=bi,
                   d2h_bytes_per_step=bo, ms_per_step=round(ms_e, 4),
                   how="copies on two copy streams, device buffers double-buffered; wall clock over drained streams")
    q.check(lib.qlmb_check_device(None))

    sampler.stop_flag = True
    clocks = sampler.summary()
    if world > 1:
        barrier()
        if hasattr(runner, "close"):
            runner.close()                               # unmap the peers' windows before the buffers go
    cpu = None
    line = None
    if rank == 0:
        line = dict(metric=METRIC, value=round(value, 2), unit=UNIT, n_gpus=world, steps=args.steps, warmup=max(args.warmup, 3),
                    ms_per_step=round(ms, 4), higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                    data="synthetic", burst=burst, timed_region=region, parity_check=parity, secondary=None,
                    config=dict(workload="MoE expert FFN layer fwd+bwd, 4-bit weights (BASELINE config 2)", tokens_per_gpu=c["N"],
                                d_model=c["D"], d_ff=c["F"], experts=c["E"], top_k=c["K"], parallelism=parallelism,
                                flops_per_step_per_gpu=flops_per_step(c), weight_grad="beta=0 (overwrite; one writer per expert)",
                                l2="per-step working set ~1.3 GB (arena 447 MB + 453 MB of weight gradients) exceeds the 126 MB L2"),
                    roofline=roof, cpu_baseline=cpu, e2e=e2e, gpu_launches=launches_per_step * args.steps * region["batches"],
                    clocks=clocks)
    return line


def run_secondary(args, dev, rank, world, pk):
    """After the headline: a few iterations of (1) the training step of BASELINE config 4 (data parallel over the
    batch, experts sharded: cudalm_c_b200/model.py) and (2) the integer AdamW of config 3 with its groups sharded
    over the ranks and the digits all-gathered (ZeRO-1 form), so that one scaling run carries all three curves.
    Efficiency of the training step: the N = 1 step holds and updates all 1.39 G quantised parameters, a rank of an
    N-rank run only its E/N experts, so tokens/s grows faster than N x the one-GPU figure in the optimizer part;
    forward + backward time per rank is what weak scaling should hold constant (train_fb_ms)."""
    import gc
    import torch
    import torch.distributed as dist
    import cudalm_c_b200 as q
    from cudalm_c_b200 import model, qlm
    out = {}
    # ---- (1) training step
    try:
        cfg = model.Config()
        m = model.QlmModel(cfg, dev, seed=1, aux=0.03, rank=rank, world=world)
        N = cfg.B * cfg.T
        g = torch.Generator(device="cpu"); g.manual_seed(rank)
        tok = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).pin_memory()
        tgt = torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).pin_memory()
        tok_d = torch.zeros(N, dtype=torch.int32, device=dev); tgt_d = torch.zeros(N, dtype=torch.int32, device=dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        losses = []

        def one(timed):
            tok_d.copy_(tok, non_blocking=True); tgt_d.copy_(tgt, non_blocking=True)
            if timed: ev[0].record()
            m.forward(tok_d)
            loss = m.backward(tok_d, tgt_d)
            if timed: ev[1].record()
            m.update()
            if timed: ev[2].record()
            losses.append(float(loss.mean()))
        for _ in range(3):
            one(False)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        fb, up = [], []
        for _ in range(4):
            one(True)
            torch.cuda.synchronize()
            fb.append(ev[0].elapsed_time(ev[1])); up.append(ev[1].elapsed_time(ev[2]))
        q.check(q.lib().qlmb_check_device(None))
        t = torch.tensor([sum(fb) / len(fb), sum(up) / len(up)], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dist.barrier()
            for ly in m.layers:
                ly["moe"].close()
        fb_ms, up_ms = float(t[0]), float(t[1])
        out.update(train_tokens_per_s=round(world * N / ((fb_ms + up_ms) * 1e-3), 1), train_ms_per_step=round(fb_ms + up_ms, 3),
                   train_fb_ms=round(fb_ms, 3), train_update_ms=round(up_ms, 3), train_loss_first=round(losses[0], 4),
                   train_loss_last=round(losses[-1], 4),
                   train_config="config 4: L=12 D=768 E=32 top-2 F=1536 V=16384, 8 x 1024 tokens per GPU, dp%d x ep%d, launches issued from the host" % (world, world))
        del m
    except Exception as e:                               # a secondary line must not take the headline down
        out["train_error"] = repr(e)[:200]
    gc.collect(); torch.cuda.empty_cache()
    # ---- (2) ZeRO-1 integer AdamW, 125 829 120 parameters in total
    try:
        n = 125829120
        Q = qlm.Qlm([(0, n)], n, dev)
        gen = torch.Generator(device=dev); gen.manual_seed(3)
        P = torch.randn(n, device=dev, generator=gen) * 0.02
        Q.init_from(P, render=False)
        del P
        G = torch.randn(n, device=dev, generator=gen) * 1e-3
        ngrp = n // 128
        per = ngrp // world
        gi0 = rank * per

        def one_step(t):
            Q.step(None, G, 3e-4, 0.9, 0.95, 0.1, t, gi_base=gi0, ng=per)
            if world > 1:
                dist.all_gather_into_tensor(Q.d, Q.d[gi0 * 64:(gi0 + per) * 64])
        for t in range(1, 4):
            one_step(t)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for t in range(4, 24):
            one_step(t)
        e1.record(); torch.cuda.synchronize()
        tm = torch.tensor([e0.elapsed_time(e1) / 20], device=dev)
        if world > 1:
            dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm)
        out.update(adamw_zero1_gbs=round(n * 11.15625 / (ms * 1e-3) / 1e9, 1), adamw_zero1_ms=round(ms, 4),
                   adamw_config="config 3: 125 829 120 parameters in total (strong scaling), groups sharded over %d rank(s), packed digits all-gathered in place; 11.15625 B per parameter" % world,
                   adamw_frac_of_hbm=round(n * 11.15625 / (ms * 1e-3) / 1e9 / (pk["hbm"] * world), 4))
        del Q, G
    except Exception as e:
        out["adamw_error"] = repr(e)[:200]
    gc.collect(); torch.cuda.empty_cache()
    return out


def cpu_baseline(steps=2, fast=True, warmup=1):
    """The reference's own moe_forward + moe_backward (CPU build, all host threads)
    on the config-2 shapes; weights are the rendered view of encoded N(0,0.02)."""
    import numpy as np
    from oracle import loader
    ref = loader.reference(exact=not fast)
    kind = "reference"
    if ref is None:
        return dict(value=None, unit=UNIT, cores=0, kind="reference", sample="oracle/_ref not built on this machine")
    ref.set_threads(host_threads())
    c = CFG
    rng = np.random.default_rng(1234)
    L = ref.moe_new(c["N"], c["D"], c["F"], c["E"], c["K"], 0.03)
    P = L.buf("P", (L.np,))
    nW = c["E"] * c["D"] * c["F"]
    o = loader.restatement()
    for nm in ("w1", "w3", "w2"):
        W = (rng.standard_normal(nW, dtype=np.float32) * np.float32(0.02))
        sp, nq, ng = loader.make_spans([nW])
        d = np.zeros(nW // 2, np.int8); r = np.zeros(nW, np.int8); s = np.zeros(ng, np.float32)
        ref.encode(W, d, r, s, sp)
        ref.render(W, d, s, sp)
        P[L.off(nm):L.off(nm) + nW] = W
    P[L.off("wr"):L.off("wr") + c["D"] * c["E"]] = rng.standard_normal(c["D"] * c["E"], dtype=np.float32) * np.float32(0.02)
    for nm in ("f_norm", "f_in", "dout"):
        L.buf(nm, (c["N"], c["D"]))[:] = rng.standard_normal((c["N"], c["D"]), dtype=np.float32)
    for _ in range(max(warmup, 1)):
        L.forward(); L.backward()                   # warm-up (page faults, thread pool)
    t0 = time.perf_counter()
    for _ in range(steps):
        L.forward(); L.backward()
    dt = (time.perf_counter() - t0) / steps
    return dict(value=round(flops_per_step(c) / dt / 1e12, 4), unit=UNIT, cores=ref.threads, kind=kind,
                sample="%d full steps (%d tokens) after %d warm-up, %.2f s/step, reference CPU build (moe_forward + moe_backward), stock flags, %d threads" % (steps, c["N"], max(warmup, 1), dt, ref.threads),
                ms_per_step=round(dt * 1e3, 1))


def run_reference(args):
    """The reference arm: the reference's own CPU implementation of the path (moe_forward + moe_backward of its CPU
    build, compiled from its sources into oracle/_ref) on this machine's host cores, the same shapes, --steps timed
    steps after --warmup.  Under torch.distributed.run rank 0 alone works, with all host threads (the launcher's
    OMP_NUM_THREADS=1 is meant for its GPU workers)."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    steps, warm = max(1, args.steps), max(1, args.warmup)
    cpu = cpu_baseline(steps=steps, warmup=warm)
    if cpu["value"] is None:
        print(json.dumps(dict(impl="reference", unavailable=cpu["sample"])))
        return
    c = CFG
    line = dict(impl="reference", metric=METRIC, value=cpu["value"], unit=UNIT, n_gpus=world, steps=steps, warmup=warm,
                ms_per_step=cpu["ms_per_step"], higher_is_better=True, scaling="weak", vs_baseline=None, dtype="f32",
                data="synthetic",
                config=dict(workload="MoE expert FFN layer fwd+bwd, 4-bit weights (BASELINE config 2)", tokens_per_gpu=c["N"],
                            d_model=c["D"], d_ff=c["F"], experts=c["E"], top_k=c["K"], parallelism="cpu, %d threads" % cpu["cores"],
                            flops_per_step_per_gpu=flops_per_step(c)),
                cpu_baseline=cpu, e2e=dict(value=cpu["value"], unit=UNIT, h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line))


# ---------------------------------------------------------------- CPU baselines of the secondary workloads
# Each one times the reference's own CPU code for that piece (oracle/_ref, stock flags, all host threads) on a bounded
# sample of the workload and says what the sample was.  Reported beside the GPU number, not a target.
def _ref_fast():
    from oracle import loader
    ref = loader.reference(exact=False)
    if ref is not None:
        ref.set_threads(host_threads())
    return ref


def cpu_linear(M, K, N):
    """config 1: the three SGEMMs of the reference (g_abt, g_ab, g_atb; cudalm.cu:3133-3202) on the rendered weights."""
    import numpy as np
    ref = _ref_fast()
    if ref is None:
        return None
    rng = np.random.default_rng(1)
    X = rng.standard_normal((M, K), dtype=np.float32); dY = rng.standard_normal((M, N), dtype=np.float32)
    W = rng.standard_normal((N, K), dtype=np.float32) * np.float32(0.02)
    dW = np.zeros((N, K), np.float32)
    run = lambda: (ref.g_abt(X, W), ref.g_ab(dY, W), ref.g_atb(dY, X, dW))
    run()
    t0 = time.perf_counter()
    for _ in range(3):
        run()
    dt = (time.perf_counter() - t0) / 3
    return dict(value=round(3 * 2.0 * M * K * N / dt / 1e12, 4), unit="TFLOP/s", cores=ref.threads, kind="reference",
                sample="3 full steps (forward, input gradient, weight gradient as fp32 SGEMMs on the rendered weights), %.1f ms/step" % (dt * 1e3))


def cpu_train(cfg):
    """config 4: gpu_forward + gpu_backward + gpu_adam of the reference's CPU build with QLM on, one step.  The full model
    needs about 30 GB of host memory; with less available a two-layer slice of the same widths is timed and scaled."""
    import numpy as np
    ref = _ref_fast()
    if ref is None:
        return None
    try:
        import psutil
        avail = psutil.virtual_memory().available
    except Exception:
        avail = 0
    L = cfg.L if avail > 64e9 else 2
    m = ref.model_new(cfg.V, cfg.D, L, cfg.H, cfg.KV, cfg.F, cfg.T, cfg.E, cfg.K, cfg.B, aux=0.03)
    rng = np.random.default_rng(4)
    blk = (rng.standard_normal(1 << 24, dtype=np.float32) * np.float32(0.02))
    for a in range(0, m.np, blk.size):
        m.P[a:a + blk.size] = blk[:min(blk.size, m.np - a)]
    m.qlm_init()
    N = cfg.B * cfg.T
    tok = rng.integers(0, cfg.V, N).astype(np.int32); tgt = rng.integers(0, cfg.V, N).astype(np.int32)
    t0 = time.perf_counter()
    m.forward(tok); m.backward(tgt); m.adam(3e-4, 1)
    dt = time.perf_counter() - t0
    scale = cfg.L / L
    return dict(value=round(N / (dt * scale), 1), unit="tokens/s", cores=ref.threads, kind="reference",
                sample=("one step of the %d-layer model (8192 tokens), %.1f s" % (L, dt)) +
                       ("" if L == cfg.L else "; scaled by %g to the 12-layer model (embedding and head counted %g times)" % (scale, scale)))


def cpu_decode(cfg, n_prompt):
    """config 5: the reference's CPU build has no K/V decoder; cmd_run there runs the full forward over the whole
    context for every new token (cudalm.cu:7431-7443).  Timed: that forward at a context of n_prompt + 3 tokens, B = 1."""
    import numpy as np
    ref = _ref_fast()
    if ref is None:
        return None
    T = n_prompt + 3
    m = ref.model_new(cfg.V, cfg.D, cfg.L, cfg.H, cfg.KV, cfg.F, T, cfg.E, cfg.K, 1, aux=0.0)
    rng = np.random.default_rng(5)
    blk = (rng.standard_normal(1 << 24, dtype=np.float32) * np.float32(0.02))
    for a in range(0, m.np, blk.size):
        m.P[a:a + blk.size] = blk[:min(blk.size, m.np - a)]
    tok = rng.integers(0, cfg.V, T).astype(np.int32)
    m.forward(tok)
    t0 = time.perf_counter()
    for _ in range(3):
        m.forward(tok)
    dt = (time.perf_counter() - t0) / 3
    return dict(value=round(1.0 / dt, 2), unit="tokens/s", cores=ref.threads, kind="reference",
                sample="3 full-context forwards at %d tokens of context, B = 1 (what the reference's CPU generation costs per new token at the start of the continuation; it grows with the context), %.1f ms each" % (T, dt * 1e3))


def cpu_gemv(K, N, B):
    import numpy as np
    ref = _ref_fast()
    if ref is None:
        return None
    rng = np.random.default_rng(6)
    W = rng.standard_normal((K, N), dtype=np.float32); X = rng.standard_normal((B, K), dtype=np.float32)
    ref.g_ab(X, W)
    t0 = time.perf_counter()
    for _ in range(5):
        ref.g_ab(X, W)
    dt = (time.perf_counter() - t0) / 5
    return dict(value=round(K * N * 4 / dt / 1e9, 2), unit="GB/s", cores=ref.threads, kind="reference",
                sample="5 calls of g_ab on the rendered fp32 weights (4 B per weight streamed), %.2f ms each" % (dt * 1e3))


def cpu_attn(T, H, KV):
    import numpy as np
    ref = _ref_fast()
    if ref is None:
        return None
    rng = np.random.default_rng(7)
    mk = lambda c: rng.standard_normal((T, c * 64), dtype=np.float32)
    Q, K_, V, dA = mk(H), mk(KV), mk(KV), mk(H)
    t0 = time.perf_counter()
    O, lse = ref.attn_fwd(Q, K_, V, 1, T, H, KV, 64)
    t1 = time.perf_counter()
    ref.attn_bwd(Q, K_, V, O, dA, lse, 1, T, H, KV, 64)
    t2 = time.perf_counter()
    pairs = H * (T * (T + 1) // 2)
    return (dict(value=round(2 * 2.0 * pairs * 64 / (t1 - t0) / 1e12, 4), unit="TFLOP/s", cores=ref.threads, kind="reference",
                 sample="one sequence of the eight (B = 1), forward, %.0f ms" % ((t1 - t0) * 1e3)),
            dict(value=round(5 * 2.0 * pairs * 64 / (t2 - t1) / 1e12, 4), unit="TFLOP/s", cores=ref.threads, kind="reference",
                 sample="one sequence of the eight (B = 1), backward, %.0f ms" % ((t2 - t1) * 1e3)))


def cpu_state():
    import numpy as np
    from oracle import loader
    ref = _ref_fast()
    if ref is None:
        return {}
    n = 128 * 131072
    rng = np.random.default_rng(8)
    sp, nq, ng = loader.make_spans([n])
    P = rng.standard_normal(n, dtype=np.float32) * np.float32(0.02)
    d = np.zeros(n // 2, np.int8); r = np.zeros(n, np.int8); sc = np.zeros(ng, np.float32)
    out = {}
    for name, fn, bpp in (("encode", lambda: ref.encode(P, d, r, sc, sp), 4 + 1.53125), ("render", lambda: ref.render(P, d, sc, sp), 0.53125 + 4),
                          ("gnorm", lambda: ref.gnorm(P), 4.0)):
        fn()
        t0 = time.perf_counter()
        for _ in range(3):
            fn()
        dt = (time.perf_counter() - t0) / 3
        out[name] = dict(value=round(n * bpp / dt / 1e9, 2), unit="GB/s", cores=ref.threads, kind="reference",
                         sample="3 passes over a 16.8 M-parameter span, %.1f ms each" % (dt * 1e3))
    return out


def run_adamw(args):
    """Secondary line (BASELINE config 3): integer AdamW over a flat 120 Mi-parameter 4-bit
    span, one step per launch; metric = algorithmic bytes (11.15625 B/param, no fp32 view) / time."""
    import numpy as np
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import qlm
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    n = args.params
    pk = peaks()
    Q = qlm.Qlm([(0, n)], n, dev)
    gen = torch.Generator(device=dev); gen.manual_seed(3)
    P = torch.randn(n, device=dev, generator=gen) * 0.02
    Q.init_from(P, render=False)
    del P
    G = torch.randn(n, device=dev, generator=gen) * 1e-3
    # N > 1: ZeRO-1 form.  Rank r steps the groups [gi0, gi0 + ng) of the same span (the hash uses
    # global element indices, so the result is the one-GPU result bit for bit) and the packed digits
    # are all-gathered in place; the total parameter count stays fixed (strong scaling).
    ngrp = n // 128
    per = (ngrp + world - 1) // world
    assert world == 1 or ngrp % world == 0, "the in-place all-gather needs equal shares"
    gi0, ng = rank * per, min(per, ngrp - rank * per)

    def one_step(t):
        Q.step(None, G, 3e-4, 0.9, 0.95, 0.1, t, gi_base=gi0, ng=ng)
        if world > 1:
            dist.all_gather_into_tensor(Q.d, Q.d[gi0 * 64:(gi0 + ng) * 64])
    t = 0
    for _ in range(max(args.warmup, 3)):
        t += 1; one_step(t)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start(); sampler.active = True
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        t += 1; one_step(t)
    e1.record(); torch.cuda.synchronize()
    sampler.active = False; sampler.stop_flag = True
    ms = e0.elapsed_time(e1) / args.steps
    if world > 1:
        tm = torch.tensor([ms], device=dev)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm.item())
        dist.barrier()
        if rank != 0:
            dist.destroy_process_group()
            return
    bpp = 11.15625
    gbs = n * bpp / (ms * 1e-3) / 1e9
    cpu = None
    if not args.no_cpu and world == 1:
        from oracle import loader
        ref = loader.reference(exact=False)
        if ref is not None:
            m = 128 * 131072
            rng = np.random.default_rng(3)
            sp, nq, ng = loader.make_spans([m])
            W = rng.standard_normal(m, dtype=np.float32) * np.float32(0.02)
            d = np.zeros(m // 2, np.int8); r = np.zeros(m, np.int8); sc = np.zeros(ng, np.float32)
            ref.encode(W, d, r, sc, sp)
            sp["sref"] = np.float32(sc.mean())
            m8 = np.zeros(m, np.int8); v8 = np.zeros(m, np.uint8); m8s = np.zeros(ng, np.float32); v8s = np.zeros(ng, np.float32)
            Gh = rng.standard_normal(m, dtype=np.float32) * np.float32(1e-3)
            kw = dict(lr=3e-4, b1=0.9, b2=0.95, wd=0.1, inv_bc1=10.0, inv_sqrt_bc2=4.47)
            ref.step(W, Gh, d, r, sc, m8, m8s, v8, v8s, sp, t=1, **kw)
            w0 = time.perf_counter()
            for i in range(5):
                ref.step(W, Gh, d, r, sc, m8, m8s, v8, v8s, sp, t=2 + i, **kw)
            dt = (time.perf_counter() - w0) / 5
            cpu = dict(value=round(m * 15.15625 / dt / 1e9, 2), unit="GB/s", cores=ref.threads, kind="reference",
                       sample="5 steps over a 16.8 M-parameter span (the CPU path also writes the fp32 view: 15.16 B/param), %.1f ms/step" % (dt * 1e3))
    print(json.dumps(dict(metric="integer_adamw_gbs", value=round(gbs, 1), unit="GB/s", n_gpus=world, steps=args.steps,
                          warmup=max(args.warmup, 3), ms_per_step=round(ms, 4), higher_is_better=True,
                          scaling="weak" if world == 1 else "strong (ZeRO-1: groups sharded, digits all-gathered)",
                          vs_baseline=None, dtype="int8/f32", data="synthetic",
                          config=dict(workload="integer AdamW step, flat 4-bit span (BASELINE config 3)", params=n,
                                      bytes_per_param=bpp, l2="1.4 GB of state per step exceeds the 126 MB L2"),
                          roofline=dict(bound="hbm", kernel="k_step_fast", achieved=round(gbs, 1), peak=pk["hbm"] * world, unit="GB/s",
                                        frac=round(gbs / (pk["hbm"] * world), 4), traffic=None,
                                        peak_kind="copy bandwidth x %d GPU(s), of %s" % (world, pk["src"])),
                          cpu_baseline=cpu, gparams_per_s=round(n / (ms * 1e-3) / 1e9, 2), gpu_launches=args.steps,
                          clocks=sampler.summary())))
    if world > 1:
        dist.destroy_process_group()


def _time(fn, steps, warmup):
    import torch
    for _ in range(max(warmup, 3)):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_linear(args):
    """Secondary lines (BASELINE config 1): one dequant-fused linear, forward + input gradient +
    weight gradient, X[8192,512], W[2048,512] stored [out,in] with groups along the input axis,
    once with fp32 and once with bf16 activations.  51.54 GFLOP per step."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import linear, qlm
    from cudalm_c_b200._lib import NK
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    M, K, N = 8192, 512, 2048
    gen = torch.Generator(device=dev); gen.manual_seed(1)
    W = torch.randn(N * K, device=dev, generator=gen) * 0.02
    Q = qlm.Qlm([(0, N * K)], N * K, dev); Q.init_from(W, render=False)
    flops = 3 * 2.0 * M * K * N
    for dt, name, io_bytes in ((torch.float32, "f32", 4), (torch.bfloat16, "bf16", 2)):
        X = torch.randn(M, K, device=dev, generator=gen).to(dt); dY = torch.randn(M, N, device=dev, generator=gen).to(dt)
        Y = torch.empty(M, N, device=dev, dtype=dt); dX = torch.empty(M, K, device=dev, dtype=dt)
        dW = torch.zeros(N, K, device=dev)

        def step():
            linear.linear_fwd(X, Q.d, Q.s, NK, N, out=Y)
            linear.linear_dgrad(dY, Q.d, Q.s, NK, K, out=dX)
            linear.linear_wgrad(dW, dY, X, NK, beta=0.0)
        ms = _time(step, args.steps, args.warmup)
        q.check(q.lib().qlmb_check_device(None))
        cpu = None if args.no_cpu else cpu_linear(M, K, N)
        tf = flops / (ms * 1e-3) / 1e12
        # bytes per step: fwd X + Y + codes, dgrad dY + dX + codes, wgrad dY + X + dW(fp32)
        byts = (M * K + M * N) * io_bytes * 3 + 2 * N * K * 0.53125 + N * K * 4
        print(json.dumps(dict(metric="dequant_linear_tflops", value=round(tf, 1), unit="TFLOP/s", n_gpus=1, steps=args.steps,
                              warmup=max(args.warmup, 3), ms_per_step=round(ms, 4), higher_is_better=True, scaling="weak",
                              vs_baseline=None, dtype=name, data="synthetic",
                              config=dict(workload="dequant-fused linear fwd+dgrad+wgrad (BASELINE config 1)", M=M, K=K, N=N,
                                          io=name, l2="working set %.0f MB, re-read every step (fits the 126 MB L2 only with bf16 I/O)" % (byts / 1e6)),
                              roofline=dict(bound="tensor", kernel="k_gemm_pair", achieved=round(tf, 1), peak=pk["tf_burst"], unit="TFLOP/s",
                                            frac=round(tf / pk["tf_burst"], 4), traffic=None, peak_kind="burst bf16, of " + pk["src"],
                                            byte_bound_ms=round(byts / (pk["hbm"] * 1e9) * 1e3, 4),
                                            flop_bound_ms=round(flops / (pk["tf_burst"] * 1e12) * 1e3, 4)),
                              cpu_baseline=cpu, gpu_launches=3 * args.steps)))


def run_attn(args):
    """Secondary lines (the attention of BASELINE config 4: B=8 sequences of T=1024, 12 heads of 64):
    causal flash attention forward and backward.  FLOPs are counted on the causal half only:
    forward 2 GEMMs, backward 5 (the two kernels recompute S and dP, that work is not counted)."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import attn
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    B, T, H, KV = 8, 1024, 12, 12
    gen = torch.Generator(device=dev); gen.manual_seed(1)
    mk = lambda c: torch.randn(B * T, c * 64, device=dev, generator=gen).to(torch.bfloat16)
    Q, K, V, dA = mk(H), mk(KV), mk(KV), mk(H)
    O, lse = attn.attn_fwd(Q, K, V, B, T, H, KV)
    pairs = B * H * (T * (T + 1) // 2)                      # (query, key) pairs inside the causal mask
    f_fwd, f_bwd = 2 * 2.0 * pairs * 64, 5 * 2.0 * pairs * 64
    ms_f = _time(lambda: attn.attn_fwd(Q, K, V, B, T, H, KV), args.steps, args.warmup)
    ms_b = _time(lambda: attn.attn_bwd(Q, K, V, O, dA, lse, B, T, H, KV), args.steps, args.warmup)
    q.check(q.lib().qlmb_check_device(None))
    cpus = (None, None) if args.no_cpu else (cpu_attn(T, H, KV) or (None, None))
    for name, ms, fl, nl in (("forward", ms_f, f_fwd, 1), ("backward", ms_b, f_bwd, 3)):
        tf = fl / (ms * 1e-3) / 1e12
        print(json.dumps(dict(metric="causal_attention_tflops", value=round(tf, 1), unit="TFLOP/s", n_gpus=1, steps=args.steps,
                              warmup=max(args.warmup, 3), ms_per_step=round(ms, 4), higher_is_better=True, scaling="weak",
                              vs_baseline=None, dtype="bf16", data="synthetic",
                              config=dict(workload="causal attention %s (BASELINE config 4 shape)" % name, B=B, T=T, H=H, KV=KV, hd=64,
                                          l2="Q, K, V, O, dA: 5 x 12.6 MB, resident in the 126 MB L2 between steps"),
                              roofline=dict(bound="tensor", kernel="k_attn_fwd" if nl == 1 else "k_attn_bwd_dkv + k_attn_bwd_dq",
                                            achieved=round(tf, 1), peak=pk["tf_burst"], unit="TFLOP/s",
                                            frac=round(tf / pk["tf_burst"], 4), traffic=None, peak_kind="burst bf16, of " + pk["src"]),
                              cpu_baseline=cpus[0 if nl == 1 else 1], gpu_launches=nl * args.steps)))


def run_train(args):
    """Secondary line (BASELINE config 4, one GPU): the reference's training step with QLM on --
    gpu_forward + gpu_head_bwd + gpu_backward + gpu_adam -- composed from the library's operators
    (cudalm_c_b200/model.py): L=12, D=768, 12 heads of 64, 32 experts top-2, F=1536, V=16384, B=8 x T=1024.
    metric = tokens per second; the token ids come from pinned host memory every step and the mean loss
    is read back, so this is also the end-to-end figure."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import model
    import torch.distributed as dist
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    cfg = model.Config()
    fused = bool(args.fused_update) and world == 1
    m = model.QlmModel(cfg, dev, seed=1, aux=0.03, rank=rank, world=world, fused=fused)
    N = cfg.B * cfg.T
    g = torch.Generator(device="cpu"); g.manual_seed(rank)
    toks = [torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).pin_memory() for _ in range(4)]
    tgts = [torch.randint(0, cfg.V, (N,), generator=g, dtype=torch.int32).pin_memory() for _ in range(4)]
    losses = []

    tok_d = torch.zeros(N, dtype=torch.int32, device=dev); tgt_d = torch.zeros(N, dtype=torch.int32, device=dev)
    graph = None
    loss_d = None

    def step(i):
        nonlocal loss_d
        tok_d.copy_(toks[i % 4], non_blocking=True); tgt_d.copy_(tgts[i % 4], non_blocking=True)
        if graph is not None:
            graph.replay()                               # forward + head + backward: about 700 launches, no host work
        else:
            m.forward(tok_d)
            loss_d = m.backward(tok_d, tgt_d)
        m.update()                                       # the step counter and bias corrections change every step: not captured
        losses.append(float(loss_d.mean()))              # device -> host read of the step's result

    for i in range(max(args.warmup, 3)):
        step(i)
    torch.cuda.synchronize()
    if world == 1 and not args.no_graph and not fused:   # the fused update's step counter changes inside backward: not captured
        # one GPU: the host needs about as long to issue the step's launches as the GPU to run them, so forward
        # and backward are replayed from a CUDA graph (same kernels, same order; the library keeps its side streams off
        # while a stream is captured)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            m.forward(tok_d)
            loss_d = m.backward(tok_d, tgt_d)
        step(0)
        torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    q.check(q.lib().qlmb_check_device(None))
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)            # the slowest rank sets the step time
        ms = float(t)
        dist.barrier()
        for ly in m.layers:
            ly["moe"].close()
        if rank != 0:
            dist.destroy_process_group()
            return
    pk = peaks()
    # 6 x active matmul parameters per token + causal attention (forward 2, backward 5 GEMMs of T x T/2 x 64 per head)
    act = cfg.L * (2 * cfg.D * cfg.D + 2 * cfg.D * cfg.KD + cfg.D * cfg.E + cfg.K * 3 * cfg.D * cfg.F) + cfg.V * cfg.D
    flops = 6.0 * act * N + cfg.L * 7 * 2.0 * cfg.B * cfg.H * (cfg.T * (cfg.T + 1) // 2) * cfg.hd
    tps = world * N / (ms * 1e-3)
    print(json.dumps(dict(metric="qlm_train_tokens_per_s", value=round(tps, 1), unit="tokens/s", n_gpus=world, steps=args.steps,
                          warmup=max(args.warmup, 3), ms_per_step=round(ms, 3), higher_is_better=True, scaling="weak",
                          vs_baseline=None, dtype="bf16", data="synthetic",
                          config=dict(workload="QLM training step, MoE transformer (BASELINE config 4)",
                                      parallelism="single" if world == 1 else "dp%d x ep%d (batch split, experts sharded over peer memory, replicated gradients all-reduced)" % (world, world),
                                      L=cfg.L, D=cfg.D, heads=cfg.H,
                                      experts=cfg.E, top_k=cfg.K, F=cfg.F, V=cfg.V, B=cfg.B, T=cfg.T,
                                      params_quantised=int(m.q.nq), params_float=int(m.q.nfloat),
                                      update=("fused per layer inside backward (qlm_fused_layer / _tail): one gradient block shared by all layers, "
                                              "clip multiplier of the previous step" if fused else "separate (gpu_adam): global norm, then one pass over all spans"),
                                      gradient_bytes=int(m.G.numel()) * 4,
                                      l2="weights 0.74 GB of codes, activations and gradients several GB per step: far beyond the 126 MB L2"),
                          roofline=dict(bound="tensor", kernel="whole step", achieved=round(flops / (ms * 1e-3) / 1e12, 1),   # per GPU
                                        peak=pk["tf_sustained"], unit="TFLOP/s",
                                        frac=round(flops / (ms * 1e-3) / 1e12 / pk["tf_sustained"], 4),
                                        traffic=None, peak_kind="sustained bf16, of " + pk["src"], model_flops_per_step=flops),
                          cpu_baseline=None if (args.no_cpu or world > 1) else cpu_train(cfg),
                          e2e=dict(value=round(tps, 1), unit="tokens/s", h2d_bytes_per_step=2 * N * 4, d2h_bytes_per_step=4,
                                   how="token ids and targets copied from pinned host memory inside the timed region, mean loss read back every step"),
                          loss_first=round(losses[0], 4), loss_last=round(losses[-1], 4),
                          gpu_launches=None)))
    if world > 1:
        dist.destroy_process_group()


def run_decode(args):
    """Secondary lines (BASELINE config 5, one GPU): greedy decoding with the K/V-cached decoder
    (cudalm_c_b200/model.py Decoder = dec_prefill + dec_step) on the config-4 model, random weights:
    prompts of 128 uniform ids, 256 new tokens, B = 1, 8, 64 live slots, bf16 cache of 1024 positions.
    A step is one CUDA-graph replay (no host input: token, position and pick stay on the device).
    metric = generated tokens per second over the 256 steps; prefill is reported beside it.  The roofline is
    HBM: bytes a step must read = 4-bit attention weights + the distinct experts the step's routing hit
    (counted on 8 extra steps after the timed run) + router + bf16 embedding for the head + the K/V rows read."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import model
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    cfg = model.Config()
    m = model.QlmModel(cfg, dev, seed=1, aux=0.0)
    n_prompt, n_new, Tm = 128, args.new_tokens, 1024
    assert n_prompt + n_new + 12 <= Tm, "prompt + new tokens + warm-up and probe steps must fit the cache of %d positions" % Tm
    cpu_dec = None if args.no_cpu else cpu_decode(cfg, n_prompt)
    for B in [int(x) for x in args.decode_b.split(",")]:
        g = torch.Generator(device="cpu"); g.manual_seed(B)
        ids_h = torch.randint(0, cfg.V, (B, n_prompt), generator=g, dtype=torch.int32).pin_memory()
        dec = model.Decoder(m, B, Tm)
        t0 = time.perf_counter()
        ids = ids_h.to(dev, non_blocking=True)
        dec.prefill(ids)
        torch.cuda.synchronize()
        t_prefill = time.perf_counter() - t0
        for _ in range(3):                                  # warm-up steps (also sizes every scratch buffer)
            dec.step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            dec.step()
        gen = torch.zeros(n_new, B, dtype=torch.int32, device=dev)
        dec.prefill(ids)                                    # back to the end of the prompt
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        e0.record()
        for j in range(n_new):
            gen[j].copy_(dec.tok)
            graph.replay()
        e1.record()
        out_h = gen.cpu()                                   # device -> host read of the generated ids
        t_e2e = time.perf_counter() - t0
        ms = e0.elapsed_time(e1) / n_new
        q.check(q.lib().qlmb_check_device(None))
        # distinct experts per layer on a few more steps -> bytes a step has to read
        hit = 0.0
        for _ in range(8):
            dec.step()
            for mo in dec.moes:
                hit += float(torch.unique(mo.member("assign", (cfg.K, B), torch.int32)).numel())
        hit /= 8.0                                           # summed over the 12 layers
        w = 0.53125
        pos_mid = n_prompt + n_new / 2
        byts = cfg.L * (2 * cfg.D * cfg.D + 2 * cfg.D * cfg.KD) * w + hit * 3 * cfg.D * cfg.F * w + cfg.L * cfg.D * cfg.E * 4 \
            + cfg.V * cfg.D * 2 + cfg.L * 2 * B * pos_mid * cfg.KD * 2
        gbs = byts / (ms * 1e-3) / 1e9
        tps = B / (ms * 1e-3)
        print(json.dumps(dict(metric="decode_tokens_per_s", value=round(tps, 1), unit="tokens/s", n_gpus=1, steps=n_new, warmup=3,
                              ms_per_step=round(ms, 4), higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                              data="synthetic",
                              config=dict(workload="greedy decode, K/V cache (BASELINE config 5)", B=B, prompt=n_prompt, new_tokens=n_new,
                                          cache_positions=Tm, model="config 4 (L=12, D=768, 32 experts top-2)",
                                          experts_hit_per_step=round(hit, 1), l2="weights read per step %.0f MB" % (byts / 1e6)),
                              roofline=dict(bound="hbm", kernel="whole step (one graph replay)", achieved=round(gbs, 1), peak=pk["hbm"],
                                            unit="GB/s", frac=round(gbs / pk["hbm"], 4), traffic=None, peak_kind="copy, of " + pk["src"],
                                            bytes_per_step=byts),
                              cpu_baseline=cpu_dec if B == 1 else None,
                              e2e=dict(value=round(B * n_new / t_e2e, 1), unit="tokens/s", h2d_bytes_per_step=0,
                                       d2h_bytes_per_step=B * 4, prefill_ms=round(t_prefill * 1e3, 2),
                                       how="host clock over the 256 replays and the read-back of the generated ids; the prompt upload and prefill are timed separately (prefill_ms, includes the first-use set-up of this batch size)"),
                              gpu_launches=None, sample=[int(x) for x in out_h[:4, 0]])))
        del dec, graph


def run_gemv(args):
    """Secondary lines (decode path, BASELINE config 5's building block): Y[B,N] = X[B,K] deq(W) for
    B live slots; metric = weight bytes streamed (0.53125 B per weight) / time."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import linear, qlm
    from cudalm_c_b200._lib import KN, NK
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    gen = torch.Generator(device=dev); gen.manual_seed(5)
    cases = ((768, 1536, KN, "KN 768x1536 (expert up-projection)"), (4096, 16384, KN, "KN 4096x16384"), (4096, 16384, NK, "NK 16384x4096"))
    slots = (1, 2, 4, 8, 64)
    if args.gemv_case:                                   # "KN 4096x16384:1" = one matrix, one slot count (profiler captures)
        nm, b = args.gemv_case.split(":")
        cases = tuple(c_ for c_ in cases if c_[3].startswith(nm))
        slots = (int(b),)
    for K, N, lay, tag in cases:
        # several copies of the weights, used in turn, so that a call never finds its weights in the 126 MB L2
        ncopy = max(2, int(160e6 / (K * N * 0.53125)) + 1)
        ncopy = min(ncopy, 40)
        W = torch.randn(K * N, device=dev, generator=gen) * 0.02
        Qs = []
        for _ in range(ncopy):
            Q = qlm.Qlm([(0, K * N)], K * N, dev); Q.init_from(W.clone(), render=False); Qs.append(Q)
        cpu = None if args.no_cpu else cpu_gemv(K, N, 1)
        # what a kernel that only loads the codes achieves at this size (launch, first-load latency, tail): the practical
        # ceiling of a single GEMV call, measured the same way (copies used in turn, replayed graph)
        read_us = None
        if lay == KN and (N // 2) % 256 == 0:
            best = None
            for ksl in (4, 8, 16, 32):
                if K % ksl:
                    continue
                turn_r = [0]

                def read_call():
                    Q = Qs[turn_r[0] % ncopy]; turn_r[0] += 1
                    q.check(q.lib().qlmb_selftest_stream_read(Q.d.data_ptr(), N // 2, K, ksl, torch.cuda.current_stream().cuda_stream))
                read_call()
                side_r = torch.cuda.Stream()
                side_r.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side_r):
                    gr = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gr, stream=side_r):
                        for _ in range(2 * ncopy):
                            read_call()
                torch.cuda.current_stream().wait_stream(side_r)
                t_r = _time(gr.replay, max(args.steps // 4, 3), 3) / (2 * ncopy) * 1e3
                best = t_r if best is None or t_r < best else best
            read_us = round(best, 2)
        for B in slots:
            X = torch.randn(B, K, device=dev, generator=gen).bfloat16()
            Y = torch.empty(B, N, device=dev, dtype=torch.bfloat16)
            turn = [0]

            def call():
                Q = Qs[turn[0] % ncopy]; turn[0] += 1
                linear.gemv_decode(X, Q.d, Q.s, lay, N, out=Y)
            ms_call = _time(call, args.steps, args.warmup)      # one host call per GEMV (host overhead included)
            # device time: 2 rounds over the copies captured in a CUDA graph, replayed
            ncall = 2 * ncopy
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(ncall):
                        call()
            torch.cuda.current_stream().wait_stream(side)
            ms = _time(graph.replay, max(args.steps // 4, 3), 3) / ncall
            gbs = K * N * 0.53125 / (ms * 1e-3) / 1e9
            print(json.dumps(dict(metric="decode_gemv_weight_gbs", value=round(gbs, 1), unit="GB/s", n_gpus=1, steps=args.steps,
                                  warmup=max(args.warmup, 3), ms_per_step=round(ms, 5), higher_is_better=True, scaling="weak",
                                  vs_baseline=None, dtype="bf16", data="synthetic",
                                  config=dict(workload="decode GEMV, 4-bit weights " + tag, slots=B,
                                              timing="%d calls in a replayed CUDA graph; one host call per GEMV takes %.1f us" % (ncall, ms_call * 1e3),
                                              l2="weights %.1f MB per call, %d copies used in turn (%.0f MB, more than the 126 MB L2)" % (K * N * 0.53125 / 1e6, ncopy, ncopy * K * N * 0.53125 / 1e6)),
                                  roofline=dict(bound="hbm", kernel="k_gemv", achieved=round(gbs, 1), peak=pk["hbm"], unit="GB/s",
                                                frac=round(gbs / pk["hbm"], 4), traffic=None, peak_kind="copy bandwidth, of " + pk["src"],
                                                read_only=None if read_us is None else dict(
                                                    us=read_us, gbs=round(K * N * 0.5 / (read_us * 1e-6) / 1e9, 1),
                                                    what="a kernel that only loads the code bytes once, same grid shape, best of 4-32 row slices")),
                                  cpu_baseline=cpu if B == 1 else None, gpu_launches=2 * args.steps)))
        del Qs, W
    q.check(q.lib().qlmb_check_device(None))


def run_state(args):
    """Secondary lines: the other passes over the optimizer state at config 3's size --
    encode (4 B read + 1.53 B written per parameter), render (0.53 read + 4 written) and the
    global-norm reduction (4 B read)."""
    import torch
    import cudalm_c_b200 as q
    from cudalm_c_b200 import qlm
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    n = args.params
    Q = qlm.Qlm([(0, n)], n, dev)
    gen = torch.Generator(device=dev); gen.manual_seed(3)
    P = torch.randn(n, device=dev, generator=gen) * 0.02
    G = torch.randn(n, device=dev, generator=gen) * 1e-3
    out = torch.zeros(2, device=dev)
    Q.init_from(P, render=False)
    cpus = {} if args.no_cpu else cpu_state()
    for name, fn, bpp in (("encode", lambda: qlm.qlm_encode(P, Q.d, Q.r, Q.s, Q.spanD, Q.nspan, Q.group, Q.dmax, Q.packed), 4 + 1.53125),
                          ("render", lambda: Q.render(P), 0.53125 + 4),
                          ("gnorm", lambda: qlm.gnorm(G, out=out), 4.0)):
        ms = _time(fn, args.steps, args.warmup)
        gbs = n * bpp / (ms * 1e-3) / 1e9
        print(json.dumps(dict(metric="qlm_%s_gbs" % name, value=round(gbs, 1), unit="GB/s", n_gpus=1, steps=args.steps,
                              warmup=max(args.warmup, 3), ms_per_step=round(ms, 4), higher_is_better=True, scaling="weak",
                              vs_baseline=None, dtype="f32/int8", data="synthetic",
                              config=dict(workload="QLM %s pass over a flat span (BASELINE config 3 size)" % name, params=n,
                                          bytes_per_param=bpp, l2="inputs exceed the 126 MB L2"),
                              roofline=dict(bound="hbm", kernel="k_" + name, achieved=round(gbs, 1), peak=pk["hbm"], unit="GB/s",
                                            frac=round(gbs / pk["hbm"], 4), traffic=None, peak_kind="copy bandwidth, of " + pk["src"]),
                              cpu_baseline=cpus.get(name), gpu_launches=args.steps)))
    q.check(q.lib().qlmb_check_device(None))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--min-seconds", type=float, default=1.2, help="length of the headline's timed region (batches of --steps steps are repeated until it is reached)")
    ap.add_argument("--no-secondary", action="store_true", help="skip the training-step and ZeRO-1 AdamW measurements after the headline")
    ap.add_argument("--workload", default="moe", choices=["moe", "adamw", "linear", "gemv", "state", "attn", "train", "decode"],
                    help="moe = the headline line; the others print secondary lines: adamw (config 3), linear (config 1), "
                         "gemv (decode building block), state (encode / render / gnorm passes)")
    ap.add_argument("--params", type=int, default=125829120, help="span size of --workload adamw")
    ap.add_argument("--ep", default="peer", choices=["peer", "nccl"],
                    help="N>1: peer = foreign rows read by peer loads inside the row kernels; nccl = all-to-all exchanges")
    ap.add_argument("--fused-update", action="store_true", help="--workload train, one GPU: the reference's fused per-layer update (CUDALM_QLM_FUSED) instead of the separate optimizer pass")
    ap.add_argument("--no-graph", action="store_true", help="--workload train: issue every launch from the host instead of replaying forward + backward from a CUDA graph")
    ap.add_argument("--decode-b", default="1,8,64", help="live slots of --workload decode (comma list; BASELINE config 5 has 1,8,64)")
    ap.add_argument("--new-tokens", type=int, default=256, help="generated tokens of --workload decode (256 in BASELINE config 5; fewer for profiler captures)")
    ap.add_argument("--gemv-case", default="", help="--workload gemv: one case only, e.g. 'KN 4096x16384:1' (matrix tag prefix : slots)")
    ap.add_argument("--tokens", type=int, default=0, help="tokens per GPU (default: the 8192 of config 2); smaller values are for profiler captures")
    args = ap.parse_args()
    if args.tokens > 0:
        CFG["N"] = args.tokens
    if args.workload == "adamw":
        run_adamw(args)
    elif args.workload == "linear":
        run_linear(args)
    elif args.workload == "gemv":
        run_gemv(args)
    elif args.workload == "state":
        run_state(args)
    elif args.workload == "attn":
        run_attn(args)
    elif args.workload == "train":
        run_train(args)
    elif args.workload == "decode":
        run_decode(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
