#!/usr/bin/env python
"""Benchmark of the fused layer kernels.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference] [--no-ops]

Workload (one "step"): the DDPM block kernel set of the baseline's config list
on fp32 NHWC [256, 32, 32, 256] per GPU:
    GroupNorm(32 groups)+affine+SiLU fused forward and backward,
    LayerNorm over C=256 on the same buffer viewed as [262144, 256], forward and backward,
    sinusoidal time embedding dim 512 for 256 integer timesteps.
Metric: algorithmic HBM bytes moved per second (fwd 2 tensors + bwd 3 tensors per
norm = 10 N floats per step).  With N GPUs the batch is sharded (each rank owns 256
samples, weak scaling) and the only exchange is one all-reduce of the 4*C
parameter-gradient floats.

Lines printed (one JSON object, rank 0 only):
  default        this library through its C ABI, plus `roofline`, `cpu_baseline`,
                 `e2e` (host buffers, copies inside the timed region) and `ops`
                 (every other kernel of the path at the baseline's other sizes).
  --impl reference   the reference's own kernels.cu (built for sm_100a with its own
                 flags into oracle/_ref/) on the same step; the reference has no CPU
                 path, so `cpu_baseline` on that line is the plain-C port timed on
                 the host cores.
"""
from __future__ import annotations

import argparse
import ctypes
import importlib
import json
import math
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402
import torch  # noqa: E402

B, H, W, C, G = 256, 32, 32, 256, 32
HW = H * W
NEL = B * HW * C
EMB = 512
STEP_BYTES = 10 * NEL * 4 + B * EMB * 4  # algorithmic bytes of one step
F = ctypes.c_float
P = lambda t: ctypes.c_void_p(t.data_ptr())


def set_batch(b):
    """Shrinks the per-GPU batch (profiler captures on a small case); the default 256 is the benchmark."""
    global B, NEL, STEP_BYTES, KERNEL_BYTES
    B = b
    NEL = B * HW * C
    STEP_BYTES = 10 * NEL * 4 + B * EMB * 4
    KERNEL_BYTES = {"gn_silu_fwd": 2 * NEL * 4, "gn_silu_bwd": 3 * NEL * 4, "ln_fwd": 2 * NEL * 4,
                    "ln_bwd": 3 * NEL * 4, "sinusoidal": B * EMB * 4}


def measured_peak():
    f = ROOT / "MEASURED_PEAKS.json"
    if f.exists():
        return float(json.loads(f.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier pool measurement)"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            time.sleep(0.15)
            self.proc.terminate()
            self.th.join(timeout=2)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if len(r) >= 6 and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) >= 6 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) >= 6 and r[2 + i] == "Active" for r in self.rows)]
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


# ------------------------------------------------------------------------------------ libraries
def load_capi():
    """The binding table only (signatures of the launcher set); loads no shared object."""
    return importlib.import_module("cuda-c-diffusion_b200.capi")


BIN = ROOT / "cuda-c-diffusion_b200" / "build" / "bin"  # host programs (cuda-c-diffusion_b200/csrc/host/Makefile)


def load_reference(capi):
    path = ROOT / "oracle" / "_ref" / "libref_kernels.so"
    if not path.exists():
        return None
    sigs = {k: capi.SIGNATURES[k] for k in capi.REFERENCE_LAUNCHERS}
    return capi.bind(ctypes.CDLL(str(path), mode=ctypes.RTLD_LOCAL), sigs)


# ------------------------------------------------------------------------------------ the step
class Step:
    """Device-resident buffers and the kernel sequence of one step."""

    KERNELS = ["gn_silu_fwd", "gn_silu_bwd", "ln_fwd", "ln_bwd", "sinusoidal"]

    def __init__(self, lib, fused, dev, seed):
        self.lib, self.fused, self.dev = lib, fused, dev
        g = torch.Generator(device=dev).manual_seed(seed)
        rn = lambda *s: torch.randn(*s, device=dev, generator=g)
        self.x, self.dy = rn(B, HW, C), rn(B, HW, C)
        self.y, self.dx = torch.empty_like(self.x), torch.empty_like(self.x)
        self.gamma, self.beta = 1 + 0.1 * rn(C), 0.1 * rn(C)
        self.mu, self.rstd = torch.empty(B * G, device=dev), torch.empty(B * G, device=dev)
        self.lmu, self.lrstd = torch.empty(B * HW, device=dev), torch.empty(B * HW, device=dev)
        # parameter gradients of the step, double-buffered: the all-reduce of step i runs while step i+1 computes
        self.dgams = [torch.empty(4 * C, device=dev), torch.empty(4 * C, device=dev)]
        self.dgam, self.dbet = self.dgams[0], None
        self.pending = [None, None]
        self.k = 0
        self.t = torch.randint(0, 1000, (B,), device=dev, generator=g).float()
        self.emb = torch.empty(B, EMB, device=dev)
        if not fused:
            self.h, self.gh = torch.empty_like(self.x), torch.empty_like(self.x)
        self.lmp = F(np.float32(math.log(1e4)))

    def stream(self):
        return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def run(self, marks=None):
        """One step.  `marks`, if given, receives a CUDA event before every kernel and one at the end."""
        L, s = self.lib, self.stream()
        self.k ^= 1
        self.dgam = self.dgams[self.k]
        if self.pending[self.k] is not None:  # the exchange that last used this buffer (two steps ago)
            self.pending[self.k].wait()
            self.pending[self.k] = None
        dg, db, lg, lb = (ctypes.c_void_p(self.dgam.data_ptr() + 4 * C * i) for i in range(4))

        def mark():
            if marks is not None:
                ev = torch.cuda.Event(enable_timing=True)
                ev.record()
                marks.append(ev)

        mark()
        if self.fused:
            L.launch_groupnorm_act_forward(P(self.y), P(self.mu), P(self.rstd), P(self.x), P(self.gamma), P(self.beta),
                                           B, HW, C, G, F(1e-5), 3, s)
            mark()
            L.launch_groupnorm_act_backward(P(self.dx), dg, db, P(self.dy), P(self.x), P(self.gamma), P(self.beta),
                                            P(self.mu), P(self.rstd), B, HW, C, G, 3, s)
        else:  # the reference's composition (conv_residual.c:28-29, :51-52)
            L.launch_groupnorm_forward(P(self.h), P(self.mu), P(self.rstd), P(self.x), P(self.gamma), P(self.beta),
                                       B, HW, C, G, F(1e-5), s)
            L.launch_activation_forward(P(self.y), P(self.h), NEL, 3, s)
            mark()
            L.launch_activation_backward(P(self.gh), P(self.dy), P(self.h), NEL, 3, s)
            L.launch_groupnorm_backward(P(self.dx), dg, db, P(self.gh), P(self.x), P(self.gamma), P(self.mu),
                                        P(self.rstd), B, HW, C, G, s)
        mark()
        L.launch_layernorm_forward(P(self.y), P(self.lmu), P(self.lrstd), P(self.x), P(self.gamma), P(self.beta),
                                   B * HW, C, F(1e-5), s)
        mark()
        L.launch_layernorm_backward(P(self.dx), lg, lb, P(self.dy), P(self.x), P(self.gamma), P(self.lmu),
                                    P(self.lrstd), B * HW, C, s)
        mark()
        L.launch_sinusoidal(P(self.emb), P(self.t), B, EMB, self.lmp, s)
        mark()

    def exchange(self):
        """Batch-sharded parameter gradients: one all-reduce of 4*C floats, issued asynchronously so that it
        overlaps the next step's kernels (nothing in a step reads the reduced gradients of the previous one)."""
        if torch.distributed.is_initialized() and torch.distributed.get_world_size() > 1:
            self.pending[self.k] = torch.distributed.all_reduce(self.dgam, async_op=True)

    def finish(self):
        """Makes the current stream wait for every exchange still in flight."""
        for i, w in enumerate(self.pending):
            if w is not None:
                w.wait()
                self.pending[i] = None


def timed_block(step, steps, world, per_kernel_events=False):
    """EXACTLY `steps` steps between two events, bracketed by barrier + synchronize on both sides; returns the
    block's milliseconds (max over ranks) and, with `per_kernel_events`, the per-kernel milliseconds per step of
    this rank (a CUDA event between every two kernels: each costs the launch overlap of the kernel behind it,
    about 4 us, so the blocks that give the headline number run without them)."""
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    all_marks = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(steps):
        marks = [] if per_kernel_events else None
        step.run(marks)
        step.exchange()
        if marks is not None:
            all_marks.append(marks)
    step.finish()  # the last exchanges complete inside the timed region
    e1.record()
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    per_kernel = None
    if per_kernel_events:
        per_kernel = [0.0] * len(Step.KERNELS)
        for marks in all_marks:
            for i in range(len(Step.KERNELS)):
                per_kernel[i] += marks[i].elapsed_time(marks[i + 1])
        per_kernel = [v / steps for v in per_kernel]
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms, per_kernel


def timed_steps(step, steps, warmup, world, blocks=5):
    """`warmup` untimed steps, then `blocks` timed blocks of exactly `steps` steps each; the reported block is the
    median one (one block of 20 steps lasts about 10 ms, too short a window to trust alone).  One more block of
    the same steps, with an event between kernels, gives the per-kernel times."""
    for _ in range(warmup):
        step.run()
        step.exchange()
    step.finish()
    runs = [timed_block(step, steps, world)[0] for _ in range(max(1, blocks))]
    ms = sorted(runs)[len(runs) // 2]
    marked_ms, per_kernel = timed_block(step, steps, world, per_kernel_events=True)
    return ms, per_kernel, [round(r, 4) for r in runs], marked_ms


def e2e_steps(step, steps, warmup, world):
    """Same step through the C ABI with HOST buffers: every step uploads x, dy, t from pinned memory and downloads
    every result (y, dx of GroupNorm+SiLU and of LayerNorm, the parameter gradients, the embedding) inside the
    timed region.  Copies and kernels are pipelined the way a host application would drive the library: an upload
    stream, a compute stream and a download stream over two device buffer sets, so that the upload of step i+1
    and the download of step i share the full-duplex link.  Both arms use this same driver."""
    dev, fused, L = step.dev, step.fused, step.lib
    hx = torch.empty(B, HW, C).pin_memory(); hdy = torch.empty(B, HW, C).pin_memory(); ht = torch.empty(B).pin_memory()
    hx.copy_(step.x); hdy.copy_(step.dy); ht.copy_(step.t)
    big = lambda: torch.empty(B, HW, C).pin_memory()
    hy, hdx, hy2, hdx2 = big(), big(), big(), big()
    hdgam, hemb = torch.empty(4 * C).pin_memory(), torch.empty(B, EMB).pin_memory()
    h2d = (hx.numel() + hdy.numel() + ht.numel()) * 4
    d2h = (hy.numel() + hdx.numel() + hy2.numel() + hdx2.numel() + hdgam.numel() + hemb.numel()) * 4

    class Set:
        def __init__(self):
            e = lambda *shape: torch.empty(*shape, device=dev)
            self.x, self.dy, self.y, self.dx, self.y2, self.dx2 = (e(B, HW, C) for _ in range(6))
            self.t, self.emb, self.dgam = e(B), e(B, EMB), e(4 * C)
            self.mu, self.rstd, self.lmu, self.lrstd = e(B * G), e(B * G), e(B * HW), e(B * HW)
            if not fused:
                self.h, self.gh = e(B, HW, C), e(B, HW, C)

    sets = [Set(), Set()]
    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    ev_in = [torch.cuda.Event() for _ in range(2)]
    ev_cmp = [torch.cuda.Event() for _ in range(2)]
    ev_out = [torch.cuda.Event() for _ in range(2)]

    def one(i):
        k = i & 1
        S = sets[k]
        with torch.cuda.stream(s_in):
            s_in.wait_event(ev_cmp[k])  # step i-2 has finished reading this set's inputs
            S.x.copy_(hx, non_blocking=True); S.dy.copy_(hdy, non_blocking=True); S.t.copy_(ht, non_blocking=True)
            ev_in[k].record(s_in)
        with torch.cuda.stream(s_cmp):
            s_cmp.wait_event(ev_in[k])
            s_cmp.wait_event(ev_out[k])  # the results of step i-2 have left this set
            st = ctypes.c_void_p(s_cmp.cuda_stream)
            dg, db, lg, lb = (ctypes.c_void_p(S.dgam.data_ptr() + 4 * C * j) for j in range(4))
            if fused:
                L.launch_groupnorm_act_forward(P(S.y), P(S.mu), P(S.rstd), P(S.x), P(step.gamma), P(step.beta),
                                               B, HW, C, G, F(1e-5), 3, st)
                L.launch_groupnorm_act_backward(P(S.dx), dg, db, P(S.dy), P(S.x), P(step.gamma), P(step.beta),
                                                P(S.mu), P(S.rstd), B, HW, C, G, 3, st)
            else:
                L.launch_groupnorm_forward(P(S.h), P(S.mu), P(S.rstd), P(S.x), P(step.gamma), P(step.beta),
                                           B, HW, C, G, F(1e-5), st)
                L.launch_activation_forward(P(S.y), P(S.h), NEL, 3, st)
                L.launch_activation_backward(P(S.gh), P(S.dy), P(S.h), NEL, 3, st)
                L.launch_groupnorm_backward(P(S.dx), dg, db, P(S.gh), P(S.x), P(step.gamma), P(S.mu), P(S.rstd),
                                            B, HW, C, G, st)
            L.launch_layernorm_forward(P(S.y2), P(S.lmu), P(S.lrstd), P(S.x), P(step.gamma), P(step.beta),
                                       B * HW, C, F(1e-5), st)
            L.launch_layernorm_backward(P(S.dx2), lg, lb, P(S.dy), P(S.x), P(step.gamma), P(S.lmu), P(S.lrstd),
                                        B * HW, C, st)
            L.launch_sinusoidal(P(S.emb), P(S.t), B, EMB, step.lmp, st)
            if world > 1:
                torch.distributed.all_reduce(S.dgam)
            ev_cmp[k].record(s_cmp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_cmp[k])
            hy.copy_(S.y, non_blocking=True); hdx.copy_(S.dx, non_blocking=True)
            hy2.copy_(S.y2, non_blocking=True); hdx2.copy_(S.dx2, non_blocking=True)
            hdgam.copy_(S.dgam, non_blocking=True); hemb.copy_(S.emb, non_blocking=True)
            ev_out[k].record(s_out)

    for i in range(warmup):
        one(i)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    cur = torch.cuda.current_stream()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(cur)
    for s_ in (s_in, s_cmp, s_out):
        s_.wait_event(e0)
    for i in range(steps):
        one(warmup + i)
    for ev in ev_out:
        cur.wait_event(ev)
    e1.record(cur)
    torch.cuda.synchronize()
    if world > 1:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([ms], device="cuda")
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms, h2d, d2h


# ------------------------------------------------------------------------------------ per-op table
def graph_time(lib, fn, nsets, reps, scratch_bytes=0):
    """Average device time of fn(i) over `reps` launches replayed from a CUDA graph
    (removes host launch overhead; fn cycles through `nsets` buffer sets larger than L2).
    The graph is replayed once untimed (warm-up of `reps` launches) and once timed."""
    s = torch.cuda.Stream()
    if scratch_bytes and hasattr(lib, "b200_scratch_reserve"):
        lib.b200_scratch_reserve(ctypes.c_void_p(s.cuda_stream), ctypes.c_longlong(scratch_bytes))
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(min(nsets, 3)):
            fn(i)
    s.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g, stream=s):
        for i in range(reps):
            fn(i % nsets)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e-3 / reps


def ops_table(lib, fused, peak, only=None):
    """Every other kernel of the path at the baseline's sizes: seconds per launch and algorithmic GB/s.
    `only` = "cfg0" restricts the table to the first configuration (profiler captures of that shape)."""
    dev = torch.device("cuda")
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    out = {}

    def add(name, secs, nbytes=None):
        rec = {"us": round(secs * 1e6, 2)}
        if nbytes:
            rec["GBps"] = round(nbytes / secs / 1e9, 1)
            rec["frac_of_measured_peak"] = round(nbytes / secs / 1e9 / peak, 3)
            rec["frac_of_nominal_8TBs"] = round(nbytes / secs / 1e9 / 8000.0, 3)
        out[name] = rec

    # ---- config 0: GroupNorm fwd+bwd [128,28,28,64], G=32 (25.7 MB tensors: rotate 8 sets to defeat L2)
    b, hw, c, g = 128, 784, 64, 32
    n = b * hw * c
    ns = 8
    xs = [torch.randn(b, hw, c, device=dev) for _ in range(ns)]
    ys = [torch.empty(b, hw, c, device=dev) for _ in range(ns)]
    dys = [torch.randn(b, hw, c, device=dev) for _ in range(ns)]
    gam, bet = 1 + 0.1 * torch.randn(c, device=dev), 0.1 * torch.randn(c, device=dev)
    mu, rs = torch.empty(b * g, device=dev), torch.empty(b * g, device=dev)
    dg, db = torch.empty(c, device=dev), torch.empty(c, device=dev)
    fw = lambda i: lib.launch_groupnorm_forward(P(ys[i]), P(mu), P(rs), P(xs[i]), P(gam), P(bet), b, hw, c, g, F(1e-5), st())
    bw = lambda i: lib.launch_groupnorm_backward(P(ys[i]), P(dg), P(db), P(dys[i]), P(xs[i]), P(gam), P(mu), P(rs), b, hw, c, g, st())
    add("cfg0_groupnorm_fwd", graph_time(lib, fw, ns, 100), 2 * n * 4)
    add("cfg0_groupnorm_bwd", graph_time(lib, bw, ns, 100, 2 * b * c * 4), 3 * n * 4)
    del xs, ys, dys
    if only == "cfg0":
        return out

    # ---- config 1: EDM magnitude-preserving ops on [256,28,28,128]
    n = 256 * 28 * 28 * 128
    rows = n // 128
    ns = 3
    A = [torch.randn(n, device=dev) for _ in range(ns)]
    Bb = [torch.randn(n, device=dev) for _ in range(ns)]
    O = [torch.empty(n, device=dev) for _ in range(ns)]
    add("cfg1_mp_silu_fwd", graph_time(lib, lambda i: lib.launch_activation_forward(P(O[i]), P(A[i]), n, 5, st()), ns, 100), 2 * n * 4)
    add("cfg1_mp_silu_bwd", graph_time(lib, lambda i: lib.launch_activation_backward(P(O[i]), P(Bb[i]), P(A[i]), n, 5, st()), ns, 100), 3 * n * 4)
    add("cfg1_mp_sum_fwd", graph_time(lib, lambda i: lib.launch_mp_sum(P(O[i]), P(A[i]), P(Bb[i]), F(0.3), n, st()), ns, 100), 3 * n * 4)
    if fused:
        add("cfg1_mp_sum_bwd", graph_time(lib, lambda i: lib.launch_mp_sum_backward(P(O[i]), P(Bb[i]), P(A[i]), F(0.3), n, st()), ns, 100), 3 * n * 4)
    else:
        def two(i):
            lib.launch_weighted_sum(P(O[i]), P(A[i]), P(A[i]), F(0.919), F(0.0), n, st())
            lib.launch_weighted_sum(P(Bb[i]), P(A[i]), P(A[i]), F(0.394), F(0.0), n, st())
        add("cfg1_mp_sum_bwd", graph_time(lib, two, ns, 100), 3 * n * 4)
    add("cfg1_mp_cat_fwd", graph_time(lib, lambda i: lib.launch_mp_channel_cat(P(O[i]), P(A[i]), P(Bb[i]), F(0.5), rows, 64, 64, st()), ns, 100), 2 * n * 4)
    add("cfg1_mp_cat_bwd", graph_time(lib, lambda i: lib.launch_mp_channel_split(P(A[i]), P(Bb[i]), P(O[i]), F(0.5), rows, 64, 64, st()), ns, 100), 2 * n * 4)
    if fused:  # pixel norm has no counterpart in the reference
        add("cfg1_pixel_norm_fwd", graph_time(lib, lambda i: lib.launch_pixel_norm_forward(P(O[i]), P(A[i]), rows, 128, F(1e-4), st()), ns, 100), 2 * n * 4)
        add("cfg1_pixel_norm_bwd", graph_time(lib, lambda i: lib.launch_pixel_norm_backward(P(O[i]), P(Bb[i]), P(A[i]), rows, 128, F(1e-4), st()), ns, 100), 3 * n * 4)
    del A, Bb, O
    Wm, Mm = torch.randn(1152, 128, device=dev), torch.randn(1152, 128, device=dev)
    gain, gg = torch.ones(1, device=dev), torch.zeros(1, device=dev)
    add("cfg1_weight_norm_fwd_1152x128", graph_time(lib, lambda i: lib.launch_weight_normalize(P(Wm), 1152, 128, F(1e-4), st()), 1, 100), 2 * Wm.numel() * 4)
    add("cfg1_weight_norm_bwd_1152x128", graph_time(lib, lambda i: lib.launch_weight_normalize_backward(P(Mm), P(Wm), P(gain), P(gg), 1152, 128, st()), 1, 100), 3 * Wm.numel() * 4)

    # ---- config 2: the two GroupNorm+SiLU kernels of the step and LayerNorm, each ALONE (the step's per-kernel
    # times also carry the write-backs of whatever ran before)
    b2, hw2, c2, g2 = 256, 1024, 256, 32
    n2 = b2 * hw2 * c2
    X2 = [torch.randn(b2, hw2, c2, device=dev) for _ in range(2)]
    D2 = [torch.randn(b2, hw2, c2, device=dev) for _ in range(2)]
    Y2 = [torch.empty(b2, hw2, c2, device=dev) for _ in range(2)]
    gam2, bet2 = 1 + 0.1 * torch.randn(c2, device=dev), 0.1 * torch.randn(c2, device=dev)
    mu2, rs2 = torch.empty(b2 * hw2, device=dev), torch.empty(b2 * hw2, device=dev)
    dg2, db2 = torch.empty(c2, device=dev), torch.empty(c2, device=dev)
    if fused:
        add("cfg2_groupnorm_silu_fwd_alone", graph_time(lib, lambda i: lib.launch_groupnorm_act_forward(
            P(Y2[i]), P(mu2), P(rs2), P(X2[i]), P(gam2), P(bet2), b2, hw2, c2, g2, F(1e-5), 3, st()), 2, 40), 2 * n2 * 4)
        add("cfg2_groupnorm_silu_bwd_alone", graph_time(lib, lambda i: lib.launch_groupnorm_act_backward(
            P(Y2[i]), P(dg2), P(db2), P(D2[i]), P(X2[i]), P(gam2), P(bet2), P(mu2), P(rs2), b2, hw2, c2, g2, 3, st()),
            2, 40, 2 * b2 * c2 * 4), 3 * n2 * 4)
    add("cfg2_layernorm_fwd_alone", graph_time(lib, lambda i: lib.launch_layernorm_forward(
        P(Y2[i]), P(mu2), P(rs2), P(X2[i]), P(gam2), P(bet2), b2 * hw2, c2, F(1e-5), st()), 2, 40 if fused else 4), 2 * n2 * 4)
    add("cfg2_layernorm_bwd_alone", graph_time(lib, lambda i: lib.launch_layernorm_backward(
        P(Y2[i]), P(dg2), P(db2), P(D2[i]), P(X2[i]), P(gam2), P(mu2), P(rs2), b2 * hw2, c2, st()), 2, 40 if fused else 4,
        64 << 20), 3 * n2 * 4)
    del X2, D2, Y2

    # ---- embeddings (latency-bound)
    tt = torch.randint(0, 1000, (256,), device=dev).float(); e1 = torch.empty(256, 512, device=dev)
    add("cfg2_sinusoidal_256x512", graph_time(lib, lambda i: lib.launch_sinusoidal(P(e1), P(tt), 256, 512, F(9.2103404), st()), 1, 100), e1.numel() * 4)
    xx, fr, ph = torch.randn(256, device=dev), torch.randn(128, device=dev), torch.rand(128, device=dev)
    e2 = torch.empty(256, 128, device=dev)
    add("cfg3_mp_fourier_256x128", graph_time(lib, lambda i: lib.launch_mp_fourier(P(e2), P(xx), P(fr), P(ph), 256, 128, st()), 1, 100), e2.numel() * 4)

    # ---- config 4: optimizer, 64M parameters
    npar = 64 * 2 ** 20
    p_, m_, v_, s_, g_ = (torch.randn(npar, device=dev) * 0.02 for _ in range(5))
    v_.abs_()
    hp = (F(1e-4), F(0.9), F(0.999), F(1e-8), F(0.19), F(0.002))
    if fused:
        add("cfg4_adam_ema_fused_64M", graph_time(lib, lambda i: lib.launch_adam_ema_step(P(p_), P(m_), P(v_), P(s_), P(g_), *hp, F(0.999), F(1.0), ctypes.c_longlong(npar), st()), 1, 100), 36 * npar)
    else:
        def two_pass(i):
            lib.launch_adam_step(P(p_), P(m_), P(v_), P(g_), *hp, npar, st())
            lib.launch_weighted_sum(P(s_), P(s_), P(p_), F(0.999), F(0.001), npar, st())
        add("cfg4_adam_then_ema_64M", graph_time(lib, two_pass, 1, 100), 36 * npar)
    add("cfg4_adam_64M", graph_time(lib, lambda i: lib.launch_adam_step(P(p_), P(m_), P(v_), P(g_), *hp, npar, st()), 1, 100), 28 * npar)
    return out


# ------------------------------------------------------------------------------------ CPU baseline
def cpu_baseline(threads=None, samples=16, min_seconds=10.0, single_seconds=6.0):
    """The plain-C port (oracle/layer_oracle.c, fp32 accumulation) on the host cores over a bounded
    sample of the step: `samples` of the 256 images per GPU, same kernel sequence, repeated until
    about `min_seconds` of wall time with every host thread, then about `single_seconds` with one."""
    sys.path.insert(0, str(ROOT / "oracle"))
    orc = importlib.import_module("oracle")
    orc.load()
    orc.set_accumulate_double(False)
    threads = threads or orc.max_threads()
    rng = np.random.default_rng(0)
    x = rng.standard_normal((samples, HW, C), dtype=np.float32)
    dy = rng.standard_normal((samples, HW, C), dtype=np.float32)
    gam = (1 + 0.1 * rng.standard_normal(C)).astype(np.float32); bet = (0.1 * rng.standard_normal(C)).astype(np.float32)
    tt = rng.integers(0, 1000, samples).astype(np.float32)

    def one():
        y, mu, rstd = orc.groupnorm_forward(x, gam, bet, G, 1e-5, "silu")
        orc.groupnorm_backward(dy, x, gam, bet, mu, rstd, G, "silu")
        y2, lmu, lrs = orc.layernorm_forward(x.reshape(-1, C), gam, bet, 1e-5)
        orc.layernorm_backward(dy.reshape(-1, C), x.reshape(-1, C), gam, lmu, lrs)
        orc.sinusoidal(tt, EMB, np.float32(math.log(1e4)))

    def timed(nthreads, seconds):
        orc.set_threads(nthreads)
        one()  # warm-up (page faults, thread pool)
        reps, t0 = 0, time.perf_counter()
        while True:
            one()
            reps += 1
            dt = time.perf_counter() - t0
            if dt >= seconds or reps >= 5000:
                break
        return STEP_BYTES * samples / B * reps / dt / 1e9, reps, dt

    gbs, reps, dt = timed(threads, min_seconds)
    gbs1, reps1, dt1 = timed(1, single_seconds)
    orc.set_accumulate_double(True)
    orc.set_threads(1)
    return {"value": round(gbs, 3), "unit": "GB/s", "cores": threads, "kind": "port",
            "single_thread": {"value": round(gbs1, 3), "unit": "GB/s", "cores": 1,
                              "sample": f"same sample x {reps1} repeats, {dt1:.1f} s"},
            "sample": f"{samples} of the {B} samples of one step (same kernel sequence) x {reps} repeats, {dt:.1f} s of "
                      f"wall time, OpenMP over {threads} threads; the reference has no CPU path, so this is the "
                      f"plain-C port of its kernels"}


# ------------------------------------------------------------------------------------ range-sharded optimizer
def run_rank_program(exe, args, world, rank, local_rank, tag, key, timeout=120):
    """Starts one process of a C program of build/bin on this rank's GPU (RANK / WORLD_SIZE / LOCAL_RANK in its
    environment); the processes of one run meet through a file whose name carries a per-run nonce chosen by rank 0,
    so that a file left behind by a crashed or killed earlier run (or another job on the machine) is never picked
    up.  Rank 0 returns the object under `key` of the program's JSON line, the other ranks None."""
    import tempfile
    if not exe.exists():
        return None
    env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(local_rank))
    nonce = [f"{os.getpid()}_{time.time_ns()}"]
    if world > 1:
        torch.distributed.broadcast_object_list(nonce, src=0)
    id_file = os.path.join(tempfile.gettempdir(), f"{tag}_{nonce[0]}.ncclid")
    try:
        res = subprocess.run([str(exe), *args, "--id-file", id_file], env=env, capture_output=True, text=True,
                             timeout=timeout)
    except subprocess.TimeoutExpired:
        return {"error": "timeout"} if rank == 0 else None
    finally:
        if rank == 0 and os.path.exists(id_file):
            os.unlink(id_file)
    if rank != 0:
        return None
    if res.returncode != 0:
        return {"error": (res.stderr or res.stdout)[-300:]}
    for ln in res.stdout.splitlines():
        if ln.startswith("{"):
            return json.loads(ln)[key]
    return {"error": "no result line"}


def sharded_adam_ema(world, rank, local_rank):
    """Optimizer config: flat 64M-parameter vector, fused Adam+EMA on this rank's range, new parameters published
    to the other ranks -- csrc/host/sharded_adam_bench.c on csrc/host/b200_sharded_optimizer.c (C, NCCL, CUDA IPC).
    Three device-timed figures (events around the launches only, max over ranks): the update kernel alone, update
    then in-place ncclAllGather, and the update whose store phase writes the peers' copies directly."""
    return run_rank_program(BIN / "sharded_adam_bench", ["--iters", "20", "--warmup", "3"], world, rank, local_rank,
                            "sharded_adam", "sharded_adam_ema")


# ------------------------------------------------------------------------------------ EDM UNet training step
def write_edm_config(folder, batch, train_steps):
    """Writes the synthetic image file and an .ini for the reference's EDM trainer into `folder`; returns the
    .ini path.  Also reachable as `bench.py --write-edm-config FOLDER` for profiler captures of the trainer."""
    os.makedirs(folder, exist_ok=True)
    images = os.path.join(folder, "images.bin")
    if not os.path.exists(images):
        rng = np.random.default_rng(0)
        n = 4096
        img = np.where(rng.random((n, 28, 28)) < 0.8, -1.0, rng.uniform(-1, 1, (n, 28, 28))).astype(np.float32)
        img.tofile(images)
    ini = os.path.join(folder, f"edm_{train_steps}.ini")
    with open(ini, "w") as f:
        f.write(f"channels = 64,128,128\nemb_dim = 128\nheads = 1\nt = 0.3\nbatch_size = {batch}\n"
                f"train_steps = {train_steps}\nlr = 1e-3\nlr_warmup = 500\nlr_ref = 5000\nema_decay = 0.999\n"
                f"tf32 = 1\nsample_steps = 1\nvis_batch = 1\nimages = {images}\nH = 28\nW = 28\nC = 1\n")
    return ini


def write_ddpm_config(folder, batch, train_steps):
    """Synthetic image file and an .ini for the reference's DDPM trainer (ddpm/main_ddpm.c): the model of its own
    ddpm.ini (channels 32/64/128, emb 64, 4 heads, 32 groups, T=1000, min-SNR gamma 5), batch `batch`, TF32 GEMMs."""
    os.makedirs(folder, exist_ok=True)
    images = os.path.join(folder, "images.bin")
    if not os.path.exists(images):
        rng = np.random.default_rng(0)
        n = 4096
        img = np.where(rng.random((n, 28, 28)) < 0.8, -1.0, rng.uniform(-1, 1, (n, 28, 28))).astype(np.float32)
        img.tofile(images)
    ini = os.path.join(folder, f"ddpm_{train_steps}.ini")
    with open(ini, "w") as f:
        f.write(f"channels = 32,64,128\nemb_dim = 64\nheads = 4\nnum_groups = 32\nbatch_size = {batch}\n"
                f"train_steps = {train_steps}\nlr = 1e-3\nlr_warmup = 500\nlr_ref = 2000\nsnr_gamma = 5.0\n"
                f"ema_decay = 0.999\nT = 1000\nbeta_start = 1e-4\nbeta_end = 0.02\nddim_steps = 1\ntf32 = 1\n"
                f"images = {images}\nH = 28\nW = 28\nC = 1\n")
    return ini


def edm_train_images_per_s(binary, batch=256, steps=(50, 450), write_config=None):
    """Images/s of the reference's own EDM trainer (edm/main_edm.c + diffusion/train.c + every host module,
    unmodified) with the given kernel backend linked in.  Config: channels 64/128/128, emb 128, 1 head, t 0.3,
    batch 256, Adam lr 1e-3, EMA 0.999, TF32 GEMMs, synthetic 28x28 images (pixel -1 with p=0.8, else U(-1,1)).
    The program has no timer, so two runs with different step counts are timed and the difference is used."""
    import tempfile
    if not Path(binary).exists():
        return None
    with tempfile.TemporaryDirectory() as tmp:
        times = []
        for st in (2,) + tuple(steps):  # the first (2-step) run only warms caches and is not used
            ini = (write_config or write_edm_config)(tmp, batch, st)
            t0 = time.perf_counter()
            res = subprocess.run([str(binary), ini], cwd=tmp, capture_output=True, text=True, timeout=900)
            times.append(time.perf_counter() - t0)
            if res.returncode != 0:
                return {"error": (res.stderr or res.stdout)[-300:]}
        dt = times[2] - times[1]
        nst = steps[1] - steps[0]
        return {"images_per_s": round(batch * nst / dt, 1), "ms_per_step": round(dt / nst * 1e3, 2), "batch": batch,
                "steps_timed": nst, "how": "wall-clock difference of two runs of the unmodified reference trainer"}


def edm_dp_train(world, rank, local_rank, batch_per_gpu, steps=30, warmup=5, graph=True, fastconv=True, sharded=None):
    """Data-parallel EDM UNet training (build/bin/edm_dp_train[_fastconv]: the reference's UNet and host
    modules, this library's kernels, NCCL gradient exchange; `fastconv` links csrc/host/b200_conv2d.c in place of
    the reference's conv2d.c; `sharded` = "allgather" | "peer" selects the range-sharded optimizer).  Every rank of
    this benchmark starts one trainer process on its own GPU.  Rank 0 returns the trainer's JSON (device-timed,
    max over ranks), the other ranks None."""
    args = ["--batch", str(batch_per_gpu), "--steps", str(steps), "--warmup", str(warmup)]
    if graph:
        args.append("--graph")
    if sharded:
        args += ["--sharded", sharded]
    got = run_rank_program(BIN / ("edm_dp_train_fastconv" if fastconv else "edm_dp_train"), args, world, rank,
                           local_rank, f"edm_dp_train_{batch_per_gpu}_{int(fastconv)}", "edm_dp_train", timeout=90)
    if isinstance(got, dict) and "error" not in got:
        got["conv2d_host_module"] = "csrc/host/b200_conv2d.c" if fastconv else "reference src/conv2d.c"
    return got


def ddpm_dp_train(world, rank, local_rank, batch_per_gpu, steps=30, warmup=5, sharded=None):
    """Data-parallel DDPM UNet training (build/bin/ddpm_dp_train: the reference's DDPM UNet with the residual block
    on the fused GroupNorm+SiLU kernels, CUDA graph, NCCL); device-timed, max over ranks."""
    args = ["--batch", str(batch_per_gpu), "--steps", str(steps), "--warmup", str(warmup), "--graph"]
    if sharded:
        args += ["--sharded", sharded]
    return run_rank_program(BIN / "ddpm_dp_train", args, world, rank, local_rank, f"ddpm_dp_train_{batch_per_gpu}",
                            "ddpm_dp_train", timeout=90)


# ------------------------------------------------------------------------------------ main
KERNEL_BYTES = {"gn_silu_fwd": 2 * NEL * 4, "gn_silu_bwd": 3 * NEL * 4, "ln_fwd": 2 * NEL * 4, "ln_bwd": 3 * NEL * 4,
                "sinusoidal": B * EMB * 4}
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under profiles/
# (GroupNorm: captured at the full batch; LayerNorm: at batch 128 and scaled by 2, traffic grows linearly with the
# batch).  Reads match the algorithmic bytes; the write figure is low because up to an L2's worth of dirty lines
# has not been written back when the kernel ends.
NCU_TRAFFIC = {"gn_silu_bwd": 536_964_864 + 226_537_472, "gn_silu_fwd": 268_459_520 + 210_318_592,
               "ln_fwd": 2 * (134_267_904 + 83_640_064), "ln_bwd": 2 * (269_501_952 + 95_807_232)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--blocks", type=int, default=5, help="timed blocks of --steps steps; the median block is reported")
    ap.add_argument("--no-ops", action="store_true", help="skip the per-op table")
    ap.add_argument("--ops-only", metavar="CFG", help="print only the per-op table of one configuration (cfg0) and exit")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--no-trainer", action="store_true", help="skip the EDM trainer legs (profiler captures)")
    ap.add_argument("--tune", action="append", default=[], metavar="KEY=INT",
                    help="set a kernel tunable (b200_tune_set), e.g. gn_deep=0 to time the backward strips without the deeper staging")
    ap.add_argument("--batch", type=int, default=256, help="samples per GPU; values other than 256 are for profiling only")
    ap.add_argument("--write-edm-config", metavar="FOLDER", help="write images.bin + edm_<steps>.ini for the reference's "
                    "EDM trainer (same config as the timing leg) and exit")
    ap.add_argument("--edm-steps", type=int, default=6, help="train_steps for --write-edm-config")
    args = ap.parse_args()
    if args.write_edm_config:
        print(write_edm_config(args.write_edm_config, args.batch, args.edm_steps))
        return
    if args.batch != 256:
        set_batch(args.batch)
    args.warmup = max(args.warmup, 3)

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        if args.impl == "reference" and rank == 0:
            cb = cpu_baseline()
            print(json.dumps({"impl": "reference", "metric": "fused norm/act fwd+bwd HBM GB/s", "value": cb["value"],
                              "unit": "GB/s", "n_gpus": 0, "higher_is_better": True, "cpu_baseline": cb,
                              "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                                      "d2h_bytes_per_step": 0}}))
            return
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.distributed.init_process_group("nccl", device_id=torch.device("cuda", local))

    capi = load_capi()
    lib = None
    if args.impl == "b200":  # the reference arm never maps this repository's kernel library
        lib = capi.load()
        for kv in args.tune:
            key, val = kv.split("=")
            lib.b200_tune_set(key.encode(), int(val))
    peak, peak_src = measured_peak()
    if args.ops_only:
        print(json.dumps({"ops": ops_table(lib, True, peak, only=args.ops_only)}))
        return
    fused = True
    ref_note = None
    if args.impl == "reference":
        ref = load_reference(capi)
        if ref is None:
            # the reference could not be compiled where this tree was built: time the plain-C port instead
            if rank == 0:
                cb = cpu_baseline()
                print(json.dumps({"impl": "reference", "metric": "fused norm/act fwd+bwd HBM GB/s",
                                  "value": cb["value"], "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
                                  "warmup": args.warmup, "higher_is_better": True, "cpu_baseline": cb,
                                  "e2e": {"value": cb["value"], "unit": "GB/s", "h2d_bytes_per_step": 0,
                                          "d2h_bytes_per_step": 0},
                                  "note": "oracle/_ref/libref_kernels.so absent; CPU port of the path"}))
            return
        lib_run, fused = ref, False
        ref_note = ("reference src/kernels.cu compiled unmodified for sm_100a with its own flags (-O3 --use_fast_math); "
                    "GroupNorm->SiLU and SiLU'->GroupNorm' composed as conv_residual.c does")
    else:
        lib_run = lib

    step = Step(lib_run, fused, torch.device("cuda", local), seed=1234 + rank)
    launches0 = lib.b200_launch_count() if args.impl == "b200" else 0
    with ClockSampler(local) as cs:
        ms, per_kernel, block_ms, marked_ms = timed_steps(step, args.steps, args.warmup, world, args.blocks)
    launches = (lib.b200_launch_count() - launches0) if args.impl == "b200" else None
    if launches is not None:  # launches of ONE timed block of `steps` steps
        launches = int(launches * args.steps / (args.steps * (max(1, args.blocks) + 1) + args.warmup))
    clocks = cs.summary()
    e2e_k = max(3, min(args.steps, 10))
    if args.no_e2e:
        e2e_ms, h2d, d2h = float("nan"), 0, 0
    else:
        e2e_ms, h2d, d2h = e2e_steps(step, e2e_k, 3, world)

    value = world * STEP_BYTES * args.steps / (ms * 1e-3) / 1e9
    e2e_value = world * STEP_BYTES * e2e_k / (e2e_ms * 1e-3) / 1e9
    dom = max(range(len(Step.KERNELS) - 1), key=lambda i: per_kernel[i])
    dom_name = Step.KERNELS[dom]
    achieved = KERNEL_BYTES[dom_name] / (per_kernel[dom] * 1e-3) / 1e9
    line = {
        "metric": "fused norm/act fwd+bwd HBM GB/s", "value": round(value, 1), "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms / args.steps, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"batch_per_gpu": B, "workload": "configs[2]: DDPM block kernels, fp32 NHWC [256,32,32,256] per GPU: GroupNorm(32)+affine+SiLU "
                               "fused fwd+bwd, LayerNorm C=256 fwd+bwd, sinusoidal dim 512; batch-sharded",
                   "l2": "inputs larger than L2 (each tensor 268 MB vs 126 MB L2); no flush needed",
                   "algorithmic_bytes_per_step": STEP_BYTES, "seed": 1234,
                   "exchange": "all-reduce of the 4*C parameter-gradient floats, overlapped with the next step (N>1)"},
        "clocks": clocks,
        "timing": {"blocks_ms": block_ms, "reported": "median block of exactly `steps` steps, CUDA events, max over ranks",
                   "per_kernel_block_ms": round(marked_ms, 4),
                   "per_kernel": "kernels_ms and roofline come from one more block of the same steps with a CUDA event "
                                 "between kernels; those events keep a kernel's launch from overlapping its predecessor, "
                                 "so that block is a few percent slower than the reported ones"},
        "e2e": {"value": round(e2e_value, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "steps": e2e_k, "ms_per_step": round(e2e_ms / e2e_k, 3),
                "how": "C ABI on host buffers; upload, compute and download streams over two device buffer sets"},
        "kernels_ms": {k: round(v, 4) for k, v in zip(Step.KERNELS, per_kernel)},
        "roofline": {"bound": "hbm", "kernel": dom_name, "achieved": round(achieved, 1), "peak": peak, "unit": "GB/s",
                     "frac": round(achieved / peak, 3), "frac_of_nominal_8TBs": round(achieved / 8000.0, 3),
                     "traffic": NCU_TRAFFIC.get(dom_name), "peak_source": peak_src,
                     "all": {k: round(KERNEL_BYTES[k] / (v * 1e-3) / 1e9 / peak, 3)
                             for k, v in zip(Step.KERNELS[:-1], per_kernel)}},
    }
    if args.impl == "b200":
        line["gpu_launches"] = launches
    else:
        line["impl"] = "reference"
        line["reference_kind"] = ref_note
    if args.impl == "b200" and not args.no_ops:
        del step
        torch.cuda.empty_cache()
        step = None
        line["sharded_adam_ema"] = sharded_adam_ema(world, rank, local)
        # EDM UNet training, images/s: weak scaling (256 per GPU) and strong scaling (256 in total)
        if world > 1:
            torch.distributed.barrier()
    if args.impl == "b200" and not args.no_ops and not args.no_trainer:
        dp = {"weak_256_per_gpu": edm_dp_train(world, rank, local, 256)}
        if world > 1:
            torch.distributed.barrier()
            dp["strong_256_global"] = edm_dp_train(world, rank, local, 256 // world)
            torch.distributed.barrier()
            dp["strong_256_global_sharded_optimizer"] = edm_dp_train(world, rank, local, 256 // world, sharded="peer")
        else:
            dp["weak_256_per_gpu_reference_conv2d"] = edm_dp_train(world, rank, local, 256, fastconv=False)
        line["edm_dp_train"] = dp
        if world > 1:
            torch.distributed.barrier()
        ddp = {"weak_256_per_gpu": ddpm_dp_train(world, rank, local, 256)}
        if world > 1:
            torch.distributed.barrier()
            ddp["strong_256_global"] = ddpm_dp_train(world, rank, local, 256 // world)
        line["ddpm_dp_train"] = ddp
    if rank == 0:
        if not args.no_cpu and (world == 1 or args.impl == "reference"):
            line["cpu_baseline"] = cpu_baseline()
        if not args.no_ops and world == 1:
            step = None
            torch.cuda.empty_cache()
            line["ops"] = ops_table(lib_run, fused, peak)
            exe = BIN / "edm_demo_b200" if args.impl == "b200" else ROOT / "oracle" / "_ref" / "edm_demo_ref"
            edm = None if args.no_trainer else edm_train_images_per_s(exe)
            if edm is not None:
                line["edm_unet_train"] = edm
            # the reference's DDPM trainer (GroupNorm+SiLU blocks): its own kernels in the reference arm; in this
            # arm once as a plain drop-in at the launch_* ABI and once with the fused residual block linked in
            if not args.no_trainer:
                if args.impl == "b200":
                    ddpm = {"drop_in": edm_train_images_per_s(BIN / "ddpm_demo_b200", steps=(100, 700),
                                                              write_config=write_ddpm_config),
                            "fused_block": edm_train_images_per_s(BIN / "ddpm_demo_b200_fused", steps=(100, 700),
                                                                  write_config=write_ddpm_config)}
                else:
                    ddpm = edm_train_images_per_s(ROOT / "oracle" / "_ref" / "ddpm_demo_ref", steps=(20, 120),
                                                  write_config=write_ddpm_config)
                line["ddpm_unet_train"] = ddpm
        print(json.dumps(line))
    if world > 1:
        torch.distributed.barrier()
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
