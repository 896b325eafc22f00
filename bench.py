#!/usr/bin/env python
"""Benchmark of the tiled SDPA hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Headline workload (one "step" = one forward + one backward pass of the fused
flash-SDPA tile tasks over one batch of synthetic input, per GPU):
  BASELINE config 3, Llama-style GQA attention, bf16 storage / fp32 accumulate:
  32 query heads (8 KV heads x group 4, K/V replicated over the group as the
  reference does), head_dim 128, seq 4096, batch 4, causal additive mask,
  RoPE (base 10000) pre-applied to Q and K ~ N(0,1), dY ~ N(0,1); one sequence
  tile (seq-tile 4096), all calls through the C ABI of include/nntile_b200.h.
The metric is TFLOP/s under the causal convention (forward 2W, backward 5W,
W = B*Hq*S^2*D).  Scaling is strong: config 3 is ONE problem of 32 independent
(batch, kv head) units; with N GPUs every rank takes the block of 8/N kv heads
that nntile_b200.parallel.shard_range deals it (what the reference does by
placing tile tasks on N StarPU CUDA workers), `value` is the FLOPs of the whole
problem over the slowest rank's time, and there is no collective on the data
path.  (`extra.weak_scaling`, N > 1 only: every rank runs all of config 3.)

The single JSON line also carries: `roofline` (dominant kernel = the backward
tile task, timed live with CUDA events, against the measured bf16 GEMM rates of
MEASURED_PEAKS.json - burst or sustained by the rule in roofline_regime()),
`cpu_baseline` (the reference's own CPU
kernels timed on a bounded sample, rank 0, N=1), `e2e` (same metric through the
same C-ABI calls with HOST buffers: pinned host -> device copies of Q, K, V, dY
and device -> host reads of A, dQ, dK, dV inside the timed region), `clocks`
(nvidia-smi samples taken during the timed region), `gpu_launches` (kernels of
this library launched in the timed region, from the library's own counter) and
`extra` (configs 2, 4, the layout-change kernels and library comparators at N=1;
the decode config 5, its batch split over the ranks, in GB/s vs HBM peak at every N).

`--impl reference` times the reference's CPU implementation of the path (its own
src/kernel/*/cpu.cc + OpenBLAS sgemm, compiled in place as oracle/_ref; the C
port of the oracle if that is absent) on all host cores, each step a bounded
sample of the same workload, and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time
from concurrent.futures import ThreadPoolExecutor

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "sdpa_fwd_bwd_tflops"
UNIT = "TFLOP/s"
# BASELINE config 3 (per GPU)
C3 = dict(head=128, seq=4096, batch=4, group=4, kv_heads=8)
# the same kernels on 16 instead of 128 (batch, head) slices: the small case for
# profiler captures (8 tensors of 16 MB, still larger than the 126 MB L2 together)
C3_SMALL = dict(head=128, seq=4096, batch=1, group=2, kv_heads=8)
C2 = dict(head=64, seq=1024, batch=8, group=1, kv_heads=12)
C4 = dict(head=128, seq=16384, batch=1, group=1, kv_heads=16, seq_tile=2048)
C5 = dict(head=128, max_seq=8192, batch=64, group=4, kv_heads=8)
# DRAM bytes per (batch, head) slice of head 128, seq 4096 measured with ncu
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch, one-pass capture
# of the full 128-slice workload; slices are independent, so a launch on fewer
# slices moves proportionally less)
NCU_DRAM_BYTES_PER_SLICE = {"flash_bwd_kernel<128>": 1563.0e6/128, "flash_fwd_kernel<128>": 519.0e6/128}
# share of the backward tile task's device time spent in flash_bwd_kernel<128> itself
# (the rest: mask classification, delta / accumulator preparation, dQ conversion), from
# the ncu launch list of the config-3 workload (profiles/)
NCU_BWD_KERNEL_SHARE = 0.881


def causal_flops(cfg):
    W = cfg["batch"]*cfg["group"]*cfg["kv_heads"]*cfg["seq"]**2*cfg["head"]
    return 2.0*W, 5.0*W


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(bf16=d.get("bf16_tflops_sustained", 1400.0),
                    bf16_burst=d.get("bf16_tflops", 1590.0), hbm=d.get("hbm_gbs", 6650.0),
                    sustained_mhz=(d.get("clocks_under_load") or {}).get("sm_mhz_median", 1275.0),
                    source="measured")
    return dict(bf16=1400.0, bf16_burst=1590.0, hbm=6650.0, sustained_mhz=1300.0,
                source="fallback")


def roofline_regime(peaks, timed_ms, sm_mhz):
    """Which measured GEMM rate a fraction is taken against.  The sustained rate was
    measured in a seconds-long loop with the board at its power limit and the SM
    clock far below maximum; the burst rate in a short run at full clock.  A timed
    region shorter than a second, or one whose sampled median SM clock is above the
    clock at which the sustained rate was measured, is in the burst regime."""
    if timed_ms < 1000.0 or (sm_mhz is not None and sm_mhz > peaks["sustained_mhz"]):
        return "burst", peaks["bf16_burst"]
    return "sustained", peaks["bf16"]


# --------------------------------------------------------------------------
# clocks sampling (nvidia-smi, during the timed region)
# --------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.lines = []
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(gpu_index), f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def count(self) -> int:
        return len(self.lines)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, pw, reasons = [], [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
                pw.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # samples under load = those drawing most of the peak power seen (an idle GPU
        # clocks down, a power-capped busy one clocks down too: power tells them apart)
        busy = [c for c, w in zip(sm, pw) if w >= 0.6*max(pw)] or sm
        return {"sm_mhz": statistics.median(busy), "sm_mhz_min_under_load": min(busy),
                "sm_max_mhz": max(mx), "power_w_max": max(pw), "samples": len(sm),
                "reasons": sorted(reasons)}


# --------------------------------------------------------------------------
# CPU reference arm (also the cpu_baseline leg)
# --------------------------------------------------------------------------
def cpu_reference_pass(n_slices: int, seq: int, head: int, threads: int, backend: str):
    """Run the reference's unfused fp32 chain (forward + backward) on `n_slices`
    independent (batch, head) slices of [head, seq], `threads` slices at a time,
    one single-threaded BLAS per slice (the reference's own setting: tasks across
    CPU workers, OPENBLAS_NUM_THREADS=1).  Returns seconds."""
    import numpy as np

    import oracle as O
    rng = np.random.default_rng(2)
    F = np.asfortranarray
    shape = (head, seq, 1, 1, 1)
    mask = F(np.triu(np.ones((seq, seq), dtype=bool)))
    data = []
    for _ in range(n_slices):
        data.append([F(rng.standard_normal(shape).astype(np.float32)) for _ in range(4)])

    def one(d):
        Q, K, V, dY = d
        Y, attn, _ = O.vanilla_forward(Q, K, V, mask, backend=backend)
        dQ, dK, dV = (O.zeros(shape, np.float32) for _ in range(3))
        O.vanilla_backward(Q, K, V, Y, dY, attn, mask, dQ, dK, dV, backend=backend)
        return float(dQ.flat[0])

    t0 = time.perf_counter()
    with ThreadPoolExecutor(max_workers=threads) as ex:
        list(ex.map(one, data))
    return time.perf_counter() - t0


def cpu_arm_setup():
    import oracle as O
    backend = "ref" if O.have_ref() else "port"
    if backend == "ref":
        import ctypes
        from oracle import build as ob
        blas = ob.find_openblas()
        if blas:
            try:
                ctypes.CDLL(blas).scipy_openblas_set_num_threads(1)
            except (OSError, AttributeError):
                pass
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else os.cpu_count()
    return backend, max(1, int(cores))


def cpu_sample_shape(cores: int):
    """Bounded sample of config 3: two slices per thread at the full
    head size and half the sequence length, so that a pass stays near a second."""
    return dict(seq=2048, head=C3["head"], slices=2*cores)


def run_reference_arm(args):
    backend, cores = cpu_arm_setup()
    smp = cpu_sample_shape(cores)
    W = smp["slices"]*smp["seq"]**2*smp["head"]
    flops = 7.0*W
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_reference_pass(smp["slices"], smp["seq"], smp["head"], cores, backend)
    times = []
    for _ in range(args.steps):
        times.append(cpu_reference_pass(smp["slices"], smp["seq"], smp["head"], cores, backend))
    total = sum(times)
    val = flops*args.steps/total/1e12
    kind = "reference" if backend == "ref" else "port"
    sample = (f"{smp['slices']} independent (batch, head) slices of config 3 at head "
              f"{smp['head']}, seq {smp['seq']} (full config: seq 4096, 128 slices), fp32 "
              f"unfused chain forward+backward, one slice per thread")
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3*total/args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C3 llama-gqa attention fwd+bwd, CPU reference chain, bounded sample",
                   "sample": sample},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": kind,
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------
def rope_(x, base=10000.0):
    """Interleaved-pair RoPE over (H, G, B, S, D) in place (setup only; follows
    wrappers/python/nntile/model/llama_attention.py:1122-1134)."""
    import torch
    H, G, B, S, D = x.shape
    inv = base**(-torch.arange(0, D, 2, device=x.device, dtype=torch.float32)/D)
    ang = torch.arange(S, device=x.device, dtype=torch.float32)[:, None]*inv[None, :]
    cos, sin = ang.cos(), ang.sin()
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    out = torch.empty_like(xf)
    out[..., 0::2] = a*cos - b*sin
    out[..., 1::2] = a*sin + b*cos
    x.copy_(out.to(x.dtype))


def causal_mask_tile(S, kind, device, dtype=None):
    """(Sq, Sk) additive mask tile (bf16 unless `dtype` says otherwise): 'diag' = -inf
    where k > q, 'zero', 'ninf'."""
    import torch
    if dtype is not None and dtype != torch.bfloat16:
        return causal_mask_tile(S, kind, device).to(dtype)
    if kind == "zero":
        return torch.zeros((S, S), dtype=torch.bfloat16, device=device)
    if kind == "ninf":
        return torch.full((S, S), -math.inf, dtype=torch.bfloat16, device=device)
    q = torch.arange(S, device=device)[:, None]
    k = torch.arange(S, device=device)[None, :]
    return torch.where(k > q, torch.tensor(-math.inf, device=device),
                       torch.tensor(0.0, device=device)).to(torch.bfloat16)


class FlashWorkload:
    """Single-sequence-tile fused attention forward+backward through the tile-level
    C entry points (the task the reference's tile layer submits)."""

    def __init__(self, cfg, device, seed, rope=True, dtype=None):
        import torch
        from nntile_b200 import ops
        self.ops, self.torch, self.cfg = ops, torch, cfg
        dt = dtype or torch.bfloat16
        H, G, B, S, D = cfg["kv_heads"], cfg["group"], cfg["batch"], cfg["seq"], cfg["head"]
        g = torch.Generator(device=device).manual_seed(seed)
        shp = (H, G, B, S, D)
        self.q = torch.randn(shp, generator=g, device=device, dtype=torch.float32).to(dt)
        kv = torch.randn((2, H, 1, B, S, D), generator=g, device=device, dtype=torch.float32)
        # K, V ~ N(0,1) per KV head, replicated over the group as the reference does
        self.k = kv[0].expand(H, G, B, S, D).contiguous().to(dt)
        self.v = kv[1].expand(H, G, B, S, D).contiguous().to(dt)
        del kv
        if rope:
            rope_(self.q)
            rope_(self.k)
        self.dy = torch.randn(shp, generator=g, device=device, dtype=torch.float32).to(dt)
        self.mask = causal_mask_tile(S, "diag", device, dt)
        self.nb = H*G*B
        self.S, self.D = S, D
        self.y = torch.zeros(shp, dtype=dt, device=device)
        self.lse = torch.empty((H, G, B, S), dtype=torch.float32, device=device)
        self.dq, self.dk, self.dv = (torch.zeros(shp, dtype=dt, device=device)
                                     for _ in range(3))
        self.s_lse = torch.empty_like(self.lse)
        self.s1, self.s2, self.s3 = (torch.empty(shp, dtype=dt, device=device)
                                     for _ in range(3))
        self.flops_fwd, self.flops_bwd = causal_flops(cfg)

    def forward(self):
        ops = self.ops
        ops.fill(-math.inf, self.lse)
        ops.clear(self.y)
        ops.flash_sdpa_fwd(self.S, self.D, self.nb, self.k, self.q, self.mask, self.s_lse,
                           self.v, self.s1, self.lse, self.y)

    def backward(self):
        self.ops.flash_sdpa_bwd(self.S, self.D, self.nb, self.k, self.q, self.v, self.y,
                                self.dy, self.mask, self.lse, self.s1, self.s2, self.s3,
                                self.dk, self.dq, self.dv)

    def step(self):
        self.forward()
        self.backward()

    def units(self):
        """(kv head, group) pairs: with K/V replicated over the group each is an
        independent attention problem of `batch` slices."""
        return self.q.shape[0]*self.q.shape[1]

    def by_unit(self, t):
        return t.view((t.shape[0]*t.shape[1],) + tuple(t.shape[2:]))

    def step_units(self, lo, hi):
        """forward + backward of units [lo, hi) only (views of the same buffers)."""
        ops = self.ops
        H, G, B = self.q.shape[:3]
        nb = (hi - lo)*B
        v = lambda t: self.by_unit(t)[lo:hi]
        ops.fill(-math.inf, v(self.lse))
        ops.clear(v(self.y))
        ops.flash_sdpa_fwd(self.S, self.D, nb, v(self.k), v(self.q), self.mask, v(self.s_lse),
                           v(self.v), v(self.s1), v(self.lse), v(self.y))
        ops.flash_sdpa_bwd(self.S, self.D, nb, v(self.k), v(self.q), v(self.v), v(self.y),
                           v(self.dy), self.mask, v(self.lse), v(self.s1), v(self.s2), v(self.s3),
                           v(self.dk), v(self.dq), v(self.dv))


def time_steps(torch, fn, steps, warmup, barrier=None, split=None, finish=None):
    """CUDA-event timing of `steps` calls on the current stream.  `split` is an
    optional pair of callables (fwd, bwd) timed separately inside each step;
    `finish` is called after the last step, inside the timed region (a pipeline
    that runs on other streams joins the current one there)."""
    for _ in range(warmup):
        fn()
    if finish:
        finish()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = []
    start.record()
    for _ in range(steps):
        if split:
            a, b, c = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            a.record()
            split[0]()
            b.record()
            split[1]()
            c.record()
            marks.append((a, b, c))
        else:
            fn()
    if finish:
        finish()
    stop.record()
    torch.cuda.synchronize()
    if barrier:
        barrier()
    total_ms = start.elapsed_time(stop)
    fwd_ms = [a.elapsed_time(b) for a, b, _ in marks]
    bwd_ms = [b.elapsed_time(c) for _, b, c in marks]
    return total_ms, fwd_ms, bwd_ms


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from nntile_b200 import _lib, ops

    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback "
                         "(use --impl reference for the CPU arm)")
    ngpu = torch.cuda.device_count()
    oversubscribed = world > ngpu
    local = local % ngpu
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        if oversubscribed:
            # more ranks than GPUs: a functional run only (NCCL wants one GPU per rank);
            # the ranks share devices and talk over gloo, and the line says so
            dist.init_process_group("gloo")
        else:
            dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()
    peaks = measured_peaks()

    def barrier():
        if world > 1:
            dist.barrier()

    if args.workload in ("decode", "decode-small"):
        # decode-only run for profiler captures: config 5, or a quarter of its batch
        c5 = dict(C5) if args.workload == "decode" else dict(C5, batch=16)
        res = run_decode(torch, ops, dev, peaks, c5, max(args.steps, 1), args.warmup)
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload, **res}), flush=True)
        return
    if args.workload == "c2":
        # config 2 only, for profiler captures of the head-64 kernels
        wl = FlashWorkload(C2, dev, seed=1, rope=False)
        ms, _, _ = time_steps(torch, wl.step, max(args.steps, 1), args.warmup)
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": "c2",
                              "ms_per_step": ms/max(args.steps, 1)}), flush=True)
        return
    if args.workload == "hbm":
        # the HBM-bound kernels only (layout changes, unfused chain), for profiler captures
        res = run_hbm_kernels(torch, ops, dev, peaks, max(args.steps, 1))
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": "hbm", **res}), flush=True)
        return
    from nntile_b200.parallel import shard_range
    full_cfg = C3 if args.workload == "c3" else C3_SMALL
    if full_cfg["kv_heads"] % world != 0:
        raise SystemExit(f"{full_cfg['kv_heads']} kv heads do not divide over {world} ranks")
    lo, hi = shard_range(full_cfg["kv_heads"], rank, world)
    cfg = dict(full_cfg, kv_heads=hi - lo)       # this rank's block of (batch, kv head) units
    wl = FlashWorkload(cfg, dev, seed=2 + 100*lo)
    fwd_path = ops.flash_sdpa_path(cfg["seq"], cfg["head"], wl.nb)
    bwd_path = ops.flash_sdpa_path(cfg["seq"], cfg["head"], wl.nb, backward=True)

    for _ in range(args.warmup):
        wl.step()
    torch.cuda.synchronize()
    sampler = ClockSampler(local)
    n0 = lib.nntile_b200_launch_count()   # launches of the timed part only
    total_ms, fwd_ms, bwd_ms = time_steps(torch, wl.step, args.steps, 0, barrier,
                                          split=(wl.forward, wl.backward))
    launches = int(lib.nntile_b200_launch_count() - n0)
    # nvidia-smi samples every 20 ms at best: a timed region shorter than that
    # many samples is followed by identical untimed steps until enough were taken
    extra_steps = 0
    t_end = time.perf_counter() + 2.0
    while not args.profile and sampler.count() < 8 and time.perf_counter() < t_end:
        wl.step()
        torch.cuda.synchronize()
        extra_steps += 1
    clocks = sampler.stop()
    clocks["window"] = (f"timed region of {args.steps} steps plus {extra_steps} identical "
                        f"untimed steps")
    t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    total_ms = float(t.item())
    ms_per_step = total_ms/args.steps
    flops_step = wl.flops_fwd + wl.flops_bwd          # this rank's shard
    flops_job = sum(causal_flops(full_cfg))           # the whole problem
    value = flops_job/(ms_per_step*1e-3)/1e12

    # ---- roofline of the dominant kernel (backward tile task) -----------------
    bwd_med = statistics.median(bwd_ms)
    fwd_med = statistics.median(fwd_ms)
    achieved = wl.flops_bwd/(bwd_med*1e-3)/1e12
    regime, peak = roofline_regime(peaks, total_ms, clocks.get("sm_mhz"))
    kernel_ms = bwd_med*NCU_BWD_KERNEL_SHARE
    fwd_tf = wl.flops_fwd/(fwd_med*1e-3)/1e12
    roofline = {
        "bound": "tensor", "kernel": "flash_sdpa_bwd tile task",
        "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved/peak,
        "regime": regime,
        "regime_rule": "burst peak if the timed region is under 1 s or the sampled median SM "
                       "clock is above the clock the sustained peak was measured at",
        "frac_burst": achieved/peaks["bf16_burst"], "frac_sustained": achieved/peaks["bf16"],
        "peak_burst": peaks["bf16_burst"], "peak_sustained": peaks["bf16"],
        "peak_source": peaks["source"] + " bf16 GEMM (" + regime + ")",
        "timed_region_ms": total_ms,
        "kernel_alone": {"name": "flash_bwd_kernel<128>", "ms": kernel_ms,
                         "achieved": wl.flops_bwd/(kernel_ms*1e-3)/1e12,
                         "frac": wl.flops_bwd/(kernel_ms*1e-3)/1e12/peak,
                         "how": "tile-task time x the kernel's share of it in the ncu launch "
                                "list (profiles/)", "share": NCU_BWD_KERNEL_SHARE},
        "ms_x_mhz": (bwd_med*clocks["sm_mhz"] if clocks.get("sm_mhz") else None),
        "traffic": (NCU_DRAM_BYTES_PER_SLICE["flash_bwd_kernel<128>"]*wl.nb
                    if (cfg["head"], cfg["seq"]) == (128, 4096) and bwd_path == 2 else None),
        "traffic_note": "DRAM bytes per launch of flash_bwd_kernel<128> from a one-pass ncu capture "
                        "of the 128-slice workload, scaled by the slices of this launch (profiles/)",
        "fwd": {"achieved": fwd_tf, "ms": fwd_med, "frac": fwd_tf/peak,
                "frac_burst": fwd_tf/peaks["bf16_burst"], "frac_sustained": fwd_tf/peaks["bf16"]},
        "bwd_ms": bwd_med,
        "step": {"achieved": flops_step/(ms_per_step*1e-3)/1e12,
                 "frac": flops_step/(ms_per_step*1e-3)/1e12/peak},
    }

    if args.profile:
        # profiling run: the kernels above are all a profiler needs to see
        if rank == 0:
            print(json.dumps({"profile_run": True, "workload": args.workload,
                              "ms_per_step": ms_per_step, "fwd_ms": fwd_med, "bwd_ms": bwd_med,
                              "roofline": roofline}), flush=True)
        return
    # ---- e2e: host buffers, copies inside the timed region --------------------
    e2e_steps = max(1, min(args.steps, 8))
    host_in = [x.cpu().pin_memory() for x in (wl.q, wl.k, wl.v, wl.dy)]
    host_out = [torch.empty_like(x, device="cpu").pin_memory()
                for x in (wl.y, wl.dq, wl.dk, wl.dv)]
    dev_in = (wl.q, wl.k, wl.v, wl.dy)
    dev_out = (wl.y, wl.dq, wl.dk, wl.dv)

    from nntile_b200.parallel import HostStream
    pipe = HostStream(dev, wl.units(), chunks=8)
    host_in, host_out = [wl.by_unit(x) for x in host_in], [wl.by_unit(x) for x in host_out]
    dev_in, dev_out = [wl.by_unit(x) for x in dev_in], [wl.by_unit(x) for x in dev_out]

    def e2e_step():
        # copies of one chunk of units overlap the kernels of the previous one, and
        # the copy-in of the next step overlaps the copy-out of this one
        pipe.step(host_in, dev_in, wl.step_units, dev_out, host_out)

    e2e_ms, _, _ = time_steps(torch, e2e_step, e2e_steps, 1, barrier, finish=pipe.join)
    t = torch.tensor([e2e_ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())/e2e_steps
    # bytes of the whole job (every rank copies its shard)
    h2d = world*sum(x.numel()*x.element_size() for x in host_in)
    d2h = world*sum(x.numel()*x.element_size() for x in host_out)
    e2e = {"value": flops_job/(e2e_ms*1e-3)/1e12, "unit": UNIT, "ms_per_step": e2e_ms,
           "steps": e2e_steps, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
    del host_in, host_out
    if world == 1:
        # the same step through the grouped-query entry points: the host holds K, V
        # (and receives dK, dV) per kv head, not replicated over the group
        try:
            e2e["grouped_query_api"] = run_e2e_gqa(torch, ops, dev, cfg, flops_step, e2e_steps)
        except Exception as ex:                      # informational; never breaks the line
            e2e["grouped_query_api"] = {"error": repr(ex)}

    extra, cpu_baseline = None, None
    del wl
    torch.cuda.empty_cache()
    if world > 1:
        extra = run_extras_multi(torch, dist, ops, dev, peaks, args, rank, world)
    if world == 1:
        extra = run_extras(torch, ops, lib, dev, peaks, args)
        backend, cores = cpu_arm_setup()
        smp = cpu_sample_shape(cores)
        secs = cpu_reference_pass(smp["slices"], smp["seq"], smp["head"], cores, backend)
        secs = min(secs, cpu_reference_pass(smp["slices"], smp["seq"], smp["head"], cores,
                                            backend))
        cpu_baseline = {
            "value": 7.0*smp["slices"]*smp["seq"]**2*smp["head"]/secs/1e12, "unit": UNIT,
            "cores": cores, "kind": "reference" if backend == "ref" else "port",
            "sample": (f"{smp['slices']} slices of config 3 at head {smp['head']}, seq "
                       f"{smp['seq']}, fp32 unfused chain fwd+bwd, one slice per thread, "
                       f"best of 2 passes ({secs:.2f} s)")}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {
                "workload": ("C3 llama-gqa attention fwd+bwd (BASELINE configs[2]): 32 q "
                             "heads (8 kv x group 4), head_dim 128, seq 4096, batch 4, "
                             "causal, RoPE pre-applied, seq-tile 4096; the 32 (batch, kv head) "
                             "units dealt over the GPUs") if args.workload == "c3"
                            else "small profiling case of C3 (16 slices)",
                "shape": full_cfg, "per_gpu_shape": cfg, "global_batch": full_cfg["batch"],
                "flop_convention": "causal: fwd 2W, bwd 5W, W=B*Hq*S^2*D",
                "l2": ("inputs_exceed_l2 (Q,K,V,dY,A %d MB each per GPU vs 126 MB L2)"
                       % (cfg["kv_heads"]*cfg["group"]*cfg["batch"]*cfg["seq"]*cfg["head"]*2 >> 20)),
                "parallelism": f"{world} shards of {cfg['kv_heads']*cfg['batch']} (batch, kv head) "
                               "units each, no collective"
                               + (f"; FUNCTIONAL RUN ONLY: {world} ranks share {ngpu} GPU(s)"
                                  if oversubscribed else ""),
                "paths": {"fwd": fwd_path, "bwd": bwd_path,
                          "legend": "2 = tcgen05/TMEM/TMA kernel, 1 = generic CUDA kernel"},
            },
            "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "clocks": clocks, "gpu_launches": launches, "extra": extra,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_extras_multi(torch, dist, ops, dev, peaks, args, rank, world):
    """N > 1: config 5 with its batch split over the ranks (aggregate GB/s over the
    slowest rank's time), and the weak-scaling line (every rank runs all of config 3)."""
    from nntile_b200.parallel import shard_range
    out = {}
    lo, hi = shard_range(C5["batch"], rank, world)
    steps = max(12, min(args.steps*4, 40))
    res = run_decode(torch, ops, dev, peaks, dict(C5, batch=hi - lo), steps, 5,
                     barrier=dist.barrier)
    t = torch.tensor([res["ms_per_step"]], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    nbytes = 2*C5["batch"]*C5["kv_heads"]*C5["max_seq"]*C5["head"]*2 \
        + 2*C5["batch"]*C5["group"]*C5["kv_heads"]*C5["head"]*2
    gbs = nbytes/(ms*1e-3)/1e9
    out["c5_decode"] = {"gbs": gbs, "ms_per_step": ms, "bytes_per_step": nbytes,
                        "frac_of_measured_hbm": gbs/(world*peaks["hbm"]),
                        "peak_gbs": world*peaks["hbm"], "peak_source": peaks["source"],
                        "shape": C5, "per_gpu_batch": hi - lo, "scaling": "strong",
                        "note": "split-KV decode, batch split over the ranks, no collective; "
                                "aggregate bytes over the slowest rank's time"}
    wl = FlashWorkload(C3, dev, seed=2 + rank)
    wsteps = max(3, min(args.steps, 10))
    ms, _, _ = time_steps(torch, wl.step, wsteps, 3, dist.barrier)
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())/wsteps
    out["weak_scaling"] = {"tflops": world*(wl.flops_fwd + wl.flops_bwd)/(ms*1e-3)/1e12,
                           "ms_per_step": ms, "global_batch": C3["batch"]*world,
                           "note": "every rank runs all of config 3 on its own seed"}
    del wl
    return out


def run_c2(torch, dev, steps):
    """Config 2: GPT-2-small attention, seq-tile 1024, head-tile 12, batch-tile 8 - one
    tile task per pass, 33 us of tensor work: launch-bound when every call comes from
    Python, so the step is also captured once in a CUDA graph and replayed."""
    wl = FlashWorkload(C2, dev, seed=1, rope=False)
    flops = wl.flops_fwd + wl.flops_bwd
    ms, _, _ = time_steps(torch, wl.step, steps*4, 3)
    ms /= steps*4
    res = {"tflops": flops/(ms*1e-3)/1e12, "ms_per_step": ms, "shape": C2,
           "note": "one tile task per pass (batch tile 8, head tile 12); working set 63 MB "
                   "fits L2; calls issued one by one from Python"}
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(3):
                wl.step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            wl.step()
        reps = 200
        gms, _, _ = time_steps(torch, graph.replay, reps, 5)
        gms /= reps
        res["cuda_graph"] = {"tflops": flops/(gms*1e-3)/1e12, "ms_per_step": gms, "replays": reps,
                             "note": "the same step (8 launches) captured once, replayed"}
    except Exception as exc:                     # informational; never breaks the line
        res["cuda_graph"] = {"error": repr(exc)[:200]}
    del wl
    return res


def run_hbm_kernels(torch, ops, dev, peaks, steps):
    """The HBM-bound kernels next to the fused pair, each timed alone on tensors far
    larger than L2: the layout-change kernels around the SDPA layer at config 3's
    shapes, and the unfused chain's kernels at config 1's per-head shapes scaled up to
    2 GiB of logits.  GB/s = algorithmic bytes (one read + one write of the tensor,
    plus the small operands) over the CUDA-event time."""
    out = {}
    hbm = peaks["hbm"]

    def timed(fn, nbytes, reps=10):
        ms, _, _ = time_steps(torch, fn, reps, 3)
        ms /= reps
        gbs = nbytes/(ms*1e-3)/1e9
        return {"gbs": gbs, "ms": ms, "bytes": nbytes, "frac_of_measured_hbm": gbs/hbm}

    g = torch.Generator(device=dev).manual_seed(5)
    # ---- layout changes: config 3's Q (32 heads) and K (8 kv heads)
    D, S, B = C3["head"], C3["seq"], C3["batch"]
    for name, lead in (("q_32_heads", C3["group"]*C3["kv_heads"]), ("k_8_kv_heads", C3["kv_heads"])):
        src = torch.randn((B, S, D, lead), generator=g, device=dev).to(torch.bfloat16)
        dst = torch.empty((lead, B, S, D), dtype=torch.bfloat16, device=dev)
        sc = torch.randn((B, S, D//2), generator=g, device=dev).to(torch.bfloat16)
        nb = src.numel()*2
        out[f"transpose_rope_{name}"] = timed(
            lambda: ops.transpose_rope(lead, D, S, B, sc, sc, src, dst), 2*nb + 2*sc.numel()*2)
        out[f"transpose_heads_back_{name}"] = timed(
            lambda: ops.transpose_heads_back(lead, D, S, B, dst, src), 2*nb)
        del src, dst, sc
    # ---- unfused chain: logits [Sk, Sq, batch] in bf16 and fp32
    Sk = Sq = 2048
    for dt, tag in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
        nbatch = 128 if dt == torch.bfloat16 else 64
        es = 2 if dt == torch.bfloat16 else 4
        logits = torch.randn((nbatch, Sq, Sk), generator=g, device=dev).to(dt)
        nb = logits.numel()*es
        mse = torch.zeros((nbatch, Sq, 2), dtype=dt, device=dev)
        mask = torch.ones((Sq, Sk), dtype=torch.bool, device=dev).tril()
        sl = torch.zeros((nbatch, Sq), dtype=dt, device=dev)
        other = torch.randn((nbatch, Sq, Sk), generator=g, device=dev).to(dt)
        out[f"mask_scalar_{tag}"] = timed(
            lambda: ops.mask_scalar(Sk*Sq, nbatch, mask, -math.inf, logits), nb//2)
        out[f"maxsumexp_{tag}"] = timed(
            lambda: ops.maxsumexp(1, Sq*nbatch, Sk, logits, mse), nb)
        out[f"softmax_inplace_{tag}"] = timed(
            lambda: ops.softmax_inplace(1, Sq*nbatch, Sk, mse, 1.0, logits), 2*nb)
        out[f"add_slice_inplace_{tag}"] = timed(
            lambda: ops.add_slice_inplace(1, Sq*nbatch, Sk, -1.0, sl, 1.0, logits), 2*nb)
        out[f"multiply_inplace_{tag}"] = timed(
            lambda: ops.multiply_inplace(logits.numel(), 1.0, other, logits), 3*nb)
        out[f"sumprod_slice_{tag}"] = timed(
            lambda: ops.sumprod_slice(1, Sq*nbatch, Sk, 1.0, logits, other, 0.0, sl), 2*nb)
        del logits, other, mse, sl
    # a write-only kernel cannot reach the copy figure (reads + writes): a plain fill of
    # 1 GiB (torch's zero_) is the yardstick for mask_scalar, which only writes
    big = torch.empty(1 << 30, dtype=torch.uint8, device=dev)
    fill = timed(lambda: big.zero_(), 1 << 30)
    del big
    out["fill_1gib_torch_zero"] = fill
    for tag in ("bf16", "fp32"):
        out[f"mask_scalar_{tag}"]["frac_of_fill"] = out[f"mask_scalar_{tag}"]["gbs"]/fill["gbs"]
    out["note"] = ("mask_scalar writes only the masked half (causal) and reads nothing but the mask: "
                   "its yardstick is the write-only rate (fill_1gib_torch_zero), not the copy bandwidth; "
                   "bytes are algorithmic, peak = measured copy bandwidth")
    return out


def run_extras(torch, ops, lib, dev, peaks, args):
    """Configs 2, 4 and 5 and the kernels beside the fused pair at N=1 (few steps each)."""
    out = {}
    steps = max(3, min(args.steps, 10))
    out["c2_gpt2_small_attention"] = run_c2(torch, dev, steps)
    # ---- config 4: long context, seq-tile 2048, K/V tiles streamed through tasks
    out["c4_long_context"] = run_c4(torch, ops, lib, dev, steps)
    # ---- config 3 through the grouped-query entry points (K, V not replicated)
    out["c3_native_gqa"] = run_c3_gqa(torch, ops, dev, steps)
    # ---- config 3 in IEEE half: the fp16 build of the same kernels
    wl = FlashWorkload(C3, dev, seed=2, dtype=torch.float16)
    ms, _, _ = time_steps(torch, wl.step, steps, 3)
    ms /= steps
    out["c3_fp16"] = {"tflops": (wl.flops_fwd + wl.flops_bwd)/(ms*1e-3)/1e12, "ms_per_step": ms,
                      "note": "config 3 with fp16 storage through nntile_b200_flash_sdpa_{fwd,bwd}_fp16"}
    del wl
    # ---- config 5: decode, HBM-bound
    out["c5_decode"] = run_decode(torch, ops, dev, peaks, C5, steps*4, 5)
    try:
        out["hbm_bound_kernels"] = run_hbm_kernels(torch, ops, dev, peaks, steps)
    except Exception as exc:                     # informational; never breaks the line
        out["hbm_bound_kernels"] = {"error": repr(exc)[:200]}
    torch.cuda.empty_cache()
    # ---- comparators (context only, not the product): the reference's own GPU wrappers
    # of the fused pair (cuDNN graph with the mask as bias + merge / add_inplace
    # kernels), compiled in place as oracle/_ref_gpu; and cuDNN through torch
    out["reference_gpu_wrappers_c3"] = run_reference_gpu(torch, dev)
    out["cudnn_comparator_c3"] = run_cudnn_comparator(torch, dev)
    return out


def run_reference_gpu(torch, dev):
    """Config 3's tile task through the reference's src/kernel/flash_sdpa_{fwd,bwd}_cudnn
    wrappers (test infrastructure, never on the product path)."""
    import ctypes
    try:
        import oracle as O
        ref = O.ref_gpu()
        if ref is None:
            return {"unavailable": "oracle/_ref_gpu not built"}
        S, D, nb = C3["seq"], C3["head"], C3["batch"]*C3["group"]*C3["kv_heads"]
        g = torch.Generator(device=dev).manual_seed(9)
        mk = lambda: torch.randn((nb, S, D), generator=g, device=dev).to(torch.bfloat16)
        q, k, v, dy = mk(), mk(), mk(), mk()
        mask = causal_mask_tile(S, "diag", dev)
        lse = torch.empty((nb, S), dtype=torch.float32, device=dev)
        A = torch.zeros_like(q)
        s_l, s1, s2, s3 = torch.empty_like(lse), torch.empty_like(q), torch.empty_like(q), \
            torch.empty_like(q)
        dK, dQ, dV = (torch.zeros_like(q) for _ in range(3))
        p = lambda t: ctypes.c_void_p(t.data_ptr())
        side = torch.cuda.Stream()          # the wrappers refuse the null stream
        sp = ctypes.c_void_p(side.cuda_stream)
        status = []

        def step():
            lse.fill_(-math.inf)
            A.zero_()
            status.append(ref.refgpu_flash_sdpa_fwd_bf16(sp, S, D, nb, p(k), p(q), p(mask), p(s_l),
                                                         p(v), p(s1), p(lse), p(A)))
            status.append(ref.refgpu_flash_sdpa_bwd_bf16(sp, S, D, nb, p(k), p(q), p(v), p(A), p(dy),
                                                         p(mask), p(lse), p(s1), p(s2), p(s3),
                                                         p(dK), p(dQ), p(dV)))

        with torch.cuda.stream(side):
            step()
            side.synchronize()
            if any(status):
                return {"unavailable": f"reference wrapper status {status}"}
            ms, _, _ = time_steps(torch, step, 5, 2)
        ms /= 5
        f, b = causal_flops(C3)
        return {"ms_per_step": ms, "tflops": (f + b)/(ms*1e-3)/1e12,
                "note": "the reference's own GPU path for one config-3 tile task (cuDNN bias-form "
                        "graph into scratch, merge kernel, three add_inplace passes); "
                        "causal-convention FLOPs although it executes all S^2"}
    except Exception as exc:
        return {"unavailable": repr(exc)[:200]}


def run_e2e_gqa(torch, ops, dev, cfg, flops_step, steps):
    """End-to-end step with pinned host buffers through the grouped-query entry
    points, copies overlapped with kernels by HostStream (chunks of one kv head)."""
    from nntile_b200.parallel import HostStream
    H, G, B, S, D = cfg["kv_heads"], cfg["group"], cfg["batch"], cfg["seq"], cfg["head"]
    g = torch.Generator(device=dev).manual_seed(11)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)
    q, dy, k, v = rnd(H, G, B, S, D), rnd(H, G, B, S, D), rnd(H, B, S, D), rnd(H, B, S, D)
    y, dq = torch.zeros_like(q), torch.zeros_like(q)
    dk, dv = torch.zeros_like(k), torch.zeros_like(k)
    lse = torch.empty((H, G, B, S), dtype=torch.float32, device=dev)
    mask = causal_mask_tile(S, "diag", dev)
    scratch = torch.empty(ops.flash_sdpa_gqa_scratch_bytes(S, D, B, G, 1), dtype=torch.uint8,
                          device=dev)

    def body(lo, hi):
        n = hi - lo
        ops.fill(-math.inf, lse[lo:hi])
        ops.clear(y[lo:hi])
        ops.flash_sdpa_fwd_gqa(S, D, B, G, n, k[lo:hi], q[lo:hi], mask, v[lo:hi], lse[lo:hi],
                               y[lo:hi], scratch)
        ops.flash_sdpa_bwd_gqa(S, D, B, G, n, k[lo:hi], q[lo:hi], v[lo:hi], y[lo:hi], dy[lo:hi],
                               mask, lse[lo:hi], dk[lo:hi], dq[lo:hi], dv[lo:hi], scratch)

    host_in = [x.cpu().pin_memory() for x in (q, k, v, dy)]
    host_out = [torch.empty_like(x, device="cpu").pin_memory() for x in (y, dq, dk, dv)]
    pipe = HostStream(dev, H, chunks=H)
    step = lambda: pipe.step(host_in, (q, k, v, dy), body, (y, dq, dk, dv), host_out)
    ms, _, _ = time_steps(torch, step, steps, 1, finish=pipe.join)
    ms /= steps
    return {"value": flops_step/(ms*1e-3)/1e12, "unit": UNIT, "ms_per_step": ms,
            "h2d_bytes_per_step": sum(x.numel()*x.element_size() for x in host_in),
            "d2h_bytes_per_step": sum(x.numel()*x.element_size() for x in host_out),
            "note": "K, V, dK, dV [head, seq, batch, kv_heads]: a quarter of the K/V bytes "
                    "cross PCIe; same FLOPs as the headline"}


def run_c3_gqa(torch, ops, dev, steps):
    """Config 3 with K, V, dK, dV of shape [head, seq, batch, kv_heads]: the same tile
    task without the reference layer's K/V replication and gradient reduction."""
    cfg = C3
    H, G, B, S, D = cfg["kv_heads"], cfg["group"], cfg["batch"], cfg["seq"], cfg["head"]
    g = torch.Generator(device=dev).manual_seed(7)
    rnd = lambda *shape: torch.randn(shape, generator=g, device=dev).to(torch.bfloat16)
    q, dy = rnd(H, G, B, S, D), rnd(H, G, B, S, D)
    k, v = rnd(H, B, S, D), rnd(H, B, S, D)
    rope_(q)
    rope_(k.view(H, 1, B, S, D))
    mask = causal_mask_tile(S, "diag", dev)
    y, dq = torch.zeros_like(q), torch.zeros_like(q)
    dk, dv = torch.zeros_like(k), torch.zeros_like(k)
    lse = torch.empty((H, G, B, S), dtype=torch.float32, device=dev)
    scratch = torch.empty(ops.flash_sdpa_gqa_scratch_bytes(S, D, B, G, H), dtype=torch.uint8,
                          device=dev)

    def step():
        ops.fill(-math.inf, lse)
        ops.clear(y)
        ops.flash_sdpa_fwd_gqa(S, D, B, G, H, k, q, mask, v, lse, y, scratch)
        ops.flash_sdpa_bwd_gqa(S, D, B, G, H, k, q, v, y, dy, mask, lse, dk, dq, dv, scratch)

    ms, _, _ = time_steps(torch, step, steps, 3)
    ms /= steps
    f, b = causal_flops(cfg)
    return {"tflops": (f + b)/(ms*1e-3)/1e12, "ms_per_step": ms,
            "note": "K, V, dK, dV [head, seq, batch, kv_heads]; same FLOPs as the headline"}


def run_cudnn_comparator(torch, dev):
    """cuDNN fused attention through torch (the Blackwell kernel the reference's
    flash_sdpa_{fwd,bwd}_cudnn wrappers reach), config 3 shape, same FLOP convention.
    'bias' is the reference's call pattern (mask as additive bias, causal flag off,
    src/kernel/flash_sdpa_fwd_cudnn/cuda.cc:103-110) without its scratch copy, merge
    and add_inplace passes; 'causal_flag' is cuDNN's own best case."""
    import torch.nn.functional as F
    try:
        from torch.nn.attention import SDPBackend, sdpa_kernel
        B, H, S, D = C3["batch"], C3["group"]*C3["kv_heads"], C3["seq"], C3["head"]
        g = torch.Generator(device=dev).manual_seed(9)
        q, k, v = (torch.randn((B, H, S, D), generator=g, device=dev).to(torch.bfloat16)
                   .requires_grad_(True) for _ in range(3))
        do = torch.randn((B, H, S, D), generator=g, device=dev).to(torch.bfloat16)
        bias = causal_mask_tile(S, "diag", dev).view(1, 1, S, S)
        W = B*H*S*S*D
        res = {}
        for name, kw in (("bias", dict(attn_mask=bias)), ("causal_flag", dict(is_causal=True))):
            with sdpa_kernel(SDPBackend.CUDNN_ATTENTION):
                def step():
                    o = F.scaled_dot_product_attention(q, k, v, **kw)
                    o.backward(do)
                ms, _, _ = time_steps(torch, step, 5, 3)
            ms /= 5
            res[name] = {"ms_per_step": ms, "tflops": 7.0*W/(ms*1e-3)/1e12}
        res["note"] = "library comparator; causal-convention FLOPs (the bias form executes all S^2)"
        return res
    except Exception as exc:          # comparator only: never fail the benchmark
        return {"unavailable": repr(exc)[:200]}


def run_decode(torch, ops, dev, peaks, c5, steps, warmup, barrier=None):
    """One new token against the KV cache of config 5 (or a smaller batch of it)."""
    from nntile_b200.sdpa import decode_sdpa
    D, L, B, G, H = c5["head"], c5["max_seq"], c5["batch"], c5["group"], c5["kv_heads"]
    g = torch.Generator(device=dev).manual_seed(4)
    q = torch.randn((H, G, B, 1, D), generator=g, device=dev).to(torch.bfloat16)
    Kc = torch.randn((H, B, L, D), generator=g, device=dev).to(torch.bfloat16)
    Vc = torch.randn((H, B, L, D), generator=g, device=dev).to(torch.bfloat16)
    o = torch.empty_like(q)
    ws = torch.empty(ops.decode_workspace_bytes(D, L, B, G, H), dtype=torch.uint8, device=dev)
    fn = lambda: decode_sdpa(q, Kc, Vc, L, out=o, workspace=ws)
    ms, _, _ = time_steps(torch, fn, steps, warmup, barrier)
    ms /= steps
    nbytes = 2*B*H*L*D*2 + 2*B*G*H*D*2
    gbs = nbytes/(ms*1e-3)/1e9
    return {"gbs": gbs, "ms_per_step": ms, "bytes_per_step": nbytes,
            "frac_of_measured_hbm": gbs/peaks["hbm"], "peak_gbs": peaks["hbm"],
            "peak_source": peaks["source"], "shape": c5,
            "note": "K+V caches read once for all query heads of a group; far above L2"}


def run_c4(torch, ops, lib, dev, steps):
    """Config 4 through the tensor-level C entry points: 8 x 8 (Q tile, K/V tile)
    tasks per pass, every pair submitted as the reference does; the mask tiles are
    one of three buffers (zero / -inf / diagonal)."""
    import ctypes
    H, S, D, St = C4["kv_heads"], C4["seq"], C4["head"], C4["seq_tile"]
    nt = S//St
    g = torch.Generator(device=dev).manual_seed(3)

    def tiles(n, fill=None):
        if fill is None:
            return [torch.randn((H, 1, 1, St, D), generator=g, device=dev).to(torch.bfloat16)
                    for _ in range(n)]
        return [torch.full((H, 1, 1, St, D), fill, dtype=torch.bfloat16, device=dev)
                for _ in range(n)]

    Q, K, V, dY = tiles(nt), tiles(nt), tiles(nt), tiles(nt)
    A, dQ, dK, dV = tiles(nt, 0.0), tiles(nt, 0.0), tiles(nt, 0.0), tiles(nt, 0.0)
    lse = [torch.empty((H, 1, 1, St), dtype=torch.float32, device=dev) for _ in range(nt)]
    mz, mi, md = (causal_mask_tile(St, k, dev) for k in ("zero", "ninf", "diag"))
    masks = []
    for qi in range(nt):            # tile (k, q) stored at k + q*nt
        for ki in range(nt):
            masks.append(mz if ki < qi else md if ki == qi else mi)

    def parr(ts):
        return ctypes.cast((ctypes.c_void_p*len(ts))(*[t.data_ptr() for t in ts]),
                           ctypes.POINTER(ctypes.c_void_p))

    i64 = ctypes.c_int64
    shape = (i64*5)(D, S, 1, 1, H)
    base = (i64*5)(D, St, 1, 1, H)
    nbytes = lib.nntile_b200_tensor_flash_sdpa_scratch_bytes(shape, base)
    scratch = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    pk = {n: parr(t) for n, t in dict(Q=Q, K=K, V=V, dY=dY, A=A, dQ=dQ, dK=dK, dV=dV, lse=lse,
                                      m=masks).items()}
    # the same mask with the fully masked pairs marked by NULL: no task for them
    mask_ptrs = [0 if ki > qi else (mz if ki < qi else md).data_ptr()
                 for qi in range(nt) for ki in range(nt)]
    pk["m_skip"] = ctypes.cast((ctypes.c_void_p*len(mask_ptrs))(*mask_ptrs),
                               ctypes.POINTER(ctypes.c_void_p))
    stream = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def make_step(mk):
        def step():
            for t in lse:
                ops.fill(-math.inf, t)
            for t in A:
                ops.clear(t)
            st = lib.nntile_b200_tensor_flash_sdpa_fwd_bf16(
                stream(), shape, base, pk["K"], pk["Q"], pk[mk], pk["lse"], pk["V"], pk["A"],
                ctypes.c_void_p(scratch.data_ptr()), nbytes)
            assert st == 0, st
            st = lib.nntile_b200_tensor_flash_sdpa_bwd_bf16(
                stream(), shape, base, pk["K"], pk["Q"], pk["V"], pk["A"], pk["dY"], pk[mk],
                pk["lse"], pk["dK"], pk["dQ"], pk["dV"], ctypes.c_void_p(scratch.data_ptr()),
                nbytes)
            assert st == 0, st
        return step

    f, b = causal_flops(dict(batch=1, group=1, kv_heads=H, seq=S, head=D))
    ms, _, _ = time_steps(torch, make_step("m"), steps, 2)
    ms /= steps
    ms2, _, _ = time_steps(torch, make_step("m_skip"), steps, 2)
    ms2 /= steps
    return {"tflops": (f + b)/(ms*1e-3)/1e12, "ms_per_step": ms, "shape": C4,
            "tasks_per_pass": nt*nt,
            "note": "all 64 tile pairs submitted per pass (28 fully masked), causal-convention flops",
            "masked_pairs_skipped": {"tflops": (f + b)/(ms2*1e-3)/1e12, "ms_per_step": ms2,
                                     "tasks_per_pass": nt*(nt + 1)//2,
                                     "note": "NULL mask entries for the 28 fully masked pairs"}}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--workload", choices=["c3", "small", "decode", "decode-small", "c2", "hbm"],
                    default="c3",
                    help="c3 = BASELINE config 3 (the headline); the others are profiler-capture "
                         "runs: small = the same kernels on 16 slices, decode / decode-small = "
                         "config 5 (a quarter of its batch), c2 = config 2 (head 64), hbm = the "
                         "HBM-bound kernels around the fused pair")
    ap.add_argument("--profile", action="store_true",
                    help="run only the timed forward/backward steps (no e2e, extras or CPU "
                         "baseline) and print a short line; for use under a profiler")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["b200", "reference"], default="b200")
    args = ap.parse_args(argv)
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup
    if args.impl == "reference":
        if int(os.environ.get("RANK", "0")) != 0:
            return 0                 # rank 0 alone runs the CPU arm
        run_reference_arm(args)
        return 0
    run_gpu_arm(args)
    return 0


if __name__ == "__main__":
    sys.exit(main())
