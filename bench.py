#!/usr/bin/env python
"""Benchmark of the block-local grid update on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (the headline configuration): 64x64x64 grid, block size 8, 4 inner x 12 outer
iterations, batch 64 per GPU, float32, forward only, LayerNorm over the whole grid
after every outer step. Inputs are synthetic: N(0,1) on the [..., 0] face, weights
N(0, 1/27), bias 0, residual scale 1, gamma 1, beta 0, silu (seeded).

One "step" is one full forward of one batch (all 12 outer steps). Metric:
neuron-updates/s = batch * grid^3 * inner * outer / seconds, whole job over all GPUs
(batch sharding: every rank runs its own batch, no collective on the data path).

The JSON line also carries
  roofline      the dominant kernel (fused step) timed alone with CUDA events: its binding
                bound at the top level (algorithmic FP32 FMA rate against the FP32 pipe rate
                measured with an FFMA-only kernel in the same run), the HBM bound nested;
  e2e           the same metric through the public op with pinned HOST buffers, copies
                inside the timed region;
  cpu_baseline  the CPU oracle (C restatement of the reference's backend_torch, OpenMP)
                on the same full batch (N = 1 only);
  c1, c3, c4    (N = 1) sub-records of the other single-GPU configurations;
  c5_slab       (every N) the 256^3 grid slab-sharded along K over the N ranks (strong scaling),
                preceded for N > 1 by a parity check of both face-exchange paths on the real ranks.
`--workload X` runs one of them alone and prints its record as the line.
`--impl reference` times that CPU oracle alone on all host threads.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GRID = (64, 64, 64)
BLOCK = 8
INNER = 4
OUTER = 12
BATCH = 64
ACT = "silu"
WORKLOAD = "C2: 64^3 grid, block 8, 4 inner x 12 outer, batch 64/GPU, fp32, forward + whole-grid LayerNorm per outer step"
METRIC = "neuron_updates_per_sec"
UNIT = "neuron-updates/s"

# FP32 pipe: 148 SMs x 128 FMA lanes x 2 FLOP at the maximum SM clock
FP32_LANES = 148 * 128
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per launch of the dominant kernel (dram__bytes_read.sum + dram__bytes_write.sum): a constant taken
# from the ncu capture summarised in the named file, not a measurement of this run
NCU_TRAFFIC = {
    "step_fwd_pair64": (143.8e6, "profiles/step_fwd_pair64_c2_ncu_full.txt"),
    "step_fwd_fast8": (173.0e6, "profiles/step_fwd_fast8_c2_ncu_full.txt"),
}


def neuron_updates(batch: int) -> float:
    return float(batch) * GRID[0] * GRID[1] * GRID[2] * INNER * OUTER


def algorithmic_bytes_per_launch(batch: int) -> float:
    # one outer step: 31 parameter floats per neuron read once (27 w + bias + scale + gamma +
    # beta), activations read once and written once
    P = GRID[0] * GRID[1] * GRID[2]
    return 124.0 * P + 8.0 * batch * P


def algorithmic_fma_per_launch(batch: int) -> float:
    P = GRID[0] * GRID[1] * GRID[2]
    return 27.0 * P * batch * INNER


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured", float(d.get("sm_max_mhz", 1965.0))
    except Exception:
        return FALLBACK_HBM_GBS, "fallback", 1965.0


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                smax.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {
            "sm_mhz": statistics.median(sm) if sm else None,
            "sm_max_mhz": max(smax) if smax else None,
            "reasons": sorted(reasons),
            "samples": len(sm),
        }


def make_inputs(torch, device, nsets: int):
    g = torch.Generator().manual_seed(0)
    M, N, K = GRID
    w = (torch.randn(27, M, N, K, generator=g) / 27 ** 0.5).to(device)
    b = torch.zeros(M, N, K, device=device)
    s = torch.ones(M, N, K, device=device)
    gamma = torch.ones(M, N, K, device=device)
    beta = torch.zeros(M, N, K, device=device)
    xs = []
    for _ in range(nsets):
        x = torch.zeros(BATCH, M, N, K)
        x[..., 0] = torch.randn(BATCH, M, N, generator=g)
        xs.append(x)
    return w, b, s, gamma, beta, xs


def cpu_inputs(batch: int):
    import numpy as np

    r = np.random.default_rng(0)
    M, N, K = GRID
    w = (r.standard_normal((27, M, N, K)) / np.sqrt(27)).astype(np.float32)
    b = np.zeros(GRID, np.float32)
    s = np.ones(GRID, np.float32)
    x = np.zeros((batch, M, N, K), np.float32)
    x[..., 0] = r.standard_normal((batch, M, N))
    return w, b, s, x


def cpu_oracle_pass(inputs) -> float:
    """Seconds for one full forward (12 outer x 4 inner + LayerNorm) of the CPU oracle."""
    from oracle import gridnet_oracle as orc

    w, b, s, x = inputs
    t0 = time.perf_counter()
    orc.outer_forward(w, b, s, s, b, x, INNER, OUTER, BLOCK, normalize=False, activation=ACT)
    return time.perf_counter() - t0


def run_reference(args, rank: int):
    """The reference arm: the CPU oracle on all host threads, on the same full batch as the GPU arm."""
    if rank != 0:
        return
    from oracle import gridnet_oracle as orc

    orc.set_threads(len(os.sched_getaffinity(0)))
    threads = orc.max_threads()
    inputs = cpu_inputs(BATCH)
    for _ in range(args.warmup):
        cpu_oracle_pass(inputs)
    dt = 0.0
    for _ in range(args.steps):
        dt += cpu_oracle_pass(inputs)
    value = neuron_updates(BATCH) * args.steps / dt
    sample = f"{BATCH} of {BATCH} samples per step, full 12 outer x 4 inner loop incl. LayerNorm"
    line = {
        "impl": "reference",
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": 0, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": BATCH,
                   "implementation": "CPU oracle (C restatement of gridnet/backend_torch.py, OpenMP)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


class Ctx:
    """What every part of a GPU run shares: rank layout, device, the process group (None at one rank)."""

    def __init__(self, args, rank, local_rank, world):
        import torch

        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
        self.args, self.rank, self.local_rank, self.world = args, rank, local_rank, world
        torch.cuda.set_device(local_rank)
        self.device = torch.device("cuda", local_rank)
        self.dist = None
        self.affinity = self._pin_cores()

    def _pin_cores(self):
        """With several ranks on one host, give each its own share of the cores this job may use, so that the
        threads that feed a GPU (and the pages of its pinned buffers, first touched by them) stay put. No GPU or
        driver setting is involved."""
        if self.world <= 1:
            return None
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = len(cores) // self.world
            if per < 1:
                return None
            mine = cores[self.local_rank * per:(self.local_rank + 1) * per]
            os.sched_setaffinity(0, mine)
            return f"{len(mine)} of {len(cores)} cores: {mine[0]}-{mine[-1]}"
        except (AttributeError, OSError):
            return None

    def need_group(self):
        """A process group, also at one rank (the slab driver issues collectives either way)."""
        import torch.distributed as dist

        if self.dist is None:
            if self.world == 1:
                os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
                os.environ.setdefault("MASTER_PORT", "29533")
                dist.init_process_group("nccl", rank=0, world_size=1, device_id=self.device)
            else:
                dist.init_process_group("nccl", device_id=self.device)
            self.dist = dist
        return self.dist

    def barrier(self):
        import torch

        if self.dist is not None:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, ms: float) -> float:
        import torch

        if self.dist is None or self.world == 1:
            return ms
        t = torch.tensor([ms], device=self.device)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def release(self):
        import gc

        import torch

        gc.collect()
        torch.cuda.empty_cache()

    def close(self):
        if self.dist is not None:
            self.dist.destroy_process_group()
            self.dist = None


def measure_fp32_peak(torch, device):
    """TFLOP/s of an FFMA-only kernel that fills every SM (CUDA events, best of 5 launches of a few ms)."""
    import ctypes

    from gridnet_b200._lib import check, lib

    sink = torch.zeros(1, device=device)
    count = ctypes.c_longlong(0)
    st = torch.cuda.current_stream().cuda_stream
    iters = 1 << 15
    check(lib.gn_probe_fp32_fma(sink.data_ptr(), iters, ctypes.byref(count), st))
    torch.cuda.synchronize()
    best = None
    for _ in range(5):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        check(lib.gn_probe_fp32_fma(sink.data_ptr(), iters, ctypes.byref(count), st))
        e1.record()
        torch.cuda.synchronize()
        ms = e0.elapsed_time(e1)
        best = ms if best is None else min(best, ms)
    return 2.0 * count.value / (best * 1e-3) / 1e12


def bench_c2(ctx: Ctx):
    import torch

    import gridnet_b200 as gb
    from gridnet_b200._lib import lib

    args, rank, world, device = ctx.args, ctx.rank, ctx.world, ctx.device
    if world > 1:
        ctx.need_group()
    NSETS = 4  # rotating input/output sets: 4 x 67 MB in + the 300 MB working set >> 126 MB L2
    w, b, s, gamma, beta, xs_host = make_inputs(torch, device, NSETS)
    xs = [x.to(device) for x in xs_host]
    ys = [torch.empty_like(x) for x in xs]
    ws = gb.outer_forward_workspace(BATCH, GRID, BLOCK, device)
    large_batch = bool(lib.gn_pair64_supported(GRID[0], GRID[1], GRID[2], BLOCK, INNER))

    def step(i):
        gb.outer_forward(w, b, s, gamma, beta, xs[i % NSETS], INNER, OUTER, BLOCK, ACT, out=ys[i % NSETS],
                         workspace=ws)

    # ---------------- device-resident timing (value)
    for i in range(max(args.warmup, 3)):
        step(i)
    ctx.barrier()
    sampler = ClockSampler(ctx.local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    ctx.barrier()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    # per outer step: step kernel + statistics finalize; plus, once per forward, the layout conversion in and out
    # (and the weight re-ordering) of the large-batch kernel, or the final normalisation of the register-patch one
    launches_per_step = OUTER * 2 + (3 if large_batch else 1)
    value = neuron_updates(BATCH) * world * args.steps / (ms * 1e-3)
    failed = gb.outer_forward_failed(ws, BATCH, GRID, BLOCK)

    # ---------------- the dominant kernel alone (roofline)
    nparts = int(lib.gn_pair64_stats_partials(*GRID)) if large_batch else gb.step_stats_partials(GRID, BLOCK)
    partials = torch.empty(BATCH, nparts, 2, dtype=torch.float64, device=device)
    stats = torch.empty(BATCH, 2, device=device)
    # any finite statistics do for timing: mean 0, rstd 1
    stats[:, 0] = 0.0
    stats[:, 1] = 1.0
    reps = max(args.steps, 3) * OUTER
    if large_batch:
        from gridnet_b200.backend_cuda import pair64_interleave, pair64_pack_weights, pair64_step

        kernel_name = "step_fwd_pair64<silu, fuse_in, stats_out>"
        packed = pair64_pack_weights(w, b, s, gamma, beta)
        xi = [pair64_interleave(x) for x in xs]
        yi = [torch.empty_like(x) for x in xi]
        flag = torch.zeros(1, dtype=torch.int32, device=device)

        def kernel(i):
            pair64_step(packed, xi[i % NSETS], yi[(i + 1) % NSETS], BATCH, GRID, INNER, ACT, stats, partials, flag)
    else:
        kernel_name = "step_fwd_fast8<silu, fuse_in, stats_out>"

        def kernel(i):
            gb.fused_step(w, b, s, xs[i % NSETS], ys[(i + 1) % NSETS], INNER, BLOCK, ACT, gamma, beta, stats, partials)

    for i in range(6):
        kernel(i)
    torch.cuda.synchronize()
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for i in range(reps):
        kernel(i)
    k1.record()
    torch.cuda.synchronize()
    kms = k0.elapsed_time(k1) / reps
    if large_batch:
        del xi, yi, packed
    fp32_measured = measure_fp32_peak(torch, device)
    hbm_peak, peak_kind, sm_max_mhz = measured_peaks()
    ach_gbs = algorithmic_bytes_per_launch(BATCH) / (kms * 1e-3) / 1e9
    fp32_nominal = FP32_LANES * 2 * sm_max_mhz * 1e6 / 1e12
    ach_tflops = 2 * algorithmic_fma_per_launch(BATCH) / (kms * 1e-3) / 1e12
    traffic, traffic_src = NCU_TRAFFIC["step_fwd_pair64" if large_batch else "step_fwd_fast8"]
    fp32 = {"bound": "fp32", "achieved": ach_tflops, "peak": fp32_measured, "unit": "TFLOP/s",
            "frac": ach_tflops / fp32_measured,
            "peak_source": "measured in this run: FFMA-only kernel on every SM, CUDA events (gn_probe_fp32_fma)",
            "peak_nominal": fp32_nominal, "frac_of_nominal": ach_tflops / fp32_nominal,
            "algorithmic_flop_per_launch": 2 * algorithmic_fma_per_launch(BATCH)}
    hbm = {"bound": "hbm", "achieved": ach_gbs, "peak": hbm_peak, "unit": "GB/s", "frac": ach_gbs / hbm_peak,
           "peak_source": f"{peak_kind} (MEASURED_PEAKS.json hbm_gbs)" if peak_kind == "measured" else "fallback 6650 GB/s",
           "algorithmic_bytes_per_launch": algorithmic_bytes_per_launch(BATCH)}
    # the binding bound is the one whose roofline time is longer
    t_fp32 = fp32["algorithmic_flop_per_launch"] / (fp32_measured * 1e12)
    t_hbm = hbm["algorithmic_bytes_per_launch"] / (hbm_peak * 1e9)
    binding, other = (fp32, hbm) if t_fp32 >= t_hbm else (hbm, fp32)
    roofline = dict(binding)
    roofline.update({"kernel": kernel_name, "kernel_ms": kms, "traffic": traffic,
                     "traffic_source": f"constant from the ncu capture summarised in {traffic_src}, not measured in this run",
                     "other_bound": other})

    # ---------------- end to end through the public op with pinned host buffers
    # Host batches go through HostPipelinedForward: host->device copy, the fused loop and the
    # device->host copy of each batch run on three streams, three device buffer sets deep, so the
    # copies of one step overlap the compute of its neighbours. All copies are inside the timed region.
    hx = [x.pin_memory() for x in xs_host[:3]]
    hy = [torch.empty_like(h).pin_memory() for h in hx]
    pipe = gb.HostPipelinedForward(w, b, s, gamma, beta, BATCH, INNER, OUTER, BLOCK, ACT)

    for i in range(4):
        pipe.submit(hx[i % 3], hy[i % 3])
    pipe.synchronize()
    ctx.barrier()
    n_e2e = max(3, args.steps)  # the same K as the device-resident figure; includes filling and draining the pipeline
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    pipe.join()  # nothing of the pipeline starts before the start event
    for i in range(n_e2e):
        pipe.submit(hx[i % 3], hy[i % 3])
    pipe.join()  # the current stream waits for the last device->host copy
    t1.record()
    ctx.barrier()
    ems = ctx.max_over_ranks(t0.elapsed_time(t1))
    ok = bool(torch.isfinite(hy[0]).all().item())
    e2e_value = neuron_updates(BATCH) * world * n_e2e / (ems * 1e-3)
    nbytes = xs[0].numel() * 4
    # The ceiling the host side sets: the same host->device and device->host copies with no compute at all, on two
    # streams, all ranks at once. End to end cannot be faster than this, whatever the kernels do.
    cs_in, cs_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    ctx.barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record()
    cs_in.wait_stream(torch.cuda.current_stream())
    cs_out.wait_stream(torch.cuda.current_stream())
    for i in range(n_e2e):
        with torch.cuda.stream(cs_in):
            xs[i % 2].copy_(hx[i % 2], non_blocking=True)
        with torch.cuda.stream(cs_out):
            hy[i % 2].copy_(ys[i % 2], non_blocking=True)
    torch.cuda.current_stream().wait_stream(cs_in)
    torch.cuda.current_stream().wait_stream(cs_out)
    c1.record()
    ctx.barrier()
    cms = ctx.max_over_ranks(c0.elapsed_time(c1))
    e2e = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes,
           "ms_per_step": ems / n_e2e, "steps": n_e2e,
           "finite": ok,
           "host_gbs_per_rank": 2 * nbytes * n_e2e / (ems * 1e-3) / 1e9,
           "copies_alone": {"ms_per_step": cms / n_e2e, "host_gbs_per_rank": 2 * nbytes * n_e2e / (cms * 1e-3) / 1e9,
                            "value_ceiling": neuron_updates(BATCH) * world * n_e2e / (cms * 1e-3),
                            "note": "the same pinned-host copies both ways with no compute, all ranks at once: the "
                                    "ceiling that host memory and PCIe set for the end-to-end figure"},
           "cpu_affinity": ctx.affinity,
           "note": "full [B,M,N,K] activations in and out through HostPipelinedForward (pinned host memory; copies of one "
                   "step overlap the compute of its neighbours on separate streams)"}

    # clocks were sampled over all three timed regions (value, kernel-only, end to end)
    clocks = sampler.stop() if rank == 0 else None

    # ---------------- CPU baseline on rank 0 at N = 1: the oracle on the same full batch
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        from oracle import gridnet_oracle as orc

        orc.set_threads(len(os.sched_getaffinity(0)))
        inputs = cpu_inputs(BATCH)
        dt, passes = 0.0, 0
        while passes < 8 and (passes == 0 or dt < 10.0):  # about 10 s of CPU work, whole passes only
            dt += cpu_oracle_pass(inputs)
            passes += 1
        rate = neuron_updates(BATCH) * passes / dt
        cpu = {"value": rate, "unit": UNIT, "cores": orc.max_threads(), "kind": "port",
               "sample": f"{passes} pass(es) over {BATCH} of {BATCH} samples, full 12 outer x 4 inner loop incl. LayerNorm, "
                         f"{dt:.1f} s", "note": "measured at N = 1 only"}

    del pipe, hx, hy, xs, ys, ws
    ctx.release()
    return {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "global_batch": BATCH * world, "parallelism": f"batch-sharded x{world}",
                   "l2": f"{NSETS} rotating input/output sets (4 x 67 MB each way) plus a 300 MB working set per step, larger than the 126 MB L2",
                   "samples_per_sec": BATCH * world * args.steps / (ms * 1e-3),
                   "step_kernel": "large-batch (step_pair64.cu)" if large_batch else "register-patch (step_fast.cu)",
                   "device_failure_flag": failed},
        "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu,
        "gpu_launches": launches_per_step * args.steps, "clocks": clocks,
    }


def slab_parity_on_ranks(ctx: Ctx) -> dict:
    """Both face-exchange paths of the slab mode on the real ranks against rank 0's single-GPU fused loop, on a
    grid small enough for one GPU: 64 x 64 x (16 * world), batch 8, 2 inner x 3 outer."""
    import torch

    import gridnet_b200 as gb
    from gridnet_b200.slab import (PeerFaceBuffers, PeerSlabBuffers, PeerStatsMailboxes, SlabLayout, make_cuda_runner,
                                   run_direct, run_distributed, run_in_place)

    dist = ctx.need_group()
    world, rank, device = ctx.world, ctx.rank, ctx.device
    M = N = 64
    K = 16 * world
    B, inner, outer = 8, 2, 3
    g = torch.Generator().manual_seed(7)  # the same full tensors on every rank
    w = torch.randn(27, M, N, K, generator=g) / 27 ** 0.5
    b = 0.1 * torch.randn(M, N, K, generator=g)
    s = 1 + 0.1 * torch.randn(M, N, K, generator=g)
    gamma = 1 + 0.1 * torch.randn(M, N, K, generator=g)
    beta = 0.1 * torch.randn(M, N, K, generator=g)
    x = torch.zeros(B, M, N, K)
    x[..., 0] = torch.randn(B, M, N, generator=g)
    lay = SlabLayout(K, world, rank)
    peers = PeerFaceBuffers(lay, B, M, N, device)
    slabs = PeerSlabBuffers(lay, B, M, N, device)
    boxes = PeerStatsMailboxes(lay, B, device)
    outs = {}
    for name in ("in-place", "direct", "nccl"):
        runner = make_cuda_runner(lay, w, b, s, gamma, beta, x, inner, ACT, device=device,
                                  work_buffers=slabs.work_buffers() if name == "in-place" else None)
        if name == "in-place":
            local = run_in_place(runner, outer, slabs, boxes)
        elif name == "direct":
            local = run_direct(runner, outer, peers, mailboxes=boxes)
        else:
            local = run_distributed(runner, outer)
        parts = [torch.empty_like(local) for _ in range(world)] if rank == 0 else None
        dist.gather(local.contiguous(), parts, dst=0)
        if rank == 0:
            outs[name] = torch.cat(parts, dim=-1)
    verdict = torch.zeros(4, device=device)
    if rank == 0:
        ref = gb.outer_forward(*(t.to(device) for t in (w, b, s, gamma, beta, x)), inner, outer, 8, ACT)
        tol = 1e-5 + 1e-4 * ref.abs()
        e_direct = (outs["direct"] - ref).abs()
        e_nccl = (outs["nccl"] - ref).abs()
        e_inplace = (outs["in-place"] - ref).abs()
        ok = all(bool((e <= tol).all().item()) for e in (e_direct, e_nccl, e_inplace))
        verdict = torch.tensor([1.0 if ok else 0.0, float(e_direct.max().item()), float(e_nccl.max().item()),
                                float(e_inplace.max().item())], device=device)
    dist.broadcast(verdict, src=0)
    mailbox_wait_failed = boxes.failed()
    del peers, boxes, slabs

    # training on the real ranks: forward + backward with the reverse face exchange and both all-reduces over NCCL,
    # gathered and compared with rank 0's single-GPU autograd through the package's ops
    from gridnet_b200.slab import make_cuda_trainer, train_distributed

    gy = torch.randn(B, M, N, K, generator=g)
    trainer = make_cuda_trainer(lay, w, b, s, gamma, beta, x, inner, ACT, device=device)
    _, res = train_distributed(trainer, outer, lambda o: gy[..., lay.k0:lay.k0 + lay.k_loc].to(device))
    gathered = []
    for t in res:
        parts = [torch.empty_like(t) for _ in range(world)] if rank == 0 else None
        dist.gather(t.contiguous(), parts, dst=0)
        gathered.append(torch.cat(parts, dim=-1) if rank == 0 else None)
    bverdict = torch.zeros(2, device=device)
    if rank == 0:
        leaves = [t.to(device).requires_grad_(True) for t in (w, b, s, gamma, beta, x)]
        h = leaves[5]
        for _ in range(outer):
            h = gb.GridNormOp.apply(gb.GridnetCudaOp.apply(leaves[0], leaves[1], leaves[2], h, inner, 8, 1e-5, False, ACT),
                                    leaves[3], leaves[4], 1e-5)
        single = torch.autograd.grad(h, leaves, gy.to(device))
        worst, okb = 0.0, True
        for a, c in zip(gathered, single):
            e = float((a - c).abs().max().item())
            worst = max(worst, e / (1.0 + float(c.abs().max().item())))
            okb = okb and bool(((a - c).abs() <= 1e-4 * (1 + c.abs().max()) + 1e-3 * c.abs()).all().item())
        bverdict = torch.tensor([1.0 if okb else 0.0, worst], device=device)
    dist.broadcast(bverdict, src=0)
    return {"slab_parity_ok": bool(verdict[0].item() > 0.5) and bool(bverdict[0].item() > 0.5) and not mailbox_wait_failed,
            "mailbox_wait_failed": mailbox_wait_failed,
            "slab_forward_parity_ok": bool(verdict[0].item() > 0.5),
            "slab_backward_parity_ok": bool(bverdict[0].item() > 0.5),
            "backward_worst_err_over_max": float(bverdict[1].item()),
            "backward_tolerance": "|slab - single GPU| <= 1e-4 (1 + max|ref|) + 1e-3 |ref| for all six gradients (two float32 "
                                  "implementations with different summation orders; the oracle comparison is in tests/test_slab.py)",
            "grid": [M, N, K], "batch": B,
            "max_abs_err_direct": float(verdict[1].item()), "max_abs_err_nccl": float(verdict[2].item()),
            "max_abs_err_in_place": float(verdict[3].item()),
            "same_bits_all_paths": None if rank != 0 else bool(torch.equal(outs["direct"], outs["nccl"])
                                                               and torch.equal(outs["in-place"], outs["nccl"])),
            "tolerance": "1e-5 + 1e-4 |ref| against outer_forward on the whole grid on rank 0"}


def bench_slab(ctx: Ctx):
    """The large-grid configuration: 256^3 grid, block 8, 2 inner x 32 outer, batch 32, forward, the grid
    slab-sharded along K over all ranks (strong scaling: the total work is fixed)."""
    import torch

    from gridnet_b200.slab import (GHOST, CudaSlabBackend, PeerFaceBuffers, PeerSlabBuffers, PeerStatsMailboxes, SlabLayout,
                                   SlabRunner, run_direct, run_distributed, run_in_place)

    args, rank, world, device = ctx.args, ctx.rank, ctx.world, ctx.device
    dist = ctx.need_group()
    parity = slab_parity_on_ranks(ctx) if world > 1 else None
    ctx.release()
    G, B, inner, outer = 256, 32, 2, 32
    lay = SlabLayout(G, world, rank)
    # The same full-grid problem on every rank and for every world size (same seed, same generator), each rank
    # keeping its slab of it: the result can then be compared with the single-GPU loop on the whole grid, and
    # the output checksum is the same number whatever N is.
    g = torch.Generator(device=device).manual_seed(100)
    w_full = torch.randn(27, G, G, G, generator=g, device=device) / 27 ** 0.5
    x_full = torch.zeros(B, G, G, G, device=device)
    x_full[..., 0] = torch.randn(B, G, G, generator=g, device=device)
    b_full = torch.zeros(G, G, G, device=device)
    s_full = torch.ones(G, G, G, device=device)
    gamma_full = torch.ones(G, G, G, device=device)
    beta_full = torch.zeros(G, G, G, device=device)
    # shard(): the rank's columns plus a ghost block either side whose adjacent column holds the neighbour's
    # boundary values (zeros beyond the ends of the grid, which normalise-on-load keeps zero)
    w, b, s, gamma, beta, x = (lay.shard(t) for t in (w_full, b_full, s_full, gamma_full, beta_full, x_full))
    backend = CudaSlabBackend(lay, w, b, s, gamma, beta, inner, ACT)

    # faces: stored by the step kernel straight into the neighbours' ghost columns (default), or into packed
    # buffers in the neighbours' memory and unpacked there (--slab-exchange direct), or packed and sent with NCCL
    # send/recv (--slab-exchange nccl)
    mode = args.slab_exchange if world > 1 else "nccl"
    direct = mode == "direct"
    peers = PeerFaceBuffers(lay, B, G, G, device) if direct else None
    slabs = PeerSlabBuffers(lay, B, G, G, device) if mode == "in-place" else None
    boxes = PeerStatsMailboxes(lay, B, device) if mode != "nccl" else None

    def one_pass():
        if mode == "in-place":
            return run_in_place(SlabRunner(lay, backend, x, G * G * G, work_buffers=slabs.work_buffers()), outer, slabs, boxes)
        runner = SlabRunner(lay, backend, x, G * G * G)
        return run_direct(runner, outer, peers, mailboxes=boxes) if direct else run_distributed(runner, outer)

    warm = max(1, min(args.warmup, 2))
    for _ in range(warm):
        one_pass()
    dist.barrier()
    torch.cuda.synchronize()
    steps = max(1, min(args.steps, 3))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        out = one_pass()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    # where a step's time goes (in-place exchange): one more pass with CUDA events between its three launches
    phases = None
    if mode == "in-place":
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(outer)]
        run_in_place(SlabRunner(lay, backend, x, G * G * G, work_buffers=slabs.work_buffers()), outer, slabs, boxes,
                     probe=lambda k, i: evs[k][i].record())
        torch.cuda.synchronize()
        mean = lambda i: sum(evs[k][i].elapsed_time(evs[k][i + 1]) for k in range(1, outer)) / (outer - 1)
        phases = {"step_kernel_ms": ctx.max_over_ranks(mean(0)), "publish_wait_finalize_ms": ctx.max_over_ranks(mean(1)),
                  "note": "CUDA events between the two launches of an outer step (the step kernel; the kernel that publishes "
                          "the sums, waits for the other ranks' and finishes the statistics), mean over steps 2..32 of one "
                          "extra pass, max over ranks (the first step has no normalise-on-load)"}
    finite = bool(torch.isfinite(out).all().item())
    chk = out.double().sum().reshape(1)  # the same bits whichever way the faces travel and whatever N is
    dist.all_reduce(chk)
    # parity at the configuration's own size, on the real ranks: every rank runs the single-GPU fused loop on the
    # whole grid and compares its slab of the result
    import gridnet_b200 as gb

    ref = gb.outer_forward(w_full, b_full, s_full, gamma_full, beta_full, x_full, inner, outer, 8, ACT)
    mine = ref[..., lay.k0:lay.k0 + lay.k_loc]
    err = (mine - out).abs()
    full_ok = torch.tensor([float(bool((err <= 1e-5 + 1e-4 * mine.abs()).all().item())),
                            float(bool(torch.equal(mine, out)))], device=device)
    worst = err.max().reshape(1)
    dist.all_reduce(full_ok, op=dist.ReduceOp.MIN)
    dist.all_reduce(worst, op=dist.ReduceOp.MAX)
    del ref, mine, err
    nu = float(B) * G ** 3 * inner * outer
    rec = {
        "metric": METRIC, "value": nu * steps / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warm, "ms_per_step": ms / steps, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C5: 256^3 grid, block 8, 2 inner x 32 outer, batch 32, fp32, forward + whole-grid "
                               "LayerNorm, slab-sharded along K", "parallelism": f"slab x{world}",
                   "exchange": ("per outer step: the step kernel stores 2 faces [32,256,256] fp32 straight into the "
                                "neighbours' ghost columns over NVLink (nothing is unpacked); the [32,2] f64 sums go to every "
                                "rank's mailbox by peer stores and flags (no collective call; two launches per step)" if mode == "in-place" else
                                "per outer step: the step kernel stores 2 faces [32,256,256] fp32 into the neighbours' memory "
                                "over NVLink; the [32,2] f64 sums go to every rank's mailbox by peer stores and flags "
                                "(no collective call)" if direct else
                                "per outer step: 2 faces [32,256,256] fp32 send/recv per neighbour + all-reduce of [32,2] f64"),
                   "samples_per_sec": B * steps / (ms * 1e-3), "finite": finite, "output_checksum": float(chk.item())},
        "gpu_launches": (outer * (2 if mode == "in-place" else 3) + 1) * steps if mode != "nccl" else (outer * 2 + 1) * steps,
    }
    if phases is not None:
        rec["phases"] = phases
    rec["full_size_parity"] = {"ok": bool(full_ok[0].item()), "bit_identical": bool(full_ok[1].item()),
                               "max_abs_err": float(worst.item()),
                               "against": "the single-GPU fused loop (gn_outer_forward_f32) on the whole 256^3 grid, run on "
                                          "every rank; tolerance 1e-5 + 1e-4 |ref|"}
    if boxes is not None:
        rec["mailbox_wait_failed"] = boxes.failed()
    if parity is not None:
        rec.update(parity)
    if not rec["full_size_parity"]["ok"]:
        rec["slab_parity_ok"] = False  # fails the run like the small-grid parity check
    del backend, peers, slabs, boxes, w, x, out, w_full, x_full
    ctx.release()
    return rec


TRAIN_WORKLOADS = {
    # name: (grid, block, inner, outer, batch, description)
    "c3": (128, 8, 2, 16, 256, "C3: 128^3 grid, block 8, 2 inner x 16 outer, batch 256, fp32, forward + backward, "
                                "whole-grid LayerNorm per outer step"),
    "c4": (64, 4, 8, 16, 128, "C4: 64^3 grid, block 4, 8 inner x 16 outer, batch 128, fp32, forward + backward, "
                              "whole-grid LayerNorm per outer step"),
}


def bench_train(ctx: Ctx, name: str, stash=None, microbatches=None, steps_cap: int = 10):
    """The forward + backward configurations: one step = the outer loop forward, then the gradient of a
    seeded random upstream gradient on the final grid back to the parameters and the input, through the
    autograd ops of the package (the step op and the whole-grid norm op per outer step). The batch is
    sharded over the ranks (strong scaling); with more than one rank the parameter gradients are
    all-reduced once per step, inside the timed region."""
    import torch

    import gridnet_b200 as gb

    args, rank, local_rank, world, device = ctx.args, ctx.rank, ctx.local_rank, ctx.world, ctx.device
    G, block, inner, outer, batch, desc = TRAIN_WORKLOADS[name]
    if args.batch:
        batch = args.batch
    if stash is None and args.stash:
        stash = True
    # keep the inner iterations' intermediate results from the forward pass (memory for time): True / False force
    # it, None leaves the package's default (kept whenever they fit comfortably in the free device memory)
    previous_stash = gb.keep_forward_stash(stash)
    ctx.release()  # what the configuration before this one held goes back to the driver first
    dist = ctx.need_group() if world > 1 else None
    if batch % world:
        raise SystemExit(f"batch {batch} does not divide over {world} ranks")
    b_loc = batch // world
    barrier = ctx.barrier

    g = torch.Generator().manual_seed(0)
    model = gb.GridnetModel((G, G, G), inner, outer, block, device, activation=ACT)
    with torch.no_grad():
        model.network.weight.copy_((torch.randn(27, G, G, G, generator=g) / 27 ** 0.5).to(device))
    params = [p for p in model.parameters()]
    gsel = torch.Generator().manual_seed(1 + rank)
    x = torch.zeros(b_loc, G, G, G, device=device)
    x[..., 0] = torch.randn(b_loc, G, G, generator=gsel).to(device)
    x.requires_grad_(True)
    gy = torch.randn(b_loc, G, G, G, device=device, generator=torch.Generator(device=device).manual_seed(2 + rank))

    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    t_fwd = t_bwd = 0.0

    nmb = max(1, args.microbatches if microbatches is None else microbatches)
    if b_loc % nmb:
        raise SystemExit(f"the per-rank batch {b_loc} does not divide into {nmb} micro-batches")
    mb = b_loc // nmb

    def step(timed: bool):
        """Forward + backward over the rank's whole batch; with --microbatches N in N slices whose parameter
        gradients are accumulated (less memory live at once: what --stash needs at C3's full batch)."""
        nonlocal t_fwd, t_bwd
        total, gxs = None, []
        for i in range(nmb):
            xs = x if nmb == 1 else x[i * mb:(i + 1) * mb].detach().requires_grad_(True)
            gys = gy if nmb == 1 else gy[i * mb:(i + 1) * mb]
            ev[0].record()
            y = model(xs)
            ev[1].record()
            grads = torch.autograd.grad(y, params + [xs], gys)
            del y
            gxs.append(grads[-1])
            if total is None:
                total = list(grads[:-1])
            else:
                for acc, gnew in zip(total, grads[:-1]):
                    acc.add_(gnew)
            ev[2].record()
            if timed:
                ev[2].synchronize()
                t_fwd += ev[0].elapsed_time(ev[1])
                t_bwd += ev[1].elapsed_time(ev[2])
        if dist is not None:
            flat = torch.cat([t.reshape(-1) for t in total])
            dist.all_reduce(flat)
        return total + gxs

    warm = max(3, args.warmup)  # the first steps also grow torch's allocator cache
    torch.cuda.reset_peak_memory_stats(device)
    free0 = torch.cuda.mem_get_info(device)[0] / 1e9
    for _ in range(warm):
        grads = step(False)
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    steps = max(1, min(args.steps, steps_cap))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    mem0 = torch.cuda.memory_stats(device)
    e0.record()
    for _ in range(steps):
        grads = step(True)
    e1.record()
    barrier()
    mem1 = torch.cuda.memory_stats(device)
    # calls of the caching allocator into the driver inside the timed region (0 once its cache is warm)
    driver_allocs = int(mem1.get("num_device_alloc", 0) - mem0.get("num_device_alloc", 0))
    alloc_retries = int(mem1.get("num_alloc_retries", 0) - mem0.get("num_alloc_retries", 0))
    peak_gb = mem1.get("allocated_bytes.all.peak", 0) / 1e9
    clocks = sampler.stop() if rank == 0 else None
    ms = ctx.max_over_ranks(e0.elapsed_time(e1))
    finite = all(bool(torch.isfinite(t_).all().item()) for t_ in grads)
    fp32_peak = measure_fp32_peak(torch, device)
    rec = None
    if True:
        nu = float(batch) * G ** 3 * inner * outer
        hbm_gbs, hbm_src, sm_max_mhz = measured_peaks()
        fp32_nominal = FP32_LANES * 2 * sm_max_mhz * 1e6 / 1e12
        flops = 162.0 * nu / world  # per GPU: 27 forward FMAs and 54 backward FMAs per neuron update
        # bytes per outer step and GPU: forward 124 P + 8 B P, backward 372 P + 12 B P
        bytes_step = (124.0 + 372.0) * G ** 3 + 20.0 * b_loc * G ** 3
        sec = ms * 1e-3 / steps
        rec = ({
            "metric": METRIC, "value": nu / sec, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warm,
            "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": desc if not args.batch else desc + f" (batch overridden to {batch})",
                       "global_batch": batch, "parallelism": f"batch-sharded x{world}",
                       "l2": "one activation tensor is %.0f MB per rank; the %d saved step and norm inputs of a step "
                             "alone are %.0f MB, larger than the 126 MB L2"
                             % (b_loc * G ** 3 * 4 / 1e6, 2 * outer, 2 * outer * b_loc * G ** 3 * 4 / 1e6),
                       "forward_ms": t_fwd / steps, "backward_ms": t_bwd / steps, "finite": finite,
                       "intermediate_results": ("kept from the forward pass" if stash else "recomputed in the backward pass"
                                                if stash is not None else
                                                "kept from the forward pass for as many of the last outer steps as fit into 70 % "
                                                "of the free device memory, recomputed for the others (package default)"),
                       "microbatches": nmb,
                       "allocator": {"driver_allocations_in_timed_region": driver_allocs,
                                     "out_of_memory_retries_in_timed_region": alloc_retries,
                                     "peak_allocated_gb": peak_gb, "free_before_gb": free0},
                       "samples_per_sec": batch / sec},
            "roofline": {"bound": "fp32", "achieved": flops / sec / 1e12, "peak": fp32_peak, "unit": "TFLOP/s",
                         "frac": flops / sec / 1e12 / fp32_peak,
                         "peak_source": "measured in this run: FFMA-only kernel on every SM, CUDA events (gn_probe_fp32_fma)",
                         "peak_nominal": fp32_nominal, "frac_of_nominal": flops / sec / 1e12 / fp32_nominal,
                         "other_bound": {"bound": "hbm", "achieved": bytes_step * outer / sec / 1e9, "peak": hbm_gbs, "unit": "GB/s",
                                 "frac": bytes_step * outer / sec / 1e9 / hbm_gbs,
                                 "peak_source": hbm_src + " (MEASURED_PEAKS.json hbm_gbs)" if hbm_src == "measured"
                                 else "fallback"},
                         "traffic": None,
                         "traffic_source": "not captured for the training step (many kernels; see profiles/train_step_c3_launch_list.txt for their shares)"},
            "clocks": clocks,
        })
    gb.keep_forward_stash(previous_stash)
    del grads, model, params, x, gy
    ctx.release()
    return rec


def bench_c1(ctx: Ctx):
    """The small MNIST-shaped configuration: 32^3 grid, block 8, 2 inner x 8 outer, batch 8, forward. Launch
    latency is what it costs, so the library runs the whole loop as one persistent cooperative kernel; it is
    timed twice: called directly, and replayed from a CUDA graph captured once (the call neither allocates nor
    synchronises, so it can be captured as is)."""
    import torch

    import gridnet_b200 as gb

    args, rank, device = ctx.args, ctx.rank, ctx.device
    G, block, inner, outer, B = 32, 8, 2, 8, 8
    g = torch.Generator().manual_seed(0)
    w = (torch.randn(27, G, G, G, generator=g) / 27 ** 0.5).to(device)
    b = torch.zeros(G, G, G, device=device)
    s = torch.ones(G, G, G, device=device)
    gamma, beta = torch.ones(G, G, G, device=device), torch.zeros(G, G, G, device=device)
    x = torch.zeros(B, G, G, G)
    x[:, 2:30, 2:30, 0] = torch.rand(B, 28, 28, generator=g)  # image placement of gridnet/scripts/train_mnist.py:59-60
    x = x.to(device)
    y = torch.empty_like(x)
    ws = gb.outer_forward_workspace(B, (G, G, G), block, device)

    def once():
        gb.outer_forward(w, b, s, gamma, beta, x, inner, outer, block, ACT, out=y, workspace=ws)

    def timed(fn, n):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    steps = max(args.steps, 20)
    eager_ms = timed(once, steps)
    eager_out = y.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        once()
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        once()
    graph_ms = timed(graph.replay, steps)
    same = bool(torch.equal(eager_out, y))
    failed = gb.outer_forward_failed(ws, B, (G, G, G), block)
    nu = float(B) * G ** 3 * inner * outer
    del graph
    from gridnet_b200._lib import lib

    plan = int(lib.gn_outer_forward_plan(B, G, G, G, inner, outer, block))
    launches = {3: 1, 2: 2 * outer + 3, 1: 2 * outer + 1}.get(plan, 4 * outer)
    if True:
        return ({
            "metric": METRIC, "value": nu / (graph_ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps,
            "warmup": max(3, args.warmup), "ms_per_step": graph_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "C1: 32^3 grid, block 8, 2 inner x 8 outer, batch 8, fp32, forward + whole-grid "
                                   "LayerNorm per outer step; replayed from a CUDA graph",
                       "kernel": {3: "one persistent cooperative kernel over all outer steps (outer_small.cu)",
                                  2: "large-batch kernel, one launch per outer step",
                                  1: "register-patch kernel, one launch per outer step"}.get(plan, "generic kernels"),
                       "launch_by_launch_ms": eager_ms, "graph_replay_ms": graph_ms,
                       "graph_equals_launch_by_launch": same, "device_failure_flag": failed,
                       "samples_per_sec": B / (graph_ms * 1e-3),
                       "l2": "working set 4 MB: L2-resident by nature of the configuration"},
            "gpu_launches": launches * steps,
        })


def brief(rec):
    """A sub-record: the full record of a workload without the keys that only make sense at the top level."""
    if rec is None:
        return None
    return {k: v for k, v in rec.items() if k not in ("metric", "unit", "higher_is_better", "vs_baseline", "dtype", "data")}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--workload", choices=["all", "c2", "c5-slab", "c3", "c4", "c1"], default="all",
                    help="all (default): the headline benchmark c2 with the other configurations as sub-records of the same "
                         "line (c5_slab at every N; c1, c3, c4 at N = 1); c2: the headline alone; c5-slab: the 256^3 grid "
                         "sharded along K over all ranks; c3 / c4: the forward + backward configurations (128^3 block 8, "
                         "64^3 block 4); c1: the small launch-bound configuration, also replayed from a CUDA graph")
    ap.add_argument("--slab-exchange", choices=["in-place", "direct", "nccl"], default="in-place",
                    help="c5-slab only: how the boundary faces travel (in-place = stored by the step kernel into the "
                         "neighbours' ghost columns; direct = into packed buffers in the neighbours' memory, unpacked there; "
                         "nccl = packed and sent with send/recv)")
    ap.add_argument("--stash", action="store_true",
                    help="c3 / c4 only: keep the forward pass's intermediate results instead of recomputing them in the "
                         "backward pass ((2 inner - 1) extra activation tensors per outer step)")
    ap.add_argument("--microbatches", type=int, default=1,
                    help="c3 / c4 only: run a step as this many slices of the batch, accumulating parameter gradients")
    ap.add_argument("--batch", type=int, default=0, help="c3 / c4 only: override the global batch size")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.gpus > 1 and world == 1:
        raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    if args.impl == "reference":
        run_reference(args, rank)
        return
    ctx = Ctx(args, rank, local_rank, world)
    line, rc = None, 0
    if args.workload == "c5-slab":
        line = bench_slab(ctx)
        if line.get("slab_parity_ok") is False:
            rc = 3
    elif args.workload in TRAIN_WORKLOADS:
        line = bench_train(ctx, args.workload)
    elif args.workload == "c1":
        line = bench_c1(ctx) if rank == 0 else None
    else:
        line = bench_c2(ctx)
        if args.workload == "all":
            # the other configurations ride on the same line; the driver only ever runs this command
            slab = bench_slab(ctx)
            line["c5_slab"] = brief(slab)
            if slab.get("slab_parity_ok") is False:
                rc = 3
            if world == 1:
                line["c1"] = brief(bench_c1(ctx))
                # C3 at its full batch in one piece: the fused training node saves only the raw step outputs, and the
                # package keeps the inner iterations of a step while they fit comfortably; C4 keeps them all
                line["c3"] = brief(bench_train(ctx, "c3", stash=None, microbatches=1, steps_cap=3))
                line["c4"] = brief(bench_train(ctx, "c4", stash=True, microbatches=1, steps_cap=5))
    if rank == 0 and line is not None:
        print(json.dumps(line), flush=True)
    ctx.close()
    if rc:
        raise SystemExit(rc)


if __name__ == "__main__":
    main()
