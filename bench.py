#!/usr/bin/env python
"""LayerNorm / RMSNorm forward + backward benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one forward + one backward (dx, dweight[, dbias]) over the workload's rows.  The
metric is achieved algorithmic HBM bandwidth in GB/s, whole job (all ranks); rows/s rides
along.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank works on
its own rows and the fp32 dweight / dbias shard sums are exchanged over NCCL on a side stream
while the next step is launched.

Prints ONE JSON line (rank 0).  `--impl reference` times the CPU oracle (the port of the
reference's algorithm) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
for p in (ROOT, ROOT / "triton-hub_b200"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))

import numpy as np
import torch

# The benchmark workloads (c1 = the reference README's Quick Start shape).  c2 is the default: the
# configuration the headline metric is quoted on.
WORKLOADS = {
    "c1": dict(op="ln", dtype="fp32", M=200, N=128, eps=1e-6, mu=0.0, sigma=1.0,
               desc="LayerNorm fp32 (2,100,128)"),
    "c2": dict(op="rms", dtype="bf16", M=32768, N=4096, eps=1e-6, mu=0.0, sigma=1.0,
               desc="RMSNorm bf16 (8,4096,4096)"),
    "c3": dict(op="ln", dtype="fp16", M=65536, N=5120, eps=1e-5, mu=3.0, sigma=2.0,
               desc="LayerNorm fp16 (65536,5120) x~N(3,2)"),
    "c4": dict(op="ln", dtype="bf16", M=32768, N=16384, eps=1e-6, mu=0.0, sigma=1.0,
               desc="LayerNorm bf16 (32768,16384)"),
    "c5_ln": dict(op="ln", dtype="bf16", M=1048576, N=4096, eps=1e-6, mu=0.0, sigma=1.0,
                  desc="LayerNorm bf16 (1048576,4096)"),
    "c5_rms": dict(op="rms", dtype="bf16", M=1048576, N=4096, eps=1e-6, mu=0.0, sigma=1.0,
                   desc="RMSNorm bf16 (1048576,4096)"),
}
TDTYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp64": torch.float64}
ESIZE = {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}
FALLBACK_HBM_GBS = 6650.0
# DRAM bytes per row (dram__bytes_read.sum + dram__bytes_write.sum) of the backward kernel, from the
# ncu captures summarised under profiles/ (taken at 16384, 16384 and 4096 rows; traffic is proportional to rows).
NCU_BWD_DRAM_BYTES_PER_ROW = {"c2": 22365.0, "c3": 28811.0, "c4": 91065.0}


def algorithmic_bytes(wl, rows):
    """Bytes the path must move for `rows` rows: forward reads x, writes y and the statistics;
    backward reads x, dy and the statistics, writes dx; plus the parameter vectors once."""
    N, s = wl["N"], ESIZE[wl["dtype"]]
    ln = wl["op"] == "ln"
    stats = 8 if ln else 4
    fwd = rows * (2 * N * s + stats) + (2 if ln else 1) * N * s
    bwd = rows * (3 * N * s + stats) + N * s + (2 if ln else 1) * N * s
    return fwd, bwd


def measured_peak():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (no MEASURED_PEAKS.json)"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML while the benchmark runs (read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.stop_flag, self.window = index, [], False, [None, None]
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.max_mhz = None

    def run(self):
        if not self.ok:
            return
        nv = self.nv
        while not self.stop_flag:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)
                reasons = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                self.samples.append((time.perf_counter(), mhz, reasons))
            except Exception:
                pass
            time.sleep(0.005)

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        nv = self.nv
        t0, t1 = self.window
        inside = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1]
        where = "timed region"
        if len(inside) < 3:
            inside, where = self.samples, "warm-up + timed region (timed region shorter than 3 samples)"
        names = {
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80): "hw_power_brake_slowdown",
        }
        seen = set()
        for _, _, r in inside:
            for bit, name in names.items():
                if r & bit:
                    seen.add(name)
        return {"sm_mhz": float(np.median([s[1] for s in inside])), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(seen), "samples": len(inside), "sampled_over": where}


def make_device_inputs(wl, rows, device, seed):
    g = torch.Generator(device=device).manual_seed(seed)
    dt = TDTYPE[wl["dtype"]]
    N = wl["N"]
    x = torch.empty((rows, N), device=device, dtype=dt)
    dy = torch.empty((rows, N), device=device, dtype=dt)
    chunk = max(1, (1 << 26) // N)  # draw in fp32 a chunk at a time, then round to the storage type
    for r0 in range(0, rows, chunk):
        r1 = min(rows, r0 + chunk)
        x[r0:r1] = (torch.randn((r1 - r0, N), device=device, generator=g) * wl["sigma"] + wl["mu"]).to(dt)
        dy[r0:r1] = torch.randn((r1 - r0, N), device=device, generator=g).to(dt)
    gp = torch.Generator(device=device).manual_seed(12345)  # parameters are replicated: same on every rank
    w = (1 + 0.1 * torch.randn(N, device=device, generator=gp)).to(dt)
    b = (0.1 * torch.randn(N, device=device, generator=gp)).to(dt) if wl["op"] == "ln" else None
    return x, dy, w, b


def run_gpu(args):
    import torch.distributed as dist
    from b200norm import _lib
    from b200norm import functional as Fn

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs torch.distributed.run with N ranks")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    _lib.load()
    if world > 1:
        dist.init_process_group("nccl", device_id=device)

    wl = dict(WORKLOADS[args.workload])
    if args.rows > 0:
        wl["M"] = args.rows
        wl["desc"] += f" cut to {args.rows} rows"
    ln = wl["op"] == "ln"
    total_rows = wl["M"] * (world if args.scaling == "weak" else 1)
    rows = total_rows // world
    N, eps = wl["N"], wl["eps"]
    x, dy, w, b = make_device_inputs(wl, rows, device, seed=1000 + rank)
    fwd_bytes, bwd_bytes = algorithmic_bytes(wl, rows)
    exchange = None
    wl_n = WORKLOADS[args.workload]["N"]
    if world > 1:
        from b200norm.parallel import GradExchange, PushExchange, sharded_layernorm_bwd, sharded_rmsnorm_bwd
        exchange = (PushExchange(max_n=wl_n, slots=2, device=device, total_shards=8 if args.g_invariant else None,
                                 device_numbering=args.graph)
                    if args.exchange == "push"
                    else GradExchange(mode=args.exchange))

    from b200norm import activations as Act
    approx = {"gelu": "none", "gelu_tanh": "tanh"}.get(args.act)
    op = "ln" if ln else "rms"
    if approx is not None and world > 1:
        raise SystemExit("--act is a single-GPU measurement")

    def step(timing=None):
        """forward + backward; with world > 1 also starts the dweight/dbias all-reduce on the
        side stream and returns its handle so that it overlaps the next step's launches."""
        if timing is not None:
            timing[0].record()
        if approx is not None:
            # norm -> GeLU (the reference's Quick Start pair): fused kernels, or the two steps one after the other
            if args.unfused:
                if ln:
                    yy, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
                else:
                    yy, rstd = Fn._rmsnorm_fwd(x, w, eps)
                    mean = None
                z = Act._gelu_fwd(yy, approx)
                if timing is not None:
                    timing[1].record()
                dyy = Act._gelu_bwd(yy, dy, approx)
                res = (Fn._layernorm_bwd(x, dyy, w, b, mean, rstd, eps) if ln else Fn._rmsnorm_bwd(x, dyy, w, rstd, eps))
            else:
                z, mean, rstd = Act._norm_gelu_fwd(op, x, w, b, eps, approx)
                if timing is not None:
                    timing[1].record()
                res = Act._norm_gelu_bwd(op, x, dy, w, b, mean, rstd, eps, approx)
            if timing is not None:
                timing[2].record()
            return (z,) + tuple(res), None
        if ln:
            y, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
        else:
            y, rstd = Fn._rmsnorm_fwd(x, w, eps)
        if timing is not None:
            timing[1].record()
        pending = None
        if world > 1:
            if args.exchange == "push":
                dx, pending = (exchange.backward_layernorm(x, dy, w, b, mean, rstd, eps) if ln
                               else exchange.backward_rmsnorm(x, dy, w, rstd, eps))
            elif ln:
                dx, pending = sharded_layernorm_bwd(x, dy, w, b, mean, rstd, eps, exchange)
            else:
                dx, pending = sharded_rmsnorm_bwd(x, dy, w, rstd, eps, exchange)
            if timing is not None:
                timing[2].record()
            out = (y, dx)
        else:
            if ln:
                dx, dw, db = Fn._layernorm_bwd(x, dy, w, b, mean, rstd, eps)
                out = (y, dx, dw, db)
            else:
                dx, dw = Fn._rmsnorm_bwd(x, dy, w, rstd, eps)
                out = (y, dx, dw)
            if timing is not None:
                timing[2].record()
        return out, pending

    def finish(pending):
        """Wait for an exchange and cast the reduced sums to the parameter type."""
        if pending is None:
            return None
        return exchange.finish(pending, w.dtype)

    sampler = ClockSampler(local)
    sampler.start()

    prev = None
    for _ in range(max(args.warmup, 3)):
        _, pend = step()
        finish(prev)
        prev = pend
    finish(prev)
    torch.cuda.synchronize()

    K = args.steps
    use_graph = args.graph and world == 1
    # With several GPUs the step can still be graph-captured when the exchange is the library's own
    # (no collective-library call inside): the kernels number the exchanges on the device.
    use_graph_multi = args.graph and world > 1 and args.exchange == "push"

    # Eager pass: every step launched from Python, with an event pair around each kernel group.
    # It gives the per-kernel split for the roofline and, without --graph, the headline time.
    KE = K if not (use_graph or use_graph_multi) else min(K, 50)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(KE)]
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    if not (use_graph or use_graph_multi):
        sampler.window[0] = time.perf_counter()
    start.record()
    prev = None
    for i in range(KE):
        _, pend = step(evs[i])
        finish(prev)
        prev = pend
    finish(prev)
    stop.record()
    torch.cuda.synchronize()
    if not (use_graph or use_graph_multi):
        sampler.window[1] = time.perf_counter()
    if world > 1:
        dist.barrier()
    eager_ms = start.elapsed_time(stop) / KE
    total_ms = eager_ms * K
    fwd_ms = float(np.mean([e[0].elapsed_time(e[1]) for e in evs]))
    bwd_ms = float(np.mean([e[1].elapsed_time(e[2]) for e in evs]))

    if use_graph:
        # Headline: one step captured into a CUDA graph (through the same public wrappers) and
        # replayed K times, so that host launch jitter cannot leak into a 0.2 ms step.
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out, _ = step()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        sampler.window[0] = time.perf_counter()
        start.record()
        for _ in range(K):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        sampler.window[1] = time.perf_counter()
        total_ms = start.elapsed_time(stop)

        # Per-kernel split for the roofline, also by graph replay: the forward and the backward
        # (+ column reduce) captured separately, an event between the two replays of each step.
        g_fwd, g_bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_fwd):
            if approx is not None:
                if args.unfused:
                    if ln:
                        gyy, gmean, grstd = Fn._layernorm_fwd(x, w, b, eps)
                    else:
                        gyy, grstd = Fn._rmsnorm_fwd(x, w, eps)
                        gmean = None
                    gy = Act._gelu_fwd(gyy, approx)
                else:
                    gy, gmean, grstd = Act._norm_gelu_fwd(op, x, w, b, eps, approx)
            elif ln:
                gy, gmean, grstd = Fn._layernorm_fwd(x, w, b, eps)
            else:
                gy, grstd = Fn._rmsnorm_fwd(x, w, eps)
        with torch.cuda.graph(g_bwd):
            if approx is not None:
                if args.unfused:
                    gdyy = Act._gelu_bwd(gyy, dy, approx)
                    gb_out = (Fn._layernorm_bwd(x, gdyy, w, b, gmean, grstd, eps) if ln
                              else Fn._rmsnorm_bwd(x, gdyy, w, grstd, eps))
                else:
                    gb_out = Act._norm_gelu_bwd(op, x, dy, w, b, gmean, grstd, eps, approx)
            elif ln:
                gb_out = Fn._layernorm_bwd(x, dy, w, b, gmean, grstd, eps)
            else:
                gb_out = Fn._rmsnorm_bwd(x, dy, w, grstd, eps)
        KS = min(K, 100)
        sevs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(KS)]
        for _ in range(3):
            g_fwd.replay()
            g_bwd.replay()
        torch.cuda.synchronize()
        for i in range(KS):
            sevs[i][0].record()
            g_fwd.replay()
            sevs[i][1].record()
            g_bwd.replay()
            sevs[i][2].record()
        torch.cuda.synchronize()
        fwd_ms = float(np.median([e[0].elapsed_time(e[1]) for e in sevs]))
        bwd_ms = float(np.median([e[1].elapsed_time(e[2]) for e in sevs]))
    if use_graph_multi:
        # One eager step opens the pipeline (push k); the captured step is
        # [forward, backward + push k+1, finish k]; a last eager finish closes it.
        _, pend = step()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            _, pend_next = step()
            graph_out = finish(pend)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        sampler.window[0] = time.perf_counter()
        start.record()
        for _ in range(K):
            graph.replay()
        stop.record()
        torch.cuda.synchronize()
        sampler.window[1] = time.perf_counter()
        total_ms = start.elapsed_time(stop)
        finish(pend_next)
        torch.cuda.synchronize()
        dist.barrier()
    if world > 1:
        t = torch.tensor([total_ms, fwd_ms, bwd_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, fwd_ms, bwd_ms = t.tolist()
    ms_per_step = total_ms / K
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    clocks = sampler.summary()

    # End to end through the public module-level API with HOST buffers: pinned x / dy in,
    # y / dx / dweight [/ dbias] out, copies inside the timed region.
    e2e = None
    if not args.no_e2e and approx is None:
        e2e = run_e2e(wl, x, dy, w, b, rows, world, device, args)

    peak, peak_src = measured_peak()
    value = (fwd_bytes + bwd_bytes) * world / (ms_per_step * 1e-3) / 1e9
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9
    launches_per_step = 3 + (1 if world > 1 else 0)  # fwd, bwd, column reduce [, finalize]
    if approx is not None and args.unfused:
        launches_per_step += 2  # the two stand-alone GeLU kernels
    line = {
        "metric": "LN/RMSNorm fwd+bwd achieved HBM GB/s",
        "value": round(value, 1),
        "unit": "GB/s",
        "n_gpus": world,
        "steps": K,
        "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 5),
        "higher_is_better": True,
        "scaling": args.scaling,
        "vs_baseline": None,
        "dtype": wl["dtype"] + " storage, fp32 arithmetic",
        "data": "synthetic (seeded normal draws with the workload's mean/std; no dataset is involved)",
        "config": {
            "workload": f"{args.workload}: {wl['desc']} fwd+bwd, eps={eps}"
                        + ("" if approx is None else f", followed by GeLU({approx}) "
                           + ("as separate kernels" if args.unfused else "fused into the norm kernels")
                           + "; bytes counted as for the fused pair (y never stored)"),
            "rows_per_gpu": rows,
            "rows_total": total_rows,
            "dim": N,
            "l2_policy": f"inputs larger than L2 ({(2 * rows * N * ESIZE[wl['dtype']]) >> 20} MiB of x+dy per GPU vs 126 MB)"
            if 2 * rows * N * ESIZE[wl["dtype"]] > 126e6 else "inputs fit in L2 (launch-bound case; GB/s not meaningful)",
            "parallelism": (f"rows sharded over {world} GPU(s); fp32 dweight/dbias exchange: "
                            + ("column reduce fused with a push into every rank's inbox over NVLink peer memory, "
                               "finished one step later" if args.exchange == "push"
                               else f"NCCL {args.exchange} on a side stream, overlapped with the next step's launches"))
            if world > 1
            else "single GPU",
        },
        "launch_mode": ("cuda graph of one step (captured through the public wrappers), replayed per step"
                        if (use_graph or use_graph_multi) else "eager: every kernel launched from Python"),
        "eager_ms_per_step": round(eager_ms, 5),
        "rows_per_s": round(total_rows / (ms_per_step * 1e-3), 1),
        "frac_of_peak": round(value / world / peak, 4),
        "frac_of_nominal_8000": round(value / world / 8000.0, 4),
        "peak_gbs_per_gpu": peak,
        "peak_source": peak_src,
        "roofline": {
            "bound": "hbm",
            "kernel": "norm_bwd_kernel (+ colreduce_kernel, same event pair)",
            "timed_by": ("CUDA events around a graph replay of the backward alone, median of the steps" if use_graph
                         else "CUDA events around the backward call in the eager loop, mean of the steps"),
            "achieved": round(bwd_gbs, 1),
            "peak": peak,
            "unit": "GB/s",
            "frac": round(bwd_gbs / peak, 4),
            "traffic": (round(NCU_BWD_DRAM_BYTES_PER_ROW[args.workload] * rows)
                        if args.workload in NCU_BWD_DRAM_BYTES_PER_ROW else None),
            "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of norm_bwd_kernel on a smaller case "
                               "(profiles/), scaled by the row count; writes still dirty in L2 at kernel end are not in it"
                               if args.workload in NCU_BWD_DRAM_BYTES_PER_ROW else None),
            "bytes_per_launch": bwd_bytes,
            "ms_per_launch": round(bwd_ms, 5),
            "fwd_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                           "bytes_per_launch": fwd_bytes, "ms_per_launch": round(fwd_ms, 5)},
            "peak_source": peak_src,
        },
        "clocks": clocks,
        "gpu_launches": launches_per_step * K,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and approx is None and not args.no_torch:
        line["gpu_baseline"] = torch_gpu_baseline(wl, x, dy, w, b, eps, fwd_bytes + bwd_bytes)
        if not args.no_triton_ref:
            line["reference_triton_gpu"] = reference_triton_gpu(wl, rows, fwd_bytes + bwd_bytes)
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(wl, budget_s=args.cpu_seconds)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


def torch_gpu_baseline(wl, x, dy, w, b, eps, step_bytes, reps=10):
    """The same fwd+bwd through torch's own CUDA kernels (F.layer_norm / F.rms_norm with autograd) on
    the same device-resident tensors: the library baseline on this box, reported beside `value`."""
    import torch.nn.functional as F
    N = x.shape[-1]
    try:
        xr = x.detach().requires_grad_(True)
        wr = w.detach().clone().requires_grad_(True)
        br = b.detach().clone().requires_grad_(True) if (wl["op"] == "ln" and b is not None) else None

        def one():
            xr.grad = None
            wr.grad = None
            if br is not None:
                br.grad = None
            y = F.layer_norm(xr, (N,), wr, br, eps) if wl["op"] == "ln" else F.rms_norm(xr, (N,), wr, eps)
            y.backward(dy)

        for _ in range(3):
            one()
        ms = float("inf")
        for _ in range(3):  # the best of three timed loops
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            for _ in range(reps):
                one()
            e.record()
            torch.cuda.synchronize()
            ms = min(ms, s.elapsed_time(e) / reps)
        xr.grad = None
        return {"kind": "torch " + torch.__version__ + (" F.layer_norm" if wl["op"] == "ln" else " F.rms_norm")
                        + " + autograd, CUDA, eager", "value": round(step_bytes / (ms * 1e-3) / 1e9, 1),
                "unit": "GB/s", "ms_per_step": round(ms, 5), "steps": reps, "trials": 3}
    except Exception as exc:  # an out-of-memory error here must not lose the measurement above
        torch.cuda.empty_cache()
        return {"kind": "torch CUDA", "unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}


def reference_triton_gpu(wl, rows, step_bytes, reps=10, timeout_s=420):
    """The reference's own Triton kernels on this GPU (its modules, unmodified, from baseline/_ref),
    timed in a child process by baseline/time_reference_gpu.py: the kernels this library replaces."""
    import subprocess
    kind = "TritonHub 1.1.1 " + ("LayerNorm" if wl["op"] == "ln" else "RMSNorm") + " module (Triton JIT, autotuned), CUDA, eager"
    if rows * wl["N"] >= 2 ** 31:
        # `row * stride_X_row` in the reference's kernels (rmsnorm.py:26-27, layernorm.py:27-28) is 32-bit:
        # from 2^31 elements on it wraps and the kernel reads and writes out of bounds.
        return {"kind": kind, "unavailable": "not run: the reference's kernels index rows with a 32-bit "
                f"row * stride, which overflows at {rows} x {wl['N']} elements (its one run at such a size ended "
                "with a CUDA error)"}
    script = ROOT / "baseline" / "time_reference_gpu.py"
    cmd = [sys.executable, str(script), wl["op"], wl["dtype"], str(rows), str(wl["N"]), str(wl["eps"]),
           str(wl["mu"]), str(wl["sigma"]), str(reps)]
    try:
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout_s)
        last = [ln for ln in res.stdout.splitlines() if ln.startswith("{")]
        if res.returncode != 0 or not last:
            lines = res.stderr.strip().splitlines() or ["no output"]
            named = [ln for ln in lines if "error" in ln.lower()]  # the line that names the error, if any
            return {"kind": kind, "unavailable": f"exit {res.returncode}: {(named[0] if named else lines[-1])[:200]}"}
        out = json.loads(last[-1])
        if "unavailable" in out:
            return {"kind": kind, **out}
        ms = out["ms_per_step"]
        return {"kind": kind + f" (triton {out['triton']})", "value": round(step_bytes / (ms * 1e-3) / 1e9, 1),
                "unit": "GB/s", "ms_per_step": round(ms, 5), "steps": out["steps"], "trials": out.get("trials", 1)}
    except subprocess.TimeoutExpired:
        return {"kind": kind, "unavailable": f"no result within {timeout_s} s"}


def run_e2e(wl, x, dy, w, b, rows, world, device, args):
    """The same step for a caller whose tensors live in pinned HOST memory, through the package's
    host-buffer API (b200norm.HostPipeline): x, dy go up, y, dx, dweight[, dbias] come down, all
    copies inside the timed region."""
    import torch.distributed as dist
    from b200norm import HostPipeline

    ln = wl["op"] == "ln"
    N, eps, dt = wl["N"], wl["eps"], TDTYPE[wl["dtype"]]
    pipe = HostPipeline(wl["op"], N, dt, device, eps, w, b)
    hx, hdy = x.cpu().pin_memory(), dy.cpu().pin_memory()
    hy = torch.empty_like(hx).pin_memory()
    hdx = torch.empty_like(hx).pin_memory()
    hdw = torch.empty((2 if ln else 1, N), dtype=dt).pin_memory()
    steps = max(1, min(args.steps, args.e2e_steps))

    def one():
        dw, db = pipe.run(hx, hdy, hy, hdx)
        hdw[0].copy_(dw, non_blocking=True)
        if ln:
            hdw[1].copy_(db, non_blocking=True)

    for _ in range(2):
        one()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(steps):
        one()
    e.record()
    torch.cuda.synchronize()
    ms = s.elapsed_time(e) / steps
    if world > 1:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = t.item()
    fwd_bytes, bwd_bytes = algorithmic_bytes(wl, rows)
    es = ESIZE[wl["dtype"]]
    # check the pipelined result against the device-resident path once (outside the timed region)
    if ln:
        from b200norm import functional as Fn
        y_ref, _, _ = Fn._layernorm_fwd(x, w, b, eps)
    else:
        from b200norm import functional as Fn
        y_ref, _ = Fn._rmsnorm_fwd(x, w, eps)
    same = bool(torch.equal(y_ref.cpu(), hy))
    return {
        "value": round((fwd_bytes + bwd_bytes) * world / (ms * 1e-3) / 1e9, 2),
        "unit": "GB/s",
        "rows_per_s": round(rows * world / (ms * 1e-3), 1),
        "ms_per_step": round(ms, 4),
        "steps": steps,
        "h2d_bytes_per_step": 2 * rows * N * es,
        "d2h_bytes_per_step": 2 * rows * N * es + (2 if ln else 1) * N * es,
        "pcie_gbs_each_way": round(2 * rows * N * es / (ms * 1e-3) / 1e9, 1),
        "chunk_rows": pipe.chunk_rows,
        "matches_device_path": same,
        "path": "pinned host x, dy -> b200norm.HostPipeline (chunked H2D | fwd+bwd kernels | D2H on three streams) "
                "-> pinned host y, dx, dweight[, dbias]",
    }


def cpu_workload(wl, rows, seed=0):
    from oracle import oracle as O
    rng = np.random.default_rng(seed)
    N = wl["N"]
    x = O.round_to(rng.standard_normal((rows, N), dtype=np.float32) * wl["sigma"] + wl["mu"], wl["dtype"])
    dy = O.round_to(rng.standard_normal((rows, N), dtype=np.float32), wl["dtype"])
    w = O.round_to(1 + 0.1 * rng.standard_normal(N, dtype=np.float32), wl["dtype"])
    b = O.round_to(0.1 * rng.standard_normal(N, dtype=np.float32), wl["dtype"]) if wl["op"] == "ln" else None
    return x, dy, w, b


def cpu_step(wl, x, dy, w, b):
    from oracle import oracle as O
    rms = wl["op"] == "rms"
    y, mean, rstd = O.norm_fwd(x, w, b, wl["eps"], rms=rms)
    return O.norm_bwd(x, dy, w, mean, rstd, rms=rms, programs=148)


def cpu_baseline(wl, budget_s=12.0):
    """The oracle (CPU port of the reference's algorithm) on the host cores, on a bounded row
    sample of the same workload."""
    from oracle import oracle as O
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    rows = min(wl["M"], max(64, (1 << 24) // wl["N"]))
    x, dy, w, b = cpu_workload(wl, rows)
    cpu_step(wl, x, dy, w, b)  # warm-up
    t0 = time.perf_counter()
    reps = 0
    while True:
        cpu_step(wl, x, dy, w, b)
        reps += 1
        if time.perf_counter() - t0 > budget_s or reps >= 200:
            break
    dt = (time.perf_counter() - t0) / reps
    fb, bb = algorithmic_bytes(wl, rows)
    O.set_threads(1)
    return {"value": round((fb + bb) / dt / 1e9, 3), "unit": "GB/s", "cores": cores, "kind": "port",
            "rows_per_s": round(rows / dt, 1),
            "sample": f"{rows} rows x {wl['N']} of the same workload, {reps} reps of fwd+bwd, mean time "
                      f"{dt * 1e3:.1f} ms; oracle/norm_oracle.c on {cores} POSIX threads; bytes counted at the "
                      f"workload's storage width"}


def run_reference(args):
    """Reference arm: the CPU port of the reference's algorithm with every host thread, on a
    bounded row sample per step of the same workload.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import oracle as O
    wl = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    O.set_threads(cores)
    rows = min(wl["M"], max(64, (1 << 24) // wl["N"]))
    x, dy, w, b = cpu_workload(wl, rows)
    for _ in range(max(1, min(args.warmup, 3))):
        cpu_step(wl, x, dy, w, b)
    K = max(1, min(args.steps, 50))
    t0 = time.perf_counter()
    for _ in range(K):
        cpu_step(wl, x, dy, w, b)
    dt = (time.perf_counter() - t0) / K
    fb, bb = algorithmic_bytes(wl, rows)
    value = round((fb + bb) / dt / 1e9, 3)
    sample = (f"{rows} rows x {wl['N']} per step (bounded sample of {args.workload}); oracle/norm_oracle.c, the CPU "
              f"port of the reference's kernels, on {cores} POSIX threads; the reference itself has no CPU path")
    line = {
        "impl": "reference", "metric": "LN/RMSNorm fwd+bwd achieved HBM GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": K, "warmup": max(1, min(args.warmup, 3)), "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": wl["dtype"] + " storage, fp32 arithmetic", "data": "synthetic (seeded)",
        "config": {"workload": f"{args.workload}: {wl['desc']} fwd+bwd, eps={wl['eps']}", "rows_per_step": rows,
                   "dim": wl["N"]},
        "rows_per_s": round(rows / dt, 1),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--rows", type=int, default=0, help="override the workload's row count (profiling on a smaller case)")
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--g-invariant", action="store_true",
                    help="push exchange over 8 fixed row shards: dweight/dbias bit-identical for any GPU count")
    ap.add_argument("--exchange", default="push", choices=["push", "all_reduce", "all_gather"],
                    help="multi-GPU dweight/dbias exchange: push = column reduce fused with stores into every "
                         "rank's inbox over NVLink peer memory (bit-exact, G-invariant); all_reduce / all_gather = "
                         "NCCL collectives on a side stream")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--graph", dest="graph", action="store_true", default=True,
                    help="time a CUDA-graph replay of the step (single GPU; default)")
    ap.add_argument("--no-graph", dest="graph", action="store_false", help="time eager launches instead")
    ap.add_argument("--act", default="none", choices=["none", "gelu", "gelu_tanh"],
                    help="time norm -> GeLU (the reference's Quick Start pair) instead of the norm alone")
    ap.add_argument("--unfused", action="store_true", help="with --act: run norm and GeLU as separate kernels")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-torch", action="store_true", help="skip the torch CUDA baseline (gpu_baseline)")
    ap.add_argument("--no-triton-ref", action="store_true",
                    help="skip timing the reference's Triton kernels on the GPU (reference_triton_gpu)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
