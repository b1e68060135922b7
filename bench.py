#!/usr/bin/env python
"""LayerNorm / RMSNorm forward + backward benchmark.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One step = one forward + one backward (dx, dweight[, dbias]) over the workload's rows.  The
metric is achieved algorithmic HBM bandwidth in GB/s, whole job (all ranks); rows/s rides
along.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank works on
its own rows; the backward's column reduce pushes the fp32 dweight / dbias shard sums into every
rank's inbox over NVLink peer memory and finishes the previous step's exchange.  The line then also
carries a bit-exactness check of dweight / dbias (`determinism`) and the two row-sharded
configurations under strong scaling (`also`).

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
# The ops built around the norm path (custom workloads only): row passes forward, backward.
# softmax / logsoftmax: x -> y; y, dout -> dx.  normalize (p = 2): x -> y; y, dout -> dx.  pnorm (p = 2): x -> (M,); x -> dx.
WIDENED_OPS = {"softmax": (2, 3), "logsoftmax": (2, 3), "normalize": (2, 3), "pnorm": (1, 2)}
TDTYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp64": torch.float64}
ESIZE = {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}
FALLBACK_HBM_GBS = 6650.0


def algorithmic_bytes(wl, rows):
    """Bytes the path must move for `rows` rows: forward reads x, writes y and the statistics;
    backward reads x, dy and the statistics, writes dx; plus the parameter vectors once."""
    N, s = wl["N"], ESIZE[wl["dtype"]]
    if wl["op"] in WIDENED_OPS:   # no parameters; forward / backward row passes of each op
        fp, bp = WIDENED_OPS[wl["op"]]
        return rows * fp * N * s, rows * bp * N * s
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


def load_traffic():
    """DRAM traffic per row of the dominant kernel from the ncu captures summarised under profiles/
    (profiles/traffic.json: written beside the summaries by the step that reads the captures)."""
    try:
        return json.loads((ROOT / "profiles" / "traffic.json").read_text())
    except Exception:
        return {}


class Measurement:
    """One workload on this rank's rows: set-up, warm-up, timed blocks, kernel split.

    The step is forward + backward (+ column reduce); with several ranks the column reduce pushes the
    shard sums into every rank's inbox and finishes the PREVIOUS step's exchange in the same kernel, so
    a step is three launches at any GPU count.  The step is captured once into a CUDA graph through
    the public wrappers and replayed (exchange numbers live on the device); --no-graph times eager
    launches instead.
    """

    def __init__(self, name, wl, scaling, args, device, world, rank, act=None, unfused=False, g_invariant=False):
        import torch.distributed as dist
        from b200norm import activations as Act
        from b200norm import functional as Fn
        self.dist, self.Fn, self.Act = dist, Fn, Act
        self.name, self.wl, self.args, self.device, self.world, self.rank = name, wl, args, device, world, rank
        self.ln = wl["op"] == "ln"
        self.total_rows = wl["M"] * (world if scaling == "weak" else 1)
        if self.total_rows % world:
            raise SystemExit(f"{self.total_rows} rows do not divide over {world} ranks")
        self.rows = self.total_rows // world
        self.N, self.eps = wl["N"], wl["eps"]
        self.x, self.dy, self.w, self.b = make_device_inputs(wl, self.rows, device, seed=1000 + rank)
        self.fwd_bytes, self.bwd_bytes = algorithmic_bytes(wl, self.rows)
        if wl["op"] == "pnorm":     # the upstream gradient of the (1, M) norms
            self.gnorm = self.dy[:, 0].contiguous().reshape(1, -1)
        self.approx = {"gelu": "none", "gelu_tanh": "tanh"}.get(act)
        self.unfused = unfused
        self.exchange = None
        if world > 1 or args.push_on_one_gpu:
            from b200norm.parallel import GradExchange, PushExchange
            self.exchange = (PushExchange(max_n=self.N, slots=2, device=device,
                                          total_shards=8 if g_invariant else None, device_numbering=args.graph)
                             if args.exchange == "push" else GradExchange(mode=args.exchange))
        self.push = self.exchange is not None and args.exchange == "push"

    # -- pieces of a step ------------------------------------------------------------------------
    def forward(self):
        Fn, Act, x, w, b, eps = self.Fn, self.Act, self.x, self.w, self.b, self.eps
        op = self.wl["op"]
        if op in WIDENED_OPS:
            from b200norm import ops as P
            from b200norm import softmax as S
            if op in ("softmax", "logsoftmax"):
                return (S._fwd(x, op == "logsoftmax"),)
            x3 = x.reshape(1, *x.shape)
            return P._normalize_fwd(x3, 2, 1e-12) if op == "normalize" else (P._norm_fwd(x3, 2, 1e-12),)
        if self.approx is not None:
            if self.unfused:
                if self.ln:
                    yy, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
                else:
                    (yy, rstd), mean = Fn._rmsnorm_fwd(x, w, eps), None
                return (Act._gelu_fwd(yy, self.approx), mean, rstd, yy)
            return Act._norm_gelu_fwd("ln" if self.ln else "rms", x, w, b, eps, self.approx) + (None,)
        if self.ln:
            return Fn._layernorm_fwd(x, w, b, eps) + (None,)
        y, rstd = Fn._rmsnorm_fwd(x, w, eps)
        return (y, None, rstd, None)

    def backward(self, saved, pending=None):
        """-> (outputs, handle of the exchange this call pushed or None).  `pending`: the previous
        step's exchange, finished here (push mode: inside the column reduce; NCCL modes: a wait)."""
        Fn, Act, x, dy, w, b, eps = self.Fn, self.Act, self.x, self.dy, self.w, self.b, self.eps
        op = self.wl["op"]
        if op in WIDENED_OPS:
            from b200norm import ops as P
            from b200norm import softmax as S
            if op in ("softmax", "logsoftmax"):
                return S._bwd(saved[0], dy, op == "logsoftmax"), None
            x3, dy3 = x.reshape(1, *x.shape), dy.reshape(1, *dy.shape)
            if op == "normalize":
                return P._normalize_bwd(x3, saved[0], saved[1], dy3, 2), None
            return P._norm_bwd(x3, saved[0], self.gnorm, 2), None
        _, mean, rstd, yy = saved
        if self.approx is not None:
            if self.unfused:
                dyy = Act._gelu_bwd(yy, dy, self.approx)
                return (Fn._layernorm_bwd(x, dyy, w, b, mean, rstd, eps) if self.ln
                        else Fn._rmsnorm_bwd(x, dyy, w, rstd, eps)), None
            return Act._norm_gelu_bwd("ln" if self.ln else "rms", x, dy, w, b, mean, rstd, eps, self.approx), None
        if self.exchange is None:
            return (Fn._layernorm_bwd(x, dy, w, b, mean, rstd, eps) if self.ln
                    else Fn._rmsnorm_bwd(x, dy, w, rstd, eps)), None
        ex = self.exchange
        if self.push:
            fin = None if pending is None else (pending, w.dtype)
            res = (ex.backward_layernorm(x, dy, w, b, mean, rstd, eps, finish=fin) if self.ln
                   else ex.backward_rmsnorm(x, dy, w, rstd, eps, finish=fin))
            return res, res[1]
        from b200norm.parallel import sharded_layernorm_bwd, sharded_rmsnorm_bwd
        dx, h = (sharded_layernorm_bwd(x, dy, w, b, mean, rstd, eps, ex) if self.ln
                 else sharded_rmsnorm_bwd(x, dy, w, rstd, eps, ex))
        grads = ex.finish(pending, w.dtype) if pending is not None else None
        return (dx, grads), h

    def close(self, pending):
        """Finish the last open exchange (a kernel of its own)."""
        if pending is not None:
            return self.exchange.finish(pending, self.w.dtype)

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, values):
        if self.world == 1:
            return list(values)
        t = torch.tensor(list(values), device=self.device, dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return t.tolist()

    # -- timing ----------------------------------------------------------------------------------
    def run(self, K, warmup, sampler=None, min_seconds=0.25, max_blocks=400):
        """Warm-up, then blocks of exactly K steps, each between a CUDA-event pair on the launching
        stream; blocks repeat until the timed region lasts `min_seconds` (so that clock samples fall
        inside it) and the MEDIAN block is reported.  All ranks start together (barrier + synchronize)
        and the block times are the max over ranks."""
        graph_mode = self.args.graph and (self.exchange is None or self.push)
        pend = None
        for _ in range(max(warmup, 3)):
            saved = self.forward()
            _, pend = self.backward(saved, pend)
        self.close(pend)
        self.barrier()

        # eager loop: the time a caller launching every kernel from Python sees
        KE = K if not graph_mode else min(K, 50)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        pend = None
        for _ in range(KE):
            saved = self.forward()
            _, pend = self.backward(saved, pend)
        self.close(pend)
        ev[1].record()
        torch.cuda.synchronize()
        eager_ms = ev[0].elapsed_time(ev[1]) / KE

        if graph_mode:
            pend = None
            if self.push:  # one eager step opens the pipeline; the captured step finishes the step before it
                saved = self.forward()
                _, pend = self.backward(saved, None)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                saved = self.forward()
                self.graph_out, pend_next = self.backward(saved, pend)
            one_step = graph.replay
            for _ in range(3):
                one_step()
        else:
            state = {"pend": None}

            def one_step():
                saved = self.forward()
                _, state["pend"] = self.backward(saved, state["pend"])
        # pilot block: how many blocks make min_seconds
        self.barrier()
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(2)]
        ev[0].record()
        for _ in range(K):
            one_step()
        ev[1].record()
        torch.cuda.synchronize()
        (pilot_ms,) = self.max_over_ranks([ev[0].elapsed_time(ev[1])])
        blocks = int(min(max_blocks, max(1, -(-min_seconds * 1e3 // max(pilot_ms, 1e-3)))))
        marks = [torch.cuda.Event(enable_timing=True) for _ in range(blocks + 1)]
        self.barrier()
        if sampler is not None:
            sampler.window[0] = time.perf_counter()
        marks[0].record()
        for i in range(blocks):
            for _ in range(K):
                one_step()
            marks[i + 1].record()
        torch.cuda.synchronize()
        if sampler is not None:
            sampler.window[1] = time.perf_counter()
        if graph_mode and self.push:
            self.close(pend_next)
        elif not graph_mode:
            self.close(state["pend"])
        self.barrier()
        per_block = [marks[i].elapsed_time(marks[i + 1]) for i in range(blocks)]
        per_block = self.max_over_ranks(per_block)          # each block: the slowest rank
        block_ms = float(np.median(per_block))

        fwd_ms, bwd_ms = self.split(graph_mode, min(K, 100))
        return {"ms_per_step": block_ms / K, "eager_ms": eager_ms, "fwd_ms": fwd_ms, "bwd_ms": bwd_ms,
                "blocks": blocks, "block_ms": [round(min(per_block), 5), round(block_ms, 5), round(max(per_block), 5)],
                "graph": graph_mode}

    def split(self, graph_mode, KS):
        """Forward and backward (+ column reduce [+ push + finish of the previous exchange]) timed apart:
        each captured into its own graph and replayed with an event between them, median over the steps
        (eager launches with --no-graph or an NCCL exchange)."""
        evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(KS)]
        pend = None
        if graph_mode:
            if self.push:
                saved = self.forward()
                _, pend = self.backward(saved, None)
            g_fwd, g_bwd = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_fwd):
                saved = self.forward()
            with torch.cuda.graph(g_bwd):
                self.split_out, pend = self.backward(saved, pend)
            for _ in range(3):
                g_fwd.replay()
                g_bwd.replay()
            self.barrier()
            for e in evs:
                e[0].record()
                g_fwd.replay()
                e[1].record()
                g_bwd.replay()
                e[2].record()
        else:
            self.barrier()
            for e in evs:
                e[0].record()
                saved = self.forward()
                e[1].record()
                _, pend = self.backward(saved, pend)
                e[2].record()
        self.close(pend)
        torch.cuda.synchronize()
        fwd = float(np.median([e[0].elapsed_time(e[1]) for e in evs]))
        bwd = float(np.median([e[1].elapsed_time(e[2]) for e in evs]))
        return self.max_over_ranks([fwd, bwd])

    def module_eager_ms(self, reps=50):
        """The public module path: LayerNorm / RMSNorm(...)(x).backward(dy), every launch from Python
        through autograd.Function."""
        import b200norm
        x = self.x.detach().requires_grad_(True)
        dt = x.dtype
        mod = (b200norm.LayerNorm(self.N, eps=self.eps, device=self.device, dtype=dt) if self.ln
               else b200norm.RMSNorm(self.N, eps=self.eps, device=self.device, dtype=dt))
        with torch.no_grad():
            mod.weight.copy_(self.w)
            if self.ln:
                mod.bias.copy_(self.b)

        def one():
            x.grad = None
            mod.weight.grad = None
            if self.ln:
                mod.bias.grad = None
            mod(x).backward(self.dy)

        for _ in range(5):
            one()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(reps):
            one()
        e.record()
        torch.cuda.synchronize()
        x.grad = None
        return s.elapsed_time(e) / reps

    def summary(self, res, peak):
        step_bytes = self.fwd_bytes + self.bwd_bytes
        value = step_bytes * self.world / (res["ms_per_step"] * 1e-3) / 1e9
        return {"value": round(value, 1), "unit": "GB/s", "ms_per_step": round(res["ms_per_step"], 5),
                "frac_of_peak_per_gpu": round(value / self.world / peak, 4),
                "rows_per_s": round(self.total_rows / (res["ms_per_step"] * 1e-3), 1),
                "rows_per_gpu": self.rows, "rows_total": self.total_rows,
                "fwd_ms": round(res["fwd_ms"], 5), "fwd_frac": round(self.fwd_bytes / (res["fwd_ms"] * 1e-3) / 1e9 / peak, 4),
                "bwd_ms": round(res["bwd_ms"], 5), "bwd_frac": round(self.bwd_bytes / (res["bwd_ms"] * 1e-3) / 1e9 / peak, 4),
                "timed_blocks": res["blocks"]}


def determinism_check(args, wl, device, world, rank):
    """BASELINE config 5's check, outside every timed region: one row-sharded backward over 8 fixed row
    shards on a seeded global batch that every rank can rebuild; dweight / dbias must be bit-identical
    on all ranks, and bit-identical to THIS GPU running the whole batch alone with row_shards = 8; no
    bounded wait may have run out on any rank."""
    import torch.distributed as dist
    from b200norm import _lib
    from b200norm import functional as Fn
    from b200norm.parallel import PushExchange, shard_bounds
    ln, N, eps = wl["op"] == "ln", wl["N"], wl["eps"]
    small = dict(wl)
    M = 8 * 512
    x, dy, w, b = make_device_inputs(small, M, device, seed=777)    # the same global batch on every rank
    r0, r1 = shard_bounds(M, world, rank)
    px = PushExchange(max_n=N, slots=2, device=device, total_shards=8)
    outs = []
    for _ in range(2):          # twice: run to run as well
        if ln:
            _, mean, rstd = Fn._layernorm_fwd(x[r0:r1], w, b, eps)
            _, _, grads = px.backward_layernorm(x[r0:r1], dy[r0:r1], w, b, mean, rstd, eps,
                                                finish=(PushExchange.SAME, w.dtype))
        else:
            _, rstd = Fn._rmsnorm_fwd(x[r0:r1], w, eps)
            _, _, grads = px.backward_rmsnorm(x[r0:r1], dy[r0:r1], w, rstd, eps, finish=(PushExchange.SAME, w.dtype))
        outs.append(torch.stack([g.float() for g in grads]))
    if ln:
        _, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
        alone = Fn._layernorm_bwd(x, dy, w, b, mean, rstd, eps, row_shards=8)[1:3]
    else:
        _, rstd = Fn._rmsnorm_fwd(x, w, eps)
        alone = Fn._rmsnorm_bwd(x, dy, w, rstd, eps, row_shards=8)[1:2]
    alone = torch.stack([g.float() for g in alone])
    torch.cuda.synchronize()
    gathered = [torch.empty_like(outs[0]) for _ in range(world)]
    dist.all_gather(gathered, outs[0])
    status = _lib.load().b200norm_device_status(0)
    flags = torch.tensor([float(torch.equal(outs[0], alone) and torch.equal(outs[1], alone)),
                          float(all(torch.equal(g, gathered[0]) for g in gathered)), -float(status)],
                         device=device, dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    vs_one, across, st = flags.tolist()
    return {"across_ranks": bool(across), "vs_one_gpu": bool(vs_one), "status": int(-st),
            "what": f"{wl['op']} {wl['dtype']} {M} x {N} global rows over {world} ranks, total_shards = 8, run twice; "
                    "compared with the same rows on one GPU (row_shards = 8) on every rank, bit for bit"}


def run_gpu(args):
    import torch.distributed as dist
    from b200norm import _lib

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

    wl = workload(args)
    if wl["op"] in WIDENED_OPS:      # kernel timing only: no host pipeline, module path or baselines for these
        if world > 1 or args.act != "none":
            raise SystemExit(f"--op {wl['op']} is a single-GPU measurement without --act")
        args.no_e2e = args.no_module = args.no_torch = args.no_cpu = True
    if args.act != "none" and world > 1:
        raise SystemExit("--act is a single-GPU measurement")
    peak, peak_src = measured_peak()
    sampler = ClockSampler(local)
    sampler.start()
    K = args.steps
    m = Measurement(args.workload, wl, args.scaling, args, device, world, rank, act=args.act, unfused=args.unfused,
                    g_invariant=args.g_invariant)
    res = m.run(K, args.warmup, sampler, min_seconds=args.min_seconds)
    sampler.stop_flag = True
    sampler.join(timeout=1.0)
    clocks = sampler.summary()
    rows, N, eps, approx = m.rows, m.N, m.eps, m.approx
    fwd_bytes, bwd_bytes = m.fwd_bytes, m.bwd_bytes
    ms_per_step, fwd_ms, bwd_ms = res["ms_per_step"], res["fwd_ms"], res["bwd_ms"]
    if world > 1:   # every rank's clocks, not rank 0's alone
        allc = [None] * world
        dist.all_gather_object(allc, clocks)
        mhz = [c["sm_mhz"] for c in allc if c.get("sm_mhz")]
        clocks["all_ranks"] = {"sm_mhz_min": min(mhz) if mhz else None, "sm_mhz_max": max(mhz) if mhz else None,
                               "reasons": sorted({r for c in allc for r in c.get("reasons", [])})}

    module_ms = m.module_eager_ms() if (world == 1 and approx is None and not args.no_module) else None

    # End to end through the public module-level API with HOST buffers: pinned x / dy in,
    # y / dx / dweight [/ dbias] out, copies inside the timed region.
    e2e = None
    if not args.no_e2e and approx is None:
        e2e = run_e2e(wl, m.x, m.dy, m.w, m.b, rows, world, device, args)

    determinism = also = None
    if world > 1 and args.exchange == "push":
        determinism = determinism_check(args, wl, device, world, rank)
        if not args.no_also:
            also = {}
            del m       # this workload's tensors make room for the next ones
            torch.cuda.empty_cache()
            for name in ("c4", "c5_rms"):     # the two row-sharded configurations, strong scaling at this GPU count
                if name == args.workload and args.scaling == "strong":
                    continue
                m2 = Measurement(name, dict(WORKLOADS[name]), "strong", args, device, world, rank)
                r2 = m2.run(min(K, 50), 5, None, min_seconds=0.1)
                also[name + "_strong"] = dict(m2.summary(r2, peak), workload=WORKLOADS[name]["desc"])
                del m2
                torch.cuda.empty_cache()
    value = (fwd_bytes + bwd_bytes) * world / (ms_per_step * 1e-3) / 1e9
    bwd_gbs = bwd_bytes / (bwd_ms * 1e-3) / 1e9
    fwd_gbs = fwd_bytes / (fwd_ms * 1e-3) / 1e9
    launches_per_step = 3  # forward, backward, column reduce (which with several GPUs also pushes and finishes)
    if world > 1 and args.exchange != "push":
        launches_per_step += 1  # the finalize kernel after the NCCL collective
    if approx is not None and args.unfused:
        launches_per_step += 2  # the two stand-alone GeLU kernels
    traffic = load_traffic().get(args.workload)  # per row: valid for any row count
    total_rows = rows * world
    graph_mode = res["graph"]
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
                            + ("column reduce fused with a push of tagged entries into every rank's inbox over NVLink "
                               "peer memory; the same kernel finishes the previous step's exchange"
                               if args.exchange == "push"
                               else f"NCCL {args.exchange} on a side stream, overlapped with the next step's launches"))
            if world > 1
            else "single GPU",
        },
        "launch_mode": ("cuda graph of one step (captured through the public wrappers), replayed per step"
                        if graph_mode else "eager: every kernel launched from Python"),
        "timed_blocks": res["blocks"],
        "block_ms_min_median_max": res["block_ms"],
        "timing": f"{res['blocks']} back-to-back blocks of exactly {K} steps, each between CUDA events on the launching "
                  "stream after a barrier + synchronize; every block is the max over ranks; ms_per_step = median block / steps",
        "eager_ms_per_step": round(res["eager_ms"], 5),
        "rows_per_s": round(total_rows / (ms_per_step * 1e-3), 1),
        "frac_of_peak": round(value / world / peak, 4),
        "frac_of_nominal_8000": round(value / world / 8000.0, 4),
        "peak_gbs_per_gpu": peak,
        "peak_source": peak_src,
        "roofline": {
            "bound": "hbm",
            "kernel": ("norm_bwd_kernel (+ the column reduce, same event pair)" if wl["op"] not in WIDENED_OPS
                       else f"the backward kernel of {wl['op']}"),
            "timed_by": ("CUDA events around a graph replay of the backward alone, median of the steps" if graph_mode
                         else "CUDA events around the backward call in an eager loop, median of the steps"),
            "achieved": round(bwd_gbs, 1),
            "peak": peak,
            "unit": "GB/s",
            "frac": round(bwd_gbs / peak, 4),
            "traffic": round(traffic["bwd_dram_bytes_per_row"] * rows) if traffic else None,
            "traffic_source": (f"ncu dram__bytes_read.sum + dram__bytes_write.sum of norm_bwd_kernel on {traffic['rows']} rows "
                               f"({traffic['summary']}, build {traffic['commit']}), scaled by the row count; writes still "
                               "dirty in L2 at kernel end are not in it" if traffic else None),
            "bytes_per_launch": bwd_bytes,
            "ms_per_launch": round(bwd_ms, 5),
            "fwd_kernel": {"achieved": round(fwd_gbs, 1), "frac": round(fwd_gbs / peak, 4),
                           "bytes_per_launch": fwd_bytes, "ms_per_launch": round(fwd_ms, 5)},
            "peak_source": peak_src,
        },
        "clocks": clocks,
        "gpu_launches": launches_per_step * K * res["blocks"],
        "gpu_launches_per_step": launches_per_step,
    }
    if module_ms is not None:
        line["module_eager_ms_per_step"] = round(module_ms, 5)
    if e2e is not None:
        line["e2e"] = e2e
    if determinism is not None:
        line["determinism"] = determinism
    if also:
        line["also"] = also
    if world == 1 and approx is None and not args.no_torch:
        line["gpu_baseline"] = torch_gpu_baseline(wl, m.x, m.dy, m.w, m.b, eps, fwd_bytes + bwd_bytes)
        if not args.no_triton_ref:
            line["reference_triton_gpu"] = reference_triton_gpu(wl, rows, fwd_bytes + bwd_bytes)
    if rank == 0 and world == 1 and not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(wl, budget_s=args.cpu_seconds)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


def workload(args):
    """The workload of this run: a named one, optionally with another row count, or --workload custom."""
    if args.workload == "custom":
        if not (args.op and args.dtype and args.dim and args.rows):
            raise SystemExit("--workload custom needs --op, --dtype, --dim and --rows")
        names = {"ln": "LayerNorm", "rms": "RMSNorm", "softmax": "Softmax", "logsoftmax": "LogSoftmax",
                 "normalize": "Ops.normalize (p=2)", "pnorm": "Ops.norm (p=2)"}
        return dict(op=args.op, dtype=args.dtype, M=args.rows, N=args.dim, eps=1e-5, mu=0.0, sigma=1.0,
                    desc=f"{names[args.op]} {args.dtype} ({args.rows},{args.dim})")
    wl = dict(WORKLOADS[args.workload])
    if args.rows > 0:
        wl["M"] = args.rows
        wl["desc"] += f" cut to {args.rows} rows"
    return wl


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
    pipe = HostPipeline(wl["op"], N, dt, device, eps, w, b, rows_hint=rows)
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
    # three blocks of `steps` steps, each the max over ranks; the median block is reported (the host link is
    # shared with the machine's other GPUs: a block that collides with a neighbour's burst reads several
    # times slower)
    block_ms = []
    for _ in range(3):
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
        block_ms.append(ms)
    ms = sorted(block_ms)[1]
    fwd_bytes, bwd_bytes = algorithmic_bytes(wl, rows)
    es = ESIZE[wl["dtype"]]
    ceiling = pcie_ceiling(hx, hdy, hy, hdx, pipe, device, world)
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
        "block_ms_per_step_min_median_max": [round(v, 4) for v in sorted(block_ms)],
        "h2d_bytes_per_step": 2 * rows * N * es,
        "d2h_bytes_per_step": 2 * rows * N * es + (2 if ln else 1) * N * es,
        "pcie_gbs_each_way": round(2 * rows * N * es / (ms * 1e-3) / 1e9, 1),
        "pcie_ceiling_gbs_each_way": ceiling,
        "pcie_ceiling_how": "the same pinned buffers copied up and down at the same time on two streams with no "
                            "kernels in between (all ranks at once, slowest rank): what the host link gives this "
                            "many ranks at best",
        "chunk_rows": pipe.chunk_rows,
        "matches_device_path": same,
        "path": "pinned host x, dy -> b200norm.HostPipeline (chunked H2D | fwd+bwd kernels | D2H on three streams) "
                "-> pinned host y, dx, dweight[, dbias]",
    }


def pcie_ceiling(hx, hdy, hy, hdx, pipe, device, world, reps=3):
    """Bare copies of the end-to-end step's bytes: x, dy up on one stream while as many bytes come down
    on another, chunked like the pipeline, nothing else running.  GB/s each way, slowest rank."""
    import torch.distributed as dist
    R = pipe.chunk_rows
    M = hx.shape[0]
    up = [torch.empty((R, hx.shape[1]), dtype=hx.dtype, device=device) for _ in range(2)]
    down = [torch.empty((R, hx.shape[1]), dtype=hx.dtype, device=device) for _ in range(2)]
    s_up, s_down = torch.cuda.Stream(device), torch.cuda.Stream(device)

    def one():
        for r0 in range(0, M, R):
            n = min(R, M - r0)
            with torch.cuda.stream(s_up):
                up[0][:n].copy_(hx[r0:r0 + n], non_blocking=True)
                up[1][:n].copy_(hdy[r0:r0 + n], non_blocking=True)
            with torch.cuda.stream(s_down):
                hy[r0:r0 + n].copy_(down[0][:n], non_blocking=True)
                hdx[r0:r0 + n].copy_(down[1][:n], non_blocking=True)

    keep_y, keep_dx = hy.clone(), hdx.clone()   # the copies overwrite the step's results: put them back afterwards
    one()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        one()
    torch.cuda.synchronize()
    dt = (time.perf_counter() - t0) / reps
    hy.copy_(keep_y)
    hdx.copy_(keep_dx)
    if world > 1:
        t = torch.tensor([dt], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dt = t.item()
    return round(2 * M * hx.shape[1] * hx.element_size() / dt / 1e9, 1)


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
            "rows_per_s": round(rows / dt, 1), "torch_cpu": torch_cpu_baseline(wl, x, dy, w, b, fb + bb),
            "sample": f"{rows} rows x {wl['N']} of the same workload, {reps} reps of fwd+bwd, mean time "
                      f"{dt * 1e3:.1f} ms; oracle/norm_oracle.c on {cores} POSIX threads; bytes counted at the "
                      f"workload's storage width"}


def torch_cpu_baseline(wl, x, dy, w, b, step_bytes, budget_s=4.0):
    """The comparator the reference's unit tests use (UnitTests/Normalization/layernorm_unittest.py:17,37,46:
    torch.nn.LayerNorm / RMSNorm), run on the host cores with autograd on the same row sample, in the
    workload's storage type."""
    import torch.nn.functional as F
    try:
        dt = TDTYPE[wl["dtype"]]
        N = wl["N"]
        xr = torch.from_numpy(x).to(dt).requires_grad_(True)
        g = torch.from_numpy(dy).to(dt)
        wr = torch.from_numpy(w).to(dt).requires_grad_(True)
        br = torch.from_numpy(b).to(dt).requires_grad_(True) if b is not None else None

        def one():
            xr.grad = wr.grad = None
            if br is not None:
                br.grad = None
            y = F.layer_norm(xr, (N,), wr, br, wl["eps"]) if wl["op"] == "ln" else F.rms_norm(xr, (N,), wr, wl["eps"])
            y.backward(g)

        one()
        t0 = time.perf_counter()
        reps = 0
        while True:
            one()
            reps += 1
            if time.perf_counter() - t0 > budget_s or reps >= 50:
                break
        sec = (time.perf_counter() - t0) / reps
        return {"value": round(step_bytes / sec / 1e9, 3), "unit": "GB/s", "threads": torch.get_num_threads(),
                "kind": "torch " + torch.__version__ + (" F.layer_norm" if wl["op"] == "ln" else " F.rms_norm")
                        + " + autograd on CPU", "reps": reps}
    except Exception as exc:
        return {"unavailable": f"{type(exc).__name__}: {str(exc)[:120]}"}


def run_reference(args):
    """Reference arm: the CPU port of the reference's algorithm with every host thread, on a
    bounded row sample per step of the same workload.  Rank 0 only."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from oracle import oracle as O
    wl = workload(args)
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
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS) + ["custom"])
    ap.add_argument("--rows", type=int, default=0, help="override the workload's row count (profiling on a smaller case)")
    ap.add_argument("--op", choices=["ln", "rms"] + sorted(WIDENED_OPS),
                    help="with --workload custom: the norms, or one of the ops built around them (single GPU, p = 2)")
    ap.add_argument("--dtype", choices=sorted(TDTYPE), help="with --workload custom: storage type")
    ap.add_argument("--dim", type=int, default=0, help="with --workload custom: row length")
    ap.add_argument("--min-seconds", type=float, default=0.25,
                    help="repeat the block of --steps steps until the timed region lasts this long (0: one block)")
    ap.add_argument("--push-on-one-gpu", action="store_true",
                    help="one GPU: run the multi-GPU step (push exchange with world = 1, the pushes land in this "
                         "GPU's own inbox) -- for profiling its kernels, which a profiler can only watch on one GPU")
    ap.add_argument("--no-also", action="store_true",
                    help="several GPUs: skip the c4 / c5 strong-scaling measurements reported under `also`")
    ap.add_argument("--no-module", action="store_true", help="skip timing the public module path (module_eager_ms_per_step)")
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
                    help="time a CUDA-graph replay of the step (default)")
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
