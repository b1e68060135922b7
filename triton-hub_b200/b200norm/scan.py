"""Throughput scan of the kernels over row lengths, storage types and ops.

    python -m b200norm.scan [--ops ln rms softmax logsoftmax ln_gelu normalize pnorm] [--dtypes bf16 fp32] [--dims 1024 4096 ...]

For every combination the forward and the backward are captured into a CUDA graph each (through
the same wrappers users call) and replayed 20 times between two CUDA events; tensors hold 1 GiB
each (far beyond the 126 MB L2).  Prints achieved algorithmic GB/s and the fraction of `--peak`
(default: the copy bandwidth measured on this pool's B200s, 6551.4 GB/s).
"""
from __future__ import annotations

import argparse

import torch

from . import activations as A
from . import functional as Fn
from . import ops as P
from . import softmax as S

DT = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "fp64": torch.float64}


def _time(fn, reps=20):
    for _ in range(3):
        fn()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        keep = fn()  # noqa: F841  (outputs live in the graph's pool)
    for _ in range(3):
        g.replay()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(reps):
        g.replay()
    e.record()
    torch.cuda.synchronize()
    return s.elapsed_time(e) / reps


def scan_one(op, dtype, N, dev, gib=1.0):
    es = torch.empty((), dtype=dtype).element_size()
    M = max(1024, int(gib * (1 << 30)) // (N * es))
    x = torch.randn(M, N, device=dev).to(dtype)
    dy = torch.randn(M, N, device=dev).to(dtype)
    w = torch.randn(N, device=dev).to(dtype)
    b = torch.randn(N, device=dev).to(dtype)
    if op in ("ln", "rms"):
        fwd = (lambda: Fn._layernorm_fwd(x, w, b, 1e-5)) if op == "ln" else (lambda: Fn._rmsnorm_fwd(x, w, 1e-5))
        out = fwd()
        bwd = ((lambda: Fn._layernorm_bwd(x, dy, w, b, out[1], out[2], 1e-5)) if op == "ln"
               else (lambda: Fn._rmsnorm_bwd(x, dy, w, out[1], 1e-5)))
    elif op in ("ln_gelu", "rms_gelu"):
        base = op.split("_")[0]
        fwd = lambda: A._norm_gelu_fwd(base, x, w, b, 1e-5, "none")
        out = fwd()
        bwd = lambda: A._norm_gelu_bwd(base, x, dy, w, b, out[1], out[2], 1e-5, "none")
    elif op in ("softmax", "logsoftmax"):
        log = op == "logsoftmax"
        fwd = lambda: S._fwd(x, log)
        y = fwd()
        bwd = lambda: S._bwd(y, dy, log)
    elif op == "normalize":  # p = 2: forward x -> y (2 row passes), backward y, dout -> dx (3)
        x3, dy3 = x.reshape(1, M, N), dy.reshape(1, M, N)
        fwd = lambda: P._normalize_fwd(x3, 2, 1e-12)
        y3, norms = fwd()
        bwd = lambda: P._normalize_bwd(x3, y3, norms, dy3, 2)
    elif op == "pnorm":      # p = 2: forward reads x (1 row pass), backward x -> dx (2)
        x3 = x.reshape(1, M, N)
        gn = torch.rand(1, M, device=dev).to(dtype)
        fwd = lambda: P._norm_fwd(x3, 2, 1e-12)
        norms = fwd()
        bwd = lambda: P._norm_bwd(x3, norms, gn, 2)
    else:
        raise ValueError(op)
    f_ms, b_ms = _time(fwd), _time(bwd)
    fp, bp = (1, 2) if op == "pnorm" else (2, 3)  # row passes forward / backward
    f_gbs, b_gbs = M * fp * N * es / f_ms / 1e6, M * bp * N * es / b_ms / 1e6
    tot = M * (fp + bp) * N * es / (f_ms + b_ms) / 1e6
    return M, f_gbs, b_gbs, tot


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ops", nargs="+", default=["ln", "rms"])
    ap.add_argument("--dtypes", nargs="+", default=["bf16", "fp32"])
    ap.add_argument("--dims", nargs="+", type=int,
                    default=[128, 512, 1024, 2048, 4096, 5120, 8192, 12288, 16384])
    ap.add_argument("--peak", type=float, default=6551.4)
    ap.add_argument("--gib", type=float, default=1.0, help="size of each (M, N) tensor")
    args = ap.parse_args()
    dev = torch.device("cuda", 0)
    for dn in args.dtypes:
        for op in args.ops:
            for N in args.dims:
                if N * torch.empty((), dtype=DT[dn]).element_size() > 65536:
                    continue
                M, f, b, t = scan_one(op, DT[dn], N, dev, args.gib)
                print(f"{dn} {op:10s} N={N:6d} M={M:8d} fwd {f:7.0f} ({f / args.peak:4.2f}) "
                      f"bwd {b:7.0f} ({b / args.peak:4.2f}) fwd+bwd {t:7.0f} ({t / args.peak:4.2f})", flush=True)


if __name__ == "__main__":
    main()
