"""Runs the UNMODIFIED reference (TritonHub, installed under baseline/_ref) on the GPU on seeded
inputs and saves what it returns, for a direct comparison with this library's kernels:

    python baseline/run_reference_ops_gpu.py out.npz

Run as a child process (tests/test_reference_on_gpu.py) so that the reference's `TritonHub` package and
this repository's drop-in of the same name never share an interpreter.  Every case stays far
below 2^31 elements: the reference's kernels form row offsets in 32-bit arithmetic.

Cases (inputs drawn on the CPU from torch.Generator(seed), so the test can rebuild them):
  ln / rms      LayerNorm / RMSNorm modules, weight ~ N(1, 0.1), bias ~ N(0, 0.1): y, dx, dweight, dbias
  gelu          GeLU(approximate) after nothing: y, dx
  softmax ...   Softmax / LogSoftmax / Softmin over the last dimension: y, dx
  norm / normalize   Ops.norm / Ops.normalize with p in {1, 2, 2.5, 3}: out, dx
"""
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"

CASES = [  # (name, kind, dtype, shape, extra)
    ("ln_fp32_c1", "ln", "fp32", (2, 100, 128), 1e-6),
    ("ln_bf16", "ln", "bf16", (64, 4096), 1e-6),
    ("ln_fp16_mean3", "ln", "fp16", (48, 5120), 1e-5),
    ("rms_bf16", "rms", "bf16", (64, 4096), 1e-6),
    ("rms_fp32", "rms", "fp32", (33, 1000), 1e-5),
    ("gelu_none_fp32", "gelu", "fp32", (50, 128), "none"),
    ("gelu_tanh_bf16", "gelu", "bf16", (16, 4096), "tanh"),
    ("softmax_fp32", "softmax", "fp32", (20, 333), None),
    ("softmax_fp16", "softmax", "fp16", (9, 1000), None),
    ("logsoftmax_fp32", "logsoftmax", "fp32", (9, 333), None),
    ("softmin_fp32", "softmin", "fp32", (9, 128), None),
    ("norm_p1_fp32", "norm", "fp32", (2, 9, 128), 1.0),
    ("norm_p2_fp32", "norm", "fp32", (2, 9, 333), 2.0),
    ("norm_p2.5_fp32", "norm", "fp32", (2, 9, 333), 2.5),
    ("norm_p3_fp32", "norm", "fp32", (1, 6, 1000), 3.0),
    ("normalize_p1_fp32", "normalize", "fp32", (2, 9, 128), 1.0),
    ("normalize_p2_fp32", "normalize", "fp32", (2, 9, 333), 2.0),
    ("normalize_p2.5_fp32", "normalize", "fp32", (2, 9, 333), 2.5),
    ("normalize_p3_fp32", "normalize", "fp32", (1, 6, 1000), 3.0),
    ("normalize_p3_fp16", "normalize", "fp16", (1, 7, 1000), 3.0),
]


def make_inputs(name, dtype, shape):
    """Seeded on the CPU (the test rebuilds the same tensors): x, dy, w, b as fp32 values already
    rounded to `dtype`."""
    import torch
    dt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[dtype]
    g = torch.Generator().manual_seed(sum(ord(c) for c in name))
    mu, sigma = (3.0, 2.0) if "mean3" in name else (0.0, 1.0)
    x = (torch.randn(shape, generator=g) * sigma + mu).to(dt)
    dy = torch.randn(shape, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(shape[-1], generator=g)).to(dt)
    b = (0.1 * torch.randn(shape[-1], generator=g)).to(dt)
    return x, dy, w, b


def main():
    out_path = sys.argv[1]
    import numpy as np
    import torch
    if not (REF / "TritonHub").is_dir():
        np.savez(out_path, unavailable=np.array("baseline/_ref holds no installed reference"))
        return
    sys.path.insert(0, str(REF))
    import TritonHub
    if not str(Path(TritonHub.__file__).resolve()).startswith(str(REF)):
        np.savez(out_path, unavailable=np.array("another TritonHub package shadows baseline/_ref"))
        return
    from TritonHub.Activations import GeLU, LogSoftmax, Softmax, Softmin
    from TritonHub.Normalization import LayerNorm, RMSNorm
    from TritonHub.Ops import norm, normalize

    dev = torch.device("cuda", 0)
    out = {}

    def keep(name, key, t):
        out[f"{name}/{key}"] = t.detach().float().cpu().numpy()

    def run_case(name, kind, dtype, shape, extra):
        x, dy, w, b = make_inputs(name, dtype, shape)
        x = x.to(dev).requires_grad_(True)
        dy = dy.to(dev)
        dt = x.dtype
        if kind in ("ln", "rms"):
            N = shape[-1]
            mod = (LayerNorm(N, eps=extra, elementwise_affine=True, bias=True, device=dev, dtype=dt) if kind == "ln"
                   else RMSNorm(N, eps=extra, elementwise_affine=True, device=dev, dtype=dt))
            with torch.no_grad():
                mod.weight.copy_(w.to(dev))
                if kind == "ln":
                    mod.bias.copy_(b.to(dev))
            y = mod(x)
            keep(name, "y", y)
            y.backward(dy)
            keep(name, "dx", x.grad), keep(name, "dw", mod.weight.grad)
            if kind == "ln":
                keep(name, "db", mod.bias.grad)
            return
        if kind == "gelu":
            y = GeLU(approximate=extra)(x)
        elif kind in ("softmax", "logsoftmax", "softmin"):
            y = {"softmax": Softmax, "logsoftmax": LogSoftmax, "softmin": Softmin}[kind]()(x)
        elif kind == "norm":
            y = norm(p=extra, eps=1e-6)(x)
        else:
            y = normalize(p=extra, eps=1e-6)(x)
        keep(name, "y", y)           # the forward result is kept even if the backward then fails
        y.backward(dy[..., 0].contiguous() if kind == "norm" else dy)
        keep(name, "dx", x.grad)

    for case in CASES:
        try:
            run_case(*case)
            torch.cuda.synchronize()
        except Exception as exc:     # a case the reference itself cannot run is recorded, not fatal
            out[f"{case[0]}/error"] = np.array(f"{type(exc).__name__}: {str(exc).strip().splitlines()[-1][:160]}")
    import triton
    np.savez(out_path, versions=np.array(f"triton {triton.__version__}, torch {torch.__version__}"), **out)


if __name__ == "__main__":
    main()
