"""Times the UNMODIFIED reference (TritonHub's Triton kernels, installed under baseline/_ref) on
the GPU for one bench workload, through its public modules, and prints one JSON line.

Run as a child process by bench.py so that the reference's `TritonHub` package and this
repository's drop-in package of the same name never share an interpreter:

    python baseline/time_reference_gpu.py ln|rms dtype M N eps mu sigma reps

The first calls trigger the reference's autotuning (five launch shapes per kernel); they are
warm-up.  Timing: CUDA events around `reps` forward+backward steps on device-resident tensors, the
best of three such loops.
"""
import json
import sys
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def main():
    op, dtype_name = sys.argv[1], sys.argv[2]
    M, N = int(sys.argv[3]), int(sys.argv[4])
    eps, mu, sigma = float(sys.argv[5]), float(sys.argv[6]), float(sys.argv[7])
    reps = int(sys.argv[8])
    if M * N >= 2 ** 31:  # the reference's `row * stride` is 32-bit: out-of-bounds accesses from here on
        print(json.dumps({"unavailable": "the reference overflows its 32-bit row offsets at this size"}))
        return
    if not (REF / "TritonHub").is_dir():
        print(json.dumps({"unavailable": "baseline/_ref holds no installed reference"}))
        return
    sys.path.insert(0, str(REF))
    import torch
    import TritonHub
    from TritonHub.Normalization import LayerNorm, RMSNorm  # the reference's own modules
    if not str(Path(TritonHub.__file__).resolve()).startswith(str(REF)):
        print(json.dumps({"unavailable": "another TritonHub package shadows baseline/_ref"}))
        return

    dt = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}[dtype_name]
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(0)
    x = torch.empty((M, N), device=dev, dtype=dt)
    dy = torch.empty((M, N), device=dev, dtype=dt)
    chunk = max(1, (1 << 26) // N)
    for r0 in range(0, M, chunk):
        r1 = min(M, r0 + chunk)
        x[r0:r1] = (torch.randn((r1 - r0, N), device=dev, generator=g) * sigma + mu).to(dt)
        dy[r0:r1] = torch.randn((r1 - r0, N), device=dev, generator=g).to(dt)
    x.requires_grad_(True)
    if op == "ln":
        mod = LayerNorm(N, eps=eps, elementwise_affine=True, bias=True, device=dev, dtype=dt)
    else:
        mod = RMSNorm(N, eps=eps, elementwise_affine=True, device=dev, dtype=dt)

    def one():
        x.grad = None
        for p in mod.parameters():
            p.grad = None
        mod(x).backward(dy)

    for _ in range(3):
        one()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):  # the best of three timed loops: the reference gets the benefit of the doubt
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(reps):
            one()
        e.record()
        torch.cuda.synchronize()
        best = min(best, s.elapsed_time(e) / reps)
    import triton
    print(json.dumps({"ms_per_step": best, "steps": reps, "trials": 3, "triton": triton.__version__,
                      "torch": torch.__version__}))


if __name__ == "__main__":
    main()
