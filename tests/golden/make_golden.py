"""Generate the golden vectors in this directory from the reference implementation.

Run once, where the reference checkout is available (it is not needed to *use* the vectors):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py /path/to/Triton-Hub [--ops-only]

The reference has no stored vectors of its own and its wrappers need a GPU, so this script
executes the reference's four Triton kernel bodies (TritonHub/Normalization/layernorm.py:14-46,
94-153; rmsnorm.py:14-38,77-122) on CPU through Triton's interpreter, restating only the host
glue around them (allocation, BLOCK_SIZE, rows_per_program and the final `.sum(0).to(dtype)`,
layernorm.py:63-72,176-208) with PROGRAMS standing in for the GPU's SM count.  Inputs are
seeded; every case is written to <name>.npz together with what the reference produced.
16-bit tensors are stored as fp16 arrays or bf16 bit patterns (uint16) to keep files small.
"""
import importlib
import math
import os
import sys
from pathlib import Path

os.environ.setdefault("TRITON_INTERPRET", "1")
import numpy as np
import torch

HERE = Path(__file__).resolve().parent
PROGRAMS = 4  # stands in for sm_count (layernorm.py:182)

# name, op, dtype, M-shape, N, eps, x mean, x std, has_weight, has_bias
CASES = [
    ("c1_ln_fp32_2x100x128", "ln", torch.float32, (2, 100), 128, 1e-6, 0.0, 1.0, True, True),
    ("rms_bf16_8x4096", "rms", torch.bfloat16, (8,), 4096, 1e-6, 0.0, 1.0, True, False),
    ("ln_fp16_6x5120_mean3", "ln", torch.float16, (6,), 5120, 1e-5, 3.0, 2.0, True, True),
    ("ln_bf16_3x16384", "ln", torch.bfloat16, (3,), 16384, 1e-6, 0.0, 1.0, True, True),
    ("ln_bf16_8x4096", "ln", torch.bfloat16, (8,), 4096, 1e-6, 0.0, 1.0, True, True),
    ("ln_fp32_7x100_nobias", "ln", torch.float32, (7,), 100, 1e-5, 0.0, 1.0, True, False),
    ("rms_fp32_5x33_noweight", "rms", torch.float32, (5,), 33, 1e-5, 0.0, 1.0, False, False),
    ("ln_fp64_4x64", "ln", torch.float64, (4,), 64, 1e-5, 0.0, 1.0, True, True),
    ("ln_fp16_5x256_noaffine", "ln", torch.float16, (5,), 256, 1e-5, 0.0, 1.0, False, False),
    ("rms_fp16_9x1000", "rms", torch.float16, (9,), 1000, 1e-5, 0.0, 1.0, True, False),
]


def next_pow2(n):
    return 1 << (n - 1).bit_length()


def store(t):
    """torch tensor -> (suffix, numpy array) in a compact, exact form."""
    if t.dtype == torch.bfloat16:
        return "__bf16bits", t.view(torch.int16).numpy().view(np.uint16)
    return "", t.numpy()


def run_case(L, R, name, op, dtype, batch, N, eps, mu, sigma, has_w, has_b):
    g = torch.Generator().manual_seed(0)
    M = int(np.prod(batch))
    x = (torch.randn(M, N, generator=g) * sigma + mu).to(dtype)
    dy = torch.randn(M, N, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype) if has_w else None
    b = (0.1 * torch.randn(N, generator=g)).to(dtype) if has_b else None
    BLOCK = min(65536 // x.element_size(), next_pow2(N))
    y = torch.empty_like(x)
    rstd = torch.empty(M, dtype=torch.float32)
    dx = torch.empty_like(x)
    rpp = math.ceil(M / PROGRAMS)
    dwp = torch.empty(PROGRAMS, N, dtype=torch.float32) if has_w else None
    out = {}
    if op == "ln":
        mean = torch.empty(M, dtype=torch.float32)
        L._layernorm_kernel_fwd.fn[(M,)](x, x.stride(0), y, y.stride(0), w, b, mean, rstd, eps, N,
                                         BLOCK_SIZE=BLOCK, HAS_WEIGHT=has_w, HAS_BIAS=has_b)
        dbp = torch.empty(PROGRAMS, N, dtype=torch.float32) if has_b else None
        L._layernorm_kernel_bwd.fn[(PROGRAMS,)](x, x.stride(0), dy, dy.stride(0), dx, dx.stride(0), w, b, dwp, dbp,
                                                mean, rstd, eps, M, N, rpp, BLOCK_SIZE=BLOCK, HAS_WEIGHT=has_w,
                                                HAS_BIAS=has_b)
        out["mean"] = mean.numpy()
        if has_b:
            k, v = store(dbp.sum(0).to(b.dtype))
            out["db" + k] = v
    else:
        R._rmsnorm_kernel_fwd.fn[(M,)](x, x.stride(0), y, y.stride(0), w, rstd, eps, N, BLOCK_SIZE=BLOCK,
                                       HAS_WEIGHT=has_w)
        R._rmsnorm_kernel_bwd.fn[(PROGRAMS,)](x, x.stride(0), dy, dy.stride(0), dx, dx.stride(0), w, dwp, rstd, eps,
                                              M, N, rpp, BLOCK_SIZE=BLOCK, HAS_WEIGHT=has_w)
    out["rstd"] = rstd.numpy()
    for key, t in (("x", x), ("dy", dy), ("w", w), ("b", b), ("y", y), ("dx", dx)):
        if t is not None:
            k, v = store(t)
            out[key + k] = v
    if has_w:
        k, v = store(dwp.sum(0).to(w.dtype))
        out["dw" + k] = v
    out["meta"] = np.array([op, str(dtype).replace("torch.", ""), str(eps), str(PROGRAMS),
                            "x".join(map(str, batch))])
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok", sum(v.nbytes for v in out.values()) // 1024, "KiB raw")


# GeLU (TritonHub/Activations/gelu.py): name, dtype, M, N, approximate
GELU_CASES = [
    ("gelu_fp32_50x128_none", torch.float32, 50, 128, "none"),
    ("gelu_fp32_50x128_tanh", torch.float32, 50, 128, "tanh"),
    ("gelu_fp16_7x1000_none", torch.float16, 7, 1000, "none"),
    ("gelu_bf16_4x4096_tanh", torch.bfloat16, 4, 4096, "tanh"),
]
# LayerNorm -> GeLU as in the Quick Start (README.md:44-48), forward and backward through both of the
# reference's kernel pairs: name, dtype, batch, N, eps, approximate
CHAIN_CASES = [
    ("quickstart_ln_gelu_fp32_2x100x128_none", torch.float32, (2, 100), 128, 1e-6, "none"),
    ("ln_gelu_bf16_8x4096_tanh", torch.bfloat16, (8,), 4096, 1e-6, "tanh"),
]


# Softmax family (TritonHub/Activations/softmax.py, logsoftmax.py): name, kind, dtype, M, N
SOFTMAX_CASES = [
    ("softmax_fp32_20x128", "softmax", torch.float32, 20, 128),
    ("softmax_fp16_6x1000", "softmax", torch.float16, 6, 1000),
    ("logsoftmax_fp32_9x333", "logsoftmax", torch.float32, 9, 333),
    ("logsoftmax_bf16_4x4096", "logsoftmax", torch.bfloat16, 4, 4096),
]


def run_softmax(S, LS, name, kind, dtype, M, N):
    g = torch.Generator().manual_seed(3)
    x = (2 * torch.randn(M, N, generator=g)).to(dtype)
    dout = torch.randn(M, N, generator=g).to(dtype)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    BLOCK = min(65536 // x.element_size(), next_pow2(N))
    if kind == "softmax":
        S._softmax_kernel_fwd.fn[(M, 1)](x, x.stride(0), y, y.stride(0), N, BLOCK_SIZE=BLOCK)
        S._softmax_kernel_bwd.fn[(M, 1)](y, y.stride(0), dout, dout.stride(0), dx, dx.stride(0), N, BLOCK_SIZE=BLOCK)
    else:
        import triton.language as tl
        tdt = {torch.float32: tl.float32, torch.float16: tl.float16, torch.bfloat16: tl.bfloat16}[dtype]
        LS._logsoftmax_kernel_fwd.fn[(M, 1)](x, x.stride(0), y, y.stride(0), N, BLOCK_SIZE=BLOCK, dtype=tdt)
        LS._logsoftmax_kernel_bwd.fn[(M, 1)](y, y.stride(0), dout, dout.stride(0), dx, dx.stride(0), N,
                                             BLOCK_SIZE=BLOCK, dtype=tdt)
    out = {}
    for key, t in (("x", x), ("dout", dout), ("y", y), ("dx", dx)):
        k, v = store(t)
        out[key + k] = v
    out["meta"] = np.array([kind, str(dtype).replace("torch.", "")])
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok")


def run_gelu(G, name, dtype, M, N, approximate):
    g = torch.Generator().manual_seed(1)
    x = (2 * torch.randn(M, N, generator=g)).to(dtype)
    dout = torch.randn(M, N, generator=g).to(dtype)
    y, dx = torch.empty_like(x), torch.empty_like(x)
    BLOCK = min(65536 // x.element_size(), next_pow2(N))
    approx = approximate == "tanh"
    G._gelu_kernel_fwd.fn[(M, 1)](x, x.stride(0), y, y.stride(0), N, BLOCK_SIZE=BLOCK, approx=approx)
    G._gelu_kernel_bwd.fn[(M, 1)](x, x.stride(0), dout, dout.stride(0), dx, dx.stride(0), N, BLOCK_SIZE=BLOCK,
                                  approx=approx)
    out = {}
    for key, t in (("x", x), ("dout", dout), ("y", y), ("dx", dx)):
        k, v = store(t)
        out[key + k] = v
    out["meta"] = np.array(["gelu", str(dtype).replace("torch.", ""), approximate])
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok")


def run_chain(L, G, name, dtype, batch, N, eps, approximate):
    g = torch.Generator().manual_seed(2)
    M = int(np.prod(batch))
    x = torch.randn(M, N, generator=g).to(dtype)
    dz = torch.randn(M, N, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(N, generator=g)).to(dtype)
    b = (0.1 * torch.randn(N, generator=g)).to(dtype)
    BLOCK = min(65536 // x.element_size(), next_pow2(N))
    approx = approximate == "tanh"
    y, z, dy, dx = (torch.empty_like(x) for _ in range(4))
    mean = torch.empty(M, dtype=torch.float32)
    rstd = torch.empty(M, dtype=torch.float32)
    L._layernorm_kernel_fwd.fn[(M,)](x, x.stride(0), y, y.stride(0), w, b, mean, rstd, eps, N, BLOCK_SIZE=BLOCK,
                                     HAS_WEIGHT=True, HAS_BIAS=True)
    G._gelu_kernel_fwd.fn[(M, 1)](y, y.stride(0), z, z.stride(0), N, BLOCK_SIZE=BLOCK, approx=approx)
    G._gelu_kernel_bwd.fn[(M, 1)](y, y.stride(0), dz, dz.stride(0), dy, dy.stride(0), N, BLOCK_SIZE=BLOCK, approx=approx)
    rpp = math.ceil(M / PROGRAMS)
    dwp = torch.empty(PROGRAMS, N, dtype=torch.float32)
    dbp = torch.empty(PROGRAMS, N, dtype=torch.float32)
    L._layernorm_kernel_bwd.fn[(PROGRAMS,)](x, x.stride(0), dy, dy.stride(0), dx, dx.stride(0), w, b, dwp, dbp, mean,
                                            rstd, eps, M, N, rpp, BLOCK_SIZE=BLOCK, HAS_WEIGHT=True, HAS_BIAS=True)
    out = {}
    for key, t in (("x", x), ("dz", dz), ("w", w), ("b", b), ("z", z), ("dx", dx),
                   ("dw", dwp.sum(0).to(dtype)), ("db", dbp.sum(0).to(dtype))):
        k, v = store(t)
        out[key + k] = v
    out["meta"] = np.array(["ln_gelu", str(dtype).replace("torch.", ""), str(eps), approximate,
                            "x".join(map(str, batch))])
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok")


# Ops.norm / Ops.normalize (TritonHub/Ops/norm.py, normalize.py): name, dtype, B, M, K, p, eps
OPS_CASES = [
    ("ops_p2_fp32_2x9x128", torch.float32, 2, 9, 128, 2, 1e-12),
    ("ops_p2_fp16_1x7x1000", torch.float16, 1, 7, 1000, 2, 1e-12),
    ("ops_p2_bf16_1x4x4096", torch.bfloat16, 1, 4, 4096, 2, 1e-6),
    ("ops_p1_fp32_1x6x333", torch.float32, 1, 6, 333, 1, 1e-12),
]
# p other than 1 and 2 goes through libdevice's pow (norm.py:4,32), which Triton's interpreter cannot
# execute ("_semantic argument must be provided outside of JIT functions"): no golden vectors for it; the
# oracle's general-p branch is pinned to torch.norm / F.normalize autograd in fp64 instead.


def run_ops(NM, NZ, name, dtype, B, M, K, p, eps):
    """The reference's host glue (norm.py:47-60, 103-126; normalize.py:35-59, 119-144) around its four
    kernels, with one fixed block shape in place of the autotuner's choice."""
    import triton
    import triton.language as tl
    tdt = {torch.float32: tl.float32, torch.float16: tl.float16, torch.bfloat16: tl.bfloat16}[dtype]
    g = torch.Generator().manual_seed(5)
    x = torch.randn(B, M, K, generator=g).to(dtype)
    dn = torch.rand(B, M, generator=g).to(dtype)
    dy = torch.randn(B, M, K, generator=g).to(dtype)
    BM, BK = 4, 64
    grid = (triton.cdiv(M, BM), B)
    norms = torch.empty(B, M, dtype=dtype)
    NM._norm_fwd_kernel.fn[grid](x, x.stride(0), x.stride(1), x.stride(2), norms, norms.stride(0), norms.stride(1),
                                 eps, p, M, K, BLOCK_SIZE_M=BM, BLOCK_SIZE_K=BK, dtype=tdt)
    dx_norm = torch.empty_like(x)
    NM._norm_bwd_kernel.fn[grid](x, x.stride(0), x.stride(1), x.stride(2), norms, norms.stride(0), norms.stride(1),
                                 dn, dn.stride(0), dn.stride(1), dx_norm, dx_norm.stride(0), dx_norm.stride(1),
                                 p, M, K, BLOCK_SIZE_M=BM, BLOCK_SIZE_K=BK, dtype=tdt)
    y = torch.empty_like(x)
    NZ._normalize_fwd_kernel.fn[grid](x, x.stride(0), x.stride(1), x.stride(2), norms, norms.stride(0),
                                      norms.stride(1), y, y.stride(0), y.stride(1), y.stride(2), M, K,
                                      BLOCK_SIZE_M=BM, BLOCK_SIZE_K=BK, dtype=tdt)
    dx = torch.empty_like(x)
    NZ._normalize_bwd_kernel.fn[grid](x, x.stride(0), x.stride(1), x.stride(2), y, y.stride(0), y.stride(1),
                                      y.stride(2), norms, norms.stride(0), norms.stride(1), dy, dy.stride(0),
                                      dy.stride(1), dy.stride(2), dx, dx.stride(0), dx.stride(1), dx.stride(2),
                                      p, M, K, BLOCK_SIZE_M=BM, BLOCK_SIZE_K=BK, dtype=tdt)
    out = {}
    for key, t in (("x", x), ("dnorm", dn), ("dy", dy), ("norms", norms), ("dx_norm", dx_norm), ("y", y), ("dx", dx)):
        k, v = store(t)
        out[key + k] = v
    out["meta"] = np.array(["ops", str(dtype).replace("torch.", ""), str(p), repr(eps)])
    np.savez_compressed(HERE / f"{name}.npz", **out)
    print(name, "ok")


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py /path/to/Triton-Hub")
    ref = sys.argv[1]
    sys.path.insert(0, ref)
    if "--ops-only" in sys.argv:
        NM, NZ = importlib.import_module("TritonHub.Ops.norm"), importlib.import_module("TritonHub.Ops.normalize")
        for case in OPS_CASES:
            run_ops(NM, NZ, *case)
        return
    from TritonHub.Normalization import layernorm as L
    from TritonHub.Normalization import rmsnorm as R
    from TritonHub.Activations import gelu as G
    for case in CASES:
        run_case(L, R, *case)
    for case in GELU_CASES:
        run_gelu(G, *case)
    for case in CHAIN_CASES:
        run_chain(L, G, *case)
    from TritonHub.Activations import logsoftmax as LS
    from TritonHub.Activations import softmax as S
    for case in SOFTMAX_CASES:
        run_softmax(S, LS, *case)
    # the package re-exports classes named like its modules, so fetch the modules themselves
    NM, NZ = importlib.import_module("TritonHub.Ops.norm"), importlib.import_module("TritonHub.Ops.normalize")
    for case in OPS_CASES:
        run_ops(NM, NZ, *case)


if __name__ == "__main__":
    main()
