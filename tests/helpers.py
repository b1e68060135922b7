"""Shared test helpers: golden-vector loading, seeded inputs, the parity metric."""
from pathlib import Path

import numpy as np
import torch

from oracle import oracle as O

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
_ALL_GOLDEN = sorted(p.stem for p in GOLDEN_DIR.glob("*.npz"))
GOLDEN = [n for n in _ALL_GOLDEN if "gelu" not in n and "softmax" not in n and not n.startswith("ops_")]  # the norm kernels alone
GOLDEN_OPS = [n for n in _ALL_GOLDEN if n.startswith("ops_")]                # the reference's Ops.norm / normalize kernels
GOLDEN_SOFTMAX = [n for n in _ALL_GOLDEN if "softmax" in n]                  # the reference's softmax kernels
GOLDEN_GELU = [n for n in _ALL_GOLDEN if n.startswith("gelu_")]          # the reference's GeLU kernels alone
GOLDEN_CHAIN = [n for n in _ALL_GOLDEN if "_gelu_" in n and not n.startswith("gelu_")]   # LayerNorm -> GeLU

TORCH_DTYPE = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16, "fp64": torch.float64}
SHORT = {"float32": "fp32", "float16": "fp16", "bfloat16": "bf16", "float64": "fp64"}

# Parity bars (relative to the tensor's largest magnitude): 1e-5 for fp32 storage (and fp64
# storage, which the kernels compute in fp32 like the reference), 1e-2 for fp16 / bf16.
TOL = O.TOL


def load_golden(name):
    """-> dict with op, dtype ('fp32'...), eps, programs, batch and float32/float64 numpy arrays
    (x, dy, w, b, y, dx, dw, db, mean, rstd; absent ones are None)."""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    op, dt, eps, programs, batch = z["meta"]
    out = {"op": op, "dtype": SHORT[dt], "eps": float(eps), "programs": int(programs),
           "batch": tuple(int(v) for v in batch.split("x"))}
    for key in ("x", "dy", "w", "b", "y", "dx", "dw", "db", "mean", "rstd"):
        if key in z:
            out[key] = z[key].astype(np.float64 if z[key].dtype == np.float64 else np.float32)
        elif key + "__bf16bits" in z:
            bits = z[key + "__bf16bits"].astype(np.uint32) << 16
            out[key] = bits.view(np.float32)
        else:
            out[key] = None
    return out


def load_golden_arrays(name):
    """Generic loader for the GeLU and LayerNorm->GeLU vectors: dict of float32/float64 arrays + 'meta' list."""
    z = np.load(GOLDEN_DIR / f"{name}.npz")
    out = {"meta": [str(v) for v in z["meta"]]}
    for key in z.files:
        if key == "meta":
            continue
        if key.endswith("__bf16bits"):
            out[key[:-10]] = (z[key].astype(np.uint32) << 16).view(np.float32)
        else:
            out[key] = z[key].astype(np.float64 if z[key].dtype == np.float64 else np.float32)
    out["dtype"] = SHORT[out["meta"][1]]
    return out


def make_inputs(M, N, dtype, *, mu=0.0, sigma=1.0, seed=0, has_w=True, has_b=True):
    """Seeded synthetic inputs with the benchmark's distributions, as float32 numpy arrays of
    values already rounded to `dtype`: x ~ N(mu, sigma), dy ~ N(0,1), w ~ N(1,0.1), b ~ N(0,0.1)."""
    rng = np.random.default_rng(seed)
    x = O.round_to(rng.standard_normal((M, N), dtype=np.float32) * sigma + mu, dtype)
    dy = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dtype)
    w = O.round_to(1 + 0.1 * rng.standard_normal(N, dtype=np.float32), dtype) if has_w else None
    b = O.round_to(0.1 * rng.standard_normal(N, dtype=np.float32), dtype) if has_b else None
    return x, dy, w, b


def to_torch(a, dtype, device="cpu"):
    return None if a is None else torch.from_numpy(np.asarray(a)).to(device=device, dtype=TORCH_DTYPE[dtype])


def to_numpy(t):
    if t is None:
        return None
    t = t.detach().cpu()
    return t.double().numpy() if t.dtype == torch.float64 else t.float().numpy()


def oracle_all(x, dy, w, b, eps, *, rms, dtype, programs=148, acc64=False):
    """Run the oracle forward + backward and round every output to its storage type, the way
    the reference's stores and `.to(dtype)` do.  Returns dict y, mean, rstd, dx, dw, db."""
    y, mean, rstd = O.norm_fwd(x, w, None if rms else b, eps, rms=rms, acc64=acc64)
    dx, dw, db = O.norm_bwd(x, dy, w, mean, rstd, rms=rms, programs=programs, acc64=acc64)
    r = lambda a: None if a is None else O.round_to(a, dtype).astype(np.float32)
    return {"y": r(y), "mean": mean, "rstd": rstd, "dx": r(dx),
            "dw": r(dw) if w is not None else None,
            "db": r(db) if (b is not None and not rms) else None}


def assert_parity(got, ref, tol, what, floor=0.0):
    """max|got - ref| <= tol * max(max|ref|, floor).  `floor` is the tensor's natural scale for
    the degenerate cases whose exact answer is all zeros (N == 1: xhat = 0 and dx = 0)."""
    got = np.asarray(got, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape, f"{what}: shape {got.shape} vs {ref.shape}"
    if ref.size == 0:
        return 0.0
    err = float(np.max(np.abs(got - ref)))
    scale = max(float(np.max(np.abs(ref))), floor)
    assert err <= tol * scale, f"{what}: max|a-ref| = {err:.3e} > {tol:.1e} * {scale:.3e}"
    return err / scale if scale > 0 else err
