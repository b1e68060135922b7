"""numpy front end of the CPU oracle (oracle/norm_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the benchmark's CPU
baseline -- never by the product package.

The C side restates the reference's kernels (TritonHub/Normalization/layernorm.py:14-46,
94-153; rmsnorm.py:14-38,77-122) and host glue (layernorm.py:48-87,155-209).  This module
adds what the reference gets from torch dtypes: rounding to the storage type on the way in and
on the way out (`round_to`), and the parity metric the tests use.
"""
from __future__ import annotations

import ctypes
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "liboracle.so"
_lib = None

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build() -> Path:
    """Compile liboracle.so with the Makefile beside this file (gcc only)."""
    subprocess.run(["make", "-C", str(_HERE), "liboracle.so"], check=True, capture_output=True)
    return _LIB_PATH


def _load():
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            build()
        lib = ctypes.CDLL(str(_LIB_PATH))
        vp, i64, i32, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float
        lib.oracle_norm_fwd.restype = None
        lib.oracle_norm_fwd.argtypes = [vp, i64, vp, vp, vp, vp, vp, i64, i64, f32, i32, i32]
        lib.oracle_norm_bwd.restype = i32
        lib.oracle_norm_bwd.argtypes = [vp, i64, vp, i64, vp, vp, vp, vp, vp, vp, i64, i64, i32, i32, i32]
        lib.oracle_gelu_fwd.restype = None
        lib.oracle_gelu_fwd.argtypes = [vp, vp, i64, i32, i32]
        lib.oracle_gelu_bwd.restype = None
        lib.oracle_gelu_bwd.argtypes = [vp, vp, vp, i64, i32, i32]
        lib.oracle_softmax_fwd.restype = None
        lib.oracle_softmax_fwd.argtypes = [vp, vp, i64, i64, i32, i32]
        lib.oracle_softmax_bwd.restype = None
        lib.oracle_softmax_bwd.argtypes = [vp, vp, vp, i64, i64, i32, i32]
        lib.oracle_pnorm_fwd.restype = None
        lib.oracle_pnorm_fwd.argtypes = [vp, vp, i64, i64, f32, f32, i32]
        lib.oracle_pnorm_bwd.restype = None
        lib.oracle_pnorm_bwd.argtypes = [vp, vp, vp, vp, i64, i64, f32, i32]
        lib.oracle_normalize_bwd.restype = None
        lib.oracle_normalize_bwd.argtypes = [vp, vp, vp, vp, vp, i64, i64, f32, i32]
        lib.oracle_set_threads.argtypes = [i32]
        lib.oracle_get_threads.restype = i32
        _lib = lib
    return _lib


def set_threads(n: int) -> None:
    """Number of POSIX threads the oracle's row loops use (1 = the scalar port)."""
    _load().oracle_set_threads(int(n))


def round_to(a: np.ndarray, dtype: str) -> np.ndarray:
    """Round values to storage type `dtype` ('fp32', 'fp16', 'bf16', 'fp64') and return them
    widened to float32 (float64 for 'fp64'), i.e. what a kernel sees after its load."""
    if dtype == "fp64":
        return np.asarray(a, dtype=np.float64)
    a32 = np.ascontiguousarray(a, dtype=np.float32)
    if dtype == "fp32":
        return a32
    if dtype == "fp16":
        return a32.astype(np.float16).astype(np.float32)
    if dtype == "bf16":  # round to nearest even on the upper 16 bits
        u = a32.view(np.uint32).astype(np.uint64)
        rounded = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        out = rounded.astype(np.uint32).view(np.float32).reshape(a32.shape).copy()
        nan = np.isnan(a32)
        out[nan] = np.nan
        return out
    raise ValueError(dtype)


def _as_f32(a):
    return None if a is None else np.ascontiguousarray(a, dtype=np.float32)


def _p(a):
    return None if a is None else a.ctypes.data


def norm_fwd(x, w, b, eps, *, rms=False, acc64=False):
    """Forward.  x: (M, N) array of storage-rounded values.  Returns (y, mean, rstd) as fp32,
    y not yet rounded to the storage type; mean is None for RMSNorm."""
    x = _as_f32(x)
    M, N = x.shape
    w, b = _as_f32(w), (None if rms else _as_f32(b))
    y = np.empty((M, N), np.float32)
    mean = None if rms else np.empty((M,), np.float32)
    rstd = np.empty((M,), np.float32)
    _load().oracle_norm_fwd(_p(x), N, _p(w), _p(b), _p(y), _p(mean), _p(rstd), M, N, float(eps), int(rms),
                            int(acc64))
    return y, mean, rstd


def norm_bwd(x, dy, w, mean, rstd, *, rms=False, programs=148, acc64=False):
    """Backward with the reference's `programs`-way row split (sm_count there).  Returns
    (dx, dw, db) as fp32 before the cast to the storage / parameter type; db is None for
    RMSNorm."""
    x, dy = _as_f32(x), _as_f32(dy)
    M, N = x.shape
    w = _as_f32(w)
    mean = None if rms else _as_f32(mean)
    rstd = _as_f32(rstd)
    dx = np.empty((M, N), np.float32)
    dw = np.empty((N,), np.float32)
    db = None if rms else np.empty((N,), np.float32)
    rc = _load().oracle_norm_bwd(_p(x), N, _p(dy), N, _p(w), _p(mean), _p(rstd), _p(dx), _p(dw), _p(db), M, N,
                                 int(programs), int(rms), int(acc64))
    if rc != 0:
        raise RuntimeError(f"oracle_norm_bwd failed ({rc})")
    return dx, dw, db


def gelu_fwd(x, approximate="none", *, acc64=False):
    """y = gelu(x) (TritonHub/Activations/gelu.py:12-29); fp32 result, not yet rounded to the storage type."""
    x = _as_f32(x)
    y = np.empty_like(x)
    _load().oracle_gelu_fwd(_p(x), _p(y), x.size, int(approximate == "tanh"), int(acc64))
    return y


def gelu_bwd(x, dout, approximate="none", *, acc64=False):
    """dx = dout * gelu'(x) (gelu.py:56-81)."""
    x, dout = _as_f32(x), _as_f32(dout)
    dx = np.empty_like(x)
    _load().oracle_gelu_bwd(_p(x), _p(dout), _p(dx), x.size, int(approximate == "tanh"), int(acc64))
    return dx


def norm_gelu(x, dz, w, b, eps, approximate, *, rms=False, programs=8, acc64=True):
    """The LayerNorm -> GeLU pair of the reference's Quick Start, forward and backward, with nothing
    rounded in between: z = gelu(norm(x)); dy = dz * gelu'(y); (dx, dw, db) = norm_bwd(dy)."""
    y, mean, rstd = norm_fwd(x, w, None if rms else b, eps, rms=rms, acc64=acc64)
    z = gelu_fwd(y, approximate, acc64=acc64)
    dy = gelu_bwd(y, dz, approximate, acc64=acc64)
    dx, dw, db = norm_bwd(x, dy, w, mean, rstd, rms=rms, programs=programs, acc64=acc64)
    return {"z": z, "mean": mean, "rstd": rstd, "dx": dx, "dw": dw, "db": db}


def softmax_fwd(x, *, log=False, acc64=False):
    """Row-wise softmax / log-softmax of an (M, N) array (softmax.py:11-22, logsoftmax.py:11-24)."""
    x = _as_f32(x)
    M, N = x.shape
    y = np.empty_like(x)
    _load().oracle_softmax_fwd(_p(x), _p(y), M, N, int(log), int(acc64))
    return y


def softmax_bwd(y, dout, *, log=False, acc64=False):
    """dx from the forward's OUTPUT y and dout (softmax.py:48-62, logsoftmax.py:51-68)."""
    y, dout = _as_f32(y), _as_f32(dout)
    M, N = y.shape
    dx = np.empty_like(y)
    _load().oracle_softmax_bwd(_p(y), _p(dout), _p(dx), M, N, int(log), int(acc64))
    return dx


def pnorm_fwd(x, *, p=2.0, eps=1e-6, dtype="fp32", acc64=False):
    """Row p-norms of an (M, N) array, clamped to eps and rounded to the storage type as the
    reference's store does (Ops/norm.py:11-45)."""
    x = _as_f32(x)
    M, N = x.shape
    norms = np.empty(M, dtype=np.float32)
    _load().oracle_pnorm_fwd(_p(x), _p(norms), M, N, float(p), float(eps), int(acc64))
    return round_to(norms, dtype).astype(np.float32)


def pnorm_bwd(x, norms, dout, *, p=2.0, acc64=True):
    """dx of the row p-norm from x, the stored norms and dout (M,) (Ops/norm.py:66-101)."""
    x, norms, dout = _as_f32(x), _as_f32(norms), _as_f32(dout)
    M, N = x.shape
    dx = np.empty_like(x)
    _load().oracle_pnorm_bwd(_p(x), _p(norms), _p(dout), _p(dx), M, N, float(p), int(acc64))
    return dx


def normalize_fwd(x, *, p=2.0, eps=1e-6, dtype="fp32", acc64=False):
    """(y, norms): norms as pnorm_fwd stores them, y = x / norms (Ops/normalize.py:11-33)."""
    x = _as_f32(x)
    norms = pnorm_fwd(x, p=p, eps=eps, dtype=dtype, acc64=acc64)
    y = (x.astype(np.float64) / norms.astype(np.float64)[:, None]).astype(np.float32)
    return y, norms


def normalize_bwd(x, y, norms, dout, *, p=2.0, acc64=True):
    """dx of normalize from x, the forward's output y, the stored norms and dout (Ops/normalize.py:61-117)."""
    x, y, norms, dout = _as_f32(x), _as_f32(y), _as_f32(norms), _as_f32(dout)
    M, N = x.shape
    dx = np.empty_like(x)
    _load().oracle_normalize_bwd(_p(x), _p(y), _p(norms), _p(dout), _p(dx), M, N, float(p), int(acc64))
    return dx


def rel_err(a, ref) -> float:
    """The parity metric: max|a - ref| / max|ref| over the whole tensor."""
    a = np.asarray(a, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    if ref.size == 0:
        return 0.0
    scale = float(np.max(np.abs(ref)))
    err = float(np.max(np.abs(a - ref)))
    return err / scale if scale > 0 else err


# Parity bars: relative to the tensor's largest magnitude.
TOL = {"fp32": 1e-5, "fp64": 1e-5, "fp16": 1e-2, "bf16": 1e-2}
