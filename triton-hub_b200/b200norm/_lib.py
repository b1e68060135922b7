"""ctypes binding of libb200norm.so (C ABI declared in include/b200norm.h).

There is no fallback: if the shared library has not been built, or a call returns a non-zero
status, a RuntimeError is raised.
"""
from __future__ import annotations

import ctypes
import threading
from pathlib import Path

LIB_PATH = Path(__file__).resolve().parent / "libb200norm.so"

# Status codes of enum b200norm_status.
OK, ERR_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT = range(5)

# Storage type codes of enum b200norm_dtype.
F32, F16, BF16, F64 = range(4)

# Fused activation codes of enum b200norm_act.
ACT_NONE, ACT_GELU_ERF, ACT_GELU_TANH = range(3)

_c = ctypes
_vp, _i64, _int, _f32, _sz = _c.c_void_p, _c.c_int64, _c.c_int, _c.c_float, _c.c_size_t

MAX_PEERS = 8


class Peers(ctypes.Structure):
    """struct b200norm_peers: where the fused column reduce pushes shard sums (see b200norm.h)."""
    _fields_ = [("world", _int), ("rank", _int), ("depth", _int), ("total_shards", _int),
                ("inbox_bytes", _sz), ("inbox", _vp * MAX_PEERS), ("counter", _vp)]


class Finish(ctypes.Structure):
    """struct b200norm_finish: an exchange for a push kernel to finish as its second phase."""
    _fields_ = [("seq", _c.c_uint64), ("slots", _int), ("w_dtype", _int), ("N", _i64), ("dw", _vp), ("db", _vp)]


_pp, _fp, _u64 = _c.POINTER(Peers), _c.POINTER(Finish), _c.c_uint64

# name -> (restype, argtypes): every symbol include/b200norm.h declares.
SIGNATURES = {
    "b200norm_version": (_int, []),
    "b200norm_query": (_int, [_c.POINTER(_int), _c.POINTER(_int)]),
    "b200norm_last_error": (_c.c_char_p, []),
    "b200norm_device_status": (_int, [_int]),
    "b200norm_bwd_workspace_bytes": (_sz, [_i64, _i64, _int, _int]),
    "b200norm_ln_fwd": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _f32, _int, _int, _vp]),
    "b200norm_rms_fwd": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _i64, _f32, _int, _int, _vp]),
    "b200norm_ln_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _vp, _sz,
                               _i64, _i64, _int, _int, _vp]),
    "b200norm_rms_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _int, _vp, _sz, _i64, _i64,
                                _int, _int, _vp]),
    "b200norm_finalize_dwdb": (_int, [_vp, _int, _int, _vp, _vp, _i64, _int, _vp]),
    "b200norm_gelu_fwd": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "b200norm_gelu_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "b200norm_softmax_fwd": (_int, [_vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "b200norm_softmax_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i64, _int, _int, _vp]),
    "b200norm_pnorm_fwd": (_int, [_vp, _i64, _vp, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200norm_pnorm_bwd": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200norm_normalize_fwd": (_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _f32, _f32, _int, _vp]),
    "b200norm_normalize_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _i64, _vp, _i64, _i64, _i64, _f32, _int, _vp]),
    "b200norm_ln_act_fwd": (_int, [_vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _i64, _i64, _f32, _int, _int, _int, _vp]),
    "b200norm_rms_act_fwd": (_int, [_vp, _i64, _vp, _vp, _i64, _vp, _i64, _i64, _f32, _int, _int, _int, _vp]),
    "b200norm_ln_act_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _vp, _i64, _vp, _vp, _vp, _int, _vp, _sz,
                                   _i64, _i64, _int, _int, _int, _vp]),
    "b200norm_rms_act_bwd": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _vp, _int, _vp, _sz, _i64, _i64,
                                    _int, _int, _int, _vp]),
    "b200norm_ln_bwd_push": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _int, _vp, _sz, _i64, _i64, _int,
                                    _int, _pp, _u64, _fp, _vp]),
    "b200norm_rms_bwd_push": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _int, _vp, _sz, _i64, _i64, _int, _int,
                                     _pp, _u64, _fp, _vp]),
    "b200norm_finalize_pushed": (_int, [_pp, _u64, _int, _vp, _vp, _i64, _int, _vp]),
    "b200norm_rms_bwd_static": (_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _i64, _vp, _i64, _i64, _int, _int, _vp]),
}

_lock = threading.Lock()
_lib = None


def load() -> ctypes.CDLL:
    """Load libb200norm.so once and set every prototype.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not LIB_PATH.exists():
                raise RuntimeError(
                    f"{LIB_PATH} is missing: build it with `python {LIB_PATH.parent / 'build.py'}` "
                    "(needs nvcc; there is no Triton, PyTorch or CPU fallback for these kernels)")
            lib = ctypes.CDLL(str(LIB_PATH))
            for name, (res, args) in SIGNATURES.items():
                fn = getattr(lib, name)
                fn.restype, fn.argtypes = res, args
            _lib = lib
    return _lib


def check(status: int) -> None:
    """Turn a non-zero status into the RuntimeError the reference's wrappers would raise."""
    if status != OK:
        msg = load().b200norm_last_error().decode() or f"b200norm status {status}"
        raise RuntimeError(msg)
