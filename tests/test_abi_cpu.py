"""The C-ABI library without a GPU: it loads, exports every symbol include/b200norm.h
declares, and its argument checks (which run before any CUDA call) return the documented
status codes."""
import ctypes
import re
from pathlib import Path

import pytest

from b200norm import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "b200norm.h"


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"B200NORM_API[^;(]*?\b(b200norm_\w+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    syms = declared_symbols()
    for name in ("b200norm_ln_fwd", "b200norm_ln_bwd", "b200norm_rms_fwd", "b200norm_rms_bwd",
                 "b200norm_finalize_dwdb", "b200norm_bwd_workspace_bytes", "b200norm_version"):
        assert name in syms


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} declared in b200norm.h but not exported"
        assert name in _lib.SIGNATURES, f"{name} has no ctypes prototype"
    assert set(_lib.SIGNATURES) == set(declared_symbols())


def test_version_matches_header():
    want = int(re.search(r"#define B200NORM_VERSION (\d+)", HEADER.read_text()).group(1))
    assert _lib.load().b200norm_version() == want


def test_bad_dtype_is_an_argument_error():
    lib = _lib.load()
    rc = lib.b200norm_ln_fwd(None, 8, None, None, None, 8, None, None, 4, 8, 1e-5, 7, 0, None)
    assert rc == _lib.ERR_ARG
    assert b"dtype" in lib.b200norm_last_error()


def test_row_wider_than_64kb_is_unsupported_with_the_reference_message():
    # layernorm.py:69-72: N > 65536 // element_size raises this text
    lib = _lib.load()
    for dtype, n in ((_lib.F32, 16385), (_lib.BF16, 32769), (_lib.F64, 8193)):
        rc = lib.b200norm_rms_fwd(None, n, None, None, n, None, 1, n, 1e-5, dtype, dtype, None)
        assert rc == _lib.ERR_UNSUPPORTED
        assert lib.b200norm_last_error() == b"This layer norm doesn't support feature dim >= 64KB."
    with pytest.raises(RuntimeError, match="feature dim >= 64KB"):
        _lib.check(rc)


def test_negative_rows_and_empty_batch():
    lib = _lib.load()
    assert lib.b200norm_ln_fwd(None, 8, None, None, None, 8, None, None, -1, 8, 1e-5, 0, 0, None) == _lib.ERR_ARG
    # M == 0 is a no-op that never touches the device
    assert lib.b200norm_ln_fwd(None, 8, None, None, None, 8, None, None, 0, 8, 1e-5, 0, 0, None) == _lib.OK


def test_bwd_rejects_row_shards_that_do_not_divide_rows():
    lib = _lib.load()
    rc = lib.b200norm_ln_bwd(None, 8, None, 8, None, None, None, None, 8, None, None, None, 3, None, 0,
                             10, 8, 0, 0, None)
    assert rc == _lib.ERR_ARG and b"row_shards" in lib.b200norm_last_error()


def test_finalize_rejects_bad_slot_count():
    lib = _lib.load()
    buf = (ctypes.c_float * 8)()
    assert lib.b200norm_finalize_dwdb(ctypes.addressof(buf), 1, 3, None, None, 8, 0, None) == _lib.ERR_ARG
