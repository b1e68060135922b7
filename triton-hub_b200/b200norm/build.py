"""Build libb200norm.so in-tree with nvcc for sm_100a.

Run as ``python build.py`` (from anywhere) or call :func:`build_library`.  Each translation
unit is compiled to an object file in parallel, then linked into
``b200norm/libb200norm.so``.  A unit is rebuilt only when it, or a header beside it, is
newer than its object file.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
import threading
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PKG_DIR = Path(__file__).resolve().parent
CSRC = PKG_DIR.parent / "csrc"
INCLUDE = PKG_DIR.parent.parent / "include"
BUILD_DIR = CSRC / "build"
LIB_PATH = PKG_DIR / "libb200norm.so"

_RETRY_LOCK = threading.Lock()

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]


def _nvcc() -> str:
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found: libb200norm.so cannot be built")
    return nvcc


def _sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _headers_mtime() -> float:
    headers = list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h")) + list(CSRC.glob("*.inc")) + list(INCLUDE.glob("*.h"))
    return max(h.stat().st_mtime for h in headers)


def _compile(src: Path, verbose: bool, ptxas_info: bool, defines: tuple = ()) -> Path:
    obj = BUILD_DIR / (src.stem + ".o")
    newest = max(src.stat().st_mtime, _headers_mtime())
    if obj.exists() and obj.stat().st_mtime >= newest:
        return obj
    cmd = [_nvcc(), *NVCC_FLAGS, *(f"-D{d}" for d in defines), f"-I{INCLUDE}", f"-I{CSRC}", "-c", str(src), "-o", str(obj)]
    if ptxas_info:
        cmd[1:1] = ["-Xptxas", "-v"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0 and "error" not in res.stderr.lower():
        # the compiler itself died (several large translation units in parallel): once more, alone
        with _RETRY_LOCK:
            res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{res.stdout}\n{res.stderr}")
    if ptxas_info:
        (BUILD_DIR / (src.stem + ".ptxas.txt")).write_text(res.stderr)
    return obj


def build_library(verbose: bool = False, force: bool = False, ptxas_info: bool = False, defines: tuple = ()) -> Path:
    """Compile every ``csrc/*.cu`` for sm_100a and link ``libb200norm.so``; returns its path.
    ``defines``: preprocessor symbols for a non-default build (``--define NAME`` on the command line), e.g.
    B200NORM_TUNING, which compiles in the environment-variable overrides of the launch table; such a
    build must be forced (``--force``), and forced again to return to the shipped configuration."""
    BUILD_DIR.mkdir(parents=True, exist_ok=True)
    if force:
        for o in BUILD_DIR.glob("*.o"):
            o.unlink()
    srcs = _sources()
    with ThreadPoolExecutor(max_workers=min(len(srcs), max(2, (os.cpu_count() or 4) - 2))) as pool:
        objs = list(pool.map(lambda s: _compile(s, verbose, ptxas_info, tuple(defines)), srcs))
    if LIB_PATH.exists() and all(LIB_PATH.stat().st_mtime >= o.stat().st_mtime for o in objs):
        return LIB_PATH
    cmd = [_nvcc(), "-shared", "-o", str(LIB_PATH), *map(str, objs),
           "-gencode", "arch=compute_100a,code=sm_100a", "-cudart", "static"]
    if verbose:
        print(" ".join(cmd), flush=True)
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError(f"link failed:\n{res.stdout}\n{res.stderr}")
    return LIB_PATH


if __name__ == "__main__":
    defs = tuple(sys.argv[i + 1] for i, a in enumerate(sys.argv[:-1]) if a == "--define")
    path = build_library(verbose=True, force="--force" in sys.argv, ptxas_info="--ptxas" in sys.argv, defines=defs)
    print(path)
