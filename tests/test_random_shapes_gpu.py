"""Seeded random shapes through every op family: row counts, row lengths (aligned and not), storage
types and padded row strides drawn at random, each checked against the CPU oracle at the usual bars
(1e-5 fp32 / fp64 storage, 1e-2 fp16 / bf16, relative to the tensor's largest magnitude)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from b200norm import activations as A
from b200norm import functional as Fn
from b200norm import ops as P
from b200norm import softmax as S
from helpers import TOL, TORCH_DTYPE, assert_parity, oracle_all, to_numpy
from oracle import oracle as O

DEV = "cuda:0"
ESIZE = {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}


def draw_case(rng):
    dt = ["fp32", "fp16", "bf16", "fp64"][rng.integers(4)]
    limit = 65536 // ESIZE[dt]
    N = int(min(limit, max(1, round(float(np.exp(rng.uniform(0, np.log(limit))))))))
    if rng.random() < 0.5:  # half of the cases on 16-byte multiples: the packet kernels
        N = max(16 // ESIZE[dt], N // (16 // ESIZE[dt]) * (16 // ESIZE[dt]))
    M = int(rng.integers(1, 200)) if N < 8192 else int(rng.integers(1, 20))
    pad = int(rng.choice([0, 0, 8, 16, 3, 1]))
    return dt, M, N, pad


def on_device(a, dt, pad):
    """(M, N) numpy -> a device view with row stride N + pad (values rounded to the storage type)."""
    M, N = a.shape
    buf = torch.zeros((M, N + pad), dtype=TORCH_DTYPE[dt], device=DEV)
    buf[:, :N] = torch.from_numpy(np.asarray(a)).to(DEV, TORCH_DTYPE[dt])
    return buf[:, :N]


@pytest.mark.parametrize("seed", range(8))
def test_norms(seed):
    rng = np.random.default_rng(1000 + seed)
    for _ in range(5):
        dt, M, N, pad = draw_case(rng)
        rms = bool(rng.integers(2))
        x = O.round_to(rng.standard_normal((M, N), dtype=np.float32) * 2 + 0.5, dt)
        dy = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        w = O.round_to(1 + 0.1 * rng.standard_normal(N, dtype=np.float32), dt)
        b = None if rms else O.round_to(0.1 * rng.standard_normal(N, dtype=np.float32), dt)
        xt, dyt = on_device(x, dt, pad), on_device(dy, dt, pad)
        wt = torch.from_numpy(np.asarray(w)).to(DEV, TORCH_DTYPE[dt])
        bt = None if b is None else torch.from_numpy(np.asarray(b)).to(DEV, TORCH_DTYPE[dt])
        ref = oracle_all(x, dy, w, b, 1e-5, rms=rms, dtype=dt, programs=8, acc64=True)
        if rms:
            y, rstd = Fn._rmsnorm_fwd(xt, wt, 1e-5)
            dx, dw = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, 1e-5)
            got = dict(y=y, dx=dx, dw=dw)
        else:
            y, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, 1e-5)
            dx, dw, db = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, 1e-5)
            got = dict(y=y, dx=dx, dw=dw, db=db)
        label = f"{'rms' if rms else 'ln'} {dt} {M}x{N}+{pad} "
        floor = 1e-2 * float(np.max(np.abs(w))) * float(np.max(np.abs(dy))) * float(np.max(ref["rstd"]))
        for k, v in got.items():
            assert_parity(to_numpy(v), ref[k], TOL[dt], label + k, floor=floor if k == "dx" else 0.0)


@pytest.mark.parametrize("seed", range(8))
def test_softmax_family_and_gelu(seed):
    rng = np.random.default_rng(2000 + seed)
    for _ in range(5):
        dt, M, N, pad = draw_case(rng)
        x = O.round_to(3 * rng.standard_normal((M, N), dtype=np.float32), dt)
        g = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        xt, gt = on_device(x, dt, pad), on_device(g, dt, pad)
        label = f"{dt} {M}x{N}+{pad} "
        for log in (False, True):
            y_ref = O.softmax_fwd(x, log=log, acc64=True)
            assert_parity(to_numpy(S._fwd(xt, log)), O.round_to(y_ref, dt), TOL[dt], label + f"softmax log={log} y")
            y_saved = O.round_to(y_ref, dt)
            dx = S._bwd(on_device(y_saved, dt, pad), gt, log)
            assert_parity(to_numpy(dx), O.round_to(O.softmax_bwd(y_saved, g, log=log, acc64=True), dt), TOL[dt],
                          label + f"softmax log={log} dx")
        approximate = ["none", "tanh"][rng.integers(2)]
        assert_parity(to_numpy(A._gelu_fwd(xt, approximate)), O.round_to(O.gelu_fwd(x, approximate, acc64=True), dt),
                      TOL[dt], label + "gelu y")
        assert_parity(to_numpy(A._gelu_bwd(xt, gt, approximate)),
                      O.round_to(O.gelu_bwd(x, g, approximate, acc64=True), dt), TOL[dt], label + "gelu dx")


@pytest.mark.parametrize("seed", range(8))
def test_pnorm_and_normalize(seed):
    rng = np.random.default_rng(3000 + seed)
    for _ in range(5):
        dt, M, N, pad = draw_case(rng)
        p = float(rng.choice([1.0, 2.0, 2.0, 3.0, 1.5]))
        x = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        g = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        gn = O.round_to(rng.random(M, dtype=np.float32), dt)
        xt = on_device(x, dt, pad).unsqueeze(0)
        label = f"p={p} {dt} {M}x{N}+{pad} "
        norms_ref = O.pnorm_fwd(x, p=p, eps=1e-12, dtype=dt, acc64=True)
        assert_parity(to_numpy(P._norm_fwd(xt, p, 1e-12)).reshape(-1), norms_ref, TOL[dt], label + "norms")
        nt = torch.from_numpy(norms_ref).to(DEV, TORCH_DTYPE[dt]).reshape(1, M)
        dxn = P._norm_bwd(xt, nt, torch.from_numpy(np.asarray(gn)).to(DEV, TORCH_DTYPE[dt]).reshape(1, M), p)
        assert_parity(to_numpy(dxn).reshape(M, N), O.round_to(O.pnorm_bwd(x, norms_ref, gn, p=p), dt), TOL[dt],
                      label + "d norm", floor=1e-3)
        y_ref, _ = O.normalize_fwd(x, p=p, eps=1e-12, dtype=dt, acc64=True)
        y_saved = O.round_to(y_ref, dt)
        y, _ = P._normalize_fwd(xt, p, 1e-12)
        assert_parity(to_numpy(y).reshape(M, N), y_saved, TOL[dt], label + "y")
        dx = P._normalize_bwd(xt, on_device(y_saved, dt, pad).unsqueeze(0), nt, on_device(g, dt, pad).unsqueeze(0), p)
        assert_parity(to_numpy(dx).reshape(M, N), O.round_to(O.normalize_bwd(x, y_saved, norms_ref, g, p=p), dt),
                      TOL[dt], label + "d normalize", floor=1.0)
