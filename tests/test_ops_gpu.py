"""Ops.norm / Ops.normalize on the GPU against the golden vectors of the reference's kernels and the
CPU oracle; plus the reference's unit tests restated (vs torch.norm / F.normalize on the GPU, its
tolerances).  Bars: 1e-5 (fp32, fp64) / 1e-2 (fp16, bf16) relative to the tensor's largest magnitude."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from TritonHub.Ops import norm, normalize
from b200norm import ops
from helpers import GOLDEN_OPS, TOL, assert_parity, load_golden_arrays, to_numpy, to_torch
from oracle import oracle as O

DEV = "cuda:0"


@pytest.mark.parametrize("name", GOLDEN_OPS)
def test_golden(name):
    g = load_golden_arrays(name)
    dt, p, eps = g["dtype"], float(g["meta"][2]), float(g["meta"][3])
    x = to_torch(g["x"], dt, DEV)
    norms = ops._norm_fwd(x, p, eps)
    assert_parity(to_numpy(norms), g["norms"], TOL[dt], f"{name}: norms")
    dxn = ops._norm_bwd(x, to_torch(g["norms"], dt, DEV), to_torch(g["dnorm"], dt, DEV), p)
    assert_parity(to_numpy(dxn), g["dx_norm"], TOL[dt], f"{name}: d norm")
    y, norms2 = ops._normalize_fwd(x, p, eps)
    assert_parity(to_numpy(y), g["y"], TOL[dt], f"{name}: y")
    assert_parity(to_numpy(norms2), g["norms"], TOL[dt], f"{name}: norms (normalize)")
    dx = ops._normalize_bwd(x, to_torch(g["y"], dt, DEV), to_torch(g["norms"], dt, DEV), to_torch(g["dy"], dt, DEV), p)
    assert_parity(to_numpy(dx), g["dx"], TOL[dt], f"{name}: d normalize")


DIMS = [1, 3, 8, 33, 64, 100, 128, 256, 512, 1000, 1024, 2048, 3000, 4096, 5120, 8192, 12288, 16384]


@pytest.mark.parametrize("dt", ["fp32", "fp16", "bf16", "fp64"])
@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 2.5])
def test_dim_sweep_vs_oracle(dt, p):
    limit = 65536 // {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}[dt]
    for N in [d for d in DIMS + [24576, 32768] if d <= limit]:
        M = 23 if N <= 4096 else 7
        rng = np.random.default_rng(N)
        x = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        g = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        gn = O.round_to(rng.random(M, dtype=np.float32), dt)
        xt = to_torch(x, dt, DEV).reshape(1, M, N)
        # norm
        norms_ref = O.pnorm_fwd(x, p=p, eps=1e-12, dtype=dt, acc64=True)
        norms = ops._norm_fwd(xt, p, 1e-12)
        assert_parity(to_numpy(norms).reshape(-1), norms_ref, TOL[dt], f"N={N} norms")
        dxn = ops._norm_bwd(xt, to_torch(norms_ref, dt, DEV).reshape(1, M), to_torch(gn, dt, DEV).reshape(1, M), p)
        assert_parity(to_numpy(dxn).reshape(M, N), O.round_to(O.pnorm_bwd(x, norms_ref, gn, p=p), dt), TOL[dt],
                      f"N={N} d norm")
        # normalize: backward from the same (storage-rounded) saved tensors on both sides
        y_ref, _ = O.normalize_fwd(x, p=p, eps=1e-12, dtype=dt, acc64=True)
        y_saved = O.round_to(y_ref, dt)
        y, norms2 = ops._normalize_fwd(xt, p, 1e-12)
        assert_parity(to_numpy(y).reshape(M, N), y_saved, TOL[dt], f"N={N} y")
        assert_parity(to_numpy(norms2).reshape(-1), norms_ref, TOL[dt], f"N={N} norms (normalize)")
        dx = ops._normalize_bwd(xt, to_torch(y_saved, dt, DEV).reshape(1, M, N), to_torch(norms_ref, dt, DEV).reshape(1, M),
                                to_torch(g, dt, DEV).reshape(1, M, N), p)
        assert_parity(to_numpy(dx).reshape(M, N), O.round_to(O.normalize_bwd(x, y_saved, norms_ref, g, p=p), dt),
                      TOL[dt], f"N={N} d normalize", floor=1.0)  # N = 1: the exact answer is 0


def test_eps_clamp_and_zero_rows():
    x = torch.zeros(2, 5, 64, device=DEV)
    x[1, 2] = 3.0
    n = ops._norm_fwd(x, 2, 1e-6)
    assert n[0, 0].item() == pytest.approx(1e-6) and n[1, 2].item() == pytest.approx(24.0)
    y, _ = ops._normalize_fwd(x, 2, 1e-6)
    assert torch.all(y[0] == 0) and torch.allclose(y[1, 2], torch.full((64,), 0.125, device=DEV))


def test_strided_and_unaligned_rows():
    torch.manual_seed(0)
    base = torch.randn(3, 40, 300, device=DEV)
    for view in (base[:, :, :257], base[:, ::2, :128], base[:, :, 4:260], base.transpose(1, 2)):
        x = view.detach().clone(memory_format=torch.preserve_format) if view.stride(-1) != 1 else view
        xr = x.detach().requires_grad_(True)
        xo = x.detach().clone().requires_grad_(True)
        y = normalize(p=2, eps=1e-12)(xr)
        yo = F.normalize(xo, p=2, dim=-1, eps=1e-12)
        torch.testing.assert_close(y, yo, rtol=1e-5, atol=1e-6)
        g = torch.randn_like(yo)
        y.backward(g)
        yo.backward(g)
        torch.testing.assert_close(xr.grad, xo.grad, rtol=1e-4, atol=1e-5)
        n = norm(p=2, eps=1e-12)(x)
        torch.testing.assert_close(n, torch.norm(x, p=2, dim=-1), rtol=1e-5, atol=1e-6)


def test_argument_errors():
    with pytest.raises(AssertionError):
        norm(p=0.5)
    with pytest.raises(AssertionError):
        normalize(p=7)
    with pytest.raises(AssertionError):
        norm()(torch.randn(4, 8, device=DEV))  # the reference wants (B, L, D)
    with pytest.raises(RuntimeError, match="64KB"):
        ops._norm_fwd(torch.randn(1, 2, 16385, device=DEV), 2, 1e-6)
    assert ops._norm_fwd(torch.empty(1, 0, 8, device=DEV), 2, 1e-6).shape == (1, 0)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32])
@pytest.mark.parametrize("kind", ["norm", "normalize"])
@pytest.mark.parametrize("p", [1, 2, 3])
def test_reference_unittests(kind, dtype, p):
    """UnitTests/Ops/norm_unittest.py and normalize_unittest.py restated (B=1, M=1000, eps=1e-12, their
    tolerances; they run p = 2, here p = 1 and 3 as well)."""
    for D in (32, 64, 128, 256, 512, 1024):
        torch.manual_seed(42)
        data = torch.randn(1, 1000, D, device="cuda", dtype=dtype)
        a, r = data.clone().requires_grad_(True), data.clone().requires_grad_(True)
        rtol, atol = (3e-4, 1e-3) if dtype == torch.float32 else (1e-2, 5e-2)
        if kind == "norm":
            out = norm(p=p, eps=1e-12)(a)
            out_ref = torch.norm(r, p=p, dim=-1, keepdim=True)
            assert torch.allclose(out, out_ref.squeeze(-1), atol=atol, rtol=rtol), 'Error in forward pass'
            g = torch.rand_like(out_ref)
            out.backward(g.squeeze(-1))
            out_ref.backward(g)
        else:
            out = normalize(p=p, eps=1e-12)(a)
            out_ref = F.normalize(r, p=p, dim=-1, eps=1e-12)
            assert torch.allclose(out, out_ref, atol=atol, rtol=rtol), 'Error in forward pass'
            g = torch.rand_like(out_ref)
            out.backward(g)
            out_ref.backward(g)
        assert torch.allclose(a.grad, r.grad, atol=atol, rtol=rtol), 'Error in backward pass'
