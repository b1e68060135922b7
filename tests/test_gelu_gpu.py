"""GeLU on the GPU, stand-alone (the reference's GeLU interface) and fused into the norms, against
the golden vectors of the reference's kernels and the CPU oracle.  Bars as for the norms: 1e-5
(fp32) / 1e-2 (fp16, bf16) relative to each tensor's largest magnitude."""
import numpy as np
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

from b200norm import GeLU, LayerNormGeLU, RMSNormGeLU, LayerNorm
from b200norm import activations as A
from b200norm import functional as Fn
from helpers import (GOLDEN_CHAIN, GOLDEN_GELU, TOL, TORCH_DTYPE, assert_parity, load_golden_arrays, make_inputs,
                     to_numpy, to_torch)
from oracle import oracle as O

DEV = "cuda:0"


@pytest.mark.parametrize("name", GOLDEN_GELU)
def test_standalone_gelu_golden(name):
    g = load_golden_arrays(name)
    approximate, dt = g["meta"][2], g["dtype"]
    x, dout = to_torch(g["x"], dt, DEV), to_torch(g["dout"], dt, DEV)
    y = A._gelu_fwd(x, approximate)
    dx = A._gelu_bwd(x, dout, approximate)
    assert_parity(to_numpy(y), g["y"], TOL[dt], f"{name}: y")
    assert_parity(to_numpy(dx), g["dx"], TOL[dt], f"{name}: dx")


@pytest.mark.parametrize("dt", ["fp32", "fp16", "bf16", "fp64"])
@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_standalone_gelu_vs_oracle(dt, approximate):
    for M, N in ((37, 1000), (5, 33), (64, 4096), (3, 7)):
        rng = np.random.default_rng(N)
        x = O.round_to(3 * rng.standard_normal((M, N), dtype=np.float32), dt)
        g = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        y = A._gelu_fwd(to_torch(x, dt, DEV), approximate)
        dx = A._gelu_bwd(to_torch(x, dt, DEV), to_torch(g, dt, DEV), approximate)
        assert_parity(to_numpy(y), O.round_to(O.gelu_fwd(x, approximate, acc64=True), dt), TOL[dt], f"{M}x{N} y")
        assert_parity(to_numpy(dx), O.round_to(O.gelu_bwd(x, g, approximate, acc64=True), dt), TOL[dt], f"{M}x{N} dx")


def test_tanh_form_saturates_where_the_reference_formula_overflows():
    """(e - 1) / (e + 1) is inf / inf = NaN once exp(2u) overflows (gelu.py:23-24, x > ~10 in fp32);
    the kernels use 1 - 2 / (e + 1) and return gelu(x) = x there."""
    x = torch.tensor([[11.0, 20.0, 50.0, -50.0, -11.0, 0.0, 1.0, 0.0]], device=DEV)
    y = A._gelu_fwd(x, "tanh")
    dx = A._gelu_bwd(x, torch.ones_like(x), "tanh")
    assert torch.isfinite(y).all() and torch.isfinite(dx).all()
    torch.testing.assert_close(y, torch.nn.functional.gelu(x, approximate="tanh"), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_reference_gelu_unittest(dtype, approximate):
    """UnitTests/Activations/gelu_unittest.py restated: GeLU vs nn.GELU, its inputs and tolerances."""
    for D in (32, 256, 2048):
        torch.manual_seed(42)
        data = torch.randn(1, 64, 64, D, device="cuda", dtype=dtype)
        a = data.clone().requires_grad_(True)
        r = data.clone().requires_grad_(True)
        rtol, atol = (3e-4, 1e-3) if dtype == torch.float32 else (5e-3, 1e-2)
        if dtype == torch.float16:
            rtol, atol = 1e-2, 5e-2
        out, out_ref = GeLU(approximate=approximate)(a), nn.GELU(approximate=approximate)(r)
        assert torch.allclose(out, out_ref, atol=atol, rtol=rtol), 'Error in forward pass'
        gr = torch.randn_like(out)
        out.backward(gr)
        out_ref.backward(gr)
        assert torch.allclose(a.grad, r.grad, atol=atol, rtol=rtol), 'Error in backward pass'


@pytest.mark.parametrize("name", GOLDEN_CHAIN)
def test_fused_layernorm_gelu_golden(name):
    g = load_golden_arrays(name)
    eps, approximate, dt = float(g["meta"][2]), g["meta"][3], g["dtype"]
    x, dz, w, b = (to_torch(g[k], dt, DEV) for k in ("x", "dz", "w", "b"))
    z, mean, rstd = A._norm_gelu_fwd("ln", x, w, b, eps, approximate)
    dx, dw, db = A._norm_gelu_bwd("ln", x, dz, w, b, mean, rstd, eps, approximate)
    # vs the reference's two-kernel chain, which rounds y to the storage type in between (the fused
    # kernels do not): two roundings of slack for 16-bit storage, the usual bar against the oracle below
    tol = TOL[dt] * (2 if dt in ("fp16", "bf16") else 1)
    for key, got in (("z", z), ("dx", dx), ("dw", dw), ("db", db)):
        assert_parity(to_numpy(got), g[key], tol, f"{name}: {key}")


DIMS = [8, 64, 128, 256, 1000, 1024, 2048, 4096, 5120, 8192, 12288, 16384]


@pytest.mark.parametrize("dt", ["fp32", "fp16", "bf16"])
@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_fused_norm_gelu_vs_oracle(dt, rms, approximate):
    limit = 65536 // {"fp32": 4, "fp16": 2, "bf16": 2}[dt]
    for N in [d for d in DIMS + [32768] if d <= limit]:
        M = 29 if N <= 4096 else 9
        x, dz, w, b = make_inputs(M, N, dt, seed=N, has_b=not rms)
        ref = O.norm_gelu(x, dz, w, b, 1e-5, approximate, rms=rms, acc64=True)
        xt, dzt, wt, bt = (to_torch(a, dt, DEV) for a in (x, dz, w, b))
        op = "rms" if rms else "ln"
        z, mean, rstd = A._norm_gelu_fwd(op, xt, wt, bt, 1e-5, approximate)
        dx, dw, db = A._norm_gelu_bwd(op, xt, dzt, wt, bt, mean, rstd, 1e-5, approximate)
        tol = TOL[dt]
        assert_parity(to_numpy(z), O.round_to(ref["z"], dt), tol, f"N={N} z")
        assert_parity(to_numpy(dx), O.round_to(ref["dx"], dt), tol, f"N={N} dx")
        assert_parity(to_numpy(dw), O.round_to(ref["dw"], dt), tol, f"N={N} dw")
        if not rms:
            assert_parity(to_numpy(db), O.round_to(ref["db"], dt), tol, f"N={N} db")
        assert_parity(to_numpy(rstd), ref["rstd"], 1e-5, f"N={N} rstd")


def test_fused_equals_the_two_step_path_and_falls_back_on_unaligned_rows():
    torch.manual_seed(0)
    N = 1024
    for approximate in ("none", "tanh"):
        fused = LayerNormGeLU(N, eps=1e-6, approximate=approximate, device=DEV, dtype=torch.float32)
        plain, act = LayerNorm(N, eps=1e-6, device=DEV, dtype=torch.float32), GeLU(approximate)
        with torch.no_grad():
            fused.weight.normal_(1, 0.1)
            fused.bias.normal_(0, 0.1)
        plain.load_state_dict(fused.state_dict())
        x = torch.randn(2, 50, N, device=DEV)
        a, r = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
        g = torch.randn_like(x)
        za, zr = fused(a), act(plain(r))
        za.backward(g)
        zr.backward(g)
        torch.testing.assert_close(za, zr, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(a.grad, r.grad, rtol=1e-4, atol=1e-5)
        torch.testing.assert_close(fused.weight.grad, plain.weight.grad, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(fused.bias.grad, plain.bias.grad, rtol=1e-4, atol=1e-4)
    # odd row length: not 16-byte aligned -> the module runs the two steps itself
    fused = RMSNormGeLU(77, approximate="none", device=DEV, dtype=torch.float16)
    x = torch.randn(31, 77, device=DEV, dtype=torch.float16, requires_grad=True)
    z = fused(x)
    z.backward(torch.ones_like(z))
    ref = torch.nn.functional.gelu(torch.nn.functional.rms_norm(x.detach().float(), (77,), None, 1e-5))
    assert_parity(to_numpy(z), to_numpy(ref.half()), 1e-2, "unaligned fused z")
    assert torch.isfinite(x.grad).all()
