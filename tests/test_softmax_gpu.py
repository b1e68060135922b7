"""Softmax / LogSoftmax / Softmin on the GPU against the golden vectors of the reference's kernels
and the CPU oracle; plus the reference's unit tests restated (vs torch.nn on the GPU, its
tolerances).  Bars: 1e-5 (fp32, fp64) / 1e-2 (fp16, bf16) relative to the tensor's largest magnitude."""
import numpy as np
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

from TritonHub.Activations import LogSoftmax, Softmax, Softmin
from b200norm import softmax as S
from helpers import GOLDEN_SOFTMAX, TOL, assert_parity, load_golden_arrays, to_numpy, to_torch
from oracle import oracle as O

DEV = "cuda:0"


@pytest.mark.parametrize("name", GOLDEN_SOFTMAX)
def test_golden(name):
    g = load_golden_arrays(name)
    log, dt = g["meta"][0] == "logsoftmax", g["dtype"]
    y = S._fwd(to_torch(g["x"], dt, DEV), log)
    dx = S._bwd(to_torch(g["y"], dt, DEV), to_torch(g["dout"], dt, DEV), log)
    assert_parity(to_numpy(y), g["y"], TOL[dt], f"{name}: y")
    assert_parity(to_numpy(dx), g["dx"], TOL[dt], f"{name}: dx")


DIMS = [1, 3, 8, 33, 64, 100, 128, 256, 512, 1000, 1024, 2048, 3000, 4096, 5120, 8192, 12288, 16384]


@pytest.mark.parametrize("dt", ["fp32", "fp16", "bf16", "fp64"])
@pytest.mark.parametrize("log", [False, True])
def test_dim_sweep_vs_oracle(dt, log):
    limit = 65536 // {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}[dt]
    for N in [d for d in DIMS + [24576, 32768] if d <= limit]:
        M = 23 if N <= 4096 else 7
        rng = np.random.default_rng(N)
        x = O.round_to(3 * rng.standard_normal((M, N), dtype=np.float32), dt)
        g = O.round_to(rng.standard_normal((M, N), dtype=np.float32), dt)
        y = S._fwd(to_torch(x, dt, DEV), log)
        y_ref = O.softmax_fwd(x, log=log, acc64=True)
        assert_parity(to_numpy(y), O.round_to(y_ref, dt), TOL[dt], f"N={N} y")
        # backward from the same (storage-rounded) saved output on both sides
        y_saved = O.round_to(y_ref, dt)
        dx = S._bwd(to_torch(y_saved, dt, DEV), to_torch(g, dt, DEV), log)
        assert_parity(to_numpy(dx), O.round_to(O.softmax_bwd(y_saved, g, log=log, acc64=True), dt), TOL[dt], f"N={N} dx")


def test_rows_sum_to_one_and_extremes_do_not_overflow():
    x = torch.tensor([[1000.0, 1000.0, -1000.0, 0.0] * 8, [-1e4] * 31 + [1e4]], device=DEV)
    y = S._softmax_fwd(x)
    assert torch.isfinite(y).all()
    torch.testing.assert_close(y.sum(-1), torch.ones(2, device=DEV))
    ly = S._logsoftmax_fwd(x)
    assert torch.isfinite(ly).all()
    torch.testing.assert_close(ly, torch.log_softmax(x, -1))


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("kind", ["softmax", "logsoftmax", "softmin"])
def test_reference_unittests(kind, dtype):
    """UnitTests/Activations/{softmax,logsoftmax,softmin}_unittest.py restated."""
    ours = {"softmax": Softmax, "logsoftmax": LogSoftmax, "softmin": Softmin}[kind]()
    ref = {"softmax": nn.Softmax(dim=-1), "logsoftmax": nn.LogSoftmax(dim=-1), "softmin": nn.Softmin(dim=-1)}[kind]
    for D in (32, 256, 2048):
        torch.manual_seed(42)
        data = torch.randn(1, 64, 64, D, device="cuda", dtype=dtype)
        a, r = data.clone().requires_grad_(True), data.clone().requires_grad_(True)
        rtol, atol = (3e-4, 1e-3) if dtype == torch.float32 else (5e-3, 1e-2)
        if dtype == torch.float16:
            rtol, atol = 1e-2, 5e-2
        out, out_ref = ours(a), ref(r)
        assert torch.allclose(out, out_ref, atol=atol, rtol=rtol), 'Error in forward pass'
        g = torch.randn_like(out)
        out.backward(g)
        out_ref.backward(g)
        assert torch.allclose(a.grad, r.grad, atol=atol, rtol=rtol), 'Error in backward pass'


def test_strided_and_unaligned_rows():
    big = torch.randn(10, 600, device=DEV)
    x = big[:, :300]                       # row stride 600, N = 300: aligned rows, strided
    torch.testing.assert_close(S._softmax_fwd(x), torch.softmax(x, -1), rtol=1e-5, atol=1e-6)
    flat = torch.randn(10 * 77 + 1, device=DEV, dtype=torch.float16)
    xu = flat[1:].view(10, 77)             # odd offset and odd length: scalar kernels
    torch.testing.assert_close(S._logsoftmax_fwd(xu).float(), torch.log_softmax(xu.float(), -1), rtol=1e-2, atol=1e-2)
