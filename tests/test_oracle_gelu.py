"""The oracle's GeLU against the golden vectors made by the reference's own GeLU kernels
(TritonHub/Activations/gelu.py, run through Triton's interpreter) and against torch CPU, and the
LayerNorm -> GeLU chain of the reference's Quick Start against the chain of reference kernels."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import GOLDEN_CHAIN, GOLDEN_GELU, TOL, assert_parity, load_golden_arrays
from oracle import oracle as O


def test_golden_present():
    assert len(GOLDEN_GELU) >= 4 and len(GOLDEN_CHAIN) >= 2


@pytest.mark.parametrize("name", GOLDEN_GELU)
@pytest.mark.parametrize("acc64", [False, True])
def test_gelu_matches_reference_kernels(name, acc64):
    g = load_golden_arrays(name)
    approximate, dt = g["meta"][2], g["dtype"]
    y = O.round_to(O.gelu_fwd(g["x"], approximate, acc64=acc64), dt)
    dx = O.round_to(O.gelu_bwd(g["x"], g["dout"], approximate, acc64=acc64), dt)
    assert_parity(y, g["y"], TOL[dt], f"{name}: y")
    assert_parity(dx, g["dx"], TOL[dt], f"{name}: dx")


@pytest.mark.parametrize("approximate", ["none", "tanh"])
def test_gelu_matches_torch_cpu(approximate):
    rng = np.random.default_rng(0)
    x = (3 * rng.standard_normal(5000)).astype(np.float32)
    g = rng.standard_normal(5000).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    yt = F.gelu(xt, approximate=approximate)
    yt.backward(torch.tensor(g, dtype=torch.float64))
    assert_parity(O.gelu_fwd(x, approximate), yt.detach().numpy(), 1e-5, "y")
    assert_parity(O.gelu_bwd(x, g, approximate), xt.grad.numpy(), 1e-5, "dx")


@pytest.mark.parametrize("name", GOLDEN_CHAIN)
def test_norm_gelu_chain_matches_reference_kernel_chain(name):
    g = load_golden_arrays(name)
    eps, approximate, dt = float(g["meta"][2]), g["meta"][3], g["dtype"]
    out = O.norm_gelu(g["x"], g["dz"], g["w"], g["b"], eps, approximate, programs=4, acc64=True)
    # The reference writes y to memory in the storage type between its two kernels and reads it back;
    # the un-rounded chain can therefore differ from it by two storage-type roundings instead of one.
    tol = TOL[dt] * (2 if dt in ("fp16", "bf16") else 1)
    for key in ("z", "dx", "dw", "db"):
        assert_parity(O.round_to(out[key], dt), g[key], tol, f"{name}: {key}")
