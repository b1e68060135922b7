"""The oracle's p-norm / normalize against golden vectors from the reference's own kernels
(TritonHub/Ops/norm.py, normalize.py under Triton's interpreter) and torch CPU autograd in fp64
(the comparator of the reference's UnitTests/Ops/norm_unittest.py:38, normalize_unittest.py:37)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import GOLDEN_OPS, TOL, assert_parity, load_golden_arrays
from oracle import oracle as O


def test_golden_present():
    assert len(GOLDEN_OPS) >= 4


@pytest.mark.parametrize("name", GOLDEN_OPS)
@pytest.mark.parametrize("acc64", [False, True])
def test_matches_reference_kernels(name, acc64):
    g = load_golden_arrays(name)
    dt, p, eps = g["dtype"], float(g["meta"][2]), float(g["meta"][3])
    K = g["x"].shape[-1]
    x, dy, dn = g["x"].reshape(-1, K), g["dy"].reshape(-1, K), g["dnorm"].reshape(-1)
    norms = O.pnorm_fwd(x, p=p, eps=eps, dtype=dt, acc64=acc64)
    assert_parity(norms, g["norms"].reshape(-1), TOL[dt], f"{name}: norms")
    assert_parity(O.round_to(O.pnorm_bwd(x, norms, dn, p=p), dt), g["dx_norm"].reshape(-1, K), TOL[dt], f"{name}: d norm")
    y, norms2 = O.normalize_fwd(x, p=p, eps=eps, dtype=dt, acc64=acc64)
    y = O.round_to(y, dt)
    assert_parity(y, g["y"].reshape(-1, K), TOL[dt], f"{name}: y")
    dx = O.round_to(O.normalize_bwd(x, y, norms2, dy, p=p), dt)
    assert_parity(dx, g["dx"].reshape(-1, K), TOL[dt], f"{name}: d normalize")


@pytest.mark.parametrize("p", [1.0, 2.0, 3.0, 2.5, 6.0])
def test_matches_torch_cpu(p):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((13, 77)).astype(np.float32)
    gn = rng.random(13).astype(np.float32)
    g = rng.standard_normal((13, 77)).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    n = torch.norm(xt, p=p, dim=-1)
    n.backward(torch.tensor(gn, dtype=torch.float64))
    norms = O.pnorm_fwd(x, p=p, eps=1e-12, acc64=True)
    assert_parity(norms, n.detach().numpy(), 1e-6, "norms")
    assert_parity(O.pnorm_bwd(x, norms, gn, p=p), xt.grad.numpy(), 1e-6, "d norm")
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    yt = F.normalize(xt, p=p, dim=-1, eps=1e-12)
    yt.backward(torch.tensor(g, dtype=torch.float64))
    y, norms = O.normalize_fwd(x, p=p, eps=1e-12, acc64=True)
    assert_parity(y, yt.detach().numpy(), 1e-6, "y")
    assert_parity(O.normalize_bwd(x, y, norms, g, p=p), xt.grad.numpy(), 1e-6, "d normalize")


def test_eps_clamp():
    x = np.zeros((3, 16), dtype=np.float32)
    assert np.all(O.pnorm_fwd(x, p=2.0, eps=1e-6) == np.float32(1e-6))
    y, _ = O.normalize_fwd(x, p=2.0, eps=1e-6)
    assert np.all(y == 0)
