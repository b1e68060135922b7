"""The oracle's Softmax / LogSoftmax against golden vectors from the reference's own kernels
(TritonHub/Activations/softmax.py, logsoftmax.py under Triton's interpreter) and torch CPU."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import GOLDEN_SOFTMAX, TOL, assert_parity, load_golden_arrays
from oracle import oracle as O


def test_golden_present():
    assert len(GOLDEN_SOFTMAX) >= 4


@pytest.mark.parametrize("name", GOLDEN_SOFTMAX)
@pytest.mark.parametrize("acc64", [False, True])
def test_matches_reference_kernels(name, acc64):
    g = load_golden_arrays(name)
    log, dt = g["meta"][0] == "logsoftmax", g["dtype"]
    y = O.round_to(O.softmax_fwd(g["x"], log=log, acc64=acc64), dt)
    dx = O.round_to(O.softmax_bwd(g["y"], g["dout"], log=log, acc64=acc64), dt)
    assert_parity(y, g["y"], TOL[dt], f"{name}: y")
    assert_parity(dx, g["dx"], TOL[dt], f"{name}: dx")


@pytest.mark.parametrize("log", [False, True])
def test_matches_torch_cpu(log):
    rng = np.random.default_rng(0)
    x = (3 * rng.standard_normal((17, 301))).astype(np.float32)
    g = rng.standard_normal((17, 301)).astype(np.float32)
    xt = torch.tensor(x, dtype=torch.float64, requires_grad=True)
    yt = F.log_softmax(xt, -1) if log else F.softmax(xt, -1)
    yt.backward(torch.tensor(g, dtype=torch.float64))
    y = O.softmax_fwd(x, log=log)
    assert_parity(y, yt.detach().numpy(), 1e-5, "y")
    assert_parity(O.softmax_bwd(y, g, log=log), xt.grad.numpy(), 1e-5, "dx")
