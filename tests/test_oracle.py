"""The CPU oracle against the golden vectors (outputs of the reference's own Triton kernel
bodies, tests/golden/make_golden.py) and against torch's CPU layer_norm / rms_norm, the
comparator of the reference's UnitTests (UnitTests/Normalization/layernorm_unittest.py:17,37)."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from helpers import GOLDEN, TOL, TORCH_DTYPE, assert_parity, load_golden, make_inputs, oracle_all, to_torch
from oracle import oracle as O


def test_golden_files_present():
    assert len(GOLDEN) >= 10


@pytest.mark.parametrize("name", GOLDEN)
@pytest.mark.parametrize("acc64", [False, True])
def test_oracle_matches_reference_kernels(name, acc64):
    g = load_golden(name)
    rms = g["op"] == "rms"
    out = oracle_all(g["x"], g["dy"], g["w"], g["b"], g["eps"], rms=rms, dtype=g["dtype"],
                     programs=g["programs"], acc64=acc64)
    tol = TOL[g["dtype"]]
    for key in ("y", "dx", "dw", "db", "mean", "rstd"):
        if g[key] is None:
            assert out[key] is None or key in ("dw", "db")
            continue
        # statistics are fp32 whatever the storage type
        assert_parity(out[key], g[key], 1e-5 if key in ("mean", "rstd") else tol, f"{name}:{key}")


@pytest.mark.parametrize("dtype,M,N,mu,sigma,eps", [
    ("fp32", 200, 128, 0.0, 1.0, 1e-6),
    ("fp32", 33, 1000, 0.0, 1.0, 1e-5),
    ("fp16", 16, 5120, 3.0, 2.0, 1e-5),
    ("bf16", 16, 4096, 0.0, 1.0, 1e-6),
    ("fp64", 9, 96, 0.0, 1.0, 1e-5),
])
@pytest.mark.parametrize("rms", [False, True])
def test_oracle_matches_torch_cpu(dtype, M, N, mu, sigma, eps, rms):
    x, dy, w, b = make_inputs(M, N, dtype, mu=mu, sigma=sigma, has_b=not rms)
    out = oracle_all(x, dy, w, b, eps, rms=rms, dtype=dtype, programs=7)
    # torch in fp64 from the same storage-rounded values is the truth the bars are scaled by
    xt = to_torch(x, "fp64").requires_grad_(True)
    wt = to_torch(w, "fp64").requires_grad_(True)
    bt = None if rms else to_torch(b, "fp64").requires_grad_(True)
    yt = F.rms_norm(xt, (N,), wt, eps) if rms else F.layer_norm(xt, (N,), wt, bt, eps)
    yt.backward(to_torch(dy, "fp64"))
    tol = TOL[dtype]
    assert_parity(out["y"], yt.detach().numpy(), tol, "y")
    assert_parity(out["dx"], xt.grad.numpy(), tol, "dx")
    assert_parity(out["dw"], wt.grad.numpy(), tol, "dw")
    if not rms:
        assert_parity(out["db"], bt.grad.numpy(), tol, "db")


def test_oracle_thread_count_does_not_change_results():
    x, dy, w, b = make_inputs(64, 256, "fp32")
    O.set_threads(1)
    a = oracle_all(x, dy, w, b, 1e-5, rms=False, dtype="fp32", programs=8)
    O.set_threads(4)
    c = oracle_all(x, dy, w, b, 1e-5, rms=False, dtype="fp32", programs=8)
    O.set_threads(1)
    for k in a:
        assert np.array_equal(a[k], c[k]), k


def test_round_to_bf16_matches_torch():
    v = np.random.default_rng(1).standard_normal(10000).astype(np.float32) * 100
    assert np.array_equal(O.round_to(v, "bf16"), torch.from_numpy(v).bfloat16().float().numpy())
    assert np.array_equal(O.round_to(v, "fp16"), torch.from_numpy(v).half().float().numpy())
