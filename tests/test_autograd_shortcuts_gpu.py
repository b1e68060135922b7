"""Gradients that autograd does not need are not computed.

The reference's Functions always return all three gradients (TritonHub/Normalization/layernorm.py:219-223,
rmsnorm.py:177-181); this library's backward skips dweight / dbias when `ctx.needs_input_grad` says
the parameter is frozen -- and then needs no partial-row workspace and launches no column reduce.
Checked through the public modules with autograd: the frozen parameter's `.grad` stays None, dx and
the other gradients are bit-identical to the all-trainable run, and the workspace is never sized.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from b200norm import LayerNorm, RMSNorm
from b200norm import functional as Fn

DEV = "cuda:0"


def _run(mod, x, dy):
    x = x.clone().requires_grad_(True)
    mod.zero_grad(set_to_none=True)
    mod(x).backward(dy)
    torch.cuda.synchronize()
    return x.grad


@pytest.mark.parametrize("dtype,N", [(torch.bfloat16, 4096), (torch.float32, 1000), (torch.float16, 77)])
@pytest.mark.parametrize("frozen", [("weight",), ("bias",), ("weight", "bias")])
def test_layernorm_frozen_parameters(dtype, N, frozen, monkeypatch):
    torch.manual_seed(0)
    M = 300
    mod = LayerNorm(N, eps=1e-5, device=DEV, dtype=dtype)
    with torch.no_grad():
        mod.weight.normal_(1, 0.1)
        mod.bias.normal_(0, 0.1)
    x = torch.randn(M, N, device=DEV, dtype=dtype)
    dy = torch.randn(M, N, device=DEV, dtype=dtype)
    dx_all = _run(mod, x, dy)
    want = {"weight": mod.weight.grad.clone(), "bias": mod.bias.grad.clone()}

    sized = []
    real = Fn._workspace_bytes
    monkeypatch.setattr(Fn, "_workspace_bytes", lambda *a: sized.append(a) or real(*a))
    for name in frozen:
        getattr(mod, name).requires_grad_(False)
    dx = _run(mod, x, dy)
    assert torch.equal(dx, dx_all)
    for name in ("weight", "bias"):
        if name in frozen:
            assert getattr(mod, name).grad is None
        else:
            assert torch.equal(getattr(mod, name).grad, want[name])
    assert bool(sized) == (len(frozen) < 2), "the partial-row workspace is sized only when a parameter gradient is wanted"


@pytest.mark.parametrize("dtype,N", [(torch.bfloat16, 4096), (torch.float32, 1000)])
def test_rmsnorm_frozen_weight(dtype, N, monkeypatch):
    torch.manual_seed(1)
    M = 300
    mod = RMSNorm(N, eps=1e-6, device=DEV, dtype=dtype)
    with torch.no_grad():
        mod.weight.normal_(1, 0.1)
    x = torch.randn(M, N, device=DEV, dtype=dtype)
    dy = torch.randn(M, N, device=DEV, dtype=dtype)
    dx_all = _run(mod, x, dy)
    assert mod.weight.grad is not None
    sized = []
    real = Fn._workspace_bytes
    monkeypatch.setattr(Fn, "_workspace_bytes", lambda *a: sized.append(a) or real(*a))
    mod.weight.requires_grad_(False)
    dx = _run(mod, x, dy)
    assert torch.equal(dx, dx_all) and mod.weight.grad is None and not sized


def test_input_that_needs_no_gradient_still_gets_parameter_gradients():
    """x without requires_grad: autograd still asks for dweight / dbias; they match the usual run."""
    torch.manual_seed(2)
    M, N = 128, 512
    mod = LayerNorm(N, device=DEV, dtype=torch.float32)
    x = torch.randn(M, N, device=DEV)
    dy = torch.randn(M, N, device=DEV)
    _run(mod, x, dy)
    want_w, want_b = mod.weight.grad.clone(), mod.bias.grad.clone()
    mod.zero_grad(set_to_none=True)
    mod(x).backward(dy)                      # x is a leaf that needs no gradient
    torch.cuda.synchronize()
    assert torch.equal(mod.weight.grad, want_w) and torch.equal(mod.bias.grad, want_b)
