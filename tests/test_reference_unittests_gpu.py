"""The reference's own UnitTests, restated as pytest: same module construction, same inputs
(seed 42, randn(1, 256, 256, D)), same comparator (torch.nn.LayerNorm / RMSNorm on the GPU) and
the same tolerances (UnitTests/Normalization/layernorm_unittest.py:6-68, rmsnorm_unittest.py).
The reference checks y and dx only; weight.grad and bias.grad are added here."""
import pytest
import torch
import torch.nn as nn

pytestmark = pytest.mark.gpu

from TritonHub.Normalization import LayerNorm, RMSNorm


def tolerances(dtype):
    rtol, atol = (3e-4, 1e-3) if dtype == torch.float32 else (5e-3, 1e-2)   # layernorm_unittest.py:30
    if dtype == torch.float16:
        rtol, atol = 1e-2, 5e-2                                               # layernorm_unittest.py:31-32
    return rtol, atol


@pytest.mark.parametrize("dtype", [torch.float16, torch.float32, torch.float64])
@pytest.mark.parametrize("D", [32, 64, 128, 256, 512, 1024, 2048])
@pytest.mark.parametrize("kind", ["layernorm", "rmsnorm"])
def test_unittest_sweep(kind, D, dtype):
    B, N, M, eps = 1, 256, 256, 1e-5
    if kind == "layernorm":
        ours = LayerNorm(dimension=D, eps=eps, bias=True, elementwise_affine=True, device='cuda', dtype=dtype)
        ref = nn.LayerNorm(D, eps=eps, bias=True, elementwise_affine=True, device='cuda', dtype=dtype)
    else:
        ours = RMSNorm(dimension=D, eps=eps, elementwise_affine=True, device='cuda', dtype=dtype)
        ref = nn.RMSNorm(D, eps=eps, elementwise_affine=True, device='cuda', dtype=dtype)
    torch.manual_seed(42)
    input_data = torch.randn(B, M, N, D, device='cuda', dtype=dtype)
    input = input_data.clone().detach().requires_grad_(True)
    input_ref = input_data.clone().detach().requires_grad_(True)
    rtol, atol = tolerances(dtype)
    output = ours(input)
    output_ref = ref(input_ref)
    assert torch.allclose(output, output_ref, atol=atol, rtol=rtol), 'Error in forward pass'
    g = torch.randn_like(output)
    output.backward(g)
    output_ref.backward(g)
    assert torch.allclose(input.grad, input_ref.grad, atol=atol, rtol=rtol), 'Error in backward pass'
    # beyond the reference's checks: parameter gradients, relative to their largest magnitude
    tol = 1e-5 if dtype != torch.float16 else 1e-2
    for p, q in zip(ours.parameters(), ref.parameters()):
        a, b = p.grad.double(), q.grad.double()
        assert (a - b).abs().max() <= max(tol, 2e-5) * b.abs().max(), 'Error in parameter gradient'
