"""Host-side mirror of the reference's module interface (TritonHub/Normalization/layernorm.py:225-252,
rmsnorm.py:183-204): constructor signatures, attributes, parameters, state_dict -- all
checkable without a GPU -- and the refusal to run on CPU tensors."""
import inspect

import pytest
import torch

import b200norm
from b200norm import LayerNorm, RMSNorm


def test_import_path_of_the_reference_still_resolves():
    from TritonHub.Normalization import LayerNorm as L2, RMSNorm as R2
    assert L2 is LayerNorm and R2 is RMSNorm


def test_constructor_signatures_match_the_reference():
    ln = inspect.signature(LayerNorm.__init__)
    assert list(ln.parameters)[1:] == ["dimension", "eps", "elementwise_affine", "bias", "device", "dtype"]
    assert ln.parameters["eps"].default == 1e-5
    rms = inspect.signature(RMSNorm.__init__)
    assert list(rms.parameters)[1:] == ["dimension", "eps", "elementwise_affine", "device", "dtype"]


def test_layernorm_parameters_and_attributes():
    m = LayerNorm(dimension=128, eps=1e-6, elementwise_affine=True, bias=True, dtype=torch.float16)
    assert (m.dim, m.eps, m.elementwise_affine) == (128, 1e-6, True)
    assert m.weight.shape == (128,) and m.weight.dtype == torch.float16
    assert torch.all(m.weight == 1) and torch.all(m.bias == 0)
    assert m.layernorm_fn is not None
    m = LayerNorm(64, bias=False)
    assert m.bias is None and m.weight is not None
    m = LayerNorm(64, elementwise_affine=False)
    assert m.weight is None and m.bias is None


def test_rmsnorm_parameters_and_attributes():
    m = RMSNorm(dimension=32, eps=1e-6)
    assert m.bias is None and torch.all(m.weight == 1) and m.rmsnorm_fn is not None
    assert RMSNorm(32, elementwise_affine=False).weight is None


def test_state_dict_interchanges_with_torch_nn():
    ours, theirs = LayerNorm(48), torch.nn.LayerNorm(48)
    with torch.no_grad():
        theirs.weight.normal_()
        theirs.bias.normal_()
    ours.load_state_dict(theirs.state_dict())
    assert torch.equal(ours.weight, theirs.weight) and torch.equal(ours.bias, theirs.bias)
    theirs.load_state_dict(ours.state_dict())
    r_ours, r_theirs = RMSNorm(48), torch.nn.RMSNorm(48)
    r_theirs.load_state_dict(r_ours.state_dict())
    assert set(r_ours.state_dict()) == {"weight"}


def test_cpu_tensors_are_rejected_not_silently_computed():
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        LayerNorm(8)(torch.randn(2, 8))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        RMSNorm(8)(torch.randn(2, 8))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        b200norm._layernorm_fwd(torch.randn(2, 8), None, None, 1e-5)


def test_product_package_does_not_import_the_oracle():
    import sys
    mods = [m for m in sys.modules if m.startswith("b200norm")]
    assert mods
    src = "".join(open(sys.modules[m].__file__).read() for m in mods if getattr(sys.modules[m], "__file__", None))
    assert "oracle" not in src
