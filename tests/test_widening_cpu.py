"""The widened ops without a GPU: the reference's import paths resolve (TritonHub/Activations/__init__.py,
TritonHub/Ops/__init__.py), constructors keep its arguments and asserts, CPU tensors are refused, and
the C ABI's argument checks (which run before any CUDA call) answer with the documented codes."""
import inspect

import pytest
import torch

from b200norm import _lib


def test_import_paths_of_the_reference_resolve():
    from TritonHub.Activations import GeLU, LogSoftmax, Softmax, Softmin
    from TritonHub.Ops import norm, normalize
    import b200norm
    assert GeLU is b200norm.GeLU and Softmax is b200norm.Softmax and LogSoftmax is b200norm.LogSoftmax
    assert Softmin is b200norm.Softmin and norm is b200norm.norm and normalize is b200norm.normalize


def test_ops_constructors_keep_the_reference_arguments_and_asserts():
    from TritonHub.Ops import norm, normalize
    for cls in (norm, normalize):  # Ops/norm.py:146-151, Ops/normalize.py:164-169
        sig = inspect.signature(cls.__init__)
        assert list(sig.parameters)[1:] == ["p", "eps"]
        assert sig.parameters["p"].default == 2 and sig.parameters["eps"].default == 1e-6
        with pytest.raises(AssertionError, match=r"p must be in \[1, 6\]"):
            cls(p=0.5)
        with pytest.raises(AssertionError, match=r"p must be in \[1, 6\]"):
            cls(p=7)
        with pytest.raises(AssertionError, match="eps must be non-negative"):
            cls(eps=-1.0)
    assert norm(p=3).p == 3 and normalize(eps=0.0).eps == 0.0


def test_gelu_rejects_an_unknown_approximation_like_the_reference():
    from TritonHub.Activations import GeLU
    with pytest.raises(AssertionError):  # gelu.py:123
        GeLU(approximate="None")
    assert GeLU(approximate="tanh").approximate == "tanh"


def test_cpu_tensors_are_refused_by_every_op():
    from TritonHub.Activations import GeLU, LogSoftmax, Softmax, Softmin
    from TritonHub.Ops import norm, normalize
    x2, x3 = torch.randn(4, 8), torch.randn(1, 4, 8)
    for call in (lambda: GeLU()(x2), lambda: Softmax()(x2), lambda: LogSoftmax()(x2), lambda: Softmin()(x2),
                 lambda: norm()(x3), lambda: normalize()(x3)):
        with pytest.raises(RuntimeError, match="CUDA tensors only"):
            call()


def test_ops_want_three_dimensions_like_the_reference():
    from TritonHub.Ops import norm, normalize
    for cls in (norm, normalize):  # Ops/norm.py:132, Ops/normalize.py:150
        with pytest.raises(AssertionError, match="Expected Tensor to be 3D"):
            cls()(torch.randn(4, 8))


def test_abi_argument_checks_of_the_widened_entry_points():
    lib = _lib.load()
    # p outside [1, 6], negative eps, unknown dtype, row wider than 64 KB
    assert lib.b200norm_pnorm_fwd(None, 8, None, 4, 8, 0.5, 1e-6, _lib.F32, None) == _lib.ERR_ARG
    assert b"p must be in [1, 6]" in lib.b200norm_last_error()
    assert lib.b200norm_normalize_fwd(None, 8, None, 8, None, 4, 8, 2.0, -1.0, _lib.F32, None) == _lib.ERR_ARG
    assert lib.b200norm_pnorm_fwd(None, 8, None, 4, 8, 2.0, 1e-6, 9, None) == _lib.ERR_ARG
    assert lib.b200norm_pnorm_fwd(None, 16385, None, 4, 16385, 2.0, 1e-6, _lib.F32, None) == _lib.ERR_UNSUPPORTED
    assert lib.b200norm_softmax_fwd(None, 32769, None, 32769, 1, 32769, 0, _lib.BF16, None) == _lib.ERR_UNSUPPORTED
    assert lib.b200norm_softmax_fwd(None, 8, None, 8, 4, 8, 2, _lib.F32, None) == _lib.ERR_ARG  # log_softmax not 0 / 1
    # an empty batch is not an error and touches no pointer
    assert lib.b200norm_pnorm_fwd(None, 8, None, 0, 8, 2.0, 1e-6, _lib.F32, None) == _lib.OK
    assert lib.b200norm_normalize_bwd(None, 8, None, 8, None, None, 8, None, 8, 0, 8, 2.0, _lib.F32, None) == _lib.OK
    assert lib.b200norm_softmax_bwd(None, 8, None, 8, None, 8, 0, 8, 1, _lib.F32, None) == _lib.OK


def test_a_missing_library_fails_loudly(monkeypatch, tmp_path):
    """No fallback of any kind: without libb200norm.so the first use raises and says how to build it."""
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", tmp_path / "libb200norm.so")
    with pytest.raises(RuntimeError, match="is missing: build it with"):
        _lib.load()
    with pytest.raises(RuntimeError, match="is missing"):
        _lib.check(_lib.ERR_ARG)
