"""p-norm and normalisation over the last dimension on libb200norm.so, with the reference's
interface: TritonHub/Ops/norm.py (`_norm_fwd` :47-60, `_norm_bwd` :103-126, `Norm` :128-144, `norm`
:146-153) and Ops/normalize.py (`_normalize_fwd` :35-59, `_normalize_bwd` :119-144, `Normalize`
:146-162, `normalize` :164-171).  Inputs are 3-D (B, M, K) as the reference requires; the rows are
handed to the library as (B*M, K)."""
from __future__ import annotations

import torch

from . import _lib
from .functional import _code, _on_device, _raw_stream, _require_cuda, _row_stride, _rows


def _norm_fwd(x, p=2, eps=1e-6):
    _require_cuda(x)
    B, M, K = x.shape
    xr = _rows(x)
    norms_x = torch.empty((B, M), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_pnorm_fwd(xr.data_ptr(), _row_stride(xr), norms_x.data_ptr(), B * M, K, float(p),
                                          float(eps), _code(x, "input"), _raw_stream(x.device.index)))
    return norms_x


def _norm_bwd(x, norms_x, dout, p=2):
    _require_cuda(x)
    B, M = norms_x.shape
    K = x.shape[-1]
    assert x.shape == (B, M, K), "Input shape mismatch"
    assert norms_x.shape == (B, M), "Input gradient shape mismatch"
    assert dout.shape == (B, M), "Output gradient shape mismatch"
    assert x.dtype == norms_x.dtype == dout.dtype, "All tensors must have the same dtype"
    norms_x, dout = norms_x.contiguous(), dout.contiguous()
    xr = _rows(x)
    dx = torch.empty((B, M, K), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_pnorm_bwd(xr.data_ptr(), _row_stride(xr), norms_x.data_ptr(), dout.data_ptr(),
                                          dx.data_ptr(), K, B * M, K, float(p), _code(x, "input"),
                                          _raw_stream(x.device.index)))
    return dx


def _normalize_fwd(x, p=2, eps=1e-6):
    _require_cuda(x)
    B, M, K = x.shape
    xr = _rows(x)
    x_norm = torch.empty((B, M, K), dtype=x.dtype, device=x.device)
    norms_x = torch.empty((B, M), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_normalize_fwd(xr.data_ptr(), _row_stride(xr), x_norm.data_ptr(), K, norms_x.data_ptr(),
                                              B * M, K, float(p), float(eps), _code(x, "input"),
                                              _raw_stream(x.device.index)))
    return x_norm, norms_x


def _normalize_bwd(x, x_norm, norms_x, dout, p=2):
    _require_cuda(x_norm)
    B, M, K = x_norm.shape
    assert dout.shape == (B, M, K), "Output gradient shape mismatch"
    assert x_norm.dtype == norms_x.dtype == dout.dtype, "All tensors must have the same dtype"
    norms_x = norms_x.contiguous()
    xr, yr, gr = _rows(x), _rows(x_norm), _rows(dout)
    dx = torch.empty((B, M, K), dtype=x_norm.dtype, device=x_norm.device)
    lib = _lib.load()
    with _on_device(x_norm.device.index):
        _lib.check(lib.b200norm_normalize_bwd(xr.data_ptr(), _row_stride(xr), yr.data_ptr(), _row_stride(yr),
                                              norms_x.data_ptr(), gr.data_ptr(), _row_stride(gr), dx.data_ptr(), K,
                                              B * M, K, float(p), _code(x_norm, "input"),
                                              _raw_stream(x_norm.device.index)))
    return dx


class Norm(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type='cuda')
    def forward(ctx, x, p=2, eps=1e-6):
        assert len(x.shape) == 3, "Expected Tensor to be 3D (B, L, D), add batch dim input is 2D"
        ctx.p = p
        norms_x = _norm_fwd(x, p, eps)
        ctx.save_for_backward(x, norms_x)
        return norms_x

    @staticmethod
    @torch.amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        x, norms_x = ctx.saved_tensors
        return _norm_bwd(x, norms_x, grad_output, ctx.p), None, None


class Normalize(torch.autograd.Function):
    @staticmethod
    @torch.amp.custom_fwd(device_type='cuda')
    def forward(ctx, x, p=2, eps=1e-6):
        assert len(x.shape) == 3, "Expected Tensor to be 3D (B, L, D), add batch dim input is 2D"
        ctx.p = p
        x_norm, norms_x = _normalize_fwd(x, p, eps)
        ctx.save_for_backward(x, x_norm, norms_x)
        return x_norm

    @staticmethod
    @torch.amp.custom_bwd(device_type='cuda')
    def backward(ctx, grad_output):
        x, x_norm, norms_x = ctx.saved_tensors
        return _normalize_bwd(x, x_norm, norms_x, grad_output, ctx.p), None, None


class norm:
    def __init__(self, p=2, eps=1e-6):
        assert p >= 1 and p <= 6, "p must be in [1, 6] for numerical stability"
        assert eps >= 0, "eps must be non-negative"
        self.p = p
        self.eps = eps
        self.norm = Norm.apply

    def __call__(self, x):
        return self.norm(x, self.p, self.eps)


class normalize:
    def __init__(self, p=2, eps=1e-6):
        assert p >= 1 and p <= 6, "p must be in [1, 6] for numerical stability"
        assert eps >= 0, "eps must be non-negative"
        self.p = p
        self.eps = eps
        self.normalize = Normalize.apply

    def __call__(self, x):
        return self.normalize(x, self.p, self.eps)
