"""GeLU on libb200norm.so -- the activation that follows the norm in the reference's Quick Start.

Stand-alone form, mirroring TritonHub/Activations/gelu.py: `_gelu_fwd` (:31-49), `_gelu_bwd`
(:83-105), the `gelu` autograd.Function (:107-119) and the `GeLU` callable (:121-129).

Fused form: `LayerNormGeLU` / `RMSNormGeLU` compute act(norm(x)) in ONE forward kernel and ONE
backward kernel (b200norm_*_act_fwd / _bwd): the normalised tensor is never written to memory,
and the backward rebuilds it from the saved statistics.  That halves the bytes of the
LayerNorm -> GeLU pair (5 row passes instead of 10).  The reference has no fused form; these
modules keep the norms' constructor arguments and add `approximate`.
"""
from __future__ import annotations

import torch

from . import _lib
from . import functional as Fn
from .functional import _DTYPE_CODE, _code, _on_device, _params, _ptr, _raw_stream, _require_cuda, _row_stride, _rows

_APPROX = {'none': 0, 'tanh': 1}
_ACT = {'none': _lib.ACT_GELU_ERF, 'tanh': _lib.ACT_GELU_TANH}


def _gelu_fwd(x, approximate='none'):
    """y = gelu(x); any shape, flattened to rows like the reference does."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_gelu_fwd(x.data_ptr(), _row_stride(x), out.data_ptr(), N, M, N,
                                         _APPROX[approximate], _code(x, "input"), _raw_stream(x.device.index)))
    return out.reshape(*batch_shape, N)


def _gelu_bwd(x, dout, approximate='none'):
    """dx = dout * gelu'(x)."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    dout = _rows(dout)
    assert x.shape == dout.shape, 'expect input and output shape to be the same'
    if dout.dtype != x.dtype:
        dout = dout.to(x.dtype)
    M, N = x.shape
    dx = torch.empty((M, N), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_gelu_bwd(x.data_ptr(), _row_stride(x), dout.data_ptr(), _row_stride(dout),
                                         dx.data_ptr(), N, M, N, _APPROX[approximate], _code(x, "input"),
                                         _raw_stream(x.device.index)))
    return dx.reshape(*batch_shape, N)


class gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, approximate):
        output = _gelu_fwd(input, approximate)
        ctx.save_for_backward(input)
        ctx.approximate = approximate
        return output

    @staticmethod
    def backward(ctx, d_out):
        input, = ctx.saved_tensors
        return _gelu_bwd(input, d_out, ctx.approximate), None


class GeLU:
    """Callable with the reference's interface (gelu.py:121-129)."""

    def __init__(self, approximate='none'):
        assert approximate in ['none', 'tanh'], 'GeLU approximate must be either none or tanh'
        self.approximate = approximate
        self.gelu_fn = gelu.apply

    def __call__(self, x):
        return self.gelu_fn(x, self.approximate)


# ---------------------------------------------------------------------------------------------
# norm -> GeLU in one kernel each way
# ---------------------------------------------------------------------------------------------
def _unaligned(status: int) -> bool:
    return status == _lib.ERR_UNSUPPORTED and b"fused activation" in _lib.load().b200norm_last_error()


def _norm_gelu_fwd(op, x, weight, bias, eps, approximate):
    """z = gelu(norm(x)); returns (z, mean or None, rstd).  Rows that are not 16-byte aligned run
    the two steps one after the other (same result, twice the traffic)."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    weight, bias, wcode = _params(weight, bias if op == "ln" else None, N, x.device)
    Fn._check_dim(x, N)
    z = torch.empty((M, N), dtype=x.dtype, device=x.device)
    mean = torch.empty((M,), dtype=torch.float32, device=x.device) if op == "ln" else None
    rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        stream = _raw_stream(x.device.index)
        if op == "ln":
            status = lib.b200norm_ln_act_fwd(x.data_ptr(), _row_stride(x), _ptr(weight), _ptr(bias), z.data_ptr(), N,
                                             mean.data_ptr(), rstd.data_ptr(), M, N, float(eps), _ACT[approximate],
                                             _code(x, "input"), wcode, stream)
        else:
            status = lib.b200norm_rms_act_fwd(x.data_ptr(), _row_stride(x), _ptr(weight), z.data_ptr(), N,
                                              rstd.data_ptr(), M, N, float(eps), _ACT[approximate],
                                              _code(x, "input"), wcode, stream)
        if _unaligned(status):
            if op == "ln":
                y, mean, rstd = Fn._layernorm_fwd(x, weight, bias, eps)
            else:
                y, rstd = Fn._rmsnorm_fwd(x, weight, eps)
            z = _gelu_fwd(y, approximate)
        else:
            _lib.check(status)
    return z.reshape(*batch_shape, N), mean, rstd


def _norm_gelu_bwd(op, x, dz, weight, bias, mean, rstd, eps, approximate, need_dw=True, need_db=True):
    """Backward of z = gelu(norm(x)): returns (dx, dweight, dbias)."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    dz = _rows(dz)
    assert dz.shape == (M, N), 'expect input and output shape to be the same'
    if dz.dtype != x.dtype:
        dz = dz.to(x.dtype)
    weight, bias, wcode = _params(weight, bias if op == "ln" else None, N, x.device)
    dx = torch.empty((M, N), dtype=x.dtype, device=x.device)
    dw = torch.empty((N,), dtype=weight.dtype, device=x.device) if (weight is not None and need_dw) else None
    db = torch.empty((N,), dtype=bias.dtype, device=x.device) if (bias is not None and need_db) else None
    lib = _lib.load()
    with _on_device(x.device.index):
        ws, ws_bytes = None, 0
        if dw is not None or db is not None:
            ws_bytes = Fn._workspace_bytes(lib, x.device.index, M, N, _code(x, "input"), 1)
            ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=x.device)
        stream = _raw_stream(x.device.index)
        if op == "ln":
            status = lib.b200norm_ln_act_bwd(
                x.data_ptr(), _row_stride(x), dz.data_ptr(), _row_stride(dz), _ptr(weight), _ptr(bias),
                mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), N, _ptr(dw), _ptr(db), None, 1, _ptr(ws), ws_bytes,
                M, N, _ACT[approximate], _code(x, "input"), wcode, stream)
        else:
            status = lib.b200norm_rms_act_bwd(
                x.data_ptr(), _row_stride(x), dz.data_ptr(), _row_stride(dz), _ptr(weight), rstd.data_ptr(),
                dx.data_ptr(), N, _ptr(dw), None, 1, _ptr(ws), ws_bytes, M, N, _ACT[approximate],
                _code(x, "input"), wcode, stream)
        if _unaligned(status):
            # rebuild y with the norm's forward, then the two backward steps
            if op == "ln":
                y, _, _ = Fn._layernorm_fwd(x, weight, bias, eps)
                dy = _gelu_bwd(y, dz, approximate)
                dx, dw, db = Fn._layernorm_bwd(x, dy, weight, bias, mean, rstd, eps, need_dw=need_dw, need_db=need_db)
            else:
                y, _ = Fn._rmsnorm_fwd(x, weight, eps)
                dy = _gelu_bwd(y, dz, approximate)
                dx, dw = Fn._rmsnorm_bwd(x, dy, weight, rstd, eps, need_dw=need_dw)
            return dx.reshape(*batch_shape, N), dw, db
        _lib.check(status)
    return dx.reshape(*batch_shape, N), dw, db


class layernorm_gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, bias, eps, approximate):
        z, mean, rstd = _norm_gelu_fwd("ln", input, weight, bias, eps, approximate)
        ctx.save_for_backward(input, weight, bias, mean, rstd)
        ctx.eps, ctx.approximate = eps, approximate
        return z

    @staticmethod
    def backward(ctx, d_out):
        input, weight, bias, mean, rstd = ctx.saved_tensors
        dx, dw, db = _norm_gelu_bwd("ln", input, d_out, weight, bias, mean, rstd, ctx.eps, ctx.approximate,
                                    ctx.needs_input_grad[1], ctx.needs_input_grad[2])
        return dx, dw, db, None, None


class rmsnorm_gelu(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, eps, approximate):
        z, _, rstd = _norm_gelu_fwd("rms", input, weight, None, eps, approximate)
        ctx.save_for_backward(input, weight, rstd)
        ctx.eps, ctx.approximate = eps, approximate
        return z

    @staticmethod
    def backward(ctx, d_out):
        input, weight, rstd = ctx.saved_tensors
        dx, dw, _ = _norm_gelu_bwd("rms", input, d_out, weight, None, None, rstd, ctx.eps, ctx.approximate,
                                   ctx.needs_input_grad[1], False)
        return dx, dw, None, None


from .modules import LayerNorm, RMSNorm  # noqa: E402  (the fused modules reuse their parameters and init)


class LayerNormGeLU(LayerNorm):
    """LayerNorm followed by GeLU, one kernel each way.  Same constructor as LayerNorm plus
    `approximate` ('none' or 'tanh'); same parameters and state_dict."""

    def __init__(self, dimension, eps=1e-5, elementwise_affine=True, bias=True, approximate='none', device=None,
                 dtype=None):
        assert approximate in ['none', 'tanh'], 'GeLU approximate must be either none or tanh'
        super().__init__(dimension, eps, elementwise_affine, bias, device, dtype)
        self.approximate = approximate

    def forward(self, x):
        return layernorm_gelu.apply(x, self.weight, self.bias, self.eps, self.approximate)


class RMSNormGeLU(RMSNorm):
    """RMSNorm followed by GeLU, one kernel each way."""

    def __init__(self, dimension, eps=1e-5, elementwise_affine=True, approximate='none', device=None, dtype=None):
        assert approximate in ['none', 'tanh'], 'GeLU approximate must be either none or tanh'
        super().__init__(dimension, eps, elementwise_affine, device, dtype)
        self.approximate = approximate

    def forward(self, x):
        return rmsnorm_gelu.apply(x, self.weight, self.eps, self.approximate)
