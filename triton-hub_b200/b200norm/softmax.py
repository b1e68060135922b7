"""Softmax, LogSoftmax and Softmin over the last dimension on libb200norm.so, with the
reference's interface: TritonHub/Activations/softmax.py (`_softmax_fwd` :24-41, `_softmax_bwd`
:64-84, `softmax` :86-97, `Softmax` :99-103), logsoftmax.py (the same layout) and softmin.py
(Softmin = Softmax of -x, :99-103).  The backward takes the saved output, as the reference does."""
from __future__ import annotations

import torch

from . import _lib
from .functional import _code, _on_device, _raw_stream, _require_cuda, _row_stride, _rows


def _fwd(x, log):
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_softmax_fwd(x.data_ptr(), _row_stride(x), out.data_ptr(), N, M, N, int(log),
                                            _code(x, "input"), _raw_stream(x.device.index)))
    return out.reshape(*batch_shape, N)


def _bwd(y, dout, log):
    _require_cuda(y)
    batch_shape = y.shape[:-1]
    y, dout = _rows(y), _rows(dout)
    assert y.shape == dout.shape, 'expect input and output shape to be the same'
    if dout.dtype != y.dtype:
        dout = dout.to(y.dtype)
    M, N = y.shape
    dx = torch.empty((M, N), dtype=y.dtype, device=y.device)
    lib = _lib.load()
    with _on_device(y.device.index):
        _lib.check(lib.b200norm_softmax_bwd(y.data_ptr(), _row_stride(y), dout.data_ptr(), _row_stride(dout),
                                            dx.data_ptr(), N, M, N, int(log), _code(y, "input"),
                                            _raw_stream(y.device.index)))
    return dx.reshape(*batch_shape, N)


def _softmax_fwd(x):
    return _fwd(x, False)


def _softmax_bwd(x, dout):
    """`x` is the forward's OUTPUT, as in the reference (softmax.py:93-96)."""
    return _bwd(x, dout, False)


def _logsoftmax_fwd(x):
    return _fwd(x, True)


def _logsoftmax_bwd(x, dout):
    return _bwd(x, dout, True)


class softmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input):
        output = _softmax_fwd(input)
        ctx.save_for_backward(output)
        return output

    @staticmethod
    def backward(ctx, d_out):
        output, = ctx.saved_tensors
        return _softmax_bwd(output, d_out)


class logsoftmax(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input):
        output = _logsoftmax_fwd(input)
        ctx.save_for_backward(output)
        return output

    @staticmethod
    def backward(ctx, d_out):
        output, = ctx.saved_tensors
        return _logsoftmax_bwd(output, d_out)


class Softmax:
    def __init__(self):
        self.softmax_fn = softmax.apply

    def __call__(self, x):
        return self.softmax_fn(x)


class LogSoftmax:
    def __init__(self):
        self.logsoftmax_fn = logsoftmax.apply

    def __call__(self, x):
        return self.logsoftmax_fn(x)


class Softmin:
    def __init__(self):
        self.softmin_fn = softmax.apply

    def __call__(self, x):
        return self.softmin_fn(-x)
