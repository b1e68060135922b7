"""Host wrappers and autograd Functions for LayerNorm / RMSNorm on libb200norm.so.

The names, argument order and return values mirror TritonHub's host layer so that code (and
tests) written against it keep working:

  _layernorm_fwd / _layernorm_bwd / layernorm   TritonHub/Normalization/layernorm.py:48-87,155-209,211-223
  _rmsnorm_fwd   / _rmsnorm_bwd   / rmsnorm     TritonHub/Normalization/rmsnorm.py:40-70,124-167,169-181

Each wrapper flattens its input to (M, N), allocates the outputs with torch and makes one
call into the C ABI on the current CUDA stream.  CPU tensors are rejected: there is no
fallback path.
"""
from __future__ import annotations

import contextlib

import torch

from . import _lib

_DTYPE_CODE = {
    torch.float32: _lib.F32,
    torch.float16: _lib.F16,
    torch.bfloat16: _lib.BF16,
    torch.float64: _lib.F64,
}


_NULL_CTX = contextlib.nullcontext()
_WS_BYTES = {}  # (device, M, N, dtype code, row_shards) -> workspace bytes; the answer never changes

try:  # the raw cudaStream_t of the current stream without building a Stream object
    _raw_stream = torch._C._cuda_getCurrentRawStream
except AttributeError:  # pragma: no cover
    def _raw_stream(index):
        return torch.cuda.current_stream(index).cuda_stream


def _on_device(index: int):
    """Context that makes `index` the current device; free when it already is (the usual case)."""
    return _NULL_CTX if torch.cuda.current_device() == index else torch.cuda.device(index)


def _workspace_bytes(lib, index, M, N, code, row_shards):
    key = (index, M, N, code, row_shards)
    n = _WS_BYTES.get(key)
    if n is None:
        n = lib.b200norm_bwd_workspace_bytes(M, N, code, row_shards)
        if n == 0:
            _lib.check(_lib.ERR_ARG)
        _WS_BYTES[key] = n
    return n


def _code(t: torch.Tensor, what: str) -> int:
    try:
        return _DTYPE_CODE[t.dtype]
    except KeyError:
        raise RuntimeError(f"b200norm: {what} dtype {t.dtype} is not supported "
                           "(float32, float16, bfloat16, float64)") from None


def _require_cuda(x: torch.Tensor) -> None:
    if not x.is_cuda:
        raise RuntimeError("b200norm runs on CUDA tensors only (no CPU fallback); got a tensor on "
                           f"'{x.device}'")


def _rows(x: torch.Tensor) -> torch.Tensor:
    """Flatten to (M, N) with unit column stride and a row stride the kernels accept."""
    if x.stride(-1) != 1:
        x = x.contiguous()          # as the reference does (layernorm.py:49-50)
    x = x.reshape(-1, x.shape[-1])
    M, N = x.shape
    overlapping_rows = M > 1 and x.stride(0) < N      # e.g. an expanded tensor (row stride 0)
    if overlapping_rows or (N > 1 and x.stride(-1) != 1):
        x = x.contiguous()
    return x


def _row_stride(x: torch.Tensor) -> int:
    return x.stride(0) if x.shape[0] > 1 else x.shape[1]


def _params(weight, bias, N, device):
    """Contiguous parameter vectors of one storage type, or None."""
    if weight is not None:
        weight = weight.contiguous()
        assert weight.shape == (N,), 'expect weight to have shape (N,)'
    if bias is not None:
        bias = bias.contiguous()
        assert bias.shape == (N,), 'expect bias to have shape (N,)'
    if weight is not None and bias is not None and bias.dtype != weight.dtype:
        bias = bias.to(weight.dtype)
    for p in (weight, bias):
        if p is not None and p.device != device:
            raise RuntimeError(f"b200norm: parameter on {p.device}, input on {device}")
    ref = weight if weight is not None else bias
    return weight, bias, (_code(ref, "weight") if ref is not None else _lib.F32)


def _ptr(t):
    return t.data_ptr() if t is not None else None


def _check_dim(x: torch.Tensor, N: int) -> None:
    if N * x.element_size() > 65536:
        raise RuntimeError("This layer norm doesn't support feature dim >= 64KB.")


def _layernorm_fwd(x, weight, bias, eps):
    """LayerNorm forward; returns (y shaped like x, mean (M,) fp32, rstd (M,) fp32)."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    weight, bias, wcode = _params(weight, bias, N, x.device)
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    mean = torch.empty((M,), dtype=torch.float32, device=x.device)
    rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
    _check_dim(x, N)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_ln_fwd(
            x.data_ptr(), _row_stride(x), _ptr(weight), _ptr(bias), out.data_ptr(), N,
            mean.data_ptr(), rstd.data_ptr(), M, N, float(eps), _code(x, "input"), wcode,
            _raw_stream(x.device.index)))
    return out.reshape(*batch_shape, N), mean, rstd


def _rmsnorm_fwd(x, weight, eps):
    """RMSNorm forward; returns (y shaped like x, rstd (M,) fp32)."""
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    weight, _, wcode = _params(weight, None, N, x.device)
    out = torch.empty((M, N), dtype=x.dtype, device=x.device)
    rstd = torch.empty((M,), dtype=torch.float32, device=x.device)
    _check_dim(x, N)
    lib = _lib.load()
    with _on_device(x.device.index):
        _lib.check(lib.b200norm_rms_fwd(
            x.data_ptr(), _row_stride(x), _ptr(weight), out.data_ptr(), N, rstd.data_ptr(), M, N,
            float(eps), _code(x, "input"), wcode, _raw_stream(x.device.index)))
    return out.reshape(*batch_shape, N), rstd


def _bwd_common(op, x, dout, weight, bias, mean, rstd, row_shards, want_group_sums, need_dw, need_db, push=None):
    _require_cuda(x)
    batch_shape = x.shape[:-1]
    x = _rows(x)
    M, N = x.shape
    dout = _rows(dout)
    assert dout.shape == (M, N), 'expect input and output shape to be the same'
    weight, bias, wcode = _params(weight, bias, N, x.device)
    if dout.dtype != x.dtype:
        dout = dout.to(x.dtype)
    dx = torch.empty((M, N), dtype=x.dtype, device=x.device)
    _check_dim(x, N)
    dw = torch.empty((N,), dtype=weight.dtype, device=x.device) if (weight is not None and need_dw) else None
    db = torch.empty((N,), dtype=bias.dtype, device=x.device) if (bias is not None and need_db) else None
    slots = 2 if op == "ln" else 1
    gs = (torch.empty((row_shards, slots, N), dtype=torch.float32, device=x.device)
          if want_group_sums else None)
    lib = _lib.load()
    with _on_device(x.device.index):
        ws, ws_bytes = None, 0
        if dw is not None or db is not None or gs is not None or push is not None:
            ws_bytes = _workspace_bytes(lib, x.device.index, M, N, _code(x, "input"), row_shards)
            ws = torch.empty((ws_bytes,), dtype=torch.uint8, device=x.device)
        stream = _raw_stream(x.device.index)
        if push is not None:  # (Peers, sequence number[, Finish]): shard sums go to every rank's inbox
            peers, seq = push[0], push[1]
            fin = push[2] if len(push) > 2 else None
            if op == "ln":
                status = lib.b200norm_ln_bwd_push(
                    x.data_ptr(), _row_stride(x), dout.data_ptr(), _row_stride(dout), _ptr(weight),
                    mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), N, row_shards, _ptr(ws), ws_bytes, M, N,
                    _code(x, "input"), wcode, peers, seq, fin, stream)
            else:
                status = lib.b200norm_rms_bwd_push(
                    x.data_ptr(), _row_stride(x), dout.data_ptr(), _row_stride(dout), _ptr(weight),
                    rstd.data_ptr(), dx.data_ptr(), N, row_shards, _ptr(ws), ws_bytes, M, N,
                    _code(x, "input"), wcode, peers, seq, fin, stream)
        elif op == "ln":
            status = lib.b200norm_ln_bwd(
                x.data_ptr(), _row_stride(x), dout.data_ptr(), _row_stride(dout), _ptr(weight),
                mean.data_ptr(), rstd.data_ptr(), dx.data_ptr(), N, _ptr(dw), _ptr(db), _ptr(gs),
                row_shards, _ptr(ws), ws_bytes, M, N, _code(x, "input"), wcode, stream)
        else:
            status = lib.b200norm_rms_bwd(
                x.data_ptr(), _row_stride(x), dout.data_ptr(), _row_stride(dout), _ptr(weight),
                rstd.data_ptr(), dx.data_ptr(), N, _ptr(dw), _ptr(gs), row_shards, _ptr(ws), ws_bytes,
                M, N, _code(x, "input"), wcode, stream)
        _lib.check(status)
    return dx.reshape(*batch_shape, N), dw, db, gs


def _layernorm_bwd(x, dout, weight, bias, mean, rstd, eps, *, row_shards=1, group_sums=False,
                   need_dw=True, need_db=True, push=None):
    """LayerNorm backward; returns (dx, dweight, dbias), the last two in the parameters' dtype
    (None for a missing parameter).  With ``group_sums=True`` a fourth value is returned: the
    fp32 (row_shards, 2, N) dweight/dbias sums per row shard, for a multi-GPU exchange.
    ``eps`` is accepted and unused, as in the reference.  ``push=(peers, seq[, finish])`` sends the shard
    sums to every rank's inbox instead (b200norm_ln_bwd_push; `finish` = a pointer to a _lib.Finish naming
    an exchange for the same kernel to finish); pass need_dw=need_db=False with it."""
    dx, dw, db, gs = _bwd_common("ln", x, dout, weight, bias, mean, rstd, row_shards, group_sums,
                                 need_dw, need_db, push)
    return (dx, dw, db, gs) if group_sums else (dx, dw, db)


def _rmsnorm_bwd(x, dout, weight, rstd, eps, *, row_shards=1, group_sums=False, need_dw=True, push=None):
    """RMSNorm backward; returns (dx, dweight) and, with ``group_sums=True``, the fp32
    (row_shards, 1, N) per-shard dweight sums."""
    dx, dw, _, gs = _bwd_common("rms", x, dout, weight, None, None, rstd, row_shards, group_sums,
                                need_dw, False, push)
    return (dx, dw, gs) if group_sums else (dx, dw)


def finalize_dwdb(group_sums: torch.Tensor, w_dtype: torch.dtype):
    """dweight (and dbias) from gathered shard sums (groups, slots, N): added left to right in
    fp32, then cast.  Returns a tuple of ``slots`` tensors."""
    _require_cuda(group_sums)
    assert group_sums.dtype == torch.float32 and group_sums.dim() == 3 and group_sums.is_contiguous()
    groups, slots, N = group_sums.shape
    outs = [torch.empty((N,), dtype=w_dtype, device=group_sums.device) for _ in range(slots)]
    code = _DTYPE_CODE[w_dtype]
    lib = _lib.load()
    with _on_device(group_sums.device.index):
        _lib.check(lib.b200norm_finalize_dwdb(
            group_sums.data_ptr(), groups, slots, outs[0].data_ptr(),
            outs[1].data_ptr() if slots == 2 else None, N, code, _raw_stream(group_sums.device.index)))
    return tuple(outs)


def finish_request(seq, slots, N, w_dtype, device):
    """-> (_lib.Finish, outs): a request for a push kernel to finish exchange `seq` as its second phase,
    and the freshly allocated dweight[, dbias] it will fill.  Keep both alive until the call returns."""
    outs = tuple(torch.empty((N,), dtype=w_dtype, device=device) for _ in range(slots))
    fin = _lib.Finish()
    fin.seq, fin.slots, fin.w_dtype, fin.N = seq, slots, _DTYPE_CODE[w_dtype], N
    fin.dw = outs[0].data_ptr()
    fin.db = outs[1].data_ptr() if slots == 2 else None
    return fin, outs


def finalize_pushed(peers, seq, slots, N, w_dtype, device):
    """dweight (and dbias) of exchange `seq` from this rank's inbox, once every rank has pushed
    (b200norm_finalize_pushed; the wait happens on the GPU, bounded)."""
    outs = [torch.empty((N,), dtype=w_dtype, device=device) for _ in range(slots)]
    lib = _lib.load()
    index = torch.device(device).index
    with _on_device(index):
        _lib.check(lib.b200norm_finalize_pushed(
            peers, seq, slots, outs[0].data_ptr(), outs[1].data_ptr() if slots == 2 else None, N,
            _DTYPE_CODE[w_dtype], _raw_stream(index)))
    return tuple(outs)


class layernorm(torch.autograd.Function):
    """autograd.Function with the reference's contract (layernorm.py:211-223): saves
    (input, weight, bias, mean, rstd); backward returns (dx, dweight, dbias, None)."""

    @staticmethod
    def forward(ctx, input, weight, bias, eps):
        output, mean, rstd = _layernorm_fwd(input, weight, bias, eps)
        ctx.save_for_backward(input, weight, bias, mean, rstd)
        ctx.eps = eps
        return output

    @staticmethod
    def backward(ctx, d_out):
        input, weight, bias, mean, rstd = ctx.saved_tensors
        grad, dw, db = _layernorm_bwd(input, d_out, weight, bias, mean, rstd, ctx.eps,
                                      need_dw=ctx.needs_input_grad[1], need_db=ctx.needs_input_grad[2])
        return grad, dw, db, None


class rmsnorm(torch.autograd.Function):
    """autograd.Function with the reference's contract (rmsnorm.py:169-181): saves
    (input, weight, rstd); backward returns (dx, dweight, None)."""

    @staticmethod
    def forward(ctx, input, weight, eps):
        output, rstd = _rmsnorm_fwd(input, weight, eps)
        ctx.save_for_backward(input, weight, rstd)
        ctx.eps = eps
        return output

    @staticmethod
    def backward(ctx, d_out):
        input, weight, rstd = ctx.saved_tensors
        grad, dw = _rmsnorm_bwd(input, d_out, weight, rstd, ctx.eps, need_dw=ctx.needs_input_grad[1])
        return grad, dw, None
