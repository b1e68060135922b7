"""Parity of the CUDA kernels, called through the C ABI (ctypes) exactly as the modules call
them, with the CPU oracle and the golden vectors.

Bars (north star): max|a-ref| <= tol * max|ref| per tensor with tol = 1e-5 for fp32 storage
and 1e-2 for fp16 / bf16, on y, dx, dweight and dbias.  `ref` is the oracle evaluated in
fp64 and rounded to the storage type, or the golden output of the reference's own kernels.
"""
import numpy as np
import pytest
import torch

from helpers import (GOLDEN, TOL, TORCH_DTYPE, assert_parity, load_golden, make_inputs, oracle_all, to_numpy,
                     to_torch)

pytestmark = pytest.mark.gpu

import b200norm
from b200norm import LayerNorm, RMSNorm, _lib
from b200norm import functional as Fn

DEV = "cuda:0"


def run_ours(x, dy, w, b, eps, *, rms, dtype, wdtype=None, row_shards=1):
    """numpy in -> our kernels through the functional wrappers -> numpy out."""
    wdtype = wdtype or dtype
    xt, dyt = to_torch(x, dtype, DEV), to_torch(dy, dtype, DEV)
    wt, bt = to_torch(w, wdtype, DEV), to_torch(b, wdtype, DEV)
    if rms:
        y, rstd = Fn._rmsnorm_fwd(xt, wt, eps)
        dx, dw = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, eps, row_shards=row_shards)
        mean, db = None, None
    else:
        y, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, eps)
        dx, dw, db = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, eps, row_shards=row_shards)
    torch.cuda.synchronize()
    return {k: to_numpy(v) for k, v in dict(y=y, mean=mean, rstd=rstd, dx=dx, dw=dw, db=db).items()}


def check_against_oracle(x, dy, w, b, eps, *, rms, dtype, wdtype=None, row_shards=1, label=""):
    got = run_ours(x, dy, w, b, eps, rms=rms, dtype=dtype, wdtype=wdtype, row_shards=row_shards)
    ref = oracle_all(x, dy, w, b, eps, rms=rms, dtype=dtype, programs=8, acc64=True)
    if wdtype is not None and wdtype != dtype:
        # parameter gradients are rounded to the parameter type, not the activation type
        from oracle import oracle as O
        y, mean, rstd = O.norm_fwd(x, w, None if rms else b, eps, rms=rms, acc64=True)
        _, dw, db = O.norm_bwd(x, dy, w, mean, rstd, rms=rms, programs=8, acc64=True)
        ref["dw"] = O.round_to(dw, wdtype) if w is not None else None
        ref["db"] = O.round_to(db, wdtype) if (b is not None and not rms) else None
    tol = TOL[dtype]
    # natural magnitude of dx, |w * dy| * rstd: the bar's scale when the exact dx is all zeros
    wmax = 1.0 if w is None else float(np.max(np.abs(w)))
    dx_floor = 1e-2 * wmax * float(np.max(np.abs(dy))) * float(np.max(ref["rstd"]))
    for key in ("y", "dx", "dw", "db"):
        if ref[key] is None:
            assert got[key] is None, f"{label}{key} should be None"
            continue
        assert_parity(got[key], ref[key], tol, f"{label}{key}", floor=dx_floor if key == "dx" else 0.0)
    assert_parity(got["rstd"], ref["rstd"], 1e-5, f"{label}rstd")
    if not rms:
        assert_parity(got["mean"], ref["mean"], 1e-5, f"{label}mean")
    return got


def test_library_is_loaded_and_device_is_a_b200_class_gpu():
    lib = _lib.load()
    sm, mp = np.zeros(1, np.int32), np.zeros(1, np.int32)
    import ctypes
    a, c = ctypes.c_int(), ctypes.c_int()
    with torch.cuda.device(0):
        _lib.check(lib.b200norm_query(ctypes.byref(a), ctypes.byref(c)))
    assert a.value == torch.cuda.get_device_properties(0).multi_processor_count
    assert c.value >= a.value


@pytest.mark.parametrize("name", GOLDEN)
def test_golden_vectors(name):
    g = load_golden(name)
    rms = g["op"] == "rms"
    got = run_ours(g["x"], g["dy"], g["w"], g["b"], g["eps"], rms=rms, dtype=g["dtype"])
    tol = TOL[g["dtype"]]
    for key in ("y", "dx", "dw", "db"):
        if g[key] is None:
            continue
        assert_parity(got[key], g[key], tol, f"{name}:{key}")
    assert_parity(got["rstd"], g["rstd"], 1e-5, f"{name}:rstd")
    if not rms:
        assert_parity(got["mean"], g["mean"], 1e-5, f"{name}:mean")


DIMS = [1, 3, 8, 33, 100, 128, 256, 1000, 1024, 2048, 3000, 4096, 5120, 8192, 12288, 16384]


@pytest.mark.parametrize("dtype", ["fp32", "fp16", "bf16", "fp64"])
@pytest.mark.parametrize("rms", [False, True])
def test_dim_sweep_vs_oracle(dtype, rms):
    limit = 65536 // {"fp32": 4, "fp16": 2, "bf16": 2, "fp64": 8}[dtype]
    dims = [d for d in DIMS + [24576, 32768] if d <= limit]
    for N in dims:
        M = 37 if N <= 4096 else 11
        x, dy, w, b = make_inputs(M, N, dtype, seed=N, has_b=not rms)
        check_against_oracle(x, dy, w, b, 1e-5, rms=rms, dtype=dtype, label=f"N={N} ")


@pytest.mark.parametrize("rms", [False, True])
def test_longer_row_after_a_shorter_one_on_the_same_kernel(rms):
    """One kernel instantiation serves a range of row lengths, each with its own staging size; a
    shorter row in between must not shrink what a longer row may use (its launch shape is cached)."""
    for N in (5120, 4160, 5120, 16384, 12296, 16384):
        x, dy, w, b = make_inputs(9, N, "bf16", seed=N, has_b=not rms)
        check_against_oracle(x, dy, w, b, 1e-5, rms=rms, dtype="bf16", label=f"N={N} ")


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_every_small_dim(dtype):
    """Every N from 1 to 257 at a few row counts: exercises each packet-count predicate and the
    any-alignment kernels."""
    for N in range(1, 258):
        M = 1 + N % 5
        x, dy, w, b = make_inputs(M, N, dtype, seed=1000 + N)
        check_against_oracle(x, dy, w, b, 1e-5, rms=bool(N % 2), dtype=dtype, label=f"N={N} M={M} ")


@pytest.mark.parametrize("has_w,has_b", [(True, True), (True, False), (False, False), (False, True)])
def test_optional_weight_and_bias(has_w, has_b):
    for dtype, N in (("fp32", 384), ("bf16", 4096), ("fp16", 77)):
        x, dy, w, b = make_inputs(19, N, dtype, has_w=has_w, has_b=has_b)
        check_against_oracle(x, dy, w, b, 1e-6, rms=False, dtype=dtype)
    x, dy, w, _ = make_inputs(19, 512, "bf16", has_w=has_w, has_b=False)
    check_against_oracle(x, dy, w, None, 1e-6, rms=True, dtype="bf16")


@pytest.mark.parametrize("M", [1, 2, 147, 149, 593, 4099])
def test_row_counts_around_the_grid_size(M):
    x, dy, w, b = make_inputs(M, 1024, "bf16", seed=M)
    check_against_oracle(x, dy, w, b, 1e-5, rms=False, dtype="bf16")
    check_against_oracle(x, dy, w, None, 1e-5, rms=True, dtype="bf16")


def test_fp32_parameters_with_16bit_activations():
    for dtype in ("bf16", "fp16"):
        x, dy, _, _ = make_inputs(64, 2048, dtype)
        _, _, w, b = make_inputs(1, 2048, "fp32", seed=5)
        check_against_oracle(x, dy, w, b, 1e-5, rms=False, dtype=dtype, wdtype="fp32")


def test_row_strided_and_non_contiguous_inputs():
    torch.manual_seed(0)
    N = 512
    big = torch.randn(40, 2 * N, device=DEV, dtype=torch.float16)
    x = big[:, :N]                      # row stride 2N, unit column stride: used without a copy
    assert x.stride() == (2 * N, 1)
    dy = torch.randn(40, N, device=DEV, dtype=torch.float16)
    w = torch.randn(N, device=DEV, dtype=torch.float16)
    b = torch.randn(N, device=DEV, dtype=torch.float16)
    y, mean, rstd = Fn._layernorm_fwd(x, w, b, 1e-5)
    yc, meanc, rstdc = Fn._layernorm_fwd(x.contiguous(), w, b, 1e-5)
    assert torch.equal(y, yc) and torch.equal(mean, meanc) and torch.equal(rstd, rstdc)
    dx, dw, db = Fn._layernorm_bwd(x, dy, w, b, mean, rstd, 1e-5)
    dxc, dwc, dbc = Fn._layernorm_bwd(x.contiguous(), dy, w, b, mean, rstd, 1e-5)
    assert torch.equal(dx, dxc) and torch.equal(dw, dwc) and torch.equal(db, dbc)
    # unaligned view (odd element offset) goes through the any-alignment kernels
    flat = torch.randn(40 * N + 1, device=DEV, dtype=torch.float16)
    xu = flat[1:].view(40, N)
    yu, _, _ = Fn._layernorm_fwd(xu, w, b, 1e-5)
    yuc, _, _ = Fn._layernorm_fwd(xu.clone(), w, b, 1e-5)
    torch.testing.assert_close(yu, yuc, rtol=1e-2, atol=1e-2)
    # non-unit last stride is made contiguous, as the reference does (layernorm.py:49-50)
    xt = torch.randn(N, 24, device=DEV, dtype=torch.float16).t()
    y1, _, _ = Fn._layernorm_fwd(xt, w, b, 1e-5)
    y2, _, _ = Fn._layernorm_fwd(xt.contiguous(), w, b, 1e-5)
    assert torch.equal(y1, y2)


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("dtype,N,M", [("bf16", 4097, 2600), ("bf16", 1025, 3000), ("fp16", 2050, 2400), ("fp32", 1027, 2400),
                                       ("fp32", 4101, 1300), ("fp64", 1031, 1300), ("bf16", 12289, 700),
                                       ("bf16", 16391, 400), ("fp32", 16383, 400), ("bf16", 20001, 300),
                                       ("bf16", 513, 3000), ("fp16", 777, 3000), ("fp32", 257, 3000), ("fp32", 1001, 3000),
                                       ("fp64", 129, 1300), ("bf16", 511, 3000)])
def test_rows_of_odd_length_in_contiguous_tensors(dtype, N, M, rms):
    """Contiguous rows of an odd length: x, dy, y and dx start every row at the same offset within a
    16-byte line, which the vector row kernels need; more rows than resident CTAs, so that every CTA
    walks several rows (all with the same alignment, by the grid's size)."""
    x, dy, w, b = make_inputs(M, N, dtype, seed=N, has_b=not rms)
    check_against_oracle(x, dy, w, b, 1e-5, rms=rms, dtype=dtype, label=f"N={N} ")


@pytest.mark.parametrize("has_w,has_b", [(True, False), (False, False), (False, True)])
def test_rows_of_odd_length_optional_parameters_and_fp32_parameters(has_w, has_b):
    x, dy, w, b = make_inputs(900, 4099, "bf16", has_w=has_w, has_b=has_b)
    check_against_oracle(x, dy, w, b, 1e-6, rms=False, dtype="bf16")
    x, dy, w, _ = make_inputs(900, 2051, "fp16", has_w=has_w, has_b=False)
    check_against_oracle(x, dy, w, None, 1e-6, rms=True, dtype="fp16")
    x, dy, _, _ = make_inputs(900, 4099, "bf16")
    _, _, w, b = make_inputs(1, 4099, "fp32", seed=5)
    check_against_oracle(x, dy, w, b, 1e-5, rms=False, dtype="bf16", wdtype="fp32")
    _, _, w, b = make_inputs(1, 4099, "fp64", seed=6)
    check_against_oracle(x, dy, w, None, 1e-5, rms=True, dtype="bf16", wdtype="fp64")


def test_row_shards_with_rows_of_odd_length():
    """dweight / dbias of one launch over 8 shards == those of 8 launches over one shard each, also
    through the vector row kernels (shards of 600 rows start at the same alignment)."""
    M, N, S = 8 * 600, 4097, 8
    x, dy, w, b = make_inputs(M, N, "bf16")
    check_against_oracle(x, dy, w, b, 1e-6, rms=False, dtype="bf16", row_shards=S)
    xt, dyt, wt, bt = (to_torch(a, "bf16", DEV) for a in (x, dy, w, b))
    y, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, 1e-6)
    dx, dw, db, gs = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, 1e-6, row_shards=S, group_sums=True)
    R = M // S
    parts = []
    for s in range(S):
        sl = slice(s * R, (s + 1) * R)
        parts.append(Fn._layernorm_bwd(xt[sl], dyt[sl], wt, bt, mean[sl], rstd[sl], 1e-6, group_sums=True)[3])
    gathered = torch.cat(parts, 0).contiguous()
    assert torch.equal(gathered, gs)
    outs = Fn.finalize_dwdb(gathered, torch.bfloat16)
    assert torch.equal(outs[0], dw) and torch.equal(outs[1], db)


@pytest.mark.parametrize("offset,stride", [(3, 4096 + 16), (1, 4096 + 5), (4, 4096)])
def test_offset_views_through_the_c_abi(offset, stride):
    """Views that start `offset` elements into their buffers (x, y, dy and dx alike, so every row has
    the same alignment in all four) against the same rows in aligned buffers; and the same x with an
    aligned y, whose rows are aligned differently (the kernels that stage whole rows)."""
    M, N = 1500, 4096
    torch.manual_seed(offset)
    lib = _lib.load()

    def view():
        return torch.randn(M * stride + 32, device=DEV).bfloat16()[offset:offset + M * stride].view(M, stride)[:, :N]

    x, dy, y, dx = view(), view(), view(), view()
    w = torch.randn(N, device=DEV).bfloat16()
    b = torch.randn(N, device=DEV).bfloat16()
    mean = torch.empty(M, device=DEV)
    rstd = torch.empty(M, device=DEV)
    code = Fn._code(x, "input")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.b200norm_ln_fwd(x.data_ptr(), stride, w.data_ptr(), b.data_ptr(), y.data_ptr(), stride,
                                   mean.data_ptr(), rstd.data_ptr(), M, N, 1e-5, code, code, stream))
    yc, meanc, rstdc = Fn._layernorm_fwd(x.contiguous(), w, b, 1e-5)
    torch.testing.assert_close(y.float(), yc.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(mean, meanc, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(rstd, rstdc, rtol=1e-5, atol=1e-5)
    ws_bytes = lib.b200norm_bwd_workspace_bytes(M, N, code, 1)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=DEV)
    dw = torch.empty(N, device=DEV, dtype=torch.bfloat16)
    db = torch.empty(N, device=DEV, dtype=torch.bfloat16)
    _lib.check(lib.b200norm_ln_bwd(x.data_ptr(), stride, dy.data_ptr(), stride, w.data_ptr(), meanc.data_ptr(),
                                   rstdc.data_ptr(), dx.data_ptr(), stride, dw.data_ptr(), db.data_ptr(), None, 1,
                                   ws.data_ptr(), ws_bytes, M, N, code, code, stream))
    dxc, dwc, dbc = Fn._layernorm_bwd(x.contiguous(), dy.contiguous(), w, b, meanc, rstdc, 1e-5)
    torch.testing.assert_close(dx.float(), dxc.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dw.float(), dwc.float(), rtol=2e-2, atol=0.3)
    torch.testing.assert_close(db.float(), dbc.float(), rtol=2e-2, atol=0.3)
    # x in the view, y and dx aligned: rows aligned differently in the two
    y2, mean2, rstd2 = Fn._layernorm_fwd(x, w, b, 1e-5)
    torch.testing.assert_close(y2.float(), yc.float(), rtol=1e-2, atol=1e-2)
    dx2, dw2, db2 = Fn._layernorm_bwd(x, dy.contiguous(), w, b, meanc, rstdc, 1e-5)
    torch.testing.assert_close(dx2.float(), dxc.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dw2.float(), dwc.float(), rtol=2e-2, atol=0.3)
    assert lib.b200norm_device_status(0) == 0


def test_batch_shape_is_restored():
    m = LayerNorm(128, eps=1e-6, device=DEV, dtype=torch.float32)
    x = torch.randn(2, 100, 128, device=DEV, requires_grad=True)
    y = m(x)
    assert y.shape == x.shape and y.is_contiguous()
    y.backward(torch.randn_like(y))
    assert x.grad.shape == x.shape and m.weight.grad.shape == (128,) and m.bias.grad.shape == (128,)


def test_run_to_run_bitwise_determinism():
    x, dy, w, b = make_inputs(3000, 4096, "bf16")
    a = run_ours(x, dy, w, b, 1e-6, rms=False, dtype="bf16")
    c = run_ours(x, dy, w, b, 1e-6, rms=False, dtype="bf16")
    for k in a:
        assert np.array_equal(a[k], c[k]), k


@pytest.mark.parametrize("rms", [False, True])
def test_row_shards_equal_separate_launches_bit_for_bit(rms):
    """One launch over 8 row shards == 8 launches over one shard each + finalize: the property
    that makes a row-sharded multi-GPU run reproduce the single-GPU dweight / dbias exactly."""
    M, N, S = 8 * 600, 4096, 8
    x, dy, w, b = make_inputs(M, N, "bf16", has_b=not rms)
    xt, dyt, wt = (to_torch(a, "bf16", DEV) for a in (x, dy, w))
    bt = to_torch(b, "bf16", DEV)
    if rms:
        y, rstd = Fn._rmsnorm_fwd(xt, wt, 1e-6)
        dx, dw, gs = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, 1e-6, row_shards=S, group_sums=True)
        db = None
    else:
        y, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, 1e-6)
        dx, dw, db, gs = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, 1e-6, row_shards=S, group_sums=True)
    parts, dxs = [], []
    R = M // S
    for s in range(S):
        sl = slice(s * R, (s + 1) * R)
        if rms:
            dxi, _, gi = Fn._rmsnorm_bwd(xt[sl], dyt[sl], wt, rstd[sl], 1e-6, group_sums=True)
        else:
            dxi, _, _, gi = Fn._layernorm_bwd(xt[sl], dyt[sl], wt, bt, mean[sl], rstd[sl], 1e-6, group_sums=True)
        parts.append(gi)
        dxs.append(dxi)
    gathered = torch.cat(parts, 0).contiguous()
    assert torch.equal(gathered, gs)
    outs = Fn.finalize_dwdb(gathered, torch.bfloat16)
    assert torch.equal(outs[0], dw)
    if not rms:
        assert torch.equal(outs[1], db)
    assert torch.equal(torch.cat(dxs, 0), dx)


def _emulated_peers(world, depth, S, slots, N):
    """`world` ranks on one GPU: each has its own inbox and counter, all in one address space."""
    inbox_bytes = depth * S * slots * N * 8          # 8-byte {value, tag} entries
    bufs = [torch.zeros(inbox_bytes, dtype=torch.uint8, device=DEV) for _ in range(world)]
    counters = [torch.zeros(32, dtype=torch.int32, device=DEV) for _ in range(world)]
    peers = []
    for r in range(world):
        pr = _lib.Peers()
        pr.world, pr.rank, pr.depth, pr.total_shards, pr.inbox_bytes = world, r, depth, S, inbox_bytes
        for q in range(world):
            pr.inbox[q] = bufs[q].data_ptr()
        pr.counter = counters[r].data_ptr()
        peers.append(pr)
    return peers, (bufs, counters)


@pytest.mark.parametrize("rms", [False, True])
@pytest.mark.parametrize("world", [1, 4])
@pytest.mark.parametrize("fused_finish", [False, True])
def test_fused_push_exchange_emulated_on_one_gpu(rms, world, fused_finish):
    """The column reduce that pushes shard sums into every rank's inbox, with the ranks emulated as
    consecutive launches on one GPU (each 'rank' has its own inbox and counter; an entry is always
    written by an earlier launch before a finish looks at it, so nothing waits).  Every rank's
    finished dweight / dbias must equal the single-launch 8-shard result bit for bit, over several
    exchanges that reuse the inbox slots -- finished by the stand-alone kernel, or (fused_finish) as
    the second phase of the NEXT exchange's push kernel, with a different row length in between."""
    import ctypes
    M, N, S, depth = 8 * 300, 2048, 8, 4
    slots = 1 if rms else 2
    lib = _lib.load()
    peers, keep = _emulated_peers(world, depth, S, slots, N)
    per = M // world
    pending = None      # (seq, N, expected dw, expected db) of the exchange still to be finished
    for seq in range(1, 8):       # more exchanges than inbox slots
        if seq == 4:              # an exchange of another shape in between must not disturb the slots
            N = 1024
        if seq == 6:              # an odd row length: single entries instead of pairs
            N = 1001
        x, dy, w, b = make_inputs(M, N, "bf16", seed=seq, has_b=not rms)
        xt, dyt, wt, bt = (to_torch(a, "bf16", DEV) for a in (x, dy, w, b))
        if rms:
            _, rstd = Fn._rmsnorm_fwd(xt, wt, 1e-6)
            dx1, dw1 = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, 1e-6, row_shards=S)
            db1 = None
        else:
            _, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, 1e-6)
            dx1, dw1, db1 = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, 1e-6, row_shards=S)
        fused = []
        for r in range(world):
            sl = slice(r * per, (r + 1) * per)
            fin = outs = None
            if fused_finish and pending is not None:
                fin, outs = Fn.finish_request(pending[0], slots, pending[1], torch.bfloat16, torch.device(DEV))
            push = (ctypes.byref(peers[r]), seq, ctypes.byref(fin) if fin is not None else None)
            if rms:
                dx, _ = Fn._rmsnorm_bwd(xt[sl], dyt[sl], wt, rstd[sl], 1e-6, row_shards=S // world, need_dw=False,
                                        push=push)
            else:
                dx, _, _ = Fn._layernorm_bwd(xt[sl], dyt[sl], wt, bt, mean[sl], rstd[sl], 1e-6,
                                             row_shards=S // world, need_dw=False, need_db=False, push=push)
            assert torch.equal(dx, dx1[sl])
            fused.append(outs)
        if fused_finish:
            if pending is not None:
                for r in range(world):
                    assert torch.equal(fused[r][0], pending[2]), f"rank {r} seq {pending[0]}: dweight differs"
                    if not rms:
                        assert torch.equal(fused[r][1], pending[3]), f"rank {r} seq {pending[0]}: dbias differs"
            pending = (seq, N, dw1, db1)
            continue
        for r in range(world):
            outs = Fn.finalize_pushed(ctypes.byref(peers[r]), seq, slots, N, torch.bfloat16, torch.device(DEV))
            assert torch.equal(outs[0], dw1), f"rank {r} seq {seq}: dweight differs"
            if not rms:
                assert torch.equal(outs[1], db1), f"rank {r} seq {seq}: dbias differs"
    if pending is not None:     # the last exchange of the fused pipeline is closed by the stand-alone kernel
        for r in range(world):
            outs = Fn.finalize_pushed(ctypes.byref(peers[r]), pending[0], slots, pending[1], torch.bfloat16,
                                      torch.device(DEV))
            assert torch.equal(outs[0], pending[2])
    torch.cuda.synchronize()
    with torch.cuda.device(0):
        assert lib.b200norm_device_status(0) == 0


@pytest.mark.parametrize("device_numbering", [False, True])
def test_push_exchange_finishing_its_own_exchange_on_one_rank(device_numbering):
    """world = 1 through the PushExchange class: every backward finishes the exchange it pushes in the
    same kernel (the CTAs wait for entries other CTAs of the grid write); with device_numbering the
    kernels count the exchanges themselves.  Bit-identical to the plain backward with 8 row shards."""
    from b200norm.parallel import PushExchange
    M, N = 8 * 200, 4096
    px = PushExchange(max_n=N, slots=2, total_shards=8, device=torch.device(DEV), device_numbering=device_numbering)
    for it in range(6):
        x, dy, w, b = make_inputs(M, N, "bf16", seed=40 + it)
        xt, dyt, wt, bt = (to_torch(a, "bf16", DEV) for a in (x, dy, w, b))
        _, mean, rstd = Fn._layernorm_fwd(xt, wt, bt, 1e-6)
        dx1, dw1, db1 = Fn._layernorm_bwd(xt, dyt, wt, bt, mean, rstd, 1e-6, row_shards=8)
        dx, _, (dw, db) = px.backward_layernorm(xt, dyt, wt, bt, mean, rstd, 1e-6,
                                                finish=(PushExchange.SAME, torch.bfloat16))
        assert torch.equal(dx, dx1) and torch.equal(dw, dw1) and torch.equal(db, db1)
        _, rstd = Fn._rmsnorm_fwd(xt, wt, 1e-6)
        dx1, dw1 = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, 1e-6, row_shards=8)
        dx, _, (dw,) = px.backward_rmsnorm(xt, dyt, wt, rstd, 1e-6, finish=(PushExchange.SAME, torch.bfloat16))
        assert torch.equal(dx, dx1) and torch.equal(dw, dw1)
    torch.cuda.synchronize()
    with torch.cuda.device(0):
        assert _lib.load().b200norm_device_status(0) == 0


def test_push_exchange_refuses_more_open_exchanges_than_the_slots_allow():
    """Slot reuse: at depth 4 at most two exchanges may be pushed-but-unfinished when another starts
    (finish s before starting s + depth // 2).  p1 p2 [p3 refused] f1 p3 [p4 refused] f2 p4 -- and
    every finished exchange is still bit-exact at that maximum."""
    from b200norm.parallel import PushExchange
    M, N = 8 * 64, 1024
    px = PushExchange(max_n=N, slots=1, total_shards=8, depth=4, device=torch.device(DEV))
    x, dy, w, _ = make_inputs(M, N, "bf16", seed=3, has_b=False)
    xt, dyt, wt = (to_torch(a, "bf16", DEV) for a in (x, dy, w))
    _, rstd = Fn._rmsnorm_fwd(xt, wt, 1e-6)
    _, dw1 = Fn._rmsnorm_bwd(xt, dyt, wt, rstd, 1e-6, row_shards=8)
    push = lambda: px.backward_rmsnorm(xt, dyt, wt, rstd, 1e-6)[1]
    h1, h2 = push(), push()
    with pytest.raises(RuntimeError, match="too many exchanges in flight"):
        push()
    (dw,) = px.finish(h1, torch.bfloat16)
    assert torch.equal(dw, dw1)
    h3 = push()
    with pytest.raises(RuntimeError, match="too many exchanges in flight"):
        push()
    (dw,) = px.finish(h2, torch.bfloat16)
    assert torch.equal(dw, dw1)
    # a finish that rides in the call itself counts: h3 is open, h4 is pushed while finishing h3
    _, h4, (dw,) = px.backward_rmsnorm(xt, dyt, wt, rstd, 1e-6, finish=(h3, torch.bfloat16))
    assert torch.equal(dw, dw1)
    (dw,) = px.finish(h4, torch.bfloat16)
    assert torch.equal(dw, dw1)
    torch.cuda.synchronize()
    with torch.cuda.device(0):
        assert _lib.load().b200norm_device_status(0) == 0


def test_finish_kernel_gives_up_on_entries_nobody_writes():
    """A bounded wait that runs out: the finish kernel is asked for an exchange that no rank has
    pushed.  It must return (after its 2 s limit), leave the context usable and raise the device
    status word -- the host-visible form of a peer that never arrived."""
    import ctypes
    import time
    N, depth, S = 256, 4, 8
    lib = _lib.load()
    (pr,), keep = _emulated_peers(1, depth, S, 1, N)
    with torch.cuda.device(0):
        assert lib.b200norm_device_status(1) == 0
        t0 = time.time()
        (dw,) = Fn.finalize_pushed(ctypes.byref(pr), 5, 1, N, torch.float32, torch.device(DEV))
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert 1.0 < waited < 10.0
        assert lib.b200norm_device_status(1) == _lib.ERR_TIMEOUT     # read and cleared
        assert lib.b200norm_device_status(0) == 0
        # the context is still usable
        assert torch.all(dw == 0)
        x = torch.randn(8, N, device=DEV)
        y, _ = Fn._rmsnorm_fwd(x, None, 1e-6)
        torch.cuda.synchronize()
        assert torch.isfinite(y).all()


def test_an_overwritten_inbox_slot_makes_the_late_finish_time_out_instead_of_adding_wrong_sums():
    """What the exchange tags buy: a finish of exchange s that comes after exchange s + depth has
    overwritten the slot does not see s's tag any more, waits out its limit and raises the status
    word -- it never adds up the other exchange's numbers as if they were its own."""
    import ctypes
    N, depth, S = 256, 4, 8
    lib = _lib.load()
    (pr,), keep = _emulated_peers(1, depth, S, 1, N)
    x = torch.randn(8 * 16, N, device=DEV)
    w = torch.ones(N, device=DEV)
    _, rstd = Fn._rmsnorm_fwd(x, w, 1e-6)
    with torch.cuda.device(0):
        assert lib.b200norm_device_status(1) == 0
        for seq in (1, 1 + depth):      # the same slot twice, nothing finished in between
            Fn._rmsnorm_bwd(x, torch.randn_like(x), w, rstd, 1e-6, row_shards=S, need_dw=False,
                            push=(ctypes.byref(pr), seq, None))
        Fn.finalize_pushed(ctypes.byref(pr), 1, 1, N, torch.float32, torch.device(DEV))
        torch.cuda.synchronize()
        assert lib.b200norm_device_status(1) == _lib.ERR_TIMEOUT
        (dw,) = Fn.finalize_pushed(ctypes.byref(pr), 1 + depth, 1, N, torch.float32, torch.device(DEV))
        torch.cuda.synchronize()
        assert lib.b200norm_device_status(0) == 0 and torch.isfinite(dw).all()


def test_outputs_do_not_write_out_of_bounds():
    """Canaries either side of y / dx / mean / rstd survive (the row-strided output path)."""
    N, M = 1000, 53
    lib = _lib.load()
    x = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    pad = 64
    ybuf = torch.full((M * N + 2 * pad,), 7.0, device=DEV, dtype=torch.bfloat16)
    sbuf = torch.full((2, M + 2 * pad), 7.0, device=DEV, dtype=torch.float32)
    y = ybuf[pad:pad + M * N]
    _lib.check(lib.b200norm_ln_fwd(x.data_ptr(), N, w.data_ptr(), None, y.data_ptr(), N,
                                   sbuf[0, pad:].data_ptr(), sbuf[1, pad:].data_ptr(), M, N, 1e-5, _lib.BF16,
                                   _lib.BF16, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.all(ybuf[:pad] == 7) and torch.all(ybuf[pad + M * N:] == 7)
    assert torch.all(sbuf[:, :pad] == 7) and torch.all(sbuf[:, pad + M:] == 7)
    ref = torch.nn.functional.layer_norm(x.float(), (N,), w.float(), None, 1e-5)
    assert_parity(to_numpy(y.view(M, N)), to_numpy(ref), 1e-2, "y")


def test_small_workspace_is_rejected():
    lib = _lib.load()
    M, N = 64, 256
    x = torch.randn(M, N, device=DEV)
    stat = torch.ones(M, device=DEV)
    dx = torch.empty_like(x)
    dw = torch.empty(N, device=DEV)
    ws = torch.empty(256, dtype=torch.uint8, device=DEV)
    rc = lib.b200norm_rms_bwd(x.data_ptr(), N, x.data_ptr(), N, None, stat.data_ptr(), dx.data_ptr(), N,
                              dw.data_ptr(), None, 1, ws.data_ptr(), 256, M, N, _lib.F32, _lib.F32, None)
    assert rc == _lib.ERR_ARG and b"workspace" in lib.b200norm_last_error()


def test_device_status_word_is_clean():
    with torch.cuda.device(0):
        assert _lib.load().b200norm_device_status(0) == 0
