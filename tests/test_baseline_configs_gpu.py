"""The benchmark configurations (c1 ... c5) at their full sizes, through the module API.

The CPU oracle cannot finish these in seconds, so each is checked three ways:
  1. every row, against a chunked torch reference on the GPU evaluated in fp32 from the same
     storage-rounded inputs (a floating-point kernel, so a torch fp32 reference is kept),
     dweight / dbias accumulated across chunks in fp64;
  2. a spread sample of rows against the CPU oracle (fp64 truth), y and dx;
  3. size-independent properties: a second run is bit-identical; the per-shard sums of an
     8-shard backward add up (left to right) to exactly the dweight / dbias it returns.
Bars: 1e-5 (fp32) / 1e-2 (fp16, bf16) relative to each tensor's largest magnitude.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from b200norm import LayerNorm, RMSNorm
from b200norm import functional as Fn
from helpers import TOL, assert_parity, to_numpy
from oracle import oracle as O

DEV = "cuda:0"
T = {"fp32": torch.float32, "fp16": torch.float16, "bf16": torch.bfloat16}

CONFIGS = {
    # name: op, dtype, batch shape, N, eps, x mean, x std
    "c1": ("ln", "fp32", (2, 100), 128, 1e-6, 0.0, 1.0),
    "c2": ("rms", "bf16", (8, 4096), 4096, 1e-6, 0.0, 1.0),
    "c3": ("ln", "fp16", (65536,), 5120, 1e-5, 3.0, 2.0),
    "c4": ("ln", "bf16", (32768,), 16384, 1e-6, 0.0, 1.0),
    "c5_ln": ("ln", "bf16", (1048576,), 4096, 1e-6, 0.0, 1.0),
    "c5_rms": ("rms", "bf16", (1048576,), 4096, 1e-6, 0.0, 1.0),
}


def draw(shape, N, dtype, mu, sigma, seed):
    g = torch.Generator(device=DEV).manual_seed(seed)
    M = int(np.prod(shape))
    out = torch.empty((M, N), device=DEV, dtype=dtype)
    step = max(1, (1 << 26) // N)
    for r in range(0, M, step):
        e = min(M, r + step)
        out[r:e] = (torch.randn((e - r, N), device=DEV, generator=g) * sigma + mu).to(dtype)
    return out.view(*shape, N)


@pytest.mark.parametrize("name", list(CONFIGS))
def test_full_size_config(name):
    op, dt, shape, N, eps, mu, sigma = CONFIGS[name]
    M = int(np.prod(shape))
    need = 4 * M * N * torch.finfo(T[dt]).bits // 8
    if torch.cuda.get_device_properties(0).total_memory < need * 1.5:
        pytest.skip("not enough device memory for this configuration")
    dtype, tol, rms = T[dt], TOL[dt], op == "rms"
    x = draw(shape, N, dtype, mu, sigma, 0).requires_grad_(True)
    dy = draw(shape, N, dtype, 0.0, 1.0, 1)
    g = torch.Generator(device=DEV).manual_seed(2)
    w = (1 + 0.1 * torch.randn(N, device=DEV, generator=g)).to(dtype)
    b = (0.1 * torch.randn(N, device=DEV, generator=g)).to(dtype)
    mod = (RMSNorm(N, eps=eps, device=DEV, dtype=dtype) if rms
           else LayerNorm(N, eps=eps, elementwise_affine=True, bias=True, device=DEV, dtype=dtype))
    with torch.no_grad():
        mod.weight.copy_(w)
        if not rms:
            mod.bias.copy_(b)

    y = mod(x)
    y.backward(dy)
    torch.cuda.synchronize()
    assert y.shape == x.shape and x.grad.shape == x.shape
    y2, dx2 = y.detach().view(M, N), x.grad.view(M, N)
    x2, dy2 = x.detach().view(M, N), dy.view(M, N)

    # 1. every row against torch in fp32, chunk by chunk
    wf, bf = w.float(), b.float()
    dw_ref = torch.zeros(N, device=DEV, dtype=torch.float64)
    db_ref = torch.zeros(N, device=DEV, dtype=torch.float64)
    worst = {"y": 0.0, "dx": 0.0}
    scale = {"y": 0.0, "dx": 0.0}
    chunk = max(1, (1 << 25) // N)
    for r in range(0, M, chunk):
        e = min(M, r + chunk)
        xc = x2[r:e].float().requires_grad_(True)
        wc = wf.clone().requires_grad_(True)
        bc = bf.clone().requires_grad_(True)
        yc = F.rms_norm(xc, (N,), wc, eps) if rms else F.layer_norm(xc, (N,), wc, bc, eps)
        yc.backward(dy2[r:e].float())
        for key, got, ref in (("y", y2[r:e], yc.detach()), ("dx", dx2[r:e], xc.grad)):
            ref_r = ref.to(dtype).float()
            worst[key] = max(worst[key], (got.float() - ref_r).abs().max().item())
            scale[key] = max(scale[key], ref_r.abs().max().item())
        dw_ref += wc.grad.double()
        if not rms:
            db_ref += bc.grad.double()
        del xc, yc
    for key in ("y", "dx"):
        assert worst[key] <= tol * scale[key], f"{name} {key}: {worst[key]:.3e} > {tol:.0e} * {scale[key]:.3e}"
    assert_parity(to_numpy(mod.weight.grad), to_numpy(dw_ref.to(dtype)), tol, f"{name} dweight")
    if not rms:
        assert_parity(to_numpy(mod.bias.grad), to_numpy(db_ref.to(dtype)), tol, f"{name} dbias")

    # 2. a spread sample of rows against the CPU oracle (fp64 truth)
    idx = torch.linspace(0, M - 1, 48, device=DEV).long().unique()
    xs, dys = to_numpy(x2[idx]), to_numpy(dy2[idx])
    wn, bn = to_numpy(w), (None if rms else to_numpy(b))
    yo, mean, rstd = O.norm_fwd(xs, wn, bn, eps, rms=rms, acc64=True)
    dxo, _, _ = O.norm_bwd(xs, dys, wn, mean, rstd, rms=rms, programs=1, acc64=True)
    assert_parity(to_numpy(y2[idx]), O.round_to(yo, dt), tol, f"{name} sampled y vs oracle")
    assert_parity(to_numpy(dx2[idx]), O.round_to(dxo, dt), tol, f"{name} sampled dx vs oracle")

    # 3. properties that do not depend on the size
    first = (y.detach().clone(), x.grad.clone(), mod.weight.grad.clone())
    x.grad = None
    mod.weight.grad = None
    if not rms:
        mod.bias.grad = None
    y_b = mod(x)
    y_b.backward(dy)
    torch.cuda.synchronize()
    assert torch.equal(y_b, first[0]) and torch.equal(x.grad, first[1]) and torch.equal(mod.weight.grad, first[2])
    del first, y_b
    if M % 8 == 0:
        if rms:
            _, rstd_t = Fn._rmsnorm_fwd(x2, w, eps)
            _, dw8, gs = Fn._rmsnorm_bwd(x2, dy2, w, rstd_t, eps, row_shards=8, group_sums=True)
            outs = (dw8,)
        else:
            _, mean_t, rstd_t = Fn._layernorm_fwd(x2, w, b, eps)
            _, dw8, db8, gs = Fn._layernorm_bwd(x2, dy2, w, b, mean_t, rstd_t, eps, row_shards=8, group_sums=True)
            outs = (dw8, db8)
        acc = gs[0].clone()
        for s in range(1, 8):
            acc += gs[s]
        for k, o in enumerate(outs):
            assert torch.equal(acc[k].to(dtype), o), f"{name}: shard sums do not add up to output {k}"
            ref = dw_ref if k == 0 else db_ref
            assert_parity(to_numpy(o), to_numpy(ref.to(dtype)), tol, f"{name} 8-shard output {k}")
