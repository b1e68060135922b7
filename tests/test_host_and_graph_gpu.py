"""The two ways callers drive the kernels besides plain eager calls: the host-buffer pipeline
(pinned host tensors in, pinned host tensors out, chunked over three streams) and CUDA-graph
capture of the wrappers.  Both must reproduce the plain device-resident calls bit for bit."""
import pytest
import torch

pytestmark = pytest.mark.gpu

from b200norm import HostPipeline
from b200norm import functional as Fn

DEV = torch.device("cuda", 0)


@pytest.mark.parametrize("op", ["ln", "rms"])
@pytest.mark.parametrize("M,chunk", [(4096, 1000), (777, 256), (64, 0)])
def test_host_pipeline_matches_device_path(op, M, chunk):
    N, dt, eps = 2048, torch.bfloat16, 1e-6
    g = torch.Generator(device=DEV).manual_seed(3)
    x = torch.randn(M, N, device=DEV, generator=g).to(dt)
    dy = torch.randn(M, N, device=DEV, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(N, device=DEV, generator=g)).to(dt)
    b = (0.1 * torch.randn(N, device=DEV, generator=g)).to(dt) if op == "ln" else None
    hx, hdy = x.cpu().pin_memory(), dy.cpu().pin_memory()
    hy, hdx = torch.empty_like(hx).pin_memory(), torch.empty_like(hx).pin_memory()
    pipe = HostPipeline(op, N, dt, DEV, eps, w, b, chunk_rows=chunk)
    for _ in range(2):          # buffers are reused across runs
        dw, db = pipe.run(hx, hdy, hy, hdx)
    if op == "ln":
        y, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
        dx, _, _ = Fn._layernorm_bwd(x, dy, w, b, mean, rstd, eps)
    else:
        y, rstd = Fn._rmsnorm_fwd(x, w, eps)
        dx, _ = Fn._rmsnorm_bwd(x, dy, w, rstd, eps)
    torch.cuda.synchronize()
    assert torch.equal(hy, y.cpu()) and torch.equal(hdx, dx.cpu())
    # dweight / dbias: per-chunk fp32 sums added left to right -- same tolerance as everywhere (bf16: 1e-2)
    chunks = pipe.chunk_rows
    ref_dw = torch.zeros(N, device=DEV)
    ref_db = torch.zeros(N, device=DEV)
    xh = (x.float() * rstd[:, None]) if op == "rms" else ((x.float() - mean[:, None]) * rstd[:, None])
    ref_dw = (dy.float() * xh).sum(0)
    ref_db = dy.float().sum(0)
    assert (dw.float() - ref_dw).abs().max() <= 1e-2 * ref_dw.abs().max()
    if op == "ln":
        assert (db.float() - ref_db).abs().max() <= 1e-2 * ref_db.abs().max()
    else:
        assert db is None


@pytest.mark.parametrize("op", ["ln", "rms"])
def test_wrappers_can_be_captured_in_a_cuda_graph(op):
    M, N, dt, eps = 1024, 4096, torch.bfloat16, 1e-6
    g = torch.Generator(device=DEV).manual_seed(4)
    x = torch.randn(M, N, device=DEV, generator=g).to(dt)
    dy = torch.randn(M, N, device=DEV, generator=g).to(dt)
    w = (1 + 0.1 * torch.randn(N, device=DEV, generator=g)).to(dt)
    b = (0.1 * torch.randn(N, device=DEV, generator=g)).to(dt)

    def step():
        if op == "ln":
            y, mean, rstd = Fn._layernorm_fwd(x, w, b, eps)
            return (y,) + Fn._layernorm_bwd(x, dy, w, b, mean, rstd, eps)
        y, rstd = Fn._rmsnorm_fwd(x, w, eps)
        return (y,) + Fn._rmsnorm_bwd(x, dy, w, rstd, eps)

    eager = [t.clone() for t in step()]      # also the first call on the device: set-up happens before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        captured = step()
    x.copy_(torch.randn(M, N, device=DEV, generator=g).to(dt))     # new data in the same buffers
    graph.replay()
    torch.cuda.synchronize()
    fresh = step()
    torch.cuda.synchronize()
    for a, c in zip(captured, fresh):
        assert torch.equal(a, c)
    assert not torch.equal(captured[0], eager[0])
