"""Row-sharded backward on 2 (or more) GPUs against a single-GPU run: with the all_gather
exchange and the same total number of row shards, dweight and dbias must be BIT-identical to the
single-GPU result (the 1048576 x 4096 multi-GPU workload asks for this determinism check); with all_reduce they must
agree to fp32 rounding.  Skipped where fewer than 2 GPUs are visible."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(M, N, dtype, device):
    g = torch.Generator(device=device).manual_seed(7)
    x = torch.randn(M, N, device=device, generator=g).to(dtype)
    dy = torch.randn(M, N, device=device, generator=g).to(dtype)
    w = (1 + 0.1 * torch.randn(N, device=device, generator=g)).to(dtype)
    b = (0.1 * torch.randn(N, device=device, generator=g)).to(dtype)
    return x, dy, w, b


def _worker(rank, world, port, out):
    import sys
    from pathlib import Path
    root = Path(__file__).resolve().parent.parent
    sys.path[:0] = [str(root), str(root / "triton-hub_b200")]
    from b200norm import functional as Fn
    from b200norm.parallel import (GradExchange, PushExchange, shard_bounds, sharded_layernorm_bwd,
                                   sharded_rmsnorm_bwd)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    device = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        M, N, dtype, eps = 8 * 1024, 4096, torch.bfloat16, 1e-6
        x, dy, w, b = _inputs(M, N, dtype, device)          # same seed on every rank: same global tensors
        r0, r1 = shard_bounds(M, world, rank)
        res = {}
        for mode in ("all_gather", "all_reduce"):
            ex = GradExchange(mode=mode)
            y, mean, rstd = Fn._layernorm_fwd(x[r0:r1], w, b, eps)
            dx, h = sharded_layernorm_bwd(x[r0:r1], dy[r0:r1], w, b, mean, rstd, eps, ex)
            dw, db = ex.finish(h, dtype)
            yr, rstd_r = Fn._rmsnorm_fwd(x[r0:r1], w, eps)
            dxr, hr = sharded_rmsnorm_bwd(x[r0:r1], dy[r0:r1], w, rstd_r, eps, ex)
            (dwr,) = ex.finish(hr, dtype)
            torch.cuda.synchronize()
            res[mode] = (dw, db, dwr, dx, dxr)
        # the library's own exchange: column reduce fused with the push over NVLink peer memory
        px = PushExchange(max_n=N, slots=2, total_shards=8, device=device)
        push_res = []
        for it in range(6):   # more exchanges than inbox slots, two in flight at a time
            y, mean, rstd = Fn._layernorm_fwd(x[r0:r1], w, b, eps)
            dx, h = px.backward_layernorm(x[r0:r1], dy[r0:r1], w, b, mean, rstd, eps)
            yr, rstd_r = Fn._rmsnorm_fwd(x[r0:r1], w, eps)
            dxr, hr = px.backward_rmsnorm(x[r0:r1], dy[r0:r1], w, rstd_r, eps)
            dw, db = px.finish(h, dtype)
            (dwr,) = px.finish(hr, dtype)
            push_res.append((dw, db, dwr, dx, dxr))
        torch.cuda.synchronize()
        dist.barrier()
        if rank == 0:
            # the single-GPU run of the whole batch with the same 8 row shards
            y1, mean1, rstd1 = Fn._layernorm_fwd(x, w, b, eps)
            dx1, dw1, db1 = Fn._layernorm_bwd(x, dy, w, b, mean1, rstd1, eps, row_shards=8)
            _, rstd1r = Fn._rmsnorm_fwd(x, w, eps)
            dx1r, dw1r = Fn._rmsnorm_bwd(x, dy, w, rstd1r, eps, row_shards=8)
            torch.cuda.synchronize()
            dw, db, dwr, dx, dxr = res["all_gather"]
            out["gather_bit_exact"] = bool(torch.equal(dw, dw1) and torch.equal(db, db1) and torch.equal(dwr, dw1r))
            out["dx_bit_exact"] = bool(torch.equal(dx, dx1[r0:r1]) and torch.equal(dxr, dx1r[r0:r1]))
            out["push_bit_exact"] = all(
                bool(torch.equal(dw, dw1) and torch.equal(db, db1) and torch.equal(dwr, dw1r) and
                     torch.equal(dx, dx1[r0:r1]) and torch.equal(dxr, dx1r[r0:r1]))
                for dw, db, dwr, dx, dxr in push_res)
            from b200norm import _lib
            out["status"] = _lib.load().b200norm_device_status(0)
            dw, db, dwr, _, _ = res["all_reduce"]
            scale = dw1.float().abs().max().item()
            out["reduce_err"] = max((dw.float() - dw1.float()).abs().max().item(),
                                    (db.float() - db1.float()).abs().max().item(),
                                    (dwr.float() - dw1r.float()).abs().max().item()) / scale
    finally:
        dist.destroy_process_group()


def test_sharded_run_reproduces_single_gpu_gradients():
    world = min(torch.cuda.device_count(), 8)
    if world < 2:
        pytest.skip("needs at least 2 GPUs")
    world = 1 << (world.bit_length() - 1)   # 2, 4 or 8 ranks
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert out["gather_bit_exact"], "all_gather exchange must reproduce the single-GPU dweight/dbias bit for bit"
        assert out["dx_bit_exact"]
        assert out["push_bit_exact"], "fused push exchange must reproduce the single-GPU dweight/dbias bit for bit"
        assert out["status"] == 0
        assert out["reduce_err"] <= 1e-2      # bf16 parameters: one ulp of the largest gradient
