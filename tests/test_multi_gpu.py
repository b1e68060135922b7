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
        # The library's own exchange: column reduce fused with the push over NVLink peer memory.
        # Four ways of driving it, each over more exchanges than the inbox has slots:
        #   "apart"   finishes as kernels of their own, the maximum number of exchanges open (depth // 2)
        #   "next"    each push kernel finishes the previous exchange (the pipeline the benchmark times)
        #   "same"    each push kernel finishes its own exchange (waits for every peer's push)
        #   "counted" as "next" with the exchanges numbered on the device (graph-replayable form)
        xs, dys = x[r0:r1], dy[r0:r1]
        push_res = {}
        for how in ("apart", "next", "same", "counted"):
            px = PushExchange(max_n=N, slots=2, total_shards=8, device=device, device_numbering=(how == "counted"))
            got = []
            prev_ln = prev_rms = None
            for it in range(6):
                y, mean, rstd = Fn._layernorm_fwd(xs, w, b, eps)
                yr, rstd_r = Fn._rmsnorm_fwd(xs, w, eps)
                if how == "apart":
                    dx, h = px.backward_layernorm(xs, dys, w, b, mean, rstd, eps)
                    dxr, hr = px.backward_rmsnorm(xs, dys, w, rstd_r, eps)
                    dw, db = px.finish(h, dtype)
                    (dwr,) = px.finish(hr, dtype)
                    got.append((dw, db, dwr, dx, dxr))
                elif how == "same":
                    dx, _, (dw, db) = px.backward_layernorm(xs, dys, w, b, mean, rstd, eps,
                                                            finish=(PushExchange.SAME, dtype))
                    dxr, _, (dwr,) = px.backward_rmsnorm(xs, dys, w, rstd_r, eps, finish=(PushExchange.SAME, dtype))
                    got.append((dw, db, dwr, dx, dxr))
                else:
                    # LayerNorm exchange k is finished by the RMSNorm push that follows it, and that RMSNorm
                    # exchange by the next iteration's LayerNorm push: one open exchange at a time.
                    if prev_rms is None:
                        dx, h = px.backward_layernorm(xs, dys, w, b, mean, rstd, eps)
                    else:
                        dx, h, (dwr_prev,) = px.backward_layernorm(xs, dys, w, b, mean, rstd, eps,
                                                                   finish=(prev_rms, dtype))
                        got[-1] = got[-1][:2] + (dwr_prev,) + got[-1][3:]
                    dxr, hr, (dw, db) = px.backward_rmsnorm(xs, dys, w, rstd_r, eps, finish=(h, dtype))
                    got.append((dw, db, None, dx, dxr))
                    prev_rms = hr
            if how in ("next", "counted"):
                (dwr_last,) = px.finish(prev_rms, dtype)
                got[-1] = got[-1][:2] + (dwr_last,) + got[-1][3:]
            push_res[how] = got
        torch.cuda.synchronize()
        dist.barrier()
        # Every rank holds the whole batch (same seed), so every rank checks its own results against its own
        # single-GPU run of the whole batch with the same 8 row shards; the verdicts are combined over ranks.
        y1, mean1, rstd1 = Fn._layernorm_fwd(x, w, b, eps)
        dx1, dw1, db1 = Fn._layernorm_bwd(x, dy, w, b, mean1, rstd1, eps, row_shards=8)
        _, rstd1r = Fn._rmsnorm_fwd(x, w, eps)
        dx1r, dw1r = Fn._rmsnorm_bwd(x, dy, w, rstd1r, eps, row_shards=8)
        torch.cuda.synchronize()
        verdict = {}
        dw, db, dwr, dx, dxr = res["all_gather"]
        verdict["gather_bit_exact"] = bool(torch.equal(dw, dw1) and torch.equal(db, db1) and torch.equal(dwr, dw1r))
        verdict["dx_bit_exact"] = bool(torch.equal(dx, dx1[r0:r1]) and torch.equal(dxr, dx1r[r0:r1]))
        for how, got in push_res.items():
            verdict["push_bit_exact_" + how] = all(
                bool(torch.equal(dw, dw1) and torch.equal(db, db1) and torch.equal(dwr, dw1r) and
                     torch.equal(dx, dx1[r0:r1]) and torch.equal(dxr, dx1r[r0:r1]))
                for dw, db, dwr, dx, dxr in got)
        from b200norm import _lib
        verdict["status_clean"] = _lib.load().b200norm_device_status(0) == 0
        dw, db, dwr, _, _ = res["all_reduce"]
        scale = dw1.float().abs().max().item()
        err = max((dw.float() - dw1.float()).abs().max().item(), (db.float() - db1.float()).abs().max().item(),
                  (dwr.float() - dw1r.float()).abs().max().item()) / scale
        keys = sorted(verdict)
        flags = torch.tensor([float(verdict[k]) for k in keys] + [-err], device=device, dtype=torch.float64)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)       # a check holds only if it holds on every rank
        if rank == 0:
            for k, v in zip(keys, flags[:-1].tolist()):
                out[k] = bool(v)
            out["reduce_err"] = -flags[-1].item()
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
        for how in ("apart", "next", "same", "counted"):
            assert out["push_bit_exact_" + how], \
                f"fused push exchange ({how}) must reproduce the single-GPU dweight/dbias bit for bit"
        assert out["status_clean"], "a bounded wait ran out on some rank"
        assert out["reduce_err"] <= 1e-2      # bf16 parameters: one ulp of the largest gradient
