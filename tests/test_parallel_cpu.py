"""Host-side logic of the row-sharded path, run as world_size-2 gloo ranks on CPU: shard
bookkeeping, both exchange modes (against a single-process sum), and a rank that never joins
(the others must get an error from the process-group timeout, not hang).  The device call that
finishes the gradients is replaced by a host fake; no GPU is involved."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from b200norm.parallel import GradExchange, local_row_shards, shard_bounds


def fake_finalize(group_sums, w_dtype):
    """Host stand-in for b200norm_finalize_dwdb: left-to-right fp32 add over groups, then cast."""
    acc = group_sums[0].clone()
    for g in range(1, group_sums.shape[0]):
        acc = acc + group_sums[g]
    return tuple(acc[s].to(w_dtype) for s in range(acc.shape[0]))


def shard_sums(shard, slots, N):
    """Deterministic stand-in for the fp32 sums a backward call emits for global row shard `shard`."""
    g = torch.Generator().manual_seed(100 + shard)
    return torch.randn(slots, N, generator=g) * 1000.0


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, slots, N, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=30))
    try:
        ex = GradExchange(mode=mode, finalize=fake_finalize)
        per = local_row_shards(world)
        mine = torch.stack([shard_sums(rank * per + k, slots, N) for k in range(per)]).contiguous()
        handle = ex.start(mine)
        grads = ex.finish(handle, torch.float32)
        out[rank] = [g.clone() for g in grads]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode", ["all_reduce", "all_gather"])
@pytest.mark.parametrize("slots", [1, 2])
def test_exchange_matches_single_process(mode, slots):
    world, N = 2, 257
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, free_port(), mode, slots, N, out), nprocs=world, join=True)
        got = {r: out[r] for r in range(world)}
    all_shards = torch.stack([shard_sums(s, slots, N) for s in range(8)])
    want = fake_finalize(all_shards, torch.float32)
    for r in range(world):
        for s in range(slots):
            if mode == "all_gather":
                # left-to-right over the 8 global shards on every rank: bit-identical to one process
                assert torch.equal(got[r][s], want[s])
            else:
                torch.testing.assert_close(got[r][s], want[s], rtol=1e-6, atol=1e-3)
    for s in range(slots):
        assert torch.equal(got[0][s], got[1][s])  # ranks agree bit for bit in both modes


def test_shard_bookkeeping():
    assert shard_bounds(1048576, 8, 3) == (393216, 524288)
    assert [local_row_shards(w) for w in (1, 2, 4, 8)] == [8, 4, 2, 1]
    with pytest.raises(ValueError):
        shard_bounds(10, 4, 0)
    with pytest.raises(ValueError):
        local_row_shards(3)
    with pytest.raises(ValueError):
        GradExchange(mode="ring")


def test_single_rank_needs_no_process_group():
    ex = GradExchange(mode="all_gather", finalize=fake_finalize)
    gs = torch.stack([shard_sums(s, 2, 33) for s in range(8)]).contiguous()
    dw, db = ex.finish(ex.start(gs), torch.float32)
    want = fake_finalize(gs, torch.float32)
    assert torch.equal(dw, want[0]) and torch.equal(db, want[1])


def _absent_peer_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
    try:
        if rank == 1:
            out[rank] = "left before the exchange"   # host-made failure: this rank never joins
            return
        ex = GradExchange(mode="all_reduce", finalize=fake_finalize)
        try:
            ex.finish(ex.start(shard_sums(0, 2, 64).unsqueeze(0).contiguous()), torch.float32)
            out[rank] = "no error"
        except Exception as e:  # the process-group timeout ends the collective with an error
            out[rank] = f"error: {type(e).__name__}"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_missing_rank_ends_in_an_error_not_a_hang():
    world = 2
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_absent_peer_worker, args=(world, free_port(), out), nprocs=world, join=True)
        assert out[1] == "left before the exchange"
        assert out[0].startswith("error"), out[0]
