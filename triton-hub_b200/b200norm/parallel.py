"""Row-sharded LayerNorm / RMSNorm across the GPUs of one box.

Rows are independent, so each rank (one process per GPU) runs forward and backward on its own
block of rows with no communication.  Only dweight / dbias are sums over ALL rows: every rank's
backward call emits fp32 per-shard sums (``group_sums``), which are exchanged over
torch.distributed (NCCL over NVLink) on a side stream while the caller goes on launching the
next layer, and are then added and cast to the parameter dtype by ``finalize_dwdb``.

The reference is single-GPU (no torch.distributed anywhere in TritonHub); this module is the
data-parallel layer added on top of its `_layernorm_bwd` / `_rmsnorm_bwd`
(TritonHub/Normalization/layernorm.py:155-209, rmsnorm.py:124-167).

Three exchange paths:
  PushExchange  the library's own: the backward's column-reduce kernel stores its shard sums,
                each tagged with the exchange number, straight into every rank's inbox over NVLink
                peer memory; a later kernel (or the next exchange's) adds them left to right.  No collective-library kernel has to
                be co-resident with the persistent forward / backward grids, and the result is
                bit-identical across ranks, runs and GPU counts.  This is the default.
  GradExchange  over torch.distributed collectives, in one of two modes:
  "all_reduce"  one NCCL sum of the (slots, N) fp32 vector.  Equal to a single-GPU run up to fp32
                rounding: the order of the cross-rank additions is NCCL's.
  "all_gather"  every rank receives all shard sums and adds them left to right in global shard
                order.  Bit-identical on every rank, for every run, and to a single-GPU run that
                used the same total number of row shards.
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

from . import _lib
from . import functional as Fn

TOTAL_SHARDS = 8  # a box has 8 GPUs; 1, 2, 4 or 8 ranks each own 8 / world consecutive shards


def shard_bounds(rows: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous block of rows owned by `rank`: [begin, end).  Rows must divide evenly."""
    if rows % world != 0:
        raise ValueError(f"{rows} rows do not divide over {world} ranks")
    per = rows // world
    return rank * per, (rank + 1) * per


def local_row_shards(world: int, total_shards: int = TOTAL_SHARDS) -> int:
    """Row shards each rank keeps apart so that all ranks together hold `total_shards`."""
    if total_shards % world != 0:
        raise ValueError(f"world size {world} does not divide {total_shards} row shards")
    return total_shards // world


class GradExchange:
    """Cross-rank sum of the fp32 dweight / dbias shard sums of one backward call.

    start(group_sums) enqueues the collective behind the work already on the current stream and
    returns at once; finish(handle, dtype) makes the current stream wait for it and returns the
    finished (dweight[, dbias]) in `dtype`.  Between the two the caller is free to launch more
    kernels: they overlap the exchange.
    """

    def __init__(self, group: Optional[dist.ProcessGroup] = None, mode: str = "all_reduce",
                 finalize: Callable[[torch.Tensor, torch.dtype], Sequence[torch.Tensor]] = Fn.finalize_dwdb):
        if mode not in ("all_reduce", "all_gather"):
            raise ValueError(f"unknown exchange mode {mode!r}")
        self.group, self.mode, self.finalize = group, mode, finalize
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self._side = None

    def _side_stream(self, device):
        if self._side is None:
            self._side = torch.cuda.Stream(device=device)
        return self._side

    def start(self, group_sums: torch.Tensor):
        """group_sums: (local_shards, slots, N) fp32, contiguous.  Returns an opaque handle."""
        assert group_sums.dtype == torch.float32 and group_sums.dim() == 3 and group_sums.is_contiguous()
        if self.world == 1:
            return (None, group_sums)
        if self.mode == "all_reduce":
            # collapse this rank's shards first (left to right), then sum across ranks
            local = group_sums if group_sums.shape[0] == 1 else None
            buf = local if local is not None else torch.stack(self._fold(group_sums)).unsqueeze(0).contiguous()
        else:
            buf = torch.empty((self.world * group_sums.shape[0],) + tuple(group_sums.shape[1:]),
                              dtype=torch.float32, device=group_sums.device)
        if group_sums.is_cuda:
            side = self._side_stream(group_sums.device)
            side.wait_stream(torch.cuda.current_stream(group_sums.device))
            with torch.cuda.stream(side):
                work = self._collective(buf, group_sums)
            # the buffers are used on the side stream: keep the allocator from recycling them early
            buf.record_stream(side)
            group_sums.record_stream(side)
        else:
            work = self._collective(buf, group_sums)
        return (work, buf)

    def _fold(self, group_sums):
        """Left-to-right fp32 sum over this rank's shards, per slot (host-side glue for all_reduce)."""
        acc = group_sums[0].clone()
        for g in range(1, group_sums.shape[0]):
            acc += group_sums[g]
        return [acc[s] for s in range(acc.shape[0])]

    def _collective(self, buf, group_sums):
        if self.mode == "all_reduce":
            return dist.all_reduce(buf, op=dist.ReduceOp.SUM, group=self.group, async_op=True)
        return dist.all_gather_into_tensor(buf, group_sums, group=self.group, async_op=True)

    def finish(self, handle, w_dtype: torch.dtype):
        """Wait for the exchange started by `start` and return the finished gradients."""
        work, buf = handle
        if work is not None:
            work.wait()  # CUDA: a stream-side wait, the host does not block
        return tuple(self.finalize(buf, w_dtype))


def sharded_layernorm_bwd(x, dout, weight, bias, mean, rstd, eps, exchange: GradExchange):
    """Backward of one rank's rows: returns (dx, handle); `exchange.finish(handle, weight.dtype)`
    later yields the global (dweight, dbias)."""
    shards = local_row_shards(exchange.world) if exchange.mode == "all_gather" else 1
    dx, _, _, gs = Fn._layernorm_bwd(x, dout, weight, bias, mean, rstd, eps, row_shards=shards, group_sums=True,
                                     need_dw=False, need_db=False)
    return dx, exchange.start(gs)


def sharded_rmsnorm_bwd(x, dout, weight, rstd, eps, exchange: GradExchange):
    """RMSNorm twin of `sharded_layernorm_bwd`; `finish` yields (dweight,)."""
    shards = local_row_shards(exchange.world) if exchange.mode == "all_gather" else 1
    dx, _, gs = Fn._rmsnorm_bwd(x, dout, weight, rstd, eps, row_shards=shards, group_sums=True, need_dw=False)
    return dx, exchange.start(gs)


class PushExchange:
    """dweight / dbias exchange fused into the backward's column reduce (b200norm_*_bwd_push).

    Each rank owns an inbox (depth, total_shards, slots, max_n) of 8-byte {fp32 value, exchange tag}
    entries in symmetric memory (torch.distributed._symmetric_memory: CUDA VMM allocations mapped into
    every rank of the group).  `backward_*` launches the backward whose column reduce stores this
    rank's shard sums into all ranks' inboxes; finishing an exchange waits (on the GPU, bounded) for
    everyone's entries and adds the shards left to right.  Nothing blocks the host.

    An exchange is finished either by `finish(handle, dtype)` -- a kernel of its own -- or inside a
    later `backward_*(..., finish=(handle, dtype))` call, whose push kernel does it as a second phase:
    the usual pipeline finishes exchange s - 1 in exchange s, so a step costs no launch more than on
    one GPU.  `finish=(SAME, dtype)` finishes the exchange being pushed in its own kernel.

    Slot reuse: exchange s + depth overwrites the inbox slot of exchange s on every peer, so a rank
    may start it only once every peer has finished s.  All a rank learns from its own finish of
    exchange k is that every peer has PUSHED k -- hence, by the peer's stream order, that the peer
    has finished whatever it had to finish before pushing k.  With the rule "finish s before starting
    s + W" on every rank, starting s + depth implies own finish of s + depth - W, implies the peers
    pushed s + depth - W, implies they finished s + depth - 2W: safe exactly when W <= depth / 2.  So
    at most depth // 2 exchanges may be open (pushed, not finished) when another starts; `_next`
    enforces it, counting an exchange whose finish rides in the very call as finished.  (A rank that
    broke the rule would make a slower peer's wait run out, not hand it wrong sums: the tags differ.)
    With device_numbering the caller keeps the same rule.
    """

    SAME = "same"  # finish=(PushExchange.SAME, dtype): finish the exchange this call pushes

    def __init__(self, max_n: int, slots: int = 2, group: Optional[dist.ProcessGroup] = None,
                 total_shards: Optional[int] = None, depth: int = 4, device: Optional[torch.device] = None,
                 device_numbering: bool = False):
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        if self.world > _lib.MAX_PEERS:
            raise ValueError(f"at most {_lib.MAX_PEERS} ranks (one box)")
        # total_shards = world (default): one shard per rank, the fastest launch shape; results are
        # identical on all ranks and from run to run.  total_shards = 8: additionally identical to
        # a run on any other GPU count (and to one GPU using row_shards=8), at the cost of 8 / world
        # times as many, shorter-lived CTAs in the backward.
        total_shards = self.world if total_shards is None else total_shards
        self.local_shards = local_row_shards(self.world, total_shards)
        self.total_shards, self.depth, self.slots, self.max_n = total_shards, depth, slots, max_n
        self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
        self.inbox_bytes = depth * ((total_shards * slots * max_n * 8 + 15) // 16 * 16)
        # device_numbering: the kernels count the exchanges themselves (seq = 0 in the ABI), so that a
        # CUDA graph holding backward_* / finish calls can be replayed; the caller then keeps the
        # "at most depth // 2 open exchanges" rule itself.
        self.device_numbering = device_numbering
        self._seq = 0
        self._oldest_open = 1
        self.counter = torch.zeros(32, dtype=torch.int32, device=self.device)  # 128 bytes of bookkeeping
        if self.world == 1:
            self._buf = torch.zeros(self.inbox_bytes, dtype=torch.uint8, device=self.device)
            bases = [self._buf.data_ptr()]
        else:
            import torch.distributed._symmetric_memory as symm_mem
            self._buf = symm_mem.empty(self.inbox_bytes, dtype=torch.uint8, device=self.device)
            self._buf.zero_()
            self._hdl = symm_mem.rendezvous(self._buf, self.group)
            bases = [int(p) for p in self._hdl.buffer_ptrs]
            torch.cuda.synchronize(self.device)
            dist.barrier(group=self.group)  # every inbox is zero before anyone pushes
        self.peers = _lib.Peers()
        self.peers.world, self.peers.rank = self.world, self.rank
        self.peers.depth, self.peers.total_shards = depth, total_shards
        self.peers.inbox_bytes = self.inbox_bytes
        for r in range(self.world):
            self.peers.inbox[r] = bases[r]
        self.peers.counter = self.counter.data_ptr()

    def _next(self, slots, N, finishing=None):
        """Number of the exchange about to be pushed.  `finishing`: the exchange the same call finishes."""
        if N > self.max_n or slots > self.slots:
            raise ValueError(f"exchange of {slots} x {N} exceeds this PushExchange ({self.slots} x {self.max_n})")
        if self.device_numbering:
            return 0
        oldest = self._oldest_open
        if finishing is not None and finishing == oldest:
            oldest += 1
        if self._seq + 1 - oldest >= self.depth // 2:
            raise RuntimeError(f"too many exchanges in flight (at most {self.depth // 2} open at depth "
                               f"{self.depth}): finish the oldest one first")
        self._seq += 1
        return self._seq

    def _finish_arg(self, finish, slots, N):
        """-> (exchange number being finished or None, Finish struct or None, outs, (slots, N) of it)."""
        if finish is None:
            return None, None, None
        handle, w_dtype = finish
        if isinstance(handle, str) and handle == self.SAME:
            fseq, fslots, fn = (0 if self.device_numbering else self._seq + 1), slots, N
        else:
            fseq, fslots, fn = handle
        fin, outs = Fn.finish_request(fseq, fslots, fn, w_dtype, self.device)
        return fseq, fin, outs

    def _done(self, fseq):
        if fseq:
            self._oldest_open = max(self._oldest_open, fseq + 1)

    def backward_layernorm(self, x, dout, weight, bias, mean, rstd, eps, finish=None):
        """This rank's rows: returns (dx, handle); finish(handle, dtype) yields (dweight, dbias).
        With finish=(older handle | SAME, dtype) the call also finishes that exchange and returns
        (dx, handle, grads of the finished exchange)."""
        N = x.shape[-1]
        fseq, fin, outs = self._finish_arg(finish, 2, N)
        same = finish is not None and isinstance(finish[0], str)
        seq = self._next(2, N, None if same else fseq)
        dx, _, _ = Fn._layernorm_bwd(x, dout, weight, bias, mean, rstd, eps, row_shards=self.local_shards,
                                     need_dw=False, need_db=False,
                                     push=(ctypes_ref(self.peers), seq, ctypes_ref(fin) if fin is not None else None))
        self._done(seq if same else fseq)
        return (dx, (seq, 2, N)) if finish is None else (dx, (seq, 2, N), outs)

    def backward_rmsnorm(self, x, dout, weight, rstd, eps, finish=None):
        """RMSNorm twin; a finished RMSNorm exchange yields (dweight,)."""
        N = x.shape[-1]
        fseq, fin, outs = self._finish_arg(finish, 1, N)
        same = finish is not None and isinstance(finish[0], str)
        seq = self._next(1, N, None if same else fseq)
        dx, _ = Fn._rmsnorm_bwd(x, dout, weight, rstd, eps, row_shards=self.local_shards, need_dw=False,
                                push=(ctypes_ref(self.peers), seq, ctypes_ref(fin) if fin is not None else None))
        self._done(seq if same else fseq)
        return (dx, (seq, 1, N)) if finish is None else (dx, (seq, 1, N), outs)

    def finish(self, handle, w_dtype: torch.dtype):
        seq, slots, N = handle
        out = Fn.finalize_pushed(ctypes_ref(self.peers), seq, slots, N, w_dtype, self.device)
        self._done(seq)
        return out


def ctypes_ref(struct):
    """Pointer argument for a ctypes Structure (the b200norm_peers* of the C ABI)."""
    return ctypes.byref(struct)
