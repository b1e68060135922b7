"""Forward + backward for tensors that live in HOST memory.

A caller whose activations sit in pinned host buffers pays for PCIe twice (x, dy in; y, dx out),
and PCIe -- not HBM -- bounds the step.  `HostPipeline` hides as much of that as the bus allows:
rows are cut into chunks and three CUDA streams run a three-stage pipeline over them
(host->device copy | forward + backward kernels | device->host copy), so that uploads, kernels
and downloads of different chunks overlap and the bus is busy in both directions at once.

dweight / dbias are formed per chunk as fp32 shard sums and added left to right at the end
(b200norm_finalize_dwdb), so the result does not depend on timing.

The reference has no host-memory path (its wrappers take CUDA tensors only,
TritonHub/Normalization/layernorm.py:73); this is the data-movement layer a host-resident
caller puts in front of `_layernorm_fwd` / `_layernorm_bwd`.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import functional as Fn


class HostPipeline:
    """Chunked, triple-buffered host<->device pipeline around LayerNorm / RMSNorm fwd + bwd.

    op: "ln" or "rms".  weight / bias: device tensors (bias None for RMSNorm or bias-free
    LayerNorm).  chunk_rows rows are in flight per stage; `buffers` device buffer sets rotate.
    The first chunk's upload and the last chunk's download have nothing to overlap with, so a call
    of C chunks takes about (C + 1) / C of the bare transfer time: with `rows_hint` (the M the
    pipeline will be called with) the default chunk is M / 24 rows, kept between 8 and 64 MiB per
    tensor (smaller chunks would be bound by the host-side launch work per chunk); without it,
    32 MiB.
    """

    def __init__(self, op: str, N: int, dtype: torch.dtype, device, eps: float, weight: Optional[torch.Tensor],
                 bias: Optional[torch.Tensor] = None, chunk_rows: int = 0, buffers: int = 3, rows_hint: int = 0):
        assert op in ("ln", "rms")
        self.op, self.N, self.dtype, self.eps = op, N, dtype, eps
        self.device = torch.device(device)
        self.weight, self.bias = weight, (bias if op == "ln" else None)
        esize = torch.empty((), dtype=dtype).element_size()
        if chunk_rows <= 0:
            row_bytes = N * esize
            chunk_bytes = 32 << 20
            if rows_hint > 0:
                chunk_bytes = min(64 << 20, max(8 << 20, rows_hint * row_bytes // 24))
            chunk_rows = max(256, chunk_bytes // row_bytes)
        self.chunk_rows = chunk_rows
        self.nbuf = buffers
        R = self.chunk_rows
        mk = lambda: torch.empty((R, N), dtype=dtype, device=self.device)
        self.dx_in = [mk() for _ in range(buffers)]   # x chunk
        self.dy_in = [mk() for _ in range(buffers)]   # dy chunk
        self.s_in = torch.cuda.Stream(self.device)
        self.s_comp = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)

    def run(self, hx: torch.Tensor, hdy: torch.Tensor, hy: torch.Tensor, hdx: torch.Tensor
            ) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
        """hx, hdy: (M, N) pinned host inputs; hy, hdx: (M, N) pinned host outputs, filled on
        return (the call synchronises the pipeline's streams).  Returns (dweight, dbias) as
        device tensors in the parameter dtype (None where there is no parameter)."""
        M, N = hx.shape
        assert N == self.N and hdy.shape == hx.shape == hy.shape == hdx.shape
        R, nb = self.chunk_rows, self.nbuf
        chunks = [(r, min(M, r + R)) for r in range(0, M, R)]
        slots = 2 if self.op == "ln" else 1
        want_params = self.weight is not None or self.bias is not None
        gs_all = (torch.empty((len(chunks), slots, N), dtype=torch.float32, device=self.device)
                  if want_params else None)
        ev_in, ev_comp, ev_out = {}, {}, {}
        outs = {}
        cur = torch.cuda.current_stream(self.device)
        for s in (self.s_in, self.s_comp, self.s_out):
            s.wait_stream(cur)
        for c, (r0, r1) in enumerate(chunks):
            b, n = c % nb, r1 - r0
            with torch.cuda.stream(self.s_in):
                if c >= nb:
                    self.s_in.wait_event(ev_comp[c - nb])      # the kernels are done with this buffer set
                self.dx_in[b][:n].copy_(hx[r0:r1], non_blocking=True)
                self.dy_in[b][:n].copy_(hdy[r0:r1], non_blocking=True)
                ev_in[c] = torch.cuda.Event()
                ev_in[c].record(self.s_in)
            with torch.cuda.stream(self.s_comp):
                self.s_comp.wait_event(ev_in[c])
                xc, dyc = self.dx_in[b][:n], self.dy_in[b][:n]
                if self.op == "ln":
                    y, mean, rstd = Fn._layernorm_fwd(xc, self.weight, self.bias, self.eps)
                    res = Fn._layernorm_bwd(xc, dyc, self.weight, self.bias, mean, rstd, self.eps,
                                            group_sums=want_params, need_dw=False, need_db=False)
                else:
                    y, rstd = Fn._rmsnorm_fwd(xc, self.weight, self.eps)
                    res = Fn._rmsnorm_bwd(xc, dyc, self.weight, rstd, self.eps, group_sums=want_params,
                                          need_dw=False)
                dx = res[0]
                if want_params:
                    gs_all[c].copy_(res[-1][0])
                ev_comp[c] = torch.cuda.Event()
                ev_comp[c].record(self.s_comp)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev_comp[c])
                hy[r0:r1].copy_(y, non_blocking=True)
                hdx[r0:r1].copy_(dx, non_blocking=True)
                # y and dx were allocated on the compute stream: tell the allocator they are still in use here
                y.record_stream(self.s_out)
                dx.record_stream(self.s_out)
                ev_out[c] = torch.cuda.Event()
                ev_out[c].record(self.s_out)
        dw = db = None
        with torch.cuda.stream(self.s_comp):
            if want_params:
                wdt = (self.weight if self.weight is not None else self.bias).dtype
                fin = Fn.finalize_dwdb(gs_all, wdt)
                dw = fin[0] if self.weight is not None else None
                db = fin[1] if (slots == 2 and self.bias is not None) else None
        cur.wait_stream(self.s_comp)
        cur.wait_stream(self.s_out)
        cur.synchronize()
        return dw, db
