"""Per-tensor dynamic FP8 cast for callers whose tensors live in HOST memory.

The cast itself runs at HBM speed; with host buffers the PCIe copies dominate.
``HostCastPipeline`` keeps ``depth`` device buffer pairs and three streams so that the
host->device copy of call i+1, the kernels of call i and the device->host copy of call
i-1 overlap (PCIe is full duplex).  Results are bit-identical to the synchronous path.
"""

from __future__ import annotations

import torch

from .sharded import sharded_dynamic_scaled_quant


class HostCastPipeline:
    def __init__(self, shape, dtype=torch.bfloat16, fp8_dtype=torch.float8_e4m3fn, device=None, exchange=None,
                 group=None, depth: int = 3):
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.fp8_dtype = fp8_dtype
        self.exchange = exchange
        self.group = group
        self.depth = depth
        self.dev_in = [torch.empty(shape, dtype=dtype, device=self.device) for _ in range(depth)]
        self.dev_out = [torch.empty(shape, dtype=fp8_dtype, device=self.device) for _ in range(depth)]
        self.s_h2d = torch.cuda.Stream(self.device)
        self.s_cmp = torch.cuda.Stream(self.device)
        self.s_d2h = torch.cuda.Stream(self.device)
        self.h2d_done = [torch.cuda.Event() for _ in range(depth)]
        self.cmp_done = [torch.cuda.Event() for _ in range(depth)]
        self.d2h_done = [torch.cuda.Event() for _ in range(depth)]
        self.calls = 0
        self.amax = None

    def submit(self, host_in: torch.Tensor, host_out: torch.Tensor) -> None:
        """Enqueue one cast: ``host_in`` (pinned, the pipeline's shape and dtype) ->
        ``host_out`` (pinned, same shape, fp8 or uint8).  Returns immediately; the result
        is in ``host_out`` after :meth:`synchronize` (or once ``depth`` later calls have
        been submitted and the matching event has completed)."""
        if not (host_in.is_pinned() and host_out.is_pinned()):
            raise ValueError("host buffers must be pinned")
        b = self.calls % self.depth
        reuse = self.calls >= self.depth
        with torch.cuda.stream(self.s_h2d):
            if reuse:
                self.s_h2d.wait_event(self.cmp_done[b])  # the kernels that read dev_in[b] are done
            self.dev_in[b].copy_(host_in, non_blocking=True)
            self.h2d_done[b].record(self.s_h2d)
        with torch.cuda.stream(self.s_cmp):
            self.s_cmp.wait_event(self.h2d_done[b])
            if reuse:
                self.s_cmp.wait_event(self.d2h_done[b])  # dev_out[b] has been copied out
            _, self.amax = sharded_dynamic_scaled_quant(self.dev_in[b], self.group, self.fp8_dtype,
                                                         exchange=self.exchange, out=self.dev_out[b])
            self.cmp_done[b].record(self.s_cmp)
        with torch.cuda.stream(self.s_d2h):
            self.s_d2h.wait_event(self.cmp_done[b])
            host_out.view(torch.uint8).copy_(self.dev_out[b].view(torch.uint8), non_blocking=True)
            self.d2h_done[b].record(self.s_d2h)
        self.calls += 1

    def copy_only(self, host_in: torch.Tensor, host_out: torch.Tensor) -> None:
        """The two copies of :meth:`submit` on the same streams with no kernel between them (the fp8
        buffer goes back as it is).  For measuring what the host link alone sustains."""
        b = self.calls % self.depth
        with torch.cuda.stream(self.s_h2d):
            self.dev_in[b].copy_(host_in, non_blocking=True)
        with torch.cuda.stream(self.s_d2h):
            host_out.view(torch.uint8).copy_(self.dev_out[b].view(torch.uint8), non_blocking=True)
        self.calls += 1

    def synchronize(self) -> None:
        self.s_h2d.synchronize()
        self.s_cmp.synchronize()
        self.s_d2h.synchronize()
