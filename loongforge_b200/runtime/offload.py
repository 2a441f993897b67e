"""Pinned-memory activation offload on side streams: gathered vision embeddings (and their gradients) of the
full-heterogeneous-DP VLM path are parked in host memory between the encoder step and the decoder micro-batches
that consume them (reference: loongforge/train/full_hetero_cpu_offload.py:16-170).

``offload`` starts an asynchronous device->host copy on a dedicated stream and returns a handle; ``reload`` starts
the host->device copy and makes the caller's stream wait for it. On CPU tensors both are identity operations."""
from __future__ import annotations

from typing import Dict, Optional

import torch


class _Handle:
    def __init__(self, host: torch.Tensor, event, device, shape, dtype):
        self.host, self.event, self.device, self.shape, self.dtype = host, event, device, shape, dtype


class AsyncCPUOffloader:
    def __init__(self, max_pinned_bytes: Optional[int] = None):
        self.d2h = self.h2d = None
        self.max_bytes = max_pinned_bytes
        self.bytes_pinned = 0
        self.pool: Dict[tuple, list] = {}

    def _streams(self):
        if self.d2h is None:
            self.d2h, self.h2d = torch.cuda.Stream(), torch.cuda.Stream()

    def _host_buffer(self, t: torch.Tensor) -> torch.Tensor:
        key = (tuple(t.shape), t.dtype)
        free = self.pool.get(key)
        if free:
            return free.pop()
        nbytes = t.numel() * t.element_size()
        if self.max_bytes is not None and self.bytes_pinned + nbytes > self.max_bytes:
            raise MemoryError(f"pinned offload budget of {self.max_bytes} bytes exceeded")
        self.bytes_pinned += nbytes
        return torch.empty(t.shape, dtype=t.dtype, pin_memory=True)

    def offload(self, t: torch.Tensor) -> _Handle:
        if not t.is_cuda:
            return _Handle(t, None, t.device, t.shape, t.dtype)
        self._streams()
        host = self._host_buffer(t)
        self.d2h.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.d2h):
            host.copy_(t, non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(self.d2h)
        t.record_stream(self.d2h)  # the device block may be reused only after the copy has read it
        return _Handle(host, ev, t.device, t.shape, t.dtype)

    def reload(self, h: _Handle, release: bool = True) -> torch.Tensor:
        if h.event is None:
            return h.host
        self._streams()
        self.h2d.wait_event(h.event)
        with torch.cuda.stream(self.h2d):
            out = torch.empty(h.shape, dtype=h.dtype, device=h.device)
            out.copy_(h.host, non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.h2d)
        torch.cuda.current_stream().wait_event(done)
        out.record_stream(torch.cuda.current_stream())
        if release:
            done.synchronize()
            self.pool.setdefault((tuple(h.shape), h.dtype), []).append(h.host)
        return out


class OffloadedActivation(torch.autograd.Function):
    """Identity in value; the tensor saved for backward lives in pinned host memory instead of HBM."""

    @staticmethod
    def forward(ctx, x, offloader: AsyncCPUOffloader, fn_weight):
        ctx.off = offloader
        ctx.handle = offloader.offload(x.detach())
        ctx.save_for_backward(fn_weight)
        return x @ fn_weight

    @staticmethod
    def backward(ctx, g):
        (w,) = ctx.saved_tensors
        x = ctx.off.reload(ctx.handle)
        return g @ w.t(), None, x.t() @ g
