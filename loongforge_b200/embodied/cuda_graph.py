"""Per-micro-batch CUDA graphs: the forward + backward of one micro-batch is captured once with static input
buffers and replayed for every later micro-batch, removing the launch overhead of the many small kernels of action
heads (reference: loongforge/embodied/train/trainers/custom/groot_n1_6/per_microbatch_cuda_graph.py,
groot_n1_7/per_microbatch_cuda_graph.py).

Requirements: parameters and gradients resident on the device (DDP / ZeRO-1, not FSDP), gradients accumulated into
``.grad`` tensors that exist before capture; random draws inside the captured region use the device generator, whose
offset advances with every replay. Shapes are made static by padding the token fields to a multiple of ``pad_to``; every
distinct input signature gets a graph of its own. On CPU the runner pads and executes eagerly, so the calling code is
the same.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn as nn


class _Captured:
    def __init__(self):
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_in: Dict[str, torch.Tensor] = {}
        self.static_loss: Optional[torch.Tensor] = None
        self.scale: Optional[float] = None
        self.calls = 0


def pad_batch(batch: Dict[str, torch.Tensor], pad_to: int, keys=("text", "tokens", "token_mask")) -> Dict[str, torch.Tensor]:
    """Token fields ``[B, L]`` are padded with zeros (= padding id / masked) to the next multiple of ``pad_to``, so that
    instructions of different lengths share one captured shape."""
    if pad_to <= 1:
        return batch
    out = dict(batch)
    for k in keys:
        v = batch.get(k)
        if v is not None and v.dim() == 2 and v.shape[1] % pad_to:
            out[k] = torch.nn.functional.pad(v, (0, pad_to - v.shape[1] % pad_to))
    return out


def shape_key(batch: Dict[str, torch.Tensor]):
    return tuple(sorted((k, tuple(v.shape), str(v.dtype)) for k, v in batch.items()))


class MicrobatchGraphRunner:
    """One captured graph per input signature (names, shapes, dtypes of the batch), at most ``max_graphs`` of them (the
    least recently used one is dropped); every signature runs ``warmup`` eager micro-batches before it is captured."""

    def __init__(self, model: nn.Module, loss_fn: Callable[[nn.Module, Dict[str, torch.Tensor]], torch.Tensor],
                 warmup: int = 3, pad_to: int = 1, max_graphs: int = 4):
        self.model, self.loss_fn, self.warmup, self.pad_to, self.max_graphs = model, loss_fn, warmup, pad_to, max_graphs
        self.captured: "Dict[tuple, _Captured]" = {}
        self.calls = 0

    @property
    def graph(self) -> Optional[torch.cuda.CUDAGraph]:
        """Any captured graph (the trainer only asks whether gradients live in captured storage)."""
        return next((c.graph for c in self.captured.values() if c.graph is not None), None)

    def _ensure_grads(self):
        for p in self.model.parameters():
            if p.requires_grad and p.grad is None:
                p.grad = torch.zeros_like(p)

    def _eager(self, batch, scale):
        loss = self.loss_fn(self.model, batch)
        (loss * scale).backward()
        return loss.detach()

    def _slot(self, batch) -> _Captured:
        key = shape_key(batch)
        c = self.captured.pop(key, None) or _Captured()
        self.captured[key] = c                       # most recently used last
        while len(self.captured) > self.max_graphs:
            self.captured.pop(next(iter(self.captured)))
        return c

    def run(self, batch: Dict[str, torch.Tensor], scale: float = 1.0) -> torch.Tensor:
        """Accumulates ``scale * dloss`` into the parameters' ``.grad`` and returns the detached loss."""
        dev = next(self.model.parameters()).device
        batch = pad_batch(batch, self.pad_to)
        c = self._slot(batch)
        self.calls += 1
        c.calls += 1
        if dev.type != "cuda" or c.calls <= self.warmup:
            self._ensure_grads()
            return self._eager(batch, scale)
        if c.graph is None:
            self._ensure_grads()
            c.static_in = {k: v.clone() for k, v in batch.items()}
            c.scale = scale
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):  # one eager pass on the side stream before capture, as capture requires
                self._eager(c.static_in, 0.0)
            torch.cuda.current_stream().wait_stream(s)
            c.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(c.graph):
                loss = self.loss_fn(self.model, c.static_in)
                (loss * scale).backward()
                c.static_loss = loss.detach()
        assert scale == c.scale, "the accumulation scale is baked into the captured graph"
        for k, v in batch.items():
            c.static_in[k].copy_(v, non_blocking=True)
        c.graph.replay()
        return c.static_loss.clone()
