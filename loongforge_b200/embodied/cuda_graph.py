"""Per-micro-batch CUDA graphs: the forward + backward of one micro-batch is captured once with static input
buffers and replayed for every later micro-batch, removing the launch overhead of the many small kernels of action
heads (reference: loongforge/embodied/train/trainers/custom/groot_n1_6/per_microbatch_cuda_graph.py,
groot_n1_7/per_microbatch_cuda_graph.py).

Requirements: parameters and gradients resident on the device (DDP / ZeRO-1, not FSDP), static shapes, gradients
accumulated into ``.grad`` tensors that exist before capture, and randomness drawn OUTSIDE the graph (noise and
timesteps are inputs). On CPU the runner executes eagerly so the calling code is the same.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch
import torch.nn as nn


class MicrobatchGraphRunner:
    def __init__(self, model: nn.Module, loss_fn: Callable[[nn.Module, Dict[str, torch.Tensor]], torch.Tensor],
                 warmup: int = 3):
        self.model, self.loss_fn, self.warmup = model, loss_fn, warmup
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_in: Dict[str, torch.Tensor] = {}
        self.static_loss: Optional[torch.Tensor] = None
        self.calls = 0

    def _ensure_grads(self):
        for p in self.model.parameters():
            if p.requires_grad and p.grad is None:
                p.grad = torch.zeros_like(p)

    def _eager(self, batch, scale):
        loss = self.loss_fn(self.model, batch)
        (loss * scale).backward()
        return loss.detach()

    def run(self, batch: Dict[str, torch.Tensor], scale: float = 1.0) -> torch.Tensor:
        """Accumulates ``scale * dloss`` into the parameters' ``.grad`` and returns the detached loss."""
        dev = next(self.model.parameters()).device
        self.calls += 1
        if dev.type != "cuda" or self.calls <= self.warmup:
            self._ensure_grads()
            return self._eager(batch, scale)
        if self.graph is None:
            self._ensure_grads()
            self.static_in = {k: v.clone() for k, v in batch.items()}
            self.scale = scale
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):  # one eager pass on the side stream before capture, as capture requires
                self._eager(self.static_in, 0.0)
            torch.cuda.current_stream().wait_stream(s)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph):
                loss = self.loss_fn(self.model, self.static_in)
                (loss * scale).backward()
                self.static_loss = loss.detach()
        assert scale == self.scale, "the accumulation scale is baked into the captured graph"
        for k, v in batch.items():
            self.static_in[k].copy_(v, non_blocking=True)
        self.graph.replay()
        return self.static_loss.clone()
