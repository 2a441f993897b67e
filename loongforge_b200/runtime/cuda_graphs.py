"""CUDA-graph helpers for the training loop: a registry of capturable callables, a full-iteration wrapper that
captures forward + backward of a micro-batch with static inputs, and graceful eager execution on CPU (reference:
loongforge/train/training_utils.py:165-198,2568-2602, loongforge/models/common/cuda_graph_base.py)."""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Sequence

import torch


class GraphedCallable:
    """Captures ``fn(*static_inputs)`` once (after `warmup` eager calls) and replays it; inputs are copied into the
    static buffers, outputs are returned as views of the static outputs (clone them if they must outlive the next call).
    Shapes and dtypes of later calls must equal those of the captured one; otherwise the call runs eagerly."""

    def __init__(self, fn: Callable, warmup: int = 3, pool=None):
        self.fn, self.warmup, self.pool = fn, warmup, pool
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.static_in: List[torch.Tensor] = []
        self.static_out = None
        self.calls = 0
        self.replays = 0

    def _sig(self, args: Sequence[torch.Tensor]):
        return tuple((tuple(a.shape), a.dtype) for a in args)

    def __call__(self, *args: torch.Tensor):
        self.calls += 1
        if not args or not args[0].is_cuda or self.calls <= self.warmup:
            return self.fn(*args)
        if self.graph is None:
            self.static_in = [a.clone() for a in args]
            self.sig = self._sig(args)
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.fn(*self.static_in)
            torch.cuda.current_stream().wait_stream(s)
            self.graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.graph, pool=self.pool):
                self.static_out = self.fn(*self.static_in)
        if self._sig(args) != self.sig:
            return self.fn(*args)
        for dst, src in zip(self.static_in, args):
            dst.copy_(src, non_blocking=True)
        self.graph.replay()
        self.replays += 1
        return self.static_out


_REGISTRY: Dict[str, GraphedCallable] = {}


def register_graphed(name: str, fn: Callable, warmup: int = 3) -> GraphedCallable:
    g = GraphedCallable(fn, warmup)
    _REGISTRY[name] = g
    return g


def get_graphed(name: str) -> GraphedCallable:
    return _REGISTRY[name]


def reset_graphs() -> None:
    _REGISTRY.clear()


def graph_optimizer_step(step_fn: Callable[[], None], warmup: int = 3) -> Callable[[], None]:
    """The optimizer step has no inputs that change address (flat buffers), so it is captured whole; scalar
    hyper-parameters that change per step must live in device tensors that the caller updates before the replay."""
    state = {"calls": 0, "graph": None}

    def run():
        state["calls"] += 1
        if not torch.cuda.is_available() or state["calls"] <= warmup:
            return step_fn()
        if state["graph"] is None:
            g = torch.cuda.CUDAGraph()
            torch.cuda.synchronize()
            with torch.cuda.graph(g):
                step_fn()
            state["graph"] = g
        state["graph"].replay()

    return run
