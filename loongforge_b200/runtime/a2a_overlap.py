"""MoE all-to-all overlap: a layer is split into the nodes attn / dispatch / experts / combine / post and the forward of
micro-batch i is interleaved with the backward of micro-batch i-1 so that one micro-batch's expert-parallel exchange
runs (on the communication stream) under the other's compute (reference:
loongforge/models/omni_models/model_chunk_schedule_plan.py:39-647, fine_grained_callables.py:106-1176).

``LayerPlan`` is the node list of one layer; ``interleave`` produces the merged issue order for a forward plan and a
backward plan; ``OverlapExecutor`` runs such an order with compute nodes on the current stream and communication nodes
on a side stream, ordered by events. With the peer-memory dispatcher (``parallel/moe_peer.py``) the exchange nodes are
SM kernels themselves, so the side stream simply lets them co-run with the other micro-batch's GEMMs."""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, List, Optional

import torch

COMPUTE, COMM = "compute", "comm"
FORWARD_NODES = [("attn", COMPUTE), ("dispatch", COMM), ("experts", COMPUTE), ("combine", COMM), ("post", COMPUTE)]


@dataclasses.dataclass
class Node:
    name: str
    kind: str
    fn: Optional[Callable[[], None]] = None
    microbatch: int = 0
    direction: str = "fwd"
    layer: int = 0


@dataclasses.dataclass
class LayerPlan:
    nodes: List[Node]

    @staticmethod
    def forward(layer: int, mb: int, fns: Optional[Dict[str, Callable]] = None) -> "LayerPlan":
        fns = fns or {}
        return LayerPlan([Node(n, k, fns.get(n), mb, "fwd", layer) for n, k in FORWARD_NODES])

    @staticmethod
    def backward(layer: int, mb: int, fns: Optional[Dict[str, Callable]] = None) -> "LayerPlan":
        fns = fns or {}
        return LayerPlan([Node(n, k, fns.get(n), mb, "bwd", layer) for n, k in reversed(FORWARD_NODES)])


def interleave(fwd: Optional[LayerPlan], bwd: Optional[LayerPlan]) -> List[Node]:
    """Merged issue order: every communication node of one plan is issued right before a compute node of the other, so
    they overlap. Relative order inside each plan is preserved."""
    if fwd is None or bwd is None:
        return list((fwd or bwd).nodes)
    cur, other = list(bwd.nodes), list(fwd.nodes)  # backward leads: its first node (post) frees activations earliest
    out: List[Node] = []
    while cur or other:
        if not cur:
            cur, other = other, cur
        n = cur.pop(0)
        out.append(n)
        if n.kind == COMM and other:
            cur, other = other, cur  # the other plan's next compute node runs under this exchange
    return out


def overlap_pairs(order: List[Node]) -> int:
    """How many communication nodes are immediately followed by a compute node of the OTHER micro-batch."""
    return sum(1 for x, y in zip(order, order[1:]) if x.kind == COMM and y.kind == COMPUTE and
               (x.microbatch, x.direction) != (y.microbatch, y.direction))


class OverlapExecutor:
    def __init__(self):
        self.comm_stream: Optional[torch.cuda.Stream] = None
        self.trace: List[str] = []

    def run(self, order: List[Node]) -> None:
        cuda = torch.cuda.is_available()
        if cuda and self.comm_stream is None:
            self.comm_stream = torch.cuda.Stream()
        last_event: Dict[tuple, object] = {}  # (microbatch, direction) -> event of its latest node
        for n in order:
            key = (n.microbatch, n.direction)
            self.trace.append(f"{n.direction}{n.microbatch}.L{n.layer}.{n.name}")
            if n.fn is None:
                continue
            if not cuda:
                n.fn()
                continue
            stream = self.comm_stream if n.kind == COMM else torch.cuda.current_stream()
            if key in last_event:
                stream.wait_event(last_event[key])  # nodes of one micro-batch stay ordered across the two streams
            with torch.cuda.stream(stream):
                n.fn()
                ev = torch.cuda.Event()
                ev.record(stream)
            last_event[key] = ev
        if cuda:
            torch.cuda.current_stream().wait_stream(self.comm_stream)
