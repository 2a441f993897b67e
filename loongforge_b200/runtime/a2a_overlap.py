"""MoE all-to-all overlap (``--overlap-moe-expert-parallel-comm``): every MoE layer is cut into the nodes
attn / dispatch / experts / combine / post, and the forward of micro-batch i is interleaved with the backward of
micro-batch i-1 so that one micro-batch's expert-parallel exchange runs (on a communication stream) under the other's
compute (reference: loongforge/models/omni_models/model_chunk_schedule_plan.py:39-647,
fine_grained_callables.py:106-1176).

How it is built here. A micro-batch is a *program*: a list of nodes, each a function from named tensors to named
tensors (`MicrobatchProgram`). Every node is its own autograd segment: its inputs are detached leaves, so its backward
is one `torch.autograd.backward` call that can be issued whenever the schedule wants it, and gradients travel between
nodes by name (summed where a value feeds several nodes). `interleave` merges the forward node list of one micro-batch
with the backward node list of the previous one: after every communication node the issue order switches to the other
program, whose next compute node then runs under that exchange. Compute nodes are issued on the current stream,
communication nodes on a side stream, ordered within a program by events; autograd runs each backward kernel on the
stream of its forward, so the same split holds in backward. The MoE stages are the five methods of
``models/moe.py::MoELayer`` that its own ``forward`` runs back to back, so the overlapped step computes exactly what
the plain step computes. With the peer-memory dispatcher (``parallel/moe_peer.py``) the exchange nodes are SM kernels
themselves; the side stream lets them co-run with the other micro-batch's GEMMs.

Scope: one pipeline stage (pp = 1), no activation recomputation, no hyper-connections; any TP / SP / EP / ETP / CP.
Two micro-batches' activations are alive at a time instead of one."""
from __future__ import annotations

import dataclasses
from typing import Callable, Dict, Iterable, List, Optional, Sequence

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


def defer_host_syncing_nodes(order: List[Node]) -> List[Node]:
    """A forward dispatch node reads the routing counts on the host, i.e. it blocks the issuing thread until the
    compute before it has run. Issue the other program's next compute node first, so the compute stream has work
    queued during that wait (swapping neighbours of different programs never breaks a dependency)."""
    out = list(order)
    i = 0
    while i + 1 < len(out):
        a, b = out[i], out[i + 1]
        if (a.kind == COMM and a.direction == "fwd" and a.name == "dispatch" and b.kind == COMPUTE
                and (a.microbatch, a.direction) != (b.microbatch, b.direction)):
            out[i], out[i + 1] = b, a
            i += 2
        else:
            i += 1
    return out


def overlap_pairs(order: List[Node]) -> int:
    """How many communication nodes are immediately followed by a compute node of the OTHER micro-batch."""
    return sum(1 for x, y in zip(order, order[1:]) if x.kind == COMM and y.kind == COMPUTE and
               (x.microbatch, x.direction) != (y.microbatch, y.direction))


class OverlapExecutor:
    """Runs an issue order: compute nodes on the current stream, communication nodes on a side stream; the nodes of one
    (micro-batch, direction) stay ordered across the two streams by events."""

    def __init__(self):
        self.comm_stream: Optional[torch.cuda.Stream] = None
        self.trace: List[str] = []

    def streams(self):
        if self.comm_stream is None:
            self.comm_stream = torch.cuda.Stream()
        return torch.cuda.current_stream(), self.comm_stream

    def run(self, order: List[Node]) -> None:
        cuda = torch.cuda.is_available()
        if cuda:
            compute, comm = self.streams()
        last_event: Dict[tuple, object] = {}  # (microbatch, direction) -> event of its latest node
        for n in order:
            key = (n.microbatch, n.direction)
            self.trace.append(f"{n.direction}{n.microbatch}.L{n.layer}.{n.name}")
            if n.fn is None:
                continue
            if not cuda:
                n.fn()
                continue
            stream = comm if n.kind == COMM else compute
            if key in last_event:
                stream.wait_event(last_event[key])
            with torch.cuda.stream(stream):
                n.fn()
                ev = torch.cuda.Event()
                ev.record(stream)
            last_event[key] = ev
        if cuda:
            compute.wait_stream(comm)


# ------------------------------------------------------------------------------------------- autograd segments
def _is_diff(t) -> bool:
    return torch.is_tensor(t) and t.is_floating_point()


class Segment:
    """One node of a micro-batch program: ``fn(*inputs) -> outputs`` over NAMED values. `ins` / `outs` are the names;
    values that are not floating-point tensors (masks, None) pass through without gradient."""

    def __init__(self, name: str, kind: str, ins: Sequence[str], outs: Sequence[str], fn: Callable, layer: int = 0):
        self.name, self.kind, self.ins, self.outs, self.fn, self.layer = name, kind, list(ins), list(outs), fn, layer
        self.leaves: Optional[list] = None
        self.results: Optional[tuple] = None

    def forward(self, env: Dict[str, object], streams=None) -> None:
        self.leaves = [env[k].detach().requires_grad_(True) if _is_diff(env[k]) else env[k] for k in self.ins]
        with torch.enable_grad():
            res = self.fn(*self.leaves)
        res = res if isinstance(res, tuple) else (res,)
        assert len(res) == len(self.outs), f"node {self.name}: {len(res)} results for {len(self.outs)} names"
        self.results = res
        for k, v in zip(self.outs, res):
            env[k] = v
            if streams is not None and torch.is_tensor(v) and v.is_cuda:
                for s in streams:  # produced on one stream, read on the other: keep the block until both are past it
                    v.record_stream(s)

    def backward(self, genv: Dict[str, torch.Tensor], streams=None) -> None:
        roots, grads = [], []
        for k, v in zip(self.outs, self.results):
            g = genv.pop(k, None)
            if torch.is_tensor(v) and v.requires_grad and g is not None:
                roots.append(v)
                grads.append(g)
        if roots:
            torch.autograd.backward(roots, grads)
        for k, leaf in zip(self.ins, self.leaves):
            if _is_diff(leaf) and leaf.grad is not None:
                g = leaf.grad
                if streams is not None and g.is_cuda:
                    for s in streams:
                        g.record_stream(s)
                genv[k] = g if k not in genv else genv[k] + g
        self.leaves = self.results = None  # activations of this node are gone


class MicrobatchProgram:
    """The node list of one micro-batch with its value / gradient environments."""

    def __init__(self, segments: List[Segment], microbatch: int):
        self.segments, self.microbatch = segments, microbatch
        self.env: Dict[str, object] = {}
        self.genv: Dict[str, torch.Tensor] = {}

    def forward_nodes(self, streams=None) -> List[Node]:
        last_use = {k: i for i, s in enumerate(self.segments) for k in s.ins}

        def run(i, s):
            s.forward(self.env, streams)
            for k in [k for k in self.env if last_use.get(k, len(self.segments)) <= i]:
                del self.env[k]  # only what autograd saved stays alive

        return [Node(s.name, s.kind, (lambda i=i, s=s: run(i, s)), self.microbatch, "fwd", s.layer)
                for i, s in enumerate(self.segments)]

    def backward_nodes(self, streams=None) -> List[Node]:
        return [Node(s.name, s.kind, (lambda s=s: s.backward(self.genv, streams)), self.microbatch, "bwd", s.layer)
                for s in reversed(self.segments)]


def run_overlapped(programs: Iterable[MicrobatchProgram], executor: Optional[OverlapExecutor] = None,
                   before_last_backward: Optional[Callable[[], None]] = None) -> OverlapExecutor:
    """1F1B over the micro-batches of one step: forward of program 0 alone, then forward of i merged with backward of
    i - 1, then the last backward alone (after `before_last_backward`, e.g. leaving the no-sync mode of the
    data-parallel wrapper)."""
    ex = executor or OverlapExecutor()
    streams = ex.streams() if torch.cuda.is_available() else None
    prev: Optional[MicrobatchProgram] = None
    for prog in programs:
        fwd = LayerPlan(prog.forward_nodes(streams))
        bwd = LayerPlan(prev.backward_nodes(streams)) if prev is not None else None
        ex.run(defer_host_syncing_nodes(interleave(fwd, bwd)))
        prev = prog
    if prev is not None:
        if before_last_backward is not None:
            before_last_backward()
        ex.run(interleave(None, LayerPlan(prev.backward_nodes(streams))))
    return ex


# ------------------------------------------------------------------------------------------- GPT programs
def _layer_segments(model, li: int, layer, rotary, packed, state: dict) -> List[Segment]:
    """Nodes of decoder layer `li` reading ``x{li}`` and writing ``x{li+1}``."""
    cfg = layer.cfg
    xin, xout = f"x{li}", f"x{li + 1}"
    share = cfg.use_dsa and cfg.dsa_indexer_topk_freq > 1

    def run_attention(x):
        if share and hasattr(layer.self_attention, "shared_topk_indices"):
            layer.self_attention.shared_topk_indices = state.get("shared_idx")  # IndexShare
        drop = cfg.hidden_dropout if layer.training else 0.0
        h = layer.input_layernorm(x) if layer.input_layernorm is not None else x
        if drop > 0:
            from ..models.transformer import hidden_dropout
            x = x + hidden_dropout(layer.self_attention(h, rotary, packed, residual=None), drop, cfg)
        else:
            x = layer.self_attention(h, rotary, packed, residual=x)
        if share:
            state["shared_idx"] = getattr(layer.self_attention, "last_topk_indices", state.get("shared_idx"))
        return x

    from ..models.moe import MoELayer
    if not (layer.is_moe and type(layer.mlp) is MoELayer):
        def whole(x):
            x = run_attention(x)
            drop = cfg.hidden_dropout if layer.training else 0.0
            h = layer.pre_mlp_layernorm(x) if layer.pre_mlp_layernorm is not None else x
            if drop > 0:
                from ..models.transformer import hidden_dropout
                return x + hidden_dropout(layer.mlp(h), drop, cfg)
            return x + layer.mlp(h) if layer.is_moe else layer.mlp(h, residual=x)
        return [Segment("layer", COMPUTE, [xin], [xout], whole, li)]

    moe = layer.mlp
    p = f"L{li}."
    side: dict = {}  # values without gradient that travel between the nodes of this layer and micro-batch

    def attn(x):
        x1 = run_attention(x)
        h = layer.pre_mlp_layernorm(x1) if layer.pre_mlp_layernorm is not None else x1
        xl, probs, side["map"] = moe.route(h)
        return x1, h, xl, probs

    def dispatch(xl, probs):
        tokens, aux, side["tpe"] = moe.dispatch_tokens(xl, probs, side["map"])
        return tokens, aux

    def experts(tokens, aux, xl, h):
        return moe.run_experts(tokens, aux, side["tpe"], xl, h)

    def combine(y, aux, xl):
        return moe.combine_tokens(y, aux, xl)

    def post(out, ys, xl, h, x1):
        y = moe.finish(out, ys, xl, h)
        drop = cfg.hidden_dropout if layer.training else 0.0
        if drop > 0:
            from ..models.transformer import hidden_dropout
            y = hidden_dropout(y, drop, cfg)
        return x1 + y

    return [
        Segment("attn", COMPUTE, [xin], [p + "x1", p + "h", p + "xl", p + "probs"], attn, li),
        Segment("dispatch", COMM, [p + "xl", p + "probs"], [p + "tokens", p + "aux"], dispatch, li),
        Segment("experts", COMPUTE, [p + "tokens", p + "aux", p + "xl", p + "h"], [p + "y", p + "ys"], experts, li),
        Segment("combine", COMM, [p + "y", p + "aux", p + "xl"], [p + "out"], combine, li),
        Segment("post", COMPUTE, [p + "out", p + "ys", p + "xl", p + "h", p + "x1"], [xout], post, li),
    ]


def gpt_program(model, inputs: dict, loss_func: Callable, microbatch: int, reports: list) -> MicrobatchProgram:
    """Program of one micro-batch of a single-stage GPT model. `inputs` are the keyword arguments of
    ``GPTModel.forward`` (tokens, position_ids, labels, loss_mask, packed, loss_scale, ...); `loss_func` maps the
    per-token losses to (loss, report). The last node computes the loss and seeds its gradient."""
    cfg = model.cfg
    if not (model.pre_process and model.post_process):
        raise ValueError("the all-to-all overlap schedule needs the whole model on this rank (pipeline size 1)")
    if cfg.enable_hyper_connections or cfg.recompute_granularity == "full" or model.decoder.deepstack_hook is not None:
        raise ValueError("the all-to-all overlap schedule does not cover hyper-connections, full recomputation or "
                         "DeepStack injection")
    tokens, position_ids = inputs["tokens"], inputs["position_ids"]
    packed = inputs.get("packed")
    dev = tokens.device if tokens is not None else inputs["decoder_input"].device
    rotary = model.build_rotary(position_ids, position_ids.shape[-1], dev)
    state: dict = {}

    def pre():
        x = inputs["decoder_input"] if inputs.get("decoder_input") is not None else model.embed(tokens)
        if cfg.moe_n_hash_layers:
            from ..models.moe import set_current_token_ids
            set_current_token_ids(tokens)
        return x

    segs: List[Segment] = [Segment("embed", COMPUTE, [], ["x0"], pre, -1)]
    n = len(model.decoder.layers)
    for li, layer in enumerate(model.decoder.layers):
        segs.extend(_layer_segments(model, li, layer, rotary, packed, state))

    def head(x):
        if model.decoder.final_layernorm is not None:
            x = model.decoder.final_layernorm(x)
        losses = model.postprocess(x, inputs.get("labels"), inputs.get("loss_mask"), inputs.get("loss_scale"),
                                   tokens=tokens, position_ids=position_ids, rotary=rotary, packed=packed,
                                   full_batch=inputs.get("full_batch"))
        loss, rep = loss_func(losses)
        reports.append(rep)
        return loss

    segs.append(Segment("head", COMPUTE, [f"x{n}"], ["loss"], head, n))
    prog = MicrobatchProgram(segs, microbatch)
    _seed_loss_gradient(prog)
    return prog


def gpt_overlapped_forward_backward(model, microbatches, before_last_backward: Optional[Callable[[], None]] = None,
                                    executor: Optional[OverlapExecutor] = None) -> List[dict]:
    """Forward + backward of all micro-batches of one step under the overlap schedule; gradients are accumulated as by
    ``loss.backward()`` per micro-batch. `microbatches`: an iterable of (GPTModel.forward keyword arguments, loss
    function) pairs, pulled one at a time (a micro-batch is fetched when its forward is about to be issued).
    Returns the loss reports in micro-batch order."""
    reports: List[dict] = []
    programs = (gpt_program(model, inputs, loss_func, i, reports) for i, (inputs, loss_func) in enumerate(microbatches))
    run_overlapped(programs, executor, before_last_backward)
    return reports


def _seed_loss_gradient(prog: MicrobatchProgram) -> None:
    """The head node's backward needs d loss = 1; it is created when that backward runs (the loss does not exist yet)."""
    head = prog.segments[-1]
    plain_backward = head.backward

    def backward(genv, streams=None):
        loss = head.results[0]
        genv["loss"] = torch.ones_like(loss)
        plain_backward(genv, streams)

    head.backward = backward
