"""Process-group context, model wrapping (DDP / ZeRO-1 / FSDP2 / HSDP) and pattern-based activation
checkpointing for the embodied stack (reference: loongforge/embodied/distributed/context.py:12-40,
parallel.py:49-486, ddp_utils/ddp_comm_hook.py:28-60, activation_checkpointing.py:15-130)."""
from __future__ import annotations

import fnmatch
import os
from typing import Iterable, List, Optional

import torch
import torch.distributed as dist
import torch.nn as nn


class DistContext:
    """torchrun environment -> process group with backend ``cpu:gloo,cuda:nccl`` when a GPU is present."""

    def __init__(self):
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local_rank = int(os.environ.get("LOCAL_RANK", "0"))
        self.device = torch.device("cuda", self.local_rank) if torch.cuda.is_available() else torch.device("cpu")

    def init(self) -> "DistContext":
        if self.device.type == "cuda":
            torch.cuda.set_device(self.device)
        if self.world > 1 and not dist.is_initialized():
            backend = "cpu:gloo,cuda:nccl" if self.device.type == "cuda" else "gloo"
            dist.init_process_group(backend, rank=self.rank, world_size=self.world)
        return self

    @property
    def is_main(self) -> bool:
        return self.rank == 0

    def barrier(self):
        if self.world > 1:
            dist.barrier()


def apply_activation_checkpointing(model: nn.Module, patterns: Iterable[str]) -> List[str]:
    """Wrap every sub-module whose qualified name matches one of the glob `patterns` so that its forward is
    recomputed in backward. Returns the wrapped names."""
    from torch.utils.checkpoint import checkpoint

    patterns = list(patterns)
    wrapped = []
    for name, mod in list(model.named_modules()):
        if name and any(fnmatch.fnmatch(name, p) for p in patterns) and not getattr(mod, "_lf_ckpt", False):
            inner = mod.forward

            def fwd(*a, _inner=inner, **kw):
                if torch.is_grad_enabled():
                    return checkpoint(_inner, *a, use_reentrant=False, **kw)
                return _inner(*a, **kw)

            mod.forward = fwd
            mod._lf_ckpt = True
            wrapped.append(name)
    return wrapped


def bf16_compress_hook(state, bucket):
    """DDP communication hook: all-reduce the bucket in bf16, return it in the original dtype."""
    group = state if state is not None else dist.group.WORLD
    buf = bucket.buffer()
    comp = buf.to(torch.bfloat16).div_(dist.get_world_size(group))
    fut = dist.all_reduce(comp, group=group, async_op=True).get_future()

    def done(f):
        buf.copy_(f.value()[0])
        return buf

    return fut.then(done)


class FSDPWrapPlan:
    """Which sub-modules become FSDP units: every module matching a pattern, innermost first, in forward order."""

    def __init__(self, model: nn.Module, patterns: Iterable[str]):
        patterns = list(patterns)
        hits = [n for n, _ in model.named_modules() if n and any(fnmatch.fnmatch(n, p) for p in patterns)]
        # a glob also matches the children of a matching block; only the outermost match becomes a unit
        self.units = [n for n in hits if not any(n.startswith(h + ".") for h in hits)]

    def __iter__(self):
        return iter(self.units)


class FSDPAutoPlanner:
    """FSDP units without hand-written patterns (``fsdp_wrap_patterns: [auto]``), in three passes over the module tree:

    1. *repeated layers*: going down from the root, the first module on each path whose class occurs at least twice in the
       model (transformer blocks, encoder layers) is a candidate and is not descended into. Containers, classes listed in
       ``no_wrap`` and modules whose parameters have more than one dtype are never candidates: the walk continues into
       their children. Consecutive candidates with the same parent and class form a run; a run is cut into groups of at
       least ``min_num_params`` parameters (several small layers share one unit — one all-gather), and a run smaller
       than that in total is left to the root unit.
    2. *leftover leaves*: a module outside every planned unit that directly owns at least ``leftover_min_num_params``
       parameters of one dtype (a big embedding or output projection) becomes a unit of its own.
    3. the root takes the rest.

    ``reshard_after_forward`` per unit comes from ``reshard_overrides`` (glob over the unit's first module name -> bool or
    int), else ``reshard_default``; the root uses ``reshard_root`` (False keeps the root's parameters gathered between
    forward and backward, which saves one all-gather per step). (reference: loongforge/embodied/distributed/parallel.py:
    278-486 for unit resolution and prefetch edges, 488-973 for the planner)"""

    CONTAINERS = (nn.ModuleList, nn.Sequential, nn.ModuleDict)

    def __init__(self, model: nn.Module, min_num_params: int = 1_000_000, leftover_min_num_params: int = 10_000_000,
                 no_wrap: Iterable[str] = (), reshard_default=True, reshard_root=False, reshard_overrides: Optional[dict] = None):
        self.model, self.min, self.leftover_min = model, int(min_num_params), int(leftover_min_num_params)
        # a unit's parameters are gathered by hooks around ITS forward: a module that other code reaches into (joint
        # attention calling a layer's projection methods) or that has no forward of its own must not be a unit. Models
        # name such classes in ``FSDP_NO_WRAP``.
        self.no_wrap = set(no_wrap or ())
        for m in model.modules():
            self.no_wrap.update(getattr(m, "FSDP_NO_WRAP", ()))
        self.reshard_default, self.reshard_root = reshard_default, reshard_root
        self.reshard_overrides = dict(reshard_overrides or {})
        self.units: List[dict] = []   # {"names": [...], "params": int, "reshard": bool | int, "kind": "layers" | "leaf"}
        self._plan()

    @staticmethod
    def _uniform_dtype(params) -> bool:
        return len({p.dtype for p in params}) <= 1

    def _reshard_for(self, name: str):
        for pat, val in self.reshard_overrides.items():
            if fnmatch.fnmatch(name, pat):
                return val
        return self.reshard_default

    def _plan(self):
        import collections
        with_params = [m for m in self.model.modules() if any(True for _ in m.parameters())]
        counts = collections.Counter(type(m) for m in with_params)
        seen = collections.Counter(id(m) for _, m in self.model.named_modules(remove_duplicate=False))
        cands: List[tuple] = []

        def visit(prefix: str, mod: nn.Module):
            for cn, child in mod.named_children():
                name = f"{prefix}.{cn}" if prefix else cn
                params = list(child.parameters())
                if not params:
                    continue
                ok = (counts[type(child)] >= 2 and not isinstance(child, self.CONTAINERS) and seen[id(child)] == 1
                      and type(child).__name__ not in self.no_wrap and self._uniform_dtype(params)
                      and type(child).forward is not nn.Module.forward)
                if ok:
                    cands.append((name, child, prefix, sum(p.numel() for p in params)))
                else:
                    visit(name, child)

        visit("", self.model)
        planned = set()
        i = 0
        while i < len(cands):  # runs of consecutive candidates with the same parent and class
            j = i
            while j + 1 < len(cands) and cands[j + 1][2] == cands[i][2] and type(cands[j + 1][1]) is type(cands[i][1]):
                j += 1
            run = cands[i:j + 1]
            i = j + 1
            if sum(c[3] for c in run) < self.min:
                continue
            groups, cur, size = [], [], 0
            for c in run:
                cur.append(c)
                size += c[3]
                if size >= self.min:
                    groups.append(cur)
                    cur, size = [], 0
            if cur:  # a short tail joins the group before it
                groups[-1].extend(cur)
            for g in groups:
                self.units.append({"names": [c[0] for c in g], "params": sum(c[3] for c in g),
                                   "reshard": self._reshard_for(g[0][0]), "kind": "layers"})
                for c in g:
                    planned.update(id(p) for p in c[1].parameters())
        for name, mod in self.model.named_modules():
            if not name or type(mod).__name__ in self.no_wrap or type(mod).forward is nn.Module.forward:
                continue
            own = [p for p in mod.parameters(recurse=False) if id(p) not in planned]
            if own and sum(p.numel() for p in own) >= self.leftover_min and self._uniform_dtype(own):
                self.units.append({"names": [name], "params": sum(p.numel() for p in own),
                                   "reshard": self._reshard_for(name), "kind": "leaf"})
                planned.update(id(p) for p in own)
        order = {n: i for i, (n, _) in enumerate(self.model.named_modules())}
        self.units.sort(key=lambda u: order[u["names"][0]])
        self.root_params = sum(p.numel() for p in self.model.parameters() if id(p) not in planned)

    def describe(self) -> str:
        lines = [f"{u['kind']:6s} {u['params']:>12,d}  reshard={u['reshard']}  {', '.join(u['names'])}" for u in self.units]
        return "\n".join(lines + [f"root   {self.root_params:>12,d}  reshard={self.reshard_root}"])

    def apply(self, mesh, **fsdp_kw) -> List[nn.Module]:
        from torch.distributed.fsdp import fully_shard
        handles = []
        for u in self.units:
            mods = [self.model.get_submodule(n) for n in u["names"]]
            handles.append(fully_shard(mods if len(mods) > 1 else mods[0], mesh=mesh, reshard_after_forward=u["reshard"], **fsdp_kw))
        fully_shard(self.model, mesh=mesh, reshard_after_forward=self.reshard_root, **fsdp_kw)
        return [h[0] if isinstance(h, (list, tuple)) else h for h in handles]


def wrap_model(model: nn.Module, args, ctx: DistContext) -> nn.Module:
    """ddp / zero1: DistributedDataParallel (static graph, gradient-as-bucket-view, optional bf16 comm hook);
    fsdp / hsdp: FSDP2 ``fully_shard`` per planned unit (patterns, or the automatic planner with ``[auto]``) with forward
    prefetch of the next units in registration order, HSDP on a 2-D device mesh."""
    model = model.to(ctx.device)
    if ctx.world == 1:
        return model
    if args.strategy in ("ddp", "zero1"):
        ddp = nn.parallel.DistributedDataParallel(
            model, device_ids=[ctx.local_rank] if ctx.device.type == "cuda" else None,
            bucket_cap_mb=args.ddp_bucket_mb, gradient_as_bucket_view=True, static_graph=args.ddp_static_graph,
            find_unused_parameters=getattr(args, "ddp_find_unused_parameters", False),
            broadcast_buffers=getattr(args, "ddp_broadcast_buffers", True))
        if args.ddp_comm_hook == "bf16_compress":
            ddp.register_comm_hook(None, bf16_compress_hook)
        return ddp
    from torch.distributed.device_mesh import init_device_mesh
    from torch.distributed.fsdp import fully_shard

    dev_type = ctx.device.type
    if args.strategy == "hsdp":
        shard = args.hsdp_shard_size
        mesh = init_device_mesh(dev_type, (ctx.world // shard, shard), mesh_dim_names=("replicate", "shard"))
    else:
        mesh = init_device_mesh(dev_type, (ctx.world,), mesh_dim_names=("shard",))
    fsdp_kw = {}
    if getattr(args, "fsdp_param_dtype", None) or getattr(args, "fsdp_reduce_dtype", None):
        from torch.distributed.fsdp import MixedPrecisionPolicy
        to = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "float32": torch.float32, None: None}
        fsdp_kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=to[args.fsdp_param_dtype], reduce_dtype=to[args.fsdp_reduce_dtype])
    if list(args.fsdp_wrap_patterns) == ["auto"]:
        planner = FSDPAutoPlanner(model, args.fsdp_min_num_params, args.fsdp_leftover_min_num_params, args.fsdp_no_wrap_modules,
                                  args.fsdp_reshard_default, args.fsdp_reshard_root, args.fsdp_reshard_module_overrides)
        if ctx.is_main:
            print("FSDP units (automatic plan):\n" + planner.describe(), flush=True)
        units = planner.apply(mesh, **fsdp_kw)
    else:
        units = []
        for name in FSDPWrapPlan(model, args.fsdp_wrap_patterns):
            units.append(fully_shard(model.get_submodule(name), mesh=mesh,
                                     reshard_after_forward=FSDPAutoPlanner._reshard_for(_ReshardOnly(args), name), **fsdp_kw))
        fully_shard(model, mesh=mesh, reshard_after_forward=args.fsdp_reshard_root, **fsdp_kw)
    n = max(int(args.fsdp_prefetch), 0)
    for i, u in enumerate(units):  # ordered forward prefetch of the next `n` units
        nxt = units[i + 1:i + 1 + n]
        if nxt and hasattr(u, "set_modules_to_forward_prefetch"):
            u.set_modules_to_forward_prefetch(nxt)
    for i, u in enumerate(units):  # and backward prefetch of the units before it
        prv = list(reversed(units[max(i - n, 0):i]))
        if prv and hasattr(u, "set_modules_to_backward_prefetch"):
            u.set_modules_to_backward_prefetch(prv)
    return model


class _ReshardOnly:
    """The reshard options of the arguments in the shape ``FSDPAutoPlanner._reshard_for`` reads."""

    def __init__(self, args):
        self.reshard_overrides = dict(args.fsdp_reshard_module_overrides or {})
        self.reshard_default = args.fsdp_reshard_default


def grad_sync_context(model: nn.Module, sync: bool):
    """No-sync context for all but the last micro-batch of an accumulation window."""
    import contextlib

    if sync:
        return contextlib.nullcontext()
    if isinstance(model, nn.parallel.DistributedDataParallel):
        return model.no_sync()
    if hasattr(model, "set_requires_gradient_sync"):  # FSDP2

        @contextlib.contextmanager
        def ctx():
            model.set_requires_gradient_sync(False)
            try:
                yield
            finally:
                model.set_requires_gradient_sync(True)

        return ctx()
    return contextlib.nullcontext()
