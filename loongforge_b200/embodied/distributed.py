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


def wrap_model(model: nn.Module, args, ctx: DistContext) -> nn.Module:
    """ddp / zero1: DistributedDataParallel (static graph, gradient-as-bucket-view, optional bf16 comm hook);
    fsdp / hsdp: FSDP2 ``fully_shard`` per planned unit with forward prefetch, HSDP on a 2-D device mesh."""
    model = model.to(ctx.device)
    if ctx.world == 1:
        return model
    if args.strategy in ("ddp", "zero1"):
        ddp = nn.parallel.DistributedDataParallel(
            model, device_ids=[ctx.local_rank] if ctx.device.type == "cuda" else None,
            bucket_cap_mb=args.ddp_bucket_mb, gradient_as_bucket_view=True, static_graph=args.ddp_static_graph)
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
    units = []
    for name in FSDPWrapPlan(model, args.fsdp_wrap_patterns):
        units.append(fully_shard(model.get_submodule(name), mesh=mesh))
    fully_shard(model, mesh=mesh)
    n = max(int(args.fsdp_prefetch), 0)
    for i, u in enumerate(units):  # ordered forward prefetch of the next `n` units
        nxt = units[i + 1:i + 1 + n]
        if nxt and hasattr(u, "set_modules_to_forward_prefetch"):
            u.set_modules_to_forward_prefetch(nxt)
    return model


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
