"""Differentiable collectives between tensor/sequence/context/expert-parallel regions.

These are the NCCL (or gloo) versions: the correctness baseline and the CPU path. On B200 the
column/row-parallel linears bypass them with the fused peer-memory kernels of
``parallel/fused_tp.py``. Semantics follow Megatron's mappings that the reference calls
(e.g. loongforge/models/omni_models/omni_combination_model.py:299-306,
loongforge/models/foundation/language_transformer_block.py:510-515).
Sequence-parallel tensors are sharded along dim 0.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def _ws(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1


def _all_gather_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    x = x.detach().contiguous()
    out = torch.empty((n * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x, group=group)
    return out


def _reduce_scatter_dim0(x: torch.Tensor, group) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    x = x.contiguous()
    assert x.shape[0] % n == 0
    out = torch.empty((x.shape[0] // n,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    if x.is_cuda:
        dist.reduce_scatter_tensor(out, x, group=group)
    else:  # gloo has no reduce_scatter
        tmp = x.clone()
        dist.all_reduce(tmp, group=group)
        r = dist.get_rank(group)
        out.copy_(tmp.chunk(n, 0)[r])
    return out


def _split_dim(x: torch.Tensor, group, dim: int) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    return x.chunk(n, dim)[dist.get_rank(group)].contiguous()


def _gather_dim(x: torch.Tensor, group, dim: int) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        if _ws(ctx.group) > 1:
            g = g.contiguous()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        if _ws(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


class _AllReduceBoth(torch.autograd.Function):
    """Sum over the group in forward AND backward: for a statistic (e.g. a sum of squares over a sharded feature
    dimension) that every rank then uses in its OWN, different downstream computation, so each rank's input receives
    gradient from every rank's output."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        if _ws(group) > 1:
            x = x.contiguous().clone()
            dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        if _ws(ctx.group) > 1:
            g = g.contiguous().clone()
            dist.all_reduce(g, group=ctx.group)
        return g, None


class _ScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _split_dim(x, group, 0)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim0(g, ctx.group), None


class _GatherFromSP(torch.autograd.Function):
    """All-gather along the sequence; backward reduce-scatters (or just splits)."""

    @staticmethod
    def forward(ctx, x, group, tp_output_grad):
        ctx.group, ctx.rs = group, tp_output_grad
        return _all_gather_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        if ctx.rs:
            return _reduce_scatter_dim0(g, ctx.group), None, None
        return _split_dim(g, ctx.group, 0), None, None


class _ReduceScatterToSP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _reduce_scatter_dim0(x, group)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_dim0(g, ctx.group), None


class _GatherLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _gather_dim(x, group, -1)

    @staticmethod
    def backward(ctx, g):
        return _split_dim(g, ctx.group, -1), None


class _ScatterLastDim(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return _split_dim(x, group, -1)

    @staticmethod
    def backward(ctx, g):
        return _gather_dim(g, ctx.group, -1), None


class _AllToAll(torch.autograd.Function):
    """all_to_all_single with optional uneven splits along dim 0."""

    @staticmethod
    def forward(ctx, x, group, out_splits, in_splits):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        if _ws(group) == 1:
            return x
        x = x.contiguous()
        if out_splits is None:
            out = torch.empty_like(x)
        else:
            out = torch.empty((sum(out_splits),) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        all_to_all_single(out, x, out_splits, in_splits, group)
        return out

    @staticmethod
    def backward(ctx, g):
        return _AllToAll.apply(g, ctx.group, ctx.in_splits, ctx.out_splits), None, None, None


def all_to_all_single(out, x, out_splits, in_splits, group):
    """dist.all_to_all_single, emulated with all_gather-free p2p lists on gloo (CPU tests)."""
    if x.is_cuda:
        dist.all_to_all_single(out, x, out_splits, in_splits, group=group)
        return
    n = _ws(group)
    ins = list(x.split(in_splits if in_splits is not None else x.shape[0] // n, 0))
    outs = list(out.split(out_splits if out_splits is not None else out.shape[0] // n, 0))
    ins = [t.contiguous() for t in ins]
    outs_c = [torch.empty_like(t) for t in outs]
    dist.all_to_all(outs_c, ins, group=group) if dist.get_backend(group) != "gloo" else _gloo_a2a(outs_c, ins, group)
    for o, c in zip(outs, outs_c):
        o.copy_(c)


def _gloo_a2a(outs, ins, group):
    n = _ws(group)
    me = dist.get_rank(group)
    ranks = dist.get_process_group_ranks(group)
    reqs = []
    for peer in range(n):
        if peer == me:
            outs[me].copy_(ins[me])
            continue
        # zero-size point-to-point transfers never complete on gloo; both sides know the sizes and skip them
        if ins[peer].numel() > 0:
            reqs.append(dist.isend(ins[peer], ranks[peer], group=group))
        if outs[peer].numel() > 0:
            reqs.append(dist.irecv(outs[peer], ranks[peer], group=group))
    for r in reqs:
        r.wait()


# public API (names follow Megatron's tensor_parallel.mappings) ------------------------------
def copy_to_tensor_model_parallel_region(x, group): return _CopyToTP.apply(x, group)
def reduce_from_tensor_model_parallel_region(x, group): return _ReduceFromTP.apply(x, group)
def all_reduce_forward_and_backward(x, group): return _AllReduceBoth.apply(x, group)
def scatter_to_sequence_parallel_region(x, group): return _ScatterToSP.apply(x, group)
def gather_from_sequence_parallel_region(x, group, tensor_parallel_output_grad: bool = True):
    return _GatherFromSP.apply(x, group, tensor_parallel_output_grad)
def reduce_scatter_to_sequence_parallel_region(x, group): return _ReduceScatterToSP.apply(x, group)
def gather_from_tensor_model_parallel_region(x, group): return _GatherLastDim.apply(x, group)
def scatter_to_tensor_model_parallel_region(x, group): return _ScatterLastDim.apply(x, group)
def all_to_all(x, group, out_splits: Optional[List[int]] = None, in_splits: Optional[List[int]] = None):
    return _AllToAll.apply(x, group, out_splits, in_splits)


def all_to_all_sp2hp(x: torch.Tensor, group) -> torch.Tensor:
    """[s/P, H, d] (sequence-sharded, all heads) -> [s, H/P, d] (full sequence, head-sharded)."""
    n = _ws(group)
    if n == 1:
        return x
    s, H, d = x.shape
    xs = x.reshape(s, n, H // n, d).permute(1, 0, 2, 3).contiguous().reshape(n * s, H // n, d)
    return all_to_all(xs, group)


def all_to_all_hp2sp(x: torch.Tensor, group) -> torch.Tensor:
    """Inverse of :func:`all_to_all_sp2hp` ([s, H/P, d] -> [s/P, H, d])."""
    n = _ws(group)
    if n == 1:
        return x
    S, h, d = x.shape
    y = all_to_all(x.contiguous(), group)  # chunk j now holds rank j's heads for my sequence slice
    return y.reshape(n, S // n, h, d).permute(1, 0, 2, 3).reshape(S // n, n * h, d)
