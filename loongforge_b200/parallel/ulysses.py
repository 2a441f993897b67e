"""Ulysses sequence parallelism for non-causal (diffusion) attention.

Tokens are sharded contiguously over the group outside attention; for attention one all-to-all turns
``[L/P, H, d]`` (all heads of my tokens) into ``[L, H/P, d]`` (my heads of all tokens) and a second one turns the
output back. Counterpart of loongforge/models/diffusion/wan/wan_ulysses.py; the all-to-alls are the autograd-aware
ones of ``parallel/mappings.py`` (NCCL on GPUs, emulated on gloo for CPU tests).
"""
from __future__ import annotations

import torch
import torch.distributed as dist
import torch.nn.functional as F

from . import mappings as M


def _ws(group) -> int:
    return dist.get_world_size(group) if (group is not None and dist.is_initialized()) else 1


def shard_sequence(x: torch.Tensor, group, dim: int = 1) -> torch.Tensor:
    """Keep this rank's contiguous slice of `dim` (the backward all-gathers the slices)."""
    n = _ws(group)
    if n == 1:
        return x
    r = dist.get_rank(group)
    xt = x.transpose(0, dim) if dim != 0 else x
    out = M.scatter_to_sequence_parallel_region(xt.contiguous(), group) if xt.requires_grad else \
        xt.chunk(n, 0)[r].contiguous()
    return out.transpose(0, dim) if dim != 0 else out


def gather_sequence(x: torch.Tensor, group, dim: int = 1) -> torch.Tensor:
    n = _ws(group)
    if n == 1:
        return x
    xt = x.transpose(0, dim).contiguous() if dim != 0 else x
    out = M.gather_from_sequence_parallel_region(xt, group, False)
    return out.transpose(0, dim) if dim != 0 else out


def ulysses_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, group) -> torch.Tensor:
    """q, k, v [B, L/P, H, d] -> [B, L/P, H*d]; full (non-causal) attention over the gathered sequence."""
    B, Ll, H, d = q.shape
    outs = []
    for b in range(B):
        qh, kh, vh = (M.all_to_all_sp2hp(t[b].contiguous(), group) for t in (q, k, v))  # [L, H/P, d]
        o = F.scaled_dot_product_attention(qh.transpose(0, 1).unsqueeze(0), kh.transpose(0, 1).unsqueeze(0),
                                           vh.transpose(0, 1).unsqueeze(0))[0].transpose(0, 1)
        outs.append(M.all_to_all_hp2sp(o.contiguous(), group))  # [L/P, H, d]
    return torch.stack(outs, 0).reshape(B, Ll, H * d)
