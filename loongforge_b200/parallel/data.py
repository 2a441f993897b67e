"""Batch distribution inside a tensor-parallel group: rank 0 of the group reads the data, the others receive it
(``tensor_parallel.broadcast_data`` in Megatron; the reference's VLM trainer broadcasts 7-11 fields plus a 2-bit
modality flag per micro-batch, loongforge/train/pretrain/pretrain_vlm.py:88-127)."""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.distributed as dist


def broadcast_data(keys: List[str], data: Optional[Dict[str, torch.Tensor]], dtype: torch.dtype, group, src_rank: int,
                   device=None) -> Dict[str, torch.Tensor]:
    """All `keys` share `dtype`. One broadcast of the shapes, one of the flattened values. Keys whose value is None
    on the source are returned as None everywhere."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return {k: (None if data[k] is None else data[k].to(dtype)) for k in keys}
    me = dist.get_rank()
    max_dim = 6
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu")
    sizes = torch.zeros(len(keys) * (max_dim + 1), dtype=torch.long, device=dev)
    if me == src_rank:
        for i, k in enumerate(keys):
            t = data[k]
            if t is None:
                sizes[i * (max_dim + 1)] = -1
                continue
            assert t.dim() <= max_dim
            sizes[i * (max_dim + 1)] = t.dim()
            for j, s in enumerate(t.shape):
                sizes[i * (max_dim + 1) + 1 + j] = s
    dist.broadcast(sizes, src_rank, group=group)
    sz = sizes.tolist()
    shapes = []
    for i in range(len(keys)):
        nd = sz[i * (max_dim + 1)]
        shapes.append(None if nd < 0 else sz[i * (max_dim + 1) + 1:i * (max_dim + 1) + 1 + nd])
    numels = [0 if s is None else int(torch.Size(s).numel()) for s in shapes]
    if me == src_rank:
        flat = torch.cat([data[k].reshape(-1).to(device=dev, dtype=dtype) for k, s in zip(keys, shapes) if s is not None]
                         or [torch.empty(0, dtype=dtype, device=dev)])
    else:
        flat = torch.empty(sum(numels), dtype=dtype, device=dev)
    dist.broadcast(flat, src_rank, group=group)
    out, off = {}, 0
    for k, s, n in zip(keys, shapes, numels):
        out[k] = None if s is None else flat[off:off + n].view(s)
        off += n
    return out


def broadcast_flags(flags: int, group, src_rank: int, device=None) -> int:
    """Small integer (e.g. the has-image / has-video bits of a micro-batch) from the source rank to the group."""
    if group is None or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return flags
    dev = device or (torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else "cpu")
    t = torch.tensor([flags], dtype=torch.long, device=dev)
    dist.broadcast(t, src_rank, group=group)
    return int(t.item())
