"""Fully-sharded data parallelism for the language model as an alternative to DDP + distributed optimizer
(``--use-torch-fsdp2`` of the reference, loongforge/train/training_utils.py:926-941; sharding strategies of
docs/source/get_started/optimization_guide.md:42-50).

Every transformer layer becomes one FSDP2 unit, the rest (embedding, final norm, output layer) forms the root unit (parameters, gradients and
optimizer state sharded over the data-parallel mesh; all-gather before use, reduce-scatter of gradients after).
FSDP manages ``param.grad`` itself, so the fused accumulation into ``main_grad`` is switched off for wrapped models.
Strategies: ``optim_grads_params`` (reshard after forward, ZeRO-3), ``optim_grads`` (keep parameters gathered between
forward and backward, ZeRO-2)."""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist
import torch.nn as nn


def wrap_fsdp2(model: nn.Module, dp_group=None, *, strategy: str = "optim_grads_params",
               param_dtype: Optional[torch.dtype] = None, reduce_dtype: Optional[torch.dtype] = torch.float32) -> nn.Module:
    from torch.distributed.device_mesh import DeviceMesh
    from torch.distributed.fsdp import MixedPrecisionPolicy, fully_shard

    if strategy not in ("optim_grads_params", "optim_grads"):
        raise ValueError(f"unsupported sharding strategy {strategy}")
    group = dp_group if dp_group is not None else dist.group.WORLD
    ranks = dist.get_process_group_ranks(group)
    dev_type = "cuda" if next(model.parameters()).is_cuda else "cpu"
    mesh = DeviceMesh.from_group(group, dev_type, mesh=ranks, mesh_dim_names=("dp",))
    kw = dict(mesh=mesh, reshard_after_forward=(strategy == "optim_grads_params"))
    if param_dtype is not None:
        kw["mp_policy"] = MixedPrecisionPolicy(param_dtype=param_dtype, reduce_dtype=reduce_dtype)
    cfg = getattr(model, "cfg", None)
    if cfg is not None:
        cfg.gradient_accumulation_fusion = False
    # The embedding and output weights are read directly (tied weights, fused linear + cross-entropy), not through
    # their modules' forward, so they stay in the ROOT unit, which is gathered for the whole forward / backward.
    decoder = getattr(model, "decoder", None)
    if decoder is not None:
        for layer in decoder.layers:
            fully_shard(layer, **kw)
    fully_shard(model, **kw)
    return model


def fsdp_state_dict(model: nn.Module) -> dict:
    """DTensor state dict (the ``fsdp_dtensor`` checkpoint format): every rank contributes its shards to torch DCP."""
    return {k: v for k, v in model.state_dict().items()}


def full_state_dict(model: nn.Module) -> dict:
    """Un-sharded tensors gathered on every rank (for export / comparison)."""
    out = {}
    for k, v in model.state_dict().items():
        out[k] = v.full_tensor() if hasattr(v, "full_tensor") else v
    return out
