"""Sparse upcycling: initialise a mixture-of-experts model from a dense checkpoint by copying the dense MLP into every
expert (optionally splitting the FFN width across finer experts) and starting the router from small noise
(reference: MoE upcycling path in loongforge/train/training_utils.py:1087-1134)."""
from __future__ import annotations

from typing import Dict

import torch


def upcycle_state_dict(dense: Dict[str, torch.Tensor], num_experts: int, *, granularity: int = 1, glu: bool = True,
                       router_std: float = 0.02, moe_layers=None, seed: int = 0) -> Dict[str, torch.Tensor]:
    """Keys follow the Megatron layout: ``...mlp.linear_fc1.weight`` -> ``...mlp.experts.linear_fc1.weight{e}``.

    ``granularity`` g > 1 splits the dense FFN width into g slices (each expert holds ffn/g columns); experts
    e, e+g, e+2g, ... share a slice, and FC2 is scaled by g so that routing top-g experts of distinct slices with
    uniform weights reproduces the dense output. `moe_layers`: set of layer indices to convert (default all)."""
    gen = torch.Generator().manual_seed(seed)
    out: Dict[str, torch.Tensor] = {}
    if num_experts % granularity:
        raise ValueError("num_experts must divide by the granularity")
    for k, v in dense.items():
        if ".mlp.linear_fc" not in k or ".experts." in k:
            out[k] = v
            continue
        layer = int(k.split("decoder.layers.")[1].split(".")[0]) if "decoder.layers." in k else -1
        if moe_layers is not None and layer not in moe_layers:
            out[k] = v
            continue
        prefix, tail = k.split(".mlp.")
        if tail == "linear_fc1.layer_norm_weight":
            out[f"{prefix}.pre_mlp_layernorm.weight"] = v
        elif tail == "linear_fc1.weight":
            hidden = v.shape[1]
            out[f"{prefix}.mlp.router.weight"] = torch.randn(num_experts, hidden, generator=gen) * router_std
            blocks = v.chunk(2, 0) if glu else (v,)
            for e in range(num_experts):
                s = e % granularity
                parts = [b.chunk(granularity, 0)[s] for b in blocks]
                out[f"{prefix}.mlp.experts.linear_fc1.weight{e}"] = torch.cat(parts, 0).clone()
        elif tail == "linear_fc2.weight":
            for e in range(num_experts):
                s = e % granularity
                out[f"{prefix}.mlp.experts.linear_fc2.weight{e}"] = (v.chunk(granularity, 1)[s] * granularity).clone()
        else:
            out[k] = v
    return out
