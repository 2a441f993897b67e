"""Stand-alone merge utilities of the converter (reference: tools/convert_checkpoint LoRA merge, VLM merge tools,
mcore/merge_megatron.py, merge_megatron_expert.py):

* ``merge_lora_state_dict`` folds ``lora_A / lora_B`` pairs (HF-PEFT naming or this framework's naming) into the base
  weights: ``W += (alpha / r) * B @ A``;
* ``merge_vlm_state_dicts`` joins separately converted language-model, vision-encoder and projector state dicts under
  the composed model's prefixes;
* ``merge_expert_shards`` joins expert-parallel shards of a Megatron state dict (local expert index -> global)."""
from __future__ import annotations

import re
from typing import Dict, List

import torch


def merge_lora_state_dict(base: Dict[str, torch.Tensor], lora: Dict[str, torch.Tensor], alpha: float, rank: int,
                          strict: bool = True) -> Dict[str, torch.Tensor]:
    out = dict(base)
    scale = alpha / rank
    pairs = {}
    for k in lora:
        m = re.match(r"(?:base_model\.model\.)?(.*)\.(lora_A|lora_a|lora_B|lora_b)(?:\.default)?\.weight$", k)
        if m:
            pairs.setdefault(m.group(1), {})[m.group(2).lower()] = lora[k]
    for name, ab in pairs.items():
        target = name + ".weight"
        if target not in out and name + ".base.weight" in out:
            target = name + ".base.weight"
        if target not in out:
            if strict:
                raise KeyError(f"LoRA adapter for {name} has no base weight")
            continue
        w = out[target]
        out[target] = (w.float() + scale * (ab["lora_b"].float() @ ab["lora_a"].float())).to(w.dtype)
    return out


def merge_vlm_state_dicts(language: Dict[str, torch.Tensor], vision: Dict[str, torch.Tensor],
                          projector: Dict[str, torch.Tensor], *, language_prefix: str = "foundation_model.",
                          vision_prefix: str = "encoder_model.image_encoder.",
                          projector_prefix: str = "encoder_model.image_projector.") -> Dict[str, torch.Tensor]:
    out = {}
    for prefix, sd in ((language_prefix, language), (vision_prefix, vision), (projector_prefix, projector)):
        for k, v in sd.items():
            key = prefix + k
            if key in out:
                raise KeyError(f"duplicate key {key}")
            out[key] = v
    return out


def merge_expert_shards(shards: List[Dict[str, torch.Tensor]]) -> Dict[str, torch.Tensor]:
    """shards[ep_rank] holds ``...experts.linear_fcX.weight{local}``; non-expert tensors must agree across shards."""
    ep = len(shards)
    out: Dict[str, torch.Tensor] = {}
    pat = re.compile(r"^(.*\.experts\.linear_fc[12]\.(?:weight|bias))(\d+)$")
    per_rank = {}
    for sd in shards:
        for k in sd:
            m = pat.match(k)
            if m:
                per_rank[m.group(1)] = max(per_rank.get(m.group(1), 0), int(m.group(2)) + 1)
    for r, sd in enumerate(shards):
        for k, v in sd.items():
            m = pat.match(k)
            if m:
                out[f"{m.group(1)}{r * per_rank[m.group(1)] + int(m.group(2))}"] = v
            elif k in out:
                if v.shape != out[k].shape or not torch.equal(v, out[k]):
                    raise ValueError(f"replicated tensor {k} differs between expert-parallel ranks")
            else:
                out[k] = v
    assert ep >= 1
    return out
