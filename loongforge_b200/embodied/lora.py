"""LoRA injection for the embodied policies, applied before the model is wrapped (reference:
loongforge/embodied/train/lora.py): every ``nn.Linear`` whose attribute name is in `targets` gets a frozen base and a
trainable low-rank update ``y = W x + (alpha / r) * B(A x)``."""
from __future__ import annotations

import math
from typing import Dict, List

import torch
import torch.nn as nn


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, rank: int, alpha: float):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        self.lora_a = nn.Linear(base.in_features, rank, bias=False, dtype=base.weight.dtype, device=base.weight.device)
        self.lora_b = nn.Linear(rank, base.out_features, bias=False, dtype=base.weight.dtype, device=base.weight.device)
        nn.init.kaiming_uniform_(self.lora_a.weight, a=math.sqrt(5))
        nn.init.zeros_(self.lora_b.weight)
        self.scale = alpha / rank

    def forward(self, x):
        return self.base(x) + self.scale * self.lora_b(self.lora_a(x))

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight + self.scale * (self.lora_b.weight @ self.lora_a.weight)


def inject_lora(model: nn.Module, rank: int, alpha: float, targets: List[str]) -> Dict:
    """Returns adapter metadata (stored in checkpoints). Non-adapter parameters are frozen."""
    for p in model.parameters():
        p.requires_grad_(False)
    wrapped = []
    for parent_name, parent in list(model.named_modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, nn.Linear) and child_name in targets:
                setattr(parent, child_name, LoRALinear(child, rank, alpha))
                wrapped.append(f"{parent_name}.{child_name}".lstrip("."))
    return {"rank": rank, "alpha": alpha, "targets": targets, "modules": wrapped}
