"""LoRA for the embodied policies, applied before the model is wrapped: every selected ``nn.Linear`` gets a frozen base
and a trainable low-rank update ``y = W x + s * B(A(dropout(x)))`` with ``s = alpha / r`` (``alpha / sqrt(r)`` with
rank-stabilised scaling).

* selection: attribute names (``q``, ``o``), glob patterns over qualified names (``policy.decoder.expert.*.qkv``),
  ``all-linear``, or — when no targets are given — what the policy declares in ``default_lora_targets()``; ``exclude``
  patterns remove matches (heads that must stay exact);
* ``modules_to_save``: modules that are trained in full next to the adapters (new heads, embodiment projectors);
* adapter files: ``adapter_model.pt`` (adapter and fully-trained tensors only) + ``adapter_config.json``; loading re-creates
  the injection from the config, so a served policy needs the base weights and the adapter directory;
* ``merge_lora`` folds every update into its base linear for export.

(reference: loongforge/embodied/train/lora.py:30-259)
"""
from __future__ import annotations

import fnmatch
import json
import math
import os
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn as nn

ADAPTER_WEIGHTS, ADAPTER_CONFIG = "adapter_model.pt", "adapter_config.json"


class LoRALinear(nn.Module):
    def __init__(self, base: nn.Linear, rank: int, alpha: float, dropout: float = 0.0, use_rslora: bool = False,
                 init: str = "kaiming"):
        super().__init__()
        self.base = base
        for p in base.parameters():
            p.requires_grad_(False)
        kw = dict(bias=False, dtype=base.weight.dtype, device=base.weight.device)
        self.lora_a = nn.Linear(base.in_features, rank, **kw)
        self.lora_b = nn.Linear(rank, base.out_features, **kw)
        if init == "gaussian":
            nn.init.normal_(self.lora_a.weight, std=1.0 / rank)
        elif init == "kaiming":
            nn.init.kaiming_uniform_(self.lora_a.weight, a=math.sqrt(5))
        else:
            raise ValueError(f"unknown LoRA initialisation {init!r} (kaiming | gaussian)")
        nn.init.zeros_(self.lora_b.weight)  # the update starts at zero: the wrapped model equals the base model
        self.scale = alpha / math.sqrt(rank) if use_rslora else alpha / rank
        self.dropout = nn.Dropout(dropout) if dropout > 0 else nn.Identity()

    @property
    def in_features(self):
        return self.base.in_features

    @property
    def out_features(self):
        return self.base.out_features

    @property
    def weight(self):
        return self.base.weight

    @property
    def bias(self):
        return self.base.bias

    def forward(self, x):
        return self.base(x) + self.scale * self.lora_b(self.lora_a(self.dropout(x)))

    def merged_weight(self) -> torch.Tensor:
        return self.base.weight + self.scale * (self.lora_b.weight @ self.lora_a.weight)


def _matches(name: str, attr: str, patterns: Iterable[str]) -> bool:
    return any(p == attr or fnmatch.fnmatch(name, p) for p in patterns)


def resolve_targets(model: nn.Module, targets: Optional[List[str]]) -> List[str]:
    """Explicit targets, or the policy's own declaration (searched through wrappers), or the attention projections."""
    if targets:
        return list(targets)
    for m in model.modules():
        f = getattr(m, "default_lora_targets", None)
        if callable(f):
            return list(f())
    return ["q", "k", "v", "o"]


def inject_lora(model: nn.Module, rank: int, alpha: float, targets: Optional[List[str]] = None, *, dropout: float = 0.0,
                use_rslora: bool = False, init: str = "kaiming", exclude: Iterable[str] = (),
                modules_to_save: Iterable[str] = ()) -> Dict:
    """Freezes everything, wraps the selected linears, un-freezes ``modules_to_save``. Returns the adapter configuration
    (stored in checkpoints and in ``adapter_config.json``)."""
    targets = resolve_targets(model, targets)
    exclude, modules_to_save = list(exclude), list(modules_to_save)
    for p in model.parameters():
        p.requires_grad_(False)
    wrapped = []
    for parent_name, parent in list(model.named_modules()):
        if isinstance(parent, LoRALinear):
            continue
        for child_name, child in list(parent.named_children()):
            full = f"{parent_name}.{child_name}".lstrip(".")
            if not isinstance(child, nn.Linear) or _matches(full, child_name, exclude):
                continue
            if "all-linear" in targets or _matches(full, child_name, targets):
                setattr(parent, child_name, LoRALinear(child, rank, alpha, dropout, use_rslora, init))
                wrapped.append(full)
    saved = []
    for name, mod in model.named_modules():
        if name and _matches(name, name.rsplit(".", 1)[-1], modules_to_save):
            for p in mod.parameters():
                p.requires_grad_(True)
            saved.append(name)
    if not wrapped:
        raise ValueError(f"no linear layer matches the LoRA targets {targets}")
    return {"rank": rank, "alpha": alpha, "targets": targets, "dropout": dropout, "use_rslora": use_rslora, "init": init,
            "exclude": exclude, "modules_to_save": modules_to_save, "modules": wrapped, "saved_modules": saved}


def adapter_state_dict(model: nn.Module) -> Dict[str, torch.Tensor]:
    """Adapter matrices and every other trainable tensor (``modules_to_save``); frozen base weights are left out."""
    trainable = {n for n, p in model.named_parameters() if p.requires_grad}
    return {n: t.detach().cpu() for n, t in model.state_dict().items() if n in trainable or ".lora_a." in n or ".lora_b." in n}


def save_adapter(model: nn.Module, output_dir: str, meta: Dict, extra: Optional[Dict] = None) -> str:
    os.makedirs(output_dir, exist_ok=True)
    torch.save(adapter_state_dict(model), os.path.join(output_dir, ADAPTER_WEIGHTS))
    with open(os.path.join(output_dir, ADAPTER_CONFIG), "w") as f:
        json.dump({**meta, **(extra or {})}, f, indent=1)
    return output_dir


def load_adapter(model: nn.Module, adapter_dir: str, trainable: bool = False) -> Dict:
    """Injects adapters as the stored configuration says (unless the model already has them) and loads their weights."""
    with open(os.path.join(adapter_dir, ADAPTER_CONFIG)) as f:
        meta = json.load(f)
    if not any(isinstance(m, LoRALinear) for m in model.modules()):
        inject_lora(model, meta["rank"], meta["alpha"], meta["targets"], dropout=meta.get("dropout", 0.0),
                    use_rslora=meta.get("use_rslora", False), init=meta.get("init", "kaiming"),
                    exclude=meta.get("exclude", ()), modules_to_save=meta.get("modules_to_save", ()))
    sd = torch.load(os.path.join(adapter_dir, ADAPTER_WEIGHTS), map_location="cpu", weights_only=True)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if unexpected:
        raise KeyError(f"adapter tensors without a place in the model: {unexpected[:5]}")
    lost = [k for k in missing if ".lora_a." in k or ".lora_b." in k]
    if lost:
        raise KeyError(f"adapter file lacks {lost[:5]}")
    if not trainable:
        for p in model.parameters():
            p.requires_grad_(False)
    return meta


def merge_lora(model: nn.Module) -> int:
    """Replaces every ``LoRALinear`` by a plain linear holding ``W + s B A``; returns how many were merged."""
    n = 0
    for parent in list(model.modules()):
        for child_name, child in list(parent.named_children()):
            if isinstance(child, LoRALinear):
                base = child.base
                with torch.no_grad():
                    base.weight.copy_(child.merged_weight())
                setattr(parent, child_name, base)
                n += 1
    return n
