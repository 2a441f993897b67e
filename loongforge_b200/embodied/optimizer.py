"""Optimizer side of the embodied stack: parameter groups, ZeRO-1 wrapper that tolerates mixed dtypes, an fp32
master-weight adapter for bf16 models, LR schedules, gradient clipping with NaN cleaning (reference:
loongforge/embodied/optimizer/optimizer.py:37-378, lr_scheduler.py, clip_gradients.py:12-80)."""
from __future__ import annotations

import math
from typing import Dict, Iterable, List

import torch
import torch.distributed as dist
import torch.nn as nn


def build_param_groups(model: nn.Module, weight_decay: float, lr: float, lr_mults: Dict[str, float] = None) -> List[dict]:
    """Biases / norms / 1-D tensors without weight decay; optional per-prefix learning-rate multipliers."""
    groups: Dict[tuple, dict] = {}
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        wd = 0.0 if (p.dim() <= 1 or name.endswith(".bias")) else weight_decay
        mult = 1.0
        for prefix, m in (lr_mults or {}).items():
            if name.startswith(prefix):
                mult = m
        g = groups.setdefault((wd, mult), {"params": [], "weight_decay": wd, "lr": lr * mult, "lr_mult": mult})
        g["params"].append(p)
    return list(groups.values())


class FP32MasterAdapter(torch.optim.Optimizer):
    """Keeps an fp32 copy of every low-precision parameter, steps the inner optimizer on the copies and writes the
    result back, so that bf16 models train with fp32 update precision."""

    def __init__(self, params_groups: List[dict], inner_cls, **inner_kw):
        self.model_groups = params_groups
        self.masters: List[List[torch.Tensor]] = []
        master_groups = []
        for g in params_groups:
            ms = [p.detach().float().clone().requires_grad_(True) for p in g["params"]]
            self.masters.append(ms)
            master_groups.append({**{k: v for k, v in g.items() if k != "params"}, "params": ms})
        self.inner = inner_cls(master_groups, **inner_kw)
        self.param_groups = self.inner.param_groups
        self.defaults = self.inner.defaults
        self.state = self.inner.state

    @torch.no_grad()
    def step(self, closure=None):
        for g, ms in zip(self.model_groups, self.masters):
            for p, m in zip(g["params"], ms):
                m.grad = None if p.grad is None else p.grad.float()
        self.inner.step()
        for g, ms in zip(self.model_groups, self.masters):
            for p, m in zip(g["params"], ms):
                p.copy_(m)

    def zero_grad(self, set_to_none: bool = True):
        for g in self.model_groups:
            for p in g["params"]:
                p.grad = None

    def state_dict(self):
        return {"inner": self.inner.state_dict(), "masters": [[m.detach().cpu() for m in ms] for ms in self.masters]}

    def load_state_dict(self, sd):
        self.inner.load_state_dict(sd["inner"])
        for ms, src in zip(self.masters, sd["masters"]):
            for m, s in zip(ms, src):
                m.data.copy_(s)


def build_optimizer(model: nn.Module, args, world: int = 1):
    groups = build_param_groups(model, args.weight_decay, args.lr)
    kw = dict(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=1e-8)
    if args.strategy == "zero1" and world > 1:
        from torch.distributed.optim import ZeroRedundancyOptimizer

        # ZeRO partitions whole parameters; groups with different dtypes are handled by one instance per dtype
        opt = ZeroRedundancyOptimizer([p for g in groups for p in g["params"]], optimizer_class=torch.optim.AdamW,
                                      weight_decay=args.weight_decay, **kw)
        return opt
    if args.fp32_master_weights:
        return FP32MasterAdapter(groups, torch.optim.AdamW, **kw)
    return torch.optim.AdamW(groups, **kw)


class LRScheduler:
    """constant | linear | cosine | wsd (warmup - stable - decay), all with linear warm-up; per-group multipliers kept."""

    def __init__(self, optimizer, kind: str, max_lr: float, min_lr: float, warmup: int, total: int,
                 decay_fraction: float = 0.1):
        self.opt, self.kind, self.max_lr, self.min_lr = optimizer, kind, max_lr, min_lr
        self.warmup, self.total, self.decay_fraction = warmup, max(total, 1), decay_fraction
        self.step_count = 0
        self._apply()

    def lr_at(self, s: int) -> float:
        if self.warmup and s < self.warmup:
            return self.max_lr * (s + 1) / self.warmup
        if self.kind == "constant":
            return self.max_lr
        span = max(self.total - self.warmup, 1)
        frac = min(max((s - self.warmup) / span, 0.0), 1.0)
        if self.kind == "linear":
            return self.max_lr + (self.min_lr - self.max_lr) * frac
        if self.kind == "cosine":
            return self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * frac))
        if self.kind == "wsd":
            start = 1.0 - self.decay_fraction
            if frac < start:
                return self.max_lr
            return self.max_lr + (self.min_lr - self.max_lr) * (frac - start) / max(self.decay_fraction, 1e-12)
        raise ValueError(self.kind)

    def _apply(self):
        lr = self.lr_at(self.step_count)
        for g in self.opt.param_groups:
            g["lr"] = lr * g.get("lr_mult", 1.0)

    def step(self):
        self.step_count += 1
        self._apply()

    def state_dict(self):
        return {"step_count": self.step_count}

    def load_state_dict(self, sd):
        self.step_count = sd["step_count"]
        self._apply()


@torch.no_grad()
def clip_gradients(params: Iterable[torch.Tensor], max_norm: float, *, nan_clean: bool = True, group=None,
                   sharded: bool = False) -> float:
    """Global-norm clipping. With ``nan_clean`` non-finite gradient entries are zeroed first; with ``sharded``
    (FSDP) the squared norm is summed over the group."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return 0.0
    if nan_clean:
        for g in grads:
            torch.nan_to_num_(g, nan=0.0, posinf=0.0, neginf=0.0)
    locals_ = [(g.to_local() if hasattr(g, "to_local") else g) for g in grads]
    sq = torch.stack([g.float().pow(2).sum() for g in locals_]).sum()
    if sharded and dist.is_initialized():
        dist.all_reduce(sq, group=group)
    norm = float(sq.sqrt())
    if max_norm and max_norm > 0 and norm > max_norm:
        scale = max_norm / (norm + 1e-6)
        for g in locals_:
            g.mul_(scale)
    return norm
