"""Learning-rate / weight-decay schedules: constant, linear, cosine, inverse-square-root, WSD,
with linear warm-up (Megatron's ``OptimizerParamScheduler``, built by the reference at
loongforge/train/training_utils.py:1073-1084)."""
from __future__ import annotations

import math
from typing import Optional


class OptimizerParamScheduler:
    def __init__(self, optimizer, *, max_lr: float, min_lr: float = 0.0, warmup_steps: int = 0,
                 decay_steps: int = 1, decay_style: str = "cosine", init_lr: float = 0.0,
                 start_wd: Optional[float] = None, end_wd: Optional[float] = None, wd_incr_steps: int = 0,
                 wd_incr_style: str = "constant", wsd_decay_steps: Optional[int] = None,
                 lr_wsd_decay_style: str = "exponential"):
        self.optimizer = optimizer
        self.max_lr, self.min_lr, self.init_lr = max_lr, min_lr, init_lr
        self.warmup_steps, self.decay_steps, self.decay_style = warmup_steps, max(decay_steps, 1), decay_style
        self.start_wd, self.end_wd = start_wd, end_wd
        self.wd_incr_steps, self.wd_incr_style = wd_incr_steps, wd_incr_style
        self.wsd_decay_steps, self.lr_wsd_decay_style = wsd_decay_steps, lr_wsd_decay_style
        self.num_steps = 0
        self.step(0)

    def get_lr(self, steps: Optional[int] = None) -> float:
        n = self.num_steps if steps is None else steps
        if self.warmup_steps > 0 and n <= self.warmup_steps:
            return self.init_lr + (self.max_lr - self.init_lr) * n / self.warmup_steps
        if self.decay_style == "constant":
            return self.max_lr
        if n > self.decay_steps:
            return self.min_lr
        if self.decay_style == "inverse-square-root":
            w = max(self.warmup_steps, 1)
            return max(self.min_lr, self.max_lr * math.sqrt(w) / math.sqrt(max(n, 1)))
        ratio = (n - self.warmup_steps) / max(self.decay_steps - self.warmup_steps, 1)
        delta = self.max_lr - self.min_lr
        if self.decay_style == "linear":
            coeff = 1.0 - ratio
        elif self.decay_style == "cosine":
            coeff = 0.5 * (math.cos(math.pi * ratio) + 1.0)
        elif self.decay_style == "WSD":
            anneal_start = self.decay_steps - (self.wsd_decay_steps or 0)
            if n <= anneal_start:
                coeff = 1.0
            else:
                r = (n - anneal_start) / max(self.wsd_decay_steps or 1, 1)
                if self.lr_wsd_decay_style == "linear":
                    coeff = 1.0 - r
                elif self.lr_wsd_decay_style == "cosine":
                    coeff = 0.5 * (math.cos(math.pi * r) + 1.0)
                else:
                    coeff = 2.0 * math.pow(0.5, r) - 1.0
        else:
            raise ValueError(f"unknown lr decay style {self.decay_style}")
        return self.min_lr + coeff * delta

    def get_wd(self) -> Optional[float]:
        if self.start_wd is None or self.end_wd is None:
            return None
        if self.num_steps > self.wd_incr_steps or self.wd_incr_style == "constant":
            return self.end_wd
        r = self.num_steps / max(self.wd_incr_steps, 1)
        coeff = r if self.wd_incr_style == "linear" else 0.5 * (math.cos(math.pi * (1 - r)) + 1.0)
        return self.start_wd + coeff * (self.end_wd - self.start_wd)

    def step(self, increment: int = 1) -> None:
        self.num_steps += increment
        lr, wd = self.get_lr(), self.get_wd()
        for g in self.optimizer.param_groups:
            g["lr"] = lr * g.get("lr_mult", 1.0)
            if wd is not None:
                g["weight_decay"] = wd * g.get("wd_mult", 1.0)

    def state_dict(self):
        return {"num_steps": self.num_steps, "max_lr": self.max_lr, "min_lr": self.min_lr,
                "warmup_steps": self.warmup_steps, "decay_steps": self.decay_steps, "decay_style": self.decay_style}

    def load_state_dict(self, sd):
        self.num_steps = 0
        self.step(sd["num_steps"])
