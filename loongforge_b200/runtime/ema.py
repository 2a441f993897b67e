"""Exponential moving average of the model weights, kept in fp32, updated after every optimizer step and saved
beside regular checkpoints (reference: loongforge/train/training_utils.py:237-244,1209-1217,2831-2835; EMA
checkpoints under ``save_ema`` :576-585)."""
from __future__ import annotations

import contextlib
import os
from typing import Dict, Iterable, Tuple

import torch
import torch.nn as nn


class ModelEMA:
    def __init__(self, named_params: Iterable[Tuple[str, nn.Parameter]], decay: float = 0.9999, warmup: bool = True):
        self.decay, self.warmup, self.updates = decay, warmup, 0
        self.params = [(n, p) for n, p in named_params if p.requires_grad]
        self.shadow: Dict[str, torch.Tensor] = {n: p.detach().float().clone() for n, p in self.params}

    def current_decay(self) -> float:
        # ramps from 0 so that early averages are not dominated by the random initialisation
        return min(self.decay, (1 + self.updates) / (10 + self.updates)) if self.warmup else self.decay

    @torch.no_grad()
    def update(self) -> None:
        d = self.current_decay()
        self.updates += 1
        for n, p in self.params:
            self.shadow[n].lerp_(p.detach().float(), 1.0 - d)

    @contextlib.contextmanager
    def swapped_in(self):
        """Evaluate / export with the averaged weights; the live weights are restored afterwards."""
        keep = {n: p.detach().clone() for n, p in self.params}
        try:
            with torch.no_grad():
                for n, p in self.params:
                    p.copy_(self.shadow[n].to(p.dtype))
            yield
        finally:
            with torch.no_grad():
                for n, p in self.params:
                    p.copy_(keep[n])

    def state_dict(self) -> dict:
        return {"shadow": self.shadow, "updates": self.updates, "decay": self.decay}

    def load_state_dict(self, sd: dict) -> None:
        self.updates, self.decay = sd["updates"], sd["decay"]
        for n, t in sd["shadow"].items():
            self.shadow[n].copy_(t)

    def save(self, root: str, iteration: int, rank_suffix: str = "") -> str:
        d = os.path.join(root, "save_ema", f"iter_{iteration:07d}")
        os.makedirs(d, exist_ok=True)
        path = os.path.join(d, f"ema{rank_suffix}.pt")
        torch.save(self.state_dict(), path)
        return path
