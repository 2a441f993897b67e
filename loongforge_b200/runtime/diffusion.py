"""Diffusion trainers: WAN image/text-to-video flow matching and Qwen-Image (reference:
loongforge/train/diffusion/pretrain_wan.py:65-546, pretrain_qwen_image.py).

A batch holds VAE latents ``[B, C, F, H, W]``, text-encoder states ``[B, Lt, D]`` and optionally CLIP image tokens.
Per step: sample timestep ids, mix latents and noise along the rectified-flow path, predict the velocity, weighted
MSE. ``ulysses_group`` shards the token sequence for long videos."""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn

from ..models.diffusion import FlowMatchScheduler, QwenImageModel, WanModel


class WanFlowMatchTrainer:
    def __init__(self, model: WanModel, optimizer: torch.optim.Optimizer, *, shift: float = 3.0,
                 num_train_timesteps: int = 1000, ulysses_group=None, clip_grad: float = 1.0, seed: int = 0):
        self.model, self.opt, self.group, self.clip = model, optimizer, ulysses_group, clip_grad
        self.sched = FlowMatchScheduler(num_train_timesteps, shift)
        self.gen = torch.Generator().manual_seed(seed)

    def loss(self, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        x0 = batch["latents"]
        ids = self.sched.sample_timestep_ids(x0.shape[0], self.gen).to(x0.device)
        noise = torch.randn(x0.shape, generator=self.gen).to(x0.device, x0.dtype)
        xt = self.sched.add_noise(x0, noise, ids)
        t = self.sched.timesteps.to(x0.device)[ids]
        pred = self.model(xt, t, batch["text"], image_context=batch.get("image_context"), ulysses_group=self.group)
        return self.sched.loss(pred, x0, noise, ids)

    def train_step(self, batch: Dict[str, torch.Tensor]) -> Dict[str, float]:
        self.opt.zero_grad(set_to_none=True)
        loss = self.loss(batch)
        loss.backward()
        norm = float(nn.utils.clip_grad_norm_(self.model.parameters(), self.clip)) if self.clip else 0.0
        self.opt.step()
        return {"loss": float(loss.detach()), "grad_norm": norm}

    @torch.no_grad()
    def sample(self, shape, text, steps: int = 20, image_context=None, generator=None) -> torch.Tensor:
        """Euler sampler over `steps` evenly spaced timestep ids from pure noise."""
        x = torch.randn(shape, generator=generator).to(text.device, text.dtype)
        ids = torch.linspace(0, self.sched.n - 1, steps + 1).long()
        sig = self.sched.sigmas.to(x.device)
        for a, b in zip(ids[:-1], ids[1:]):
            t = self.sched.timesteps.to(x.device)[a].expand(shape[0])
            v = self.model(x, t, text, image_context=image_context)
            x = x + v * (sig[b] - sig[a])
        return x


class QwenImageTrainer:
    """Same objective on 2x2-packed image latents with the double-stream MMDiT."""

    def __init__(self, model: QwenImageModel, optimizer, *, shift: float = 3.0, seed: int = 0):
        self.model, self.opt = model, optimizer
        self.sched = FlowMatchScheduler(1000, shift)
        self.gen = torch.Generator().manual_seed(seed)

    @staticmethod
    def pack_latents(lat: torch.Tensor):
        """[B, C, H, W] -> ([B, H/2 * W/2, 4C], (H/2, W/2))."""
        B, C, H, W = lat.shape
        x = lat.view(B, C, H // 2, 2, W // 2, 2).permute(0, 2, 4, 1, 3, 5).reshape(B, (H // 2) * (W // 2), C * 4)
        return x, (H // 2, W // 2)

    def loss(self, batch):
        x0, grid = self.pack_latents(batch["latents"])
        ids = self.sched.sample_timestep_ids(x0.shape[0], self.gen).to(x0.device)
        noise = torch.randn(x0.shape, generator=self.gen).to(x0.device, x0.dtype)
        xt = self.sched.add_noise(x0, noise, ids)
        pred = self.model(xt, self.sched.sigmas.to(x0.device)[ids], batch["text"], grid)
        return self.sched.loss(pred, x0, noise, ids)

    def train_step(self, batch):
        self.opt.zero_grad(set_to_none=True)
        loss = self.loss(batch)
        loss.backward()
        self.opt.step()
        return {"loss": float(loss.detach())}
