"""Distributed training of the diffusion transformers (WAN image/text-to-video, Qwen-Image) on the common training
loop: data parallelism through the flat-buffer DDP wrapper and the distributed optimizer, Ulysses sequence parallelism
over the context-parallel group for long token sequences, checkpoints, log line, hooks
(reference: loongforge/train/diffusion/pretrain_wan.py:65-546, pretrain_qwen_image.py; model names in
loongforge/utils/config_map.py:373-390).

One micro-batch holds VAE latents ``[B, C, F, H, W]`` (``[B, C, H, W]`` for Qwen-Image), text-encoder states
``[B, Lt, D]`` and optionally CLIP image tokens. Per micro-batch: draw timestep ids and noise (one generator per
data-parallel rank, shared by the ranks of a sequence-parallel group so that they see the same noisy sample), mix along
the rectified-flow path, predict the velocity, weighted MSE.
"""
from __future__ import annotations

import glob
import os
from typing import Dict, Iterator, Optional, Sequence

import torch

from ..models.config import TransformerConfig
from ..models.diffusion import DiTConfig, FlowMatchScheduler, QwenImageModel, WanModel
from ..parallel.state import ParallelDims
from .trainer import Trainer

DIT_PRESETS: Dict[str, dict] = {
    # name: (kind, DiTConfig fields); sizes follow the public model cards
    "tiny-wan": dict(kind="wan", hidden_size=64, num_heads=4, num_layers=2, ffn_hidden_size=128, in_channels=4,
                     out_channels=4, text_dim=32, freq_dim=32),
    "tiny-qwen-image": dict(kind="qwen_image", hidden_size=64, num_heads=4, num_layers=2, ffn_hidden_size=128,
                            in_channels=4, out_channels=4, text_dim=32, freq_dim=32),
    "wan2-1-t2v-1.3b": dict(kind="wan", hidden_size=1536, num_heads=12, num_layers=30, ffn_hidden_size=8960,
                            in_channels=16, out_channels=16, text_dim=4096, freq_dim=256),
    "wan2-1-i2v": dict(kind="wan", hidden_size=5120, num_heads=40, num_layers=40, ffn_hidden_size=13824, in_channels=36,
                       out_channels=16, text_dim=4096, freq_dim=256, image_context_dim=1280),
    "wan2-2-i2v": dict(kind="wan", hidden_size=5120, num_heads=40, num_layers=40, ffn_hidden_size=13824, in_channels=36,
                       out_channels=16, text_dim=4096, freq_dim=256),
    "qwen-image-edit-2511": dict(kind="qwen_image", hidden_size=3072, num_heads=24, num_layers=60, ffn_hidden_size=12288,
                                 in_channels=16, out_channels=16, text_dim=3584, freq_dim=256),  # 16 latent channels, 2 x 2 packed
}


def dit_config(name: str, **overrides):
    """(kind, DiTConfig) of a preset name (``-`` and ``_`` are interchangeable)."""
    key = name.lower().replace("_", "-")
    if key not in DIT_PRESETS:
        raise KeyError(f"unknown diffusion model {name!r}; known: {sorted(DIT_PRESETS)}")
    fields = dict(DIT_PRESETS[key])
    kind = fields.pop("kind")
    fields.update(overrides)
    return kind, DiTConfig(**fields)


def is_diffusion_model(name: Optional[str]) -> bool:
    return bool(name) and name.lower().replace("_", "-") in DIT_PRESETS


def synthetic_latent_iterator(kind: str, cfg: DiTConfig, micro_batch_size: int, *, frames: int = 4, height: int = 16,
                              width: int = 16, text_len: int = 16, dp_rank: int = 0, dp_size: int = 1, seed: int = 0,
                              start_sample: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Random latents / text states of the model's shapes; sample i of the global stream goes to rank
    ``(i // micro_batch_size) % dp_size`` so that the union over ranks does not depend on the layout."""
    step = 0
    while True:
        items = []
        for j in range(micro_batch_size):
            idx = start_sample + (step * dp_size + dp_rank) * micro_batch_size + j
            g = torch.Generator().manual_seed(seed * 1000003 + idx)
            lat = (torch.randn(cfg.out_channels, frames, height, width, generator=g) if kind == "wan"
                   else torch.randn(cfg.in_channels, height, width, generator=g))  # packed 2 x 2 by the trainer
            it = {"latents": lat, "text": torch.randn(text_len, cfg.text_dim, generator=g)}
            if kind == "wan" and cfg.in_channels > cfg.out_channels:
                it["condition"] = torch.randn(cfg.in_channels - cfg.out_channels, frames, height, width, generator=g)
            if cfg.image_context_dim is not None:
                it["image_context"] = torch.randn(8, cfg.image_context_dim, generator=g)
            items.append(it)
        yield {k: torch.stack([it[k] for it in items]) for k in items[0]}
        step += 1


def latent_file_iterator(paths: Sequence[str], micro_batch_size: int, *, dp_rank: int = 0, dp_size: int = 1,
                         start_sample: int = 0) -> Iterator[Dict[str, torch.Tensor]]:
    """Precomputed samples: every ``*.pt`` under the given directories is a dict with ``latents``, ``text`` and
    optionally ``condition`` / ``image_context`` (what an offline VAE + text-encoder pass writes)."""
    files = sorted(f for p in paths for f in (glob.glob(os.path.join(p, "*.pt")) if os.path.isdir(p) else [p]))
    if not files:
        raise ValueError(f"no .pt latent samples under {list(paths)}")
    step = 0
    while True:
        items = []
        for j in range(micro_batch_size):
            idx = start_sample + (step * dp_size + dp_rank) * micro_batch_size + j
            items.append(torch.load(files[idx % len(files)], map_location="cpu", weights_only=True))
        same = all(it["latents"].shape == items[0]["latents"].shape and it["text"].shape == items[0]["text"].shape
                   for it in items)
        # equal shapes: one batched tensor per field; different shapes: lists, which the trainer packs into one token row
        yield {k: (torch.stack([it[k] for it in items]) if same else [it[k] for it in items]) for k in items[0]}
        step += 1


class DiffusionTrainer(Trainer):
    def __init__(self, dit_cfg: DiTConfig, train_cfg, dims: Optional[ParallelDims] = None, *, kind: str = "wan",
                 shift: float = 3.0, num_train_timesteps: int = 1000, recompute: bool = False, **kw):
        dims = dims or ParallelDims()
        if dims.tp > 1 or dims.pp > 1 or dims.ep > 1:
            raise ValueError("diffusion models train with data parallelism and Ulysses sequence parallelism "
                             "(--context-parallel-size); tensor / pipeline / expert parallel sizes must be 1")
        self.dit_cfg, self.kind, self.recompute = dit_cfg, kind, recompute
        if train_cfg.bf16:
            dit_cfg.params_dtype = torch.bfloat16
        self.sched = FlowMatchScheduler(num_train_timesteps, shift)
        # the common loop reads a few sizes from a transformer config
        stand_in = TransformerConfig(num_layers=dit_cfg.num_layers, hidden_size=dit_cfg.hidden_size,
                                     num_attention_heads=dit_cfg.num_heads, ffn_hidden_size=dit_cfg.ffn_hidden_size,
                                     vocab_size=1, model_family=kind)
        super().__init__(stand_in, train_cfg, dims, **kw)
        # one noise stream per data-parallel rank; the ranks of a sequence-parallel group share it
        self.gen = torch.Generator().manual_seed(train_cfg.seed * 7919 + self.st.dp_rank)

    def _default_model_provider(self, pre_process, post_process, layer_numbers):
        model = (WanModel if self.kind == "wan" else QwenImageModel)(self.dit_cfg, device=self.device)
        if hasattr(model, "recompute"):
            model.recompute = self.recompute
        return model

    def build_data_iterator(self, args=None):
        st, t = self.st, self.tcfg
        kw = dict(dp_rank=st.dp_rank, dp_size=st.dp_size, start_sample=self.consumed_samples)
        paths = getattr(args, "data_path", None) if args is not None else None
        if paths:
            return latent_file_iterator(paths, t.micro_batch_size, **kw)
        return synthetic_latent_iterator(self.kind, self.dit_cfg, t.micro_batch_size, seed=t.seed, **kw)

    def _default_forward_step(self, data_iterator, model):
        b = self.get_batch(data_iterator)
        st, sched = self.st, self.sched
        cp = st.dims.cp
        nmb = self.mb_calc.num_microbatches
        dt = self.dit_cfg.params_dtype
        if isinstance(b["latents"], (list, tuple)):
            return self._packed_forward_step(b, model, nmb)
        x0 = b["latents"].to(dt)
        B = x0.shape[0]
        ids = sched.sample_timestep_ids(B, self.gen).to(x0.device)
        noise = torch.randn(x0.shape, generator=self.gen).to(x0.device, dt)
        if self.kind == "wan":
            xt = sched.add_noise(x0, noise, ids)
            if "condition" in b:  # image-to-video: conditioning latents ride along as extra input channels
                xt = torch.cat([xt, b["condition"].to(dt)], dim=1)
            t = sched.timesteps.to(x0.device)[ids]
            pred = model(xt, t, b["text"].to(dt), image_context=b.get("image_context"),
                         ulysses_group=st.group("cp") if cp > 1 else None)
            per_sample = sched.loss(pred, x0, noise, ids)
        else:
            from .diffusion import QwenImageTrainer
            p0, grid = QwenImageTrainer.pack_latents(x0)
            pn, _ = QwenImageTrainer.pack_latents(noise)
            xt = sched.add_noise(p0, pn, ids)
            pred = model(xt, sched.sigmas.to(x0.device)[ids], b["text"].to(dt), grid)
            per_sample = sched.loss(pred, p0, pn, ids)

        def loss_func(loss):
            # under Ulysses every rank of the group computes the same loss from the gathered prediction and holds
            # partial parameter gradients; gradients are AVERAGED over dp x cp, hence the factor cp
            return loss * (float(cp) / nmb), {"loss": loss.detach()}

        return per_sample, loss_func

    def _packed_forward_step(self, b, model, nmb):
        """Samples of different sizes (variable resolution / length): packed into one token row by the model
        (``WanModel.forward_packed``) instead of being padded to a common shape."""
        if self.kind != "wan" or self.st.dims.cp > 1:
            raise NotImplementedError("packed variable-size samples are supported for WAN without sequence parallelism")
        sched, dt, dev = self.sched, self.dit_cfg.params_dtype, self.device
        x0 = [x.to(dev, dt) for x in b["latents"]]
        n = len(x0)
        ids = sched.sample_timestep_ids(n, self.gen).to(dev)
        noise = [torch.randn(x.shape, generator=self.gen).to(dev, dt) for x in x0]
        xt = [sched.add_noise(x[None], z[None], ids[i:i + 1])[0] for i, (x, z) in enumerate(zip(x0, noise))]
        if "condition" in b:
            xt = [torch.cat([x, c.to(dev, dt)], dim=0) for x, c in zip(xt, b["condition"])]
        img = [c.to(dev, dt) for c in b["image_context"]] if "image_context" in b else None
        module = model.module if hasattr(model, "module") else model
        pred = module.forward_packed(xt, sched.timesteps.to(dev)[ids], [c.to(dev, dt) for c in b["text"]], img)
        loss = sum(sched.loss(p[None], x[None], z[None], ids[i:i + 1])
                   for i, (p, x, z) in enumerate(zip(pred, x0, noise))) / n

        def loss_func(l):
            return l / nmb, {"loss": l.detach()}

        return loss, loss_func

    def flops_per_step(self) -> float:
        n_params = sum(p.numel() for m in self.models for p in m.module.parameters())
        return 6.0 * n_params * self.tcfg.seq_length * self.mb_calc.current_gbs


def build_diffusion_trainer(name: str, train_cfg, dims=None, **kw) -> DiffusionTrainer:
    overrides = kw.pop("dit_overrides", {}) or {}
    kind, cfg = dit_config(name, **overrides)
    return DiffusionTrainer(cfg, train_cfg, dims, kind=kind, **kw)
