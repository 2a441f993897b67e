"""Trainer template of the embodied stack: ``train -> _setup -> _training_loop -> _train_step`` with gradient
accumulation under no-sync contexts, NaN cleaning, clipping, manual garbage collection, checkpoint / RNG / data-loader
resume hooks, and a name -> trainer registry (reference: loongforge/embodied/train/trainers/base_trainer.py:45-808,
supervised/finetune_trainer.py, trainer_builder.py)."""
from __future__ import annotations

import gc
import os
from typing import Callable, Dict, Optional

import torch
import torch.nn as nn

from . import checkpoint as ckpt
from .config import EmbodiedArgs, set_global_args
from .cuda_graph import MicrobatchGraphRunner
from .data import ResumableLoader, build_dataset
from .distributed import DistContext, apply_activation_checkpointing, grad_sync_context, wrap_model
from .logging import MetricLogger, StageTimers
from .models import build_policy
from .optimizer import LRScheduler, build_optimizer, clip_gradients


def load_pretrained(model: nn.Module, path: str, strict: bool = False) -> Dict[str, object]:
    """Weights from a ``.pt`` / ``.pth`` state dict (optionally under a ``model`` key), a ``.safetensors`` file, or every such
    file of a directory; names are matched with and without the adapter's ``policy.`` prefix."""
    files = [path] if os.path.isfile(path) else sorted(
        os.path.join(path, f) for f in os.listdir(path) if f.endswith((".pt", ".pth", ".safetensors", ".bin")))
    if not files:
        raise FileNotFoundError(f"no weight file under {path}")
    sd: Dict[str, torch.Tensor] = {}
    for f in files:
        if f.endswith(".safetensors"):
            from safetensors.torch import load_file
            part = load_file(f)
        else:
            part = torch.load(f, map_location="cpu", weights_only=False)
            part = part.get("model", part) if isinstance(part, dict) else part
        sd.update(part)
    own = model.state_dict()
    fixed = {}
    for k, v in sd.items():
        for cand in (k, f"policy.{k}", k[len("policy."):] if k.startswith("policy.") else None):
            if cand in own and tuple(own[cand].shape) == tuple(v.shape):
                fixed[cand] = v
                break
    missing, unexpected = model.load_state_dict(fixed, strict=False)
    extra = [k for k in sd if k not in fixed and f"policy.{k}" not in fixed and k[len("policy."):] not in fixed]
    if strict and (missing or extra):
        raise KeyError(f"pretrained weights do not cover the model: missing {missing[:5]}, unexpected {extra[:5]}")
    return {"loaded": len(fixed), "missing": list(missing), "unexpected": extra}


def freeze_modules(model: nn.Module, patterns) -> list:
    """Sub-modules whose dotted path equals or matches (glob) a pattern stop training; a pattern that matches nothing is an
    error (a typo would silently train what was meant to stay fixed)."""
    import fnmatch
    frozen = []
    for pat in patterns:
        hits = [n for n, _ in model.named_modules() if n and (n == pat or fnmatch.fnmatch(n, pat) or n == f"policy.{pat}")]
        if not hits:
            raise KeyError(f"freeze_modules: nothing matches {pat!r}")
        for n in hits:
            for p in model.get_submodule(n).parameters():
                p.requires_grad_(False)
        frozen += hits
    return frozen


class BaseTrainer:
    def __init__(self, args: EmbodiedArgs, ctx: Optional[DistContext] = None):
        self.args = args
        self.ctx = ctx or DistContext().init()
        set_global_args(args)
        self.step = 0

    # ---- hooks subclasses override
    def build_model(self) -> nn.Module:
        raise NotImplementedError

    def compute_loss(self, model: nn.Module, batch: Dict[str, torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    # ---- template
    def _setup(self):
        a, ctx = self.args, self.ctx
        torch.manual_seed(a.seed)  # identical initial weights on every rank
        if a.deterministic_mode:
            torch.use_deterministic_algorithms(True, warn_only=True)
            torch.backends.cudnn.benchmark = False
        if a.disable_tf32:
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        model = self.build_model()
        if a.pretrained_checkpoint:
            report = load_pretrained(model, a.pretrained_checkpoint, a.pretrained_strict)
            if ctx.is_main:
                print(f" > loaded {report['loaded']} tensors from {a.pretrained_checkpoint} "
                      f"({len(report['missing'])} missing, {len(report['unexpected'])} unexpected)", flush=True)
        if a.lora_rank > 0:
            from .lora import inject_lora, load_adapter
            self.lora_meta = inject_lora(model, a.lora_rank, a.lora_alpha, a.lora_targets, dropout=a.lora_dropout,
                                         use_rslora=a.lora_use_rslora, init=a.lora_init, exclude=a.lora_exclude,
                                         modules_to_save=a.lora_modules_to_save)
            if a.lora_adapter_path:
                load_adapter(model, a.lora_adapter_path, trainable=True)
                for n, p in model.named_parameters():  # adapters and fully-trained modules train on, the base stays frozen
                    p.requires_grad_(".lora_a." in n or ".lora_b." in n or any(n.startswith(m + ".") for m in self.lora_meta["saved_modules"]))
        else:
            self.lora_meta = None
        if a.freeze_modules:
            self.frozen = freeze_modules(model, a.freeze_modules)
        if a.bf16:
            model = model.to(torch.bfloat16)
        if a.activation_checkpoint_patterns:
            apply_activation_checkpointing(model, a.activation_checkpoint_patterns)
        self.model = wrap_model(model, a, ctx)
        self.optimizer = build_optimizer(self.model, a, ctx.world)
        self.scheduler = LRScheduler(self.optimizer, a.lr_scheduler, a.lr, a.min_lr, a.warmup_steps,
                                     a.lr_decay_steps or a.train_steps, num_cycles=a.lr_num_cycles, power=a.lr_power)
        self.loader = ResumableLoader(build_dataset(a), a.per_device_batch_size, ctx.rank, ctx.world, a.seed, a.num_workers,
                                      sampler=a.sampler)
        self.logger = MetricLogger(a.output_dir, ctx.is_main, a.train_steps, tensorboard=a.tensorboard,
                                   wandb_project=a.wandb_project, run_name=a.run_name)
        self.timers = StageTimers(a.log_stage_times)
        self.logger.log_config(a)
        self.logger.log_param_stats(self.model)
        if self.lora_meta is not None:
            self.logger.note(f"LoRA rank {self.lora_meta['rank']} on {len(self.lora_meta['modules'])} linear layers"
                             + (f", fully trained: {self.lora_meta['saved_modules']}" if self.lora_meta["saved_modules"] else ""))
        self.graph_runner = (MicrobatchGraphRunner(self.model, self.compute_loss, a.cuda_graph_warmup_steps, a.cuda_graph_pad_length,
                                                   a.cuda_graph_max_graphs) if a.per_microbatch_cuda_graph else None)
        if a.resume:
            st = ckpt.load_checkpoint(a.output_dir, self.model, self.optimizer, self.scheduler, rank=ctx.rank)
            if st is None:
                self.logger.note(f"resume requested but no checkpoint under {a.output_dir}: starting from step 0")
            else:
                self.logger.note(f"resumed from step {st['step']}")
            if st is not None:
                self.step = st["step"]
                if st.get("dataloader"):
                    self.loader.load_state_dict(st["dataloader"])
        torch.manual_seed(a.seed + 1000 * ctx.rank + self.step)  # per-rank noise streams from here on

    def _to_device(self, batch):
        dev = self.ctx.device
        out = {k: v.to(dev, non_blocking=True) for k, v in batch.items()}
        if self.args.bf16:
            out = {k: (v.to(torch.bfloat16) if v.is_floating_point() else v) for k, v in out.items()}
        return out

    def _train_step(self, it) -> Dict[str, float]:
        a = self.args
        n = a.gradient_accumulation_steps
        total = 0.0
        parts: Dict[str, float] = {}
        for i in range(n):
            with self.timers("data"):
                batch = self._to_device(next(it))
            with self.timers("forward-backward"), grad_sync_context(self.model, sync=(i == n - 1)):
                if self.graph_runner is not None:
                    loss = self.graph_runner.run(batch, 1.0 / n)
                else:
                    loss = self.compute_loss(self.model, batch)
                    (loss / n).backward()
            total += float(loss.detach()) / n
            if a.check_for_nan_in_loss and not torch.isfinite(loss.detach()).all():
                raise FloatingPointError(f"loss is {float(loss.detach())} at step {self.step + 1} (micro-batch {i})")
            for k, v in self._loss_parts().items():  # what the policy reports beside the total (video / action loss ...)
                parts[k] = parts.get(k, 0.0) + float(v) / n
        with self.timers("optimizer"):
            norm = clip_gradients(self.model.parameters(), a.max_grad_norm, nan_clean=a.nan_clean,
                                  sharded=a.strategy in ("fsdp", "hsdp"))
            self.optimizer.step()
        if self.graph_runner is not None and self.graph_runner.graph is not None:
            for p in self.model.parameters():  # captured graphs accumulate into fixed .grad storage
                if p.grad is not None:
                    p.grad.zero_()
        else:
            self.optimizer.zero_grad(set_to_none=True)
        self.scheduler.step()
        return {"loss": total, **parts, "grad_norm": norm, "lr": self.optimizer.param_groups[0]["lr"]}

    def _loss_parts(self) -> Dict[str, torch.Tensor]:
        for m in self.model.modules():
            d = getattr(m, "last_losses", None)
            if isinstance(d, dict) and d:
                return d
        return {}

    def _training_loop(self):
        a = self.args
        it = iter(self.loader)
        prof = None
        while self.step < a.train_steps:
            if a.profile_step_start >= 0 and self.step == a.profile_step_start and self.ctx.is_main:
                acts = [torch.profiler.ProfilerActivity.CPU] + ([torch.profiler.ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
                prof = torch.profiler.profile(activities=acts, record_shapes=True)
                prof.__enter__()
            metrics = self._train_step(it)
            self.step += 1
            if prof is not None and self.step >= max(a.profile_step_end, a.profile_step_start + 1):
                prof.__exit__(None, None, None)
                os.makedirs(os.path.join(a.output_dir, "profile"), exist_ok=True)
                prof.export_chrome_trace(os.path.join(a.output_dir, "profile", f"trace_step{a.profile_step_start}_{self.step}.json"))
                prof = None
            if a.log_interval and self.step % a.log_interval == 0:
                self.logger.log(self.step, metrics, a.per_device_batch_size * a.gradient_accumulation_steps * self.ctx.world,
                                self.timers.summary(a.log_interval) if a.log_stage_times else None)
            if a.manual_gc_interval and self.step % a.manual_gc_interval == 0:
                gc.collect()
            if a.save_interval and self.step % a.save_interval == 0:
                self.save()
            self.last_metrics = metrics

    def save(self):
        ckpt.save_checkpoint(self.args.output_dir, self.step, self.model, self.optimizer if self.args.save_training_state else None,
                             self.scheduler, fmt=self.args.checkpoint_format, dataloader_state=self.loader.state_dict(),
                             lora_meta=self.lora_meta, rank=self.ctx.rank, world=self.ctx.world, async_save=self.args.async_save)
        if self.lora_meta is not None and self.ctx.is_main and self.args.strategy in ("ddp", "zero1"):
            from .lora import save_adapter
            save_adapter(ckpt._unwrap(self.model), os.path.join(self.args.output_dir, f"step_{self.step:08d}", "adapter"),
                         self.lora_meta, {"model_name": self.args.model_name, "step": self.step})

    def train(self):
        if self.args.manual_gc_interval:
            gc.disable()
        try:
            self._setup()
            self._training_loop()
        finally:
            ckpt.wait_async_saves()
            if hasattr(self, "logger"):
                self.logger.finish()
            if self.args.manual_gc_interval:
                gc.enable()
        return self.last_metrics if hasattr(self, "last_metrics") else {}


class FinetuneTrainer(BaseTrainer):
    """Supervised fine-tuning of a flow-matching policy on action chunks."""

    def build_model(self) -> nn.Module:
        return build_policy(self.args.model_name, self.args)

    def compute_loss(self, model, batch):
        return model(batch)


_TRAINERS: Dict[str, Callable[..., BaseTrainer]] = {}


def register_trainer(name: str):
    def deco(cls):
        _TRAINERS[name] = cls
        return cls
    return deco


for _n in ("pi05", "groot_n1_6", "groot_n1_7", "xvla", "lingbot_va", "fastwam", "dreamzero", "cosmos3"):
    _TRAINERS[_n] = FinetuneTrainer


def build_trainer(args: EmbodiedArgs, ctx: Optional[DistContext] = None) -> BaseTrainer:
    return _TRAINERS.get(args.model_name, FinetuneTrainer)(args, ctx)
