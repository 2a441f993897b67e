"""Training with fully-sharded data parallelism (``--use-torch-fsdp2`` / ``--use-megatron-fsdp`` of the reference,
loongforge/train/training_utils.py:926-941): the same step loop, data path, schedules, log line and scheduler as
:class:`~loongforge_b200.runtime.trainer.Trainer`, with the model wrapped by FSDP2 units instead of the flat-buffer
DDP wrapper, and an AdamW over the sharded (DTensor) parameters instead of the bucket-sharded optimizer.

Scope: data parallelism only (tensor / pipeline / expert parallel sizes 1), which is how the reference uses FSDP2
(its FSDP path wraps the whole GPT model over the data-parallel group). Checkpoints are torch distributed checkpoints
of the sharded model and optimizer state dicts under the usual ``iter_XXXXXXX`` directory with the same tracker file.
"""
from __future__ import annotations

import contextlib
import math
import os
from typing import List

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel import fsdp as F
from .trainer import Trainer


class _FSDPChunk(nn.Module):
    """Presents an FSDP2-wrapped model with the small surface the step loop uses on a model chunk."""

    def __init__(self, module: nn.Module):
        super().__init__()
        self.module = module
        self.is_last_microbatch = True

    def forward(self, *a, **kw):
        return self.module(*a, **kw)

    @contextlib.contextmanager
    def no_sync(self):
        # gradient reduce-scatter only on the last micro-batch; until then unsharded gradients accumulate
        self.module.set_requires_gradient_sync(False)
        try:
            yield
        finally:
            self.module.set_requires_gradient_sync(True)

    def broadcast_params(self):
        pass  # every rank initialises from the same seed and FSDP shards from rank-identical full tensors

    def zero_grad_buffer(self):
        self.module.zero_grad(set_to_none=True)

    def finish_grad_sync(self):
        pass


class _ShardedAdamW:
    """AdamW over DTensor shards with the (ok, grad_norm, num_zeros) step contract of the distributed optimizer."""

    def __init__(self, chunks: List[_FSDPChunk], tcfg):
        decay, no_decay = [], []
        for c in chunks:
            for n, p in c.module.named_parameters():
                if p.requires_grad:
                    (no_decay if (p.dim() == 1 or n.endswith(".bias")) else decay).append(p)
        self.params = decay + no_decay
        self.clip = tcfg.clip_grad
        self.opt = torch.optim.AdamW(
            [{"params": decay, "weight_decay": tcfg.weight_decay}, {"params": no_decay, "weight_decay": 0.0}],
            lr=tcfg.lr, betas=(tcfg.adam_beta1, tcfg.adam_beta2), eps=tcfg.adam_eps)
        self._wd = tcfg.weight_decay
        # the scheduler drives group 0; `step` mirrors it into the real groups
        self.param_groups = [{"lr": tcfg.lr, "weight_decay": tcfg.weight_decay}]
        self.post_sync_hooks: List = []
        self.sharded = True
        self.chunks = chunks

    def zero_grad(self):
        self.opt.zero_grad(set_to_none=True)

    def grad_norm(self) -> float:
        total = None
        for p in self.params:
            if p.grad is None:
                continue
            g = p.grad.to_local() if hasattr(p.grad, "to_local") else p.grad
            s = g.float().pow(2).sum()
            total = s if total is None else total + s
        if total is None:
            return 0.0
        if dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(total)  # shards are disjoint over the data-parallel ranks
        return float(total.sqrt())

    def step(self):
        for hook in self.post_sync_hooks:
            hook()
        norm = self.grad_norm()
        if not math.isfinite(norm):
            return False, norm, None
        if self.clip and self.clip > 0:
            c = min(1.0, self.clip / (norm + 1e-6))
            if c < 1.0:
                for p in self.params:
                    if p.grad is not None:
                        p.grad.mul_(c)
        lr, wd = self.param_groups[0]["lr"], self.param_groups[0]["weight_decay"]
        self.opt.param_groups[0].update(lr=lr, weight_decay=wd)
        self.opt.param_groups[1].update(lr=lr)
        self.opt.step()
        return True, norm, None

    def reload_model_params(self):
        pass

    def state_dict(self):
        return {"param_groups": self.param_groups}

    def load_state_dict(self, sd):
        self.param_groups = sd["param_groups"]


class FSDPMixin:
    """Overrides of model / optimizer construction and checkpointing; combine with a Trainer class."""

    def __init__(self, model_cfg, train_cfg, dims=None, **kw):
        if dims is not None and (dims.tp > 1 or dims.pp > 1 or dims.ep > 1 or dims.cp > 1):
            raise ValueError("the FSDP trainer shards over data parallelism only (tp = pp = ep = cp = 1)")
        model_cfg.gradient_accumulation_fusion = False  # FSDP owns param.grad; nothing accumulates into main_grad
        strategy = getattr(train_cfg, "fsdp_sharding_strategy", None)
        # "optim" / "no_shard" are ZeRO-1 / DDP settings of the non-FSDP path; under FSDP the default is full sharding
        self.sharding_strategy = strategy if strategy in ("optim_grads_params", "optim_grads") else "optim_grads_params"
        super().__init__(model_cfg, train_cfg, dims, **kw)

    def _build_models(self):
        module = self.model_provider(True, True, list(range(self.mcfg.num_layers)))
        if dist.is_initialized():
            F.wrap_fsdp2(module, self.st.group("dp_cp"), strategy=self.sharding_strategy,
                         param_dtype=torch.bfloat16 if self.tcfg.bf16 and self.mcfg.params_dtype != torch.bfloat16 else None)
        return [_FSDPChunk(module)]

    def _build_optimizer(self):
        return _ShardedAdamW(self.models, self.tcfg)

    # ------------------------------------------------------------------ checkpoints
    def _dcp_state(self):
        from torch.distributed.checkpoint.state_dict import get_model_state_dict, get_optimizer_state_dict

        m = self.models[0].module
        return {"model": get_model_state_dict(m), "optim": get_optimizer_state_dict(m, self.optimizer.opt)}

    def save_checkpoint(self, path: str):
        import torch.distributed.checkpoint as dcp

        from ..ckpt import checkpointing as C

        d = C.iteration_dir(path, self.iteration)
        os.makedirs(d, exist_ok=True)
        dcp.save(self._dcp_state(), checkpoint_id=d)
        if (not dist.is_initialized()) or dist.get_rank() == 0:
            torch.save({"iteration": self.iteration, "consumed_samples": self.consumed_samples,
                        "num_floating_point_operations_so_far": self.num_flops_so_far,
                        "optimizer": self.optimizer.state_dict(),
                        "opt_param_scheduler": self.scheduler.state_dict(), "format": "fsdp_dcp"},
                       os.path.join(d, "common.pt"))
            C.write_tracker(path, self.iteration)
        if dist.is_initialized():
            dist.barrier()

    def load_checkpoint(self, path: str, **kw):
        import torch.distributed.checkpoint as dcp
        from torch.distributed.checkpoint.state_dict import set_model_state_dict, set_optimizer_state_dict

        from ..ckpt import checkpointing as C

        it, release = C.read_tracker(path)
        if it is None:
            return 0
        d = C.iteration_dir(path, it, release)
        state = self._dcp_state()
        dcp.load(state, checkpoint_id=d)
        m = self.models[0].module
        set_model_state_dict(m, state["model"])
        set_optimizer_state_dict(m, self.optimizer.opt, state["optim"])
        common = torch.load(os.path.join(d, "common.pt"), weights_only=False)
        self.optimizer.load_state_dict(common["optimizer"])
        self.scheduler.load_state_dict(common["opt_param_scheduler"])
        self.iteration = common["iteration"]
        self.consumed_samples = common.get("consumed_samples", 0)
        self.num_flops_so_far = common.get("num_floating_point_operations_so_far", 0.0)
        return self.iteration


class FSDPTrainer(FSDPMixin, Trainer):
    pass


def fsdp_variant(trainer_cls):
    """The FSDP flavour of any Trainer subclass (SFT, ...)."""
    if issubclass(trainer_cls, FSDPMixin):
        return trainer_cls
    return type("FSDP" + trainer_cls.__name__, (FSDPMixin, trainer_cls), {})
