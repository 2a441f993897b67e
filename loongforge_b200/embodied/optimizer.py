"""Optimizer side of the embodied stack: parameter groups, ZeRO-1 wrapper that tolerates mixed dtypes, an fp32
master-weight adapter for bf16 models, LR schedules, gradient clipping with NaN cleaning (reference:
loongforge/embodied/optimizer/optimizer.py:37-378, lr_scheduler.py, clip_gradients.py:12-80)."""
from __future__ import annotations

import math
from typing import Dict, Iterable, List, Optional

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


class ZeroAdamW(torch.optim.Optimizer):
    """ZeRO stage 1 with fp32 masters, written against plain collectives. Every parameter has ONE owner rank (greedy
    balancing by element count); the owner keeps the fp32 master and both Adam moments, applies decoupled AdamW to the
    master from the (already data-parallel-reduced) gradient, writes the result into the model parameter and the owners'
    updated parameters are broadcast, one flat buffer per owner and dtype. Memory per rank: masters + moments of 1 / world
    of the model. Works for mixed dtypes (bf16 weights next to fp32 scalars).

    The state is keyed by parameter NAME: ``local_state_dict()`` is this rank's shard, and
    ``load_local_state_dicts(shards)`` takes the shards of ANY earlier world size and keeps what this rank owns now, so a
    checkpoint survives a change of the number of ranks (reference: the ZeRO wrappers of
    loongforge/embodied/optimizer/optimizer.py:37-104,221-250 and the shard files of distributed/checkpoint.py)."""

    def __init__(self, groups: List[dict], names: Dict[int, str], lr: float, betas=(0.9, 0.95), eps: float = 1e-8,
                 weight_decay: float = 0.0, group=None):
        super().__init__(groups, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.names = names
        params = [p for g in self.param_groups for p in g["params"]]
        load = [0] * self.world
        self.owner: Dict[int, int] = {}
        for p in sorted(params, key=lambda q: -q.numel()):          # largest first onto the lightest rank
            r = min(range(self.world), key=lambda i: load[i])
            self.owner[id(p)] = r
            load[r] += p.numel()
        self._params = params
        for p in params:
            if self.owner[id(p)] == self.rank:
                self.state[p] = {"step": 0, "master": p.detach().float().clone(),
                                 "exp_avg": torch.zeros_like(p, dtype=torch.float32),
                                 "exp_avg_sq": torch.zeros_like(p, dtype=torch.float32)}

    def owned(self):
        return [p for p in self._params if self.owner[id(p)] == self.rank]

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if self.owner[id(p)] != self.rank or p.grad is None:
                    continue
                st = self.state[p]
                st["step"] += 1
                grad = p.grad.float()
                st["exp_avg"].mul_(b1).add_(grad, alpha=1 - b1)
                st["exp_avg_sq"].mul_(b2).addcmul_(grad, grad, value=1 - b2)
                bc1, bc2 = 1 - b1 ** st["step"], 1 - b2 ** st["step"]
                m = st["master"]
                m.mul_(1 - g["lr"] * g["weight_decay"])
                m.addcdiv_(st["exp_avg"], (st["exp_avg_sq"] / bc2).sqrt_().add_(g["eps"]), value=-g["lr"] / bc1)
                p.copy_(m)
        self._broadcast_params()

    def _broadcast_params(self):
        if self.world == 1:
            return
        from torch._utils import _flatten_dense_tensors, _unflatten_dense_tensors
        for r in range(self.world):
            by_dtype: Dict[torch.dtype, List[torch.Tensor]] = {}
            for p in self._params:
                if self.owner[id(p)] == r:
                    by_dtype.setdefault(p.dtype, []).append(p.data)
            src = dist.get_global_rank(self.group, r) if self.group is not None else r
            for ts in by_dtype.values():
                flat = _flatten_dense_tensors(ts)
                dist.broadcast(flat, src=src, group=self.group)
                if r != self.rank:
                    for t, u in zip(ts, _unflatten_dense_tensors(flat, ts)):
                        t.copy_(u)

    # -- name-keyed shard state
    def local_state_dict(self) -> dict:
        return {"world": self.world, "rank": self.rank,
                "state": {self.names[id(p)]: {k: (v.cpu() if torch.is_tensor(v) else v) for k, v in self.state[p].items()}
                          for p in self.owned()},
                "param_groups": [{k: v for k, v in g.items() if k != "params"} for g in self.param_groups]}

    def load_local_state_dicts(self, shards: List[dict]) -> None:
        merged: Dict[str, dict] = {}
        for sh in shards:
            merged.update(sh["state"])
        for p in self.owned():
            src = merged[self.names[id(p)]]
            st = self.state[p]
            st["step"] = int(src["step"])
            for k in ("master", "exp_avg", "exp_avg_sq"):
                st[k].copy_(src[k])
            p.data.copy_(st["master"])
        for g, sg in zip(self.param_groups, shards[0]["param_groups"]):
            g.update({k: v for k, v in sg.items() if k in ("lr", "betas", "eps", "weight_decay")})
        self._broadcast_params()

    def consolidated_state_dict(self, to: int = 0) -> Optional[dict]:
        """All shards merged on rank ``to`` (one file for export); None elsewhere."""
        local = self.local_state_dict()
        if self.world == 1:
            return local
        out = [None] * self.world if self.rank == to else None
        dist.gather_object(local, out, dst=dist.get_global_rank(self.group, to) if self.group is not None else to, group=self.group)
        if self.rank != to:
            return None
        merged = dict(out[0])
        merged["state"] = {k: v for sh in out for k, v in sh["state"].items()}
        return merged

    def state_dict(self):
        return self.local_state_dict()

    def load_state_dict(self, sd):
        self.load_local_state_dicts([sd])


def build_optimizer(model: nn.Module, args, world: int = 1):
    """``optimizer``: adamw (default) | adam | sgd | lion; ``strategy: zero1`` always uses the sharded AdamW; ``lr_mults``
    maps parameter-name prefixes to learning-rate multipliers (a slower backbone next to a fresh head)."""
    mults = dict(getattr(args, "lr_mults", None) or {})
    groups = build_param_groups(model, args.weight_decay, args.lr, {("module." + k if hasattr(model, "module") else k): v
                                                                     for k, v in mults.items()})
    eps = getattr(args, "adam_eps", 1e-8)
    kw = dict(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2), eps=eps)
    if args.strategy == "zero1":
        names = {id(p): n[len("module."):] if n.startswith("module.") else n for n, p in model.named_parameters()}
        return ZeroAdamW(groups, names, weight_decay=args.weight_decay, **kw)
    kind = getattr(args, "optimizer", "adamw")
    if kind == "adamw":
        cls, ckw = torch.optim.AdamW, kw
    elif kind == "adam":
        cls, ckw = torch.optim.Adam, kw
    elif kind == "sgd":
        cls, ckw = torch.optim.SGD, dict(lr=args.lr, momentum=args.adam_beta1)
    elif kind == "lion":
        cls, ckw = Lion, dict(lr=args.lr, betas=(args.adam_beta1, args.adam_beta2))
    else:
        raise ValueError(f"unknown optimizer {kind!r} (adamw | adam | sgd | lion)")
    if args.fp32_master_weights:
        return FP32MasterAdapter(groups, cls, **ckw)
    return cls(groups, **ckw)


class Lion(torch.optim.Optimizer):
    """Sign-of-interpolated-momentum update with decoupled weight decay: ``u = sign(b1 m + (1 - b1) g)``,
    ``p -= lr (u + wd p)``, ``m = b2 m + (1 - b2) g``."""

    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0):
        super().__init__(params, dict(lr=lr, betas=betas, weight_decay=weight_decay))

    @torch.no_grad()
    def step(self, closure=None):
        for g in self.param_groups:
            b1, b2 = g["betas"]
            for p in g["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p)
                m = st["exp_avg"]
                p.mul_(1 - g["lr"] * g["weight_decay"])
                p.add_(torch.sign(m * b1 + p.grad * (1 - b1)), alpha=-g["lr"])
                m.mul_(b2).add_(p.grad, alpha=1 - b2)


class LRScheduler:
    """constant | linear | cosine | cosine_restarts | polynomial | wsd (warmup - stable - decay), all with linear warm-up;
    per-group multipliers kept. ``total`` is the step at which the decay ends (the learning rate stays at ``min_lr`` after
    it); ``num_cycles`` cosine periods for ``cosine_restarts``; ``power`` for ``polynomial``."""

    def __init__(self, optimizer, kind: str, max_lr: float, min_lr: float, warmup: int, total: int,
                 decay_fraction: float = 0.1, num_cycles: int = 1, power: float = 1.0):
        self.opt, self.kind, self.max_lr, self.min_lr = optimizer, kind, max_lr, min_lr
        self.warmup, self.total, self.decay_fraction = warmup, max(total, 1), decay_fraction
        self.num_cycles, self.power = max(int(num_cycles), 1), power
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
        if self.kind == "cosine_restarts":
            if frac >= 1.0:
                return self.min_lr
            within = (frac * self.num_cycles) % 1.0
            return self.min_lr + 0.5 * (self.max_lr - self.min_lr) * (1 + math.cos(math.pi * within))
        if self.kind == "polynomial":
            return self.min_lr + (self.max_lr - self.min_lr) * (1 - frac) ** self.power
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
