"""Random-number state management for model parallelism: named generator states that can be forked around a region
(dropout inside tensor-parallel regions must differ across TP ranks, dropout outside must match), seeding rules, and
activation checkpointing that restores those states for the recomputation (the ``tensor_parallel.get_cuda_rng_tracker``,
``model_parallel_cuda_manual_seed`` and ``tensor_parallel.checkpoint`` API of Megatron that the reference calls,
e.g. loongforge/train/training_utils.py and the transformer blocks)."""
from __future__ import annotations

import contextlib
from typing import Dict

import torch

MODEL_PARALLEL_RNG = "model-parallel-rng"
DATA_PARALLEL_RNG = "data-parallel-rng"
EXPERT_PARALLEL_RNG = "expert-parallel-rng"


def _get_state(device_type: str):
    return torch.cuda.get_rng_state() if device_type == "cuda" else torch.get_rng_state()


def _set_state(device_type: str, state) -> None:
    if device_type == "cuda":
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


class RNGStatesTracker:
    """Named RNG states on the default device (CUDA when available, else CPU)."""

    def __init__(self):
        self.device_type = "cuda" if torch.cuda.is_available() else "cpu"
        self.states: Dict[str, torch.Tensor] = {}
        self.seeds = set()

    def reset(self):
        self.states.clear()
        self.seeds.clear()

    def get_states(self) -> Dict[str, torch.Tensor]:
        return {k: v.clone() for k, v in self.states.items()}

    def set_states(self, states: Dict[str, torch.Tensor]) -> None:
        self.states = {k: v.clone() for k, v in states.items()}

    def add(self, name: str, seed: int) -> None:
        if seed in self.seeds:
            raise ValueError(f"seed {seed} already present")
        if name in self.states:
            raise ValueError(f"rng state {name} already present")
        self.seeds.add(seed)
        keep = _get_state(self.device_type)
        (torch.cuda.manual_seed if self.device_type == "cuda" else torch.manual_seed)(seed)
        self.states[name] = _get_state(self.device_type)
        _set_state(self.device_type, keep)

    @contextlib.contextmanager
    def fork(self, name: str = MODEL_PARALLEL_RNG):
        """Run the body on the named state; the default state is untouched and the named state advances."""
        if name not in self.states:
            raise KeyError(f"rng state {name} was not added")
        keep = _get_state(self.device_type)
        _set_state(self.device_type, self.states[name])
        try:
            yield
        finally:
            self.states[name] = _get_state(self.device_type)
            _set_state(self.device_type, keep)


_TRACKER = RNGStatesTracker()


def get_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


get_cuda_rng_tracker = get_rng_tracker  # Megatron's name


def model_parallel_manual_seed(seed: int, tp_rank: int = 0, pp_rank: int = 0, ep_rank: int = 0) -> None:
    """Default state: ``seed + 100 * pp_rank`` — equal across the TP ranks of a stage (dropout on replicated
    activations). Model-parallel state: offset 2718 + tp_rank — different per TP rank (dropout on sharded activations).
    Expert state additionally depends on the expert-parallel rank."""
    base = seed + 100 * pp_rank
    _TRACKER.reset()
    torch.manual_seed(base)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(base)
    _TRACKER.add(DATA_PARALLEL_RNG, base + 1)
    _TRACKER.add(MODEL_PARALLEL_RNG, base + 2718 + tp_rank)
    _TRACKER.add(EXPERT_PARALLEL_RNG, base + 1024 + 100 * ep_rank + tp_rank)


model_parallel_cuda_manual_seed = model_parallel_manual_seed


class _CheckpointFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensors, *args):
        ctx.fn = fn
        ctx.default_state = _get_state(_TRACKER.device_type)
        ctx.tracker_states = _TRACKER.get_states()
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        ctx.others = [a for a in args if not torch.is_tensor(a)]
        with torch.no_grad():
            return fn(*args)

    @staticmethod
    def backward(ctx, *grads):
        tensors, others = list(ctx.saved_tensors), list(ctx.others)
        args = [(tensors.pop(0).detach().requires_grad_(True) if t else others.pop(0)) for t in ctx.is_tensor]
        for a in args:
            if torch.is_tensor(a) and not a.is_floating_point():
                a.requires_grad_(False)
        keep_default, keep_tracker = _get_state(_TRACKER.device_type), _TRACKER.get_states()
        _set_state(_TRACKER.device_type, ctx.default_state)
        _TRACKER.set_states(ctx.tracker_states)
        try:
            with torch.enable_grad():
                out = ctx.fn(*args)
        finally:
            _set_state(_TRACKER.device_type, keep_default)
            _TRACKER.set_states(keep_tracker)
        outs = out if isinstance(out, tuple) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if torch.is_tensor(a) and a.requires_grad else None for a in args)


def checkpoint(fn, *args):
    """Activation checkpointing that replays the forward with the SAME random streams (default and tracked)."""
    return _CheckpointFn.apply(fn, len(args), *args)
