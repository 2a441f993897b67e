"""Named wall-clock / device timers with min-max reporting across ranks
(the Megatron timers the reference logs at loongforge/train/training_utils.py:2062-2087,2406-2426)."""
from __future__ import annotations

import time
from typing import Dict, List, Optional

import torch
import torch.distributed as dist


class _Timer:
    def __init__(self, name: str, device_sync: bool):
        self.name, self.device_sync = name, device_sync
        self.elapsed_, self.count, self._t0, self.started = 0.0, 0, 0.0, False

    def start(self, barrier: bool = False):
        assert not self.started, f"timer {self.name} already started"
        if barrier and dist.is_initialized():
            dist.barrier()
        if self.device_sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self._t0 = time.perf_counter()
        self.started = True

    def stop(self, barrier: bool = False):
        assert self.started, f"timer {self.name} not started"
        if barrier and dist.is_initialized():
            dist.barrier()
        if self.device_sync and torch.cuda.is_available():
            torch.cuda.synchronize()
        self.elapsed_ += time.perf_counter() - self._t0
        self.count += 1
        self.started = False

    def elapsed(self, reset: bool = True) -> float:
        was = self.started
        if was:
            self.stop()
        e = self.elapsed_
        if reset:
            self.elapsed_, self.count = 0.0, 0
        if was:
            self.start()
        return e


class Timers:
    """``timers('name', log_level=1).start()`` ... ``.stop()``; levels above `log_level` are no-ops."""

    def __init__(self, log_level: int = 2, device_sync: bool = False):
        self.log_level, self.device_sync = log_level, device_sync
        self.timers: Dict[str, _Timer] = {}
        self._noop = _Noop()

    def __call__(self, name: str, log_level: int = 0):
        if log_level > self.log_level:
            return self._noop
        if name not in self.timers:
            self.timers[name] = _Timer(name, self.device_sync)
        return self.timers[name]

    def report(self, names: Optional[List[str]] = None, normalizer: float = 1.0, reset: bool = True) -> str:
        names = names or sorted(self.timers)
        vals = torch.tensor([self.timers[n].elapsed(reset) * 1e3 / normalizer if n in self.timers else 0.0
                             for n in names], dtype=torch.float64)
        mn, mx = vals.clone(), vals.clone()
        if dist.is_initialized() and dist.get_world_size() > 1:
            if dist.get_backend() != "gloo":  # NCCL reduces device tensors
                mn, mx = mn.cuda(), mx.cuda()
            dist.all_reduce(mn, op=dist.ReduceOp.MIN)
            dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        return "(min, max) time across ranks (ms):" + "".join(
            f"\n    {n.ljust(40, '.')}: ({a:.2f}, {b:.2f})" for n, a, b in zip(names, mn.tolist(), mx.tolist()))


class _Noop:
    def start(self, *a, **k): pass
    def stop(self, *a, **k): pass
    def elapsed(self, *a, **k): return 0.0
