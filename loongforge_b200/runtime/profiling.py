"""Tracing and inspection hooks of the training loop: scheduled torch profiler, NVTX ranges, CUDA memory history with
an out-of-memory snapshot, periodic "detail" iterations, and tensor-inspector hooks that log statistics of chosen
modules' outputs / gradients (reference: loongforge/train/training_utils.py:247-273,325-342,486-494,2604-2662,
2741-2746; flags ``--profile``, ``--profile-step-start/end``, ``--profile-ranks``, ``--enable-log-tensor``)."""
from __future__ import annotations

import contextlib
import fnmatch
import json
import os
from typing import Callable, Dict, List, Optional

import torch
import torch.nn as nn


class StepProfiler:
    """torch.profiler with a wait / warmup / active schedule between two steps on selected ranks; writes Chrome traces."""

    def __init__(self, out_dir: str, step_start: int, step_end: int, ranks: Optional[List[int]] = None, rank: int = 0,
                 record_shapes: bool = True, with_stack: bool = False, profile_memory: bool = True):
        self.enabled = ranks is None or rank in ranks
        self.out_dir, self.rank = out_dir, rank
        self.start, self.end = step_start, step_end
        self.prof = None
        self.kw = dict(record_shapes=record_shapes, with_stack=with_stack, profile_memory=profile_memory)
        self.trace_path: Optional[str] = None

    def step(self, iteration: int) -> None:
        if not self.enabled:
            return
        from torch.profiler import ProfilerActivity, profile, schedule

        if iteration == self.start and self.prof is None:
            acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if torch.cuda.is_available() else [])
            active = max(self.end - self.start - 1, 1)
            self.prof = profile(activities=acts, schedule=schedule(wait=0, warmup=1, active=active, repeat=1), **self.kw)
            self.prof.__enter__()
        elif self.prof is not None:
            self.prof.step()
            if iteration >= self.end:
                self.prof.__exit__(None, None, None)
                os.makedirs(self.out_dir, exist_ok=True)
                self.trace_path = os.path.join(self.out_dir, f"trace_rank{self.rank}_it{self.start}-{self.end}.json")
                self.prof.export_chrome_trace(self.trace_path)
                self.prof = None
                self.enabled = False


@contextlib.contextmanager
def nvtx_range(name: str):
    """NVTX range on GPUs (visible to Nsight tools); plain pass-through on CPU."""
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class MemoryHistory:
    """Records CUDA allocator history and dumps a snapshot periodically and when an allocation fails."""

    def __init__(self, out_dir: str, rank: int = 0, max_entries: int = 100000):
        self.out_dir, self.rank, self.on = out_dir, rank, False
        if torch.cuda.is_available():
            torch.cuda.memory._record_memory_history(max_entries=max_entries)
            self.on = True
            if hasattr(torch._C, "_cuda_attach_out_of_memory_observer"):
                torch._C._cuda_attach_out_of_memory_observer(lambda *a: self.dump("oom"))

    def dump(self, tag: str) -> Optional[str]:
        if not self.on:
            return None
        os.makedirs(self.out_dir, exist_ok=True)
        path = os.path.join(self.out_dir, f"memory_rank{self.rank}_{tag}.pickle")
        torch.cuda.memory._dump_snapshot(path)
        return path


def detail_iteration(iteration: int, interval: Optional[int]) -> bool:
    """Timers synchronise the device only on one iteration out of `interval` (the "detail log" iteration)."""
    return bool(interval) and iteration % interval == 0


class TensorInspector:
    """Forward / backward hooks on modules whose qualified name matches a glob; every `interval` calls the statistics
    (mean, abs-max, L2 norm, NaN / Inf counts) of their outputs and output gradients are appended to a JSONL file."""

    def __init__(self, model: nn.Module, patterns: List[str], out_path: str, interval: int = 1, rank: int = 0,
                 backward: bool = True):
        self.out_path, self.interval, self.rank = out_path, interval, rank
        self.iteration = 0
        self.handles = []
        self.records: List[dict] = []
        for name, mod in model.named_modules():
            # wrappers (DDP, pipeline chunks) prefix the qualified name: a pattern also matches as a suffix
            if name and any(fnmatch.fnmatch(name, p) or fnmatch.fnmatch(name, "*." + p) for p in patterns):
                self.handles.append(mod.register_forward_hook(self._hook(name, "fwd")))
                if backward:
                    self.handles.append(mod.register_full_backward_hook(self._bhook(name)))

    @staticmethod
    def stats(t: torch.Tensor) -> Dict[str, float]:
        f = t.detach().float()
        return {"mean": float(f.mean()), "absmax": float(f.abs().max()), "norm": float(f.norm()),
                "nan": int(torch.isnan(f).sum()), "inf": int(torch.isinf(f).sum()), "shape": list(t.shape)}

    def _log(self, name, kind, t):
        if self.iteration % self.interval == 0 and torch.is_tensor(t) and t.numel():
            self.records.append({"iteration": self.iteration, "rank": self.rank, "module": name, "kind": kind,
                                 **self.stats(t)})

    def _hook(self, name, kind):
        def fn(mod, inp, out):
            self._log(name, kind, out[0] if isinstance(out, tuple) else out)
        return fn

    def _bhook(self, name):
        def fn(mod, gin, gout):
            self._log(name, "bwd", gout[0])
        return fn

    def step(self) -> None:
        if self.records:
            os.makedirs(os.path.dirname(self.out_path) or ".", exist_ok=True)
            with open(self.out_path, "a") as f:
                for r in self.records:
                    f.write(json.dumps(r) + "\n")
            self.records.clear()
        self.iteration += 1

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
