"""Optimizer-state CPU offload: fp32 master weights and Adam moments in pinned host memory, updated by a native
multi-threaded host kernel (``ops/csrc_cpu/cpu_adam.cpp``) — the counterpart of the DeepSpeed CPU-Adam path the
reference documents for optimizer offload (docs/source/features/optimizer_support.md:54-60).

Per step and parameter bucket: gradients are copied device -> host on a side stream, the host update runs, and the
refreshed bf16 weights are copied back. Buckets are pipelined so that bucket i+1's gradient copy overlaps bucket i's
host update. On a CPU-only machine the same code runs without the copies."""
from __future__ import annotations

import os
from typing import Iterable, List, Optional

import torch

_EXT = None


def _load_ext():
    global _EXT
    if _EXT is None:
        from torch.utils import cpp_extension

        here = os.path.dirname(os.path.abspath(__file__))
        src = os.path.join(here, "..", "ops", "csrc_cpu", "cpu_adam.cpp")
        build = os.path.join(here, "..", "ops", "_build_cpu")
        os.makedirs(build, exist_ok=True)
        _EXT = cpp_extension.load(name="lfb200_cpu", sources=[os.path.abspath(src)], build_directory=os.path.abspath(build),
                                  extra_cflags=["-O3"], verbose=False)
    return _EXT


def build() -> None:
    _load_ext()


class CPUOffloadAdam:
    def __init__(self, params: Iterable[torch.nn.Parameter], lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8,
                 weight_decay: float = 0.0, bucket_elems: int = 1 << 24):
        self.params: List[torch.nn.Parameter] = [p for p in params if p.requires_grad]
        self.lr, self.betas, self.eps, self.wd = lr, betas, eps, weight_decay
        self.step_count = 0
        self.ext = _load_ext()
        pin = torch.cuda.is_available()
        self.state = []
        for p in self.params:
            n = p.numel()
            st = {"master": torch.empty(n, dtype=torch.float32, pin_memory=pin),
                  "m": torch.zeros(n, dtype=torch.float32, pin_memory=pin),
                  "v": torch.zeros(n, dtype=torch.float32, pin_memory=pin),
                  "grad": torch.empty(n, dtype=torch.float32 if p.dtype == torch.float32 else torch.bfloat16, pin_memory=pin),
                  "out": torch.empty(n, dtype=torch.bfloat16, pin_memory=pin) if p.dtype == torch.bfloat16 else None}
            st["master"].copy_(p.detach().reshape(-1).float())
            self.state.append(st)
        self.copy_stream = torch.cuda.Stream() if torch.cuda.is_available() else None

    def zero_grad(self, set_to_none: bool = True):
        for p in self.params:
            p.grad = None

    @torch.no_grad()
    def step(self, grad_scale: float = 1.0):
        self.step_count += 1
        events: List[Optional[torch.cuda.Event]] = []
        # stage 1: queue every gradient copy (device -> pinned host) on the side stream
        for p, st in zip(self.params, self.state):
            g = p.grad if p.grad is not None else torch.zeros_like(p)
            if p.is_cuda:
                self.copy_stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(self.copy_stream):
                    st["grad"].copy_(g.reshape(-1).to(st["grad"].dtype), non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(self.copy_stream)
                events.append(ev)
            else:
                st["grad"].copy_(g.reshape(-1).to(st["grad"].dtype))
                events.append(None)
        # stage 2: host update of tensor i as soon as ITS gradient arrived; copy the result back asynchronously
        for p, st, ev in zip(self.params, self.state, events):
            if ev is not None:
                ev.synchronize()
            self.ext.cpu_adam_step(st["master"], st["grad"], st["m"], st["v"], st["out"], self.lr, self.betas[0],
                                   self.betas[1], self.eps, self.wd if p.dim() > 1 else 0.0, self.step_count, grad_scale)
            src = st["out"] if st["out"] is not None else st["master"]
            if p.is_cuda:
                with torch.cuda.stream(self.copy_stream):
                    p.reshape(-1).copy_(src, non_blocking=True)
            else:
                p.reshape(-1).copy_(src.to(p.dtype))
        if self.copy_stream is not None:
            torch.cuda.current_stream().wait_stream(self.copy_stream)

    def state_dict(self):
        return {"step": self.step_count, "state": [{k: v for k, v in st.items() if k in ("master", "m", "v")}
                                                   for st in self.state]}

    def load_state_dict(self, sd):
        self.step_count = sd["step"]
        for st, src in zip(self.state, sd["state"]):
            for k in ("master", "m", "v"):
                st[k].copy_(src[k])
