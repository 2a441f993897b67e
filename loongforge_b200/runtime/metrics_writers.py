"""Scalar sinks and side logs of the training loop: JSONL scalars (always), TensorBoard and Weights & Biases when
their packages are importable, the progress log with cumulative TFLOP/s, the energy monitor (NVML), and the one-time
dump of the first model input (reference: loongforge/train/training_utils.py:1256-1291,2103-2202,2314-2324,2988-3146)."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional

import torch


class ScalarWriter:
    def __init__(self, out_dir: str, *, tensorboard: bool = True, wandb_project: Optional[str] = None, enabled: bool = True,
                 run_name: Optional[str] = None):
        self.enabled = enabled
        self.tb = self.wandb = None
        if not enabled:
            return
        os.makedirs(out_dir, exist_ok=True)
        self.path = os.path.join(out_dir, "scalars.jsonl")
        if tensorboard:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(out_dir)
            except Exception:  # noqa: BLE001 - the tensorboard package is optional
                self.tb = None
        if wandb_project:
            try:
                import wandb
                # no network is assumed: runs are written to disk unless WANDB_MODE says otherwise
                self.wandb = wandb.init(project=wandb_project, name=run_name, dir=out_dir,
                                        mode=os.environ.get("WANDB_MODE", "offline"))
            except Exception:  # noqa: BLE001
                self.wandb = None

    def add_scalars(self, scalars: Dict[str, float], step: int) -> None:
        if not self.enabled:
            return
        with open(self.path, "a") as f:
            f.write(json.dumps({"step": step, **{k: float(v) for k, v in scalars.items()}}) + "\n")
        if self.tb is not None:
            for k, v in scalars.items():
                self.tb.add_scalar(k, float(v), step)
        if self.wandb is not None:
            self.wandb.log({k: float(v) for k, v in scalars.items()}, step=step)

    def close(self) -> None:
        if self.tb is not None:
            self.tb.close()


class ProgressLog:
    """Appends job-level lines: start, every checkpoint (iteration, tokens so far, job and cumulative TFLOP/s/GPU)."""

    def __init__(self, out_dir: str, world_size: int):
        os.makedirs(out_dir, exist_ok=True)
        self.path, self.world = os.path.join(out_dir, "progress.txt"), world_size
        self.t0 = time.time()
        self.flops_at_start: Optional[float] = None

    def _write(self, msg: str) -> None:
        with open(self.path, "a") as f:
            f.write(f"{time.strftime('%Y-%m-%d %H:%M:%S')}\t{msg}\n")

    def start(self, flops_so_far: float, job_id: str = "") -> None:
        self.flops_at_start = flops_so_far
        self._write(f"Starting job\tjob_id={job_id}\tworld_size={self.world}")

    def checkpoint(self, iteration: int, tokens_so_far: int, flops_so_far: float) -> None:
        dt = max(time.time() - self.t0, 1e-9)
        job = (flops_so_far - (self.flops_at_start or 0.0)) / dt / 1e12 / self.world
        self._write(f"Saved checkpoint\titeration={iteration}\ttokens={tokens_so_far}\tjob_tflops_per_gpu={job:.1f}")


class EnergyMonitor:
    """Integrates NVML power over time (read-only queries); returns joules since the last lap. Without NVML: zeros."""

    def __init__(self, device_index: int = 0):
        self.h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
        except Exception:  # noqa: BLE001
            self.h = None
        self.t = time.time()
        self.joules = 0.0

    def sample(self) -> None:
        now = time.time()
        if self.h is not None:
            self.joules += self.nv.nvmlDeviceGetPowerUsage(self.h) / 1000.0 * (now - self.t)
        self.t = now

    def lap(self) -> float:
        self.sample()
        j, self.joules = self.joules, 0.0
        return j


def dump_first_batch(batch: Dict[str, torch.Tensor], detokenize=None, max_tokens: int = 256) -> str:
    """Readable one-time dump of the first model input: shapes, dtypes, head of the tokens (decoded when a tokenizer is
    given) with the loss-masked positions marked."""
    lines = []
    for k, v in batch.items():
        if torch.is_tensor(v):
            lines.append(f"{k}: shape={list(v.shape)} dtype={v.dtype}")
    if "tokens" in batch:
        toks = batch["tokens"].reshape(-1)[:max_tokens].tolist()
        mask = batch.get("loss_mask")
        mask = mask.reshape(-1)[:max_tokens].tolist() if mask is not None else [1] * len(toks)
        text = [(detokenize([t]) if detokenize else str(t)) for t in toks]
        lines.append("tokens: " + " ".join(f"[{s}]" if m else s for s, m in zip(text, mask)))
    return "\n".join(lines)
