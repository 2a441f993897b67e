"""Logging of the embodied trainer: the resolved configuration as a key / value block, the Megatron-style iteration line
plus ``metrics.jsonl``, optional TensorBoard and Weights & Biases writers, per-stage timers reduced to the slowest
rank, loss components reported by the policy, smoothed loss and loss-spike notes, memory and remaining-time estimates,
parameter statistics (reference: loongforge/embodied/train/utils/logging.py:29-648)."""
from __future__ import annotations

import collections
import contextlib
import dataclasses
import json
import os
import time
from typing import Dict, Iterable, Optional

import torch
import torch.distributed as dist


def format_block(title: str, items: dict) -> str:
    lines = [f"------------------------ {title} ------------------------"]
    for k in sorted(items, key=str.lower):
        lines.append(f"  {k} {'.' * max(1, 48 - len(k))} {items[k]}")
    lines.append(f"-------------------- end of {title} ---------------------")
    return "\n".join(lines)


def flatten_config(obj, prefix: str = "") -> dict:
    """Dataclasses and dicts, nested, to dotted keys."""
    items = ({f.name: getattr(obj, f.name) for f in dataclasses.fields(obj)} if dataclasses.is_dataclass(obj) else dict(obj))
    out = {}
    for k, v in items.items():
        key = f"{prefix}.{k}" if prefix else str(k)
        if (dataclasses.is_dataclass(v) and not isinstance(v, type)) or (isinstance(v, dict) and v):
            out.update(flatten_config(v, key))
        else:
            out[key] = v
    return out


class StageTimers:
    """``with timers("data"): ...`` accumulates wall time per stage (with a device synchronisation on each side when a GPU
    is in use, so that a stage owns the kernels it launched); ``summary`` reports, per stage, the time of the slowest rank."""

    def __init__(self, enabled: bool = True):
        self.enabled = enabled
        self.total: Dict[str, float] = collections.defaultdict(float)
        self.count: Dict[str, int] = collections.defaultdict(int)

    @contextlib.contextmanager
    def __call__(self, name: str):
        if not self.enabled:
            yield
            return
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        t0 = time.perf_counter()
        try:
            yield
        finally:
            if torch.cuda.is_available():
                torch.cuda.synchronize()
            self.total[name] += time.perf_counter() - t0
            self.count[name] += 1

    def reset(self):
        self.total.clear()
        self.count.clear()

    def summary(self, normalizer: int = 1, reset: bool = True) -> Dict[str, float]:
        """Milliseconds per stage (divided by ``normalizer`` steps), the maximum over ranks."""
        names = sorted(self.total)
        vals = torch.tensor([self.total[n] for n in names], dtype=torch.float64)
        if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1 and names:
            if torch.cuda.is_available() and dist.get_backend() != "gloo":
                vals = vals.cuda()
            dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        out = {n: float(v) * 1e3 / max(normalizer, 1) for n, v in zip(names, vals.cpu())}
        if reset:
            self.reset()
        return out

    @staticmethod
    def line(times: Dict[str, float]) -> str:
        return "    time (ms) | " + " | ".join(f"{k}: {v:.2f}" for k, v in times.items())


class MetricLogger:
    def __init__(self, output_dir: str, is_main: bool = True, total_steps: Optional[int] = None, *, tensorboard: bool = False,
                 wandb_project: Optional[str] = None, run_name: Optional[str] = None, smoothing: int = 20,
                 spike_factor: float = 3.0):
        self.is_main, self.total = is_main, total_steps
        self.path = os.path.join(output_dir, "metrics.jsonl")
        self.output_dir = output_dir
        self.window = collections.deque(maxlen=max(smoothing, 1))
        self.spike_factor = spike_factor
        self.spikes = 0
        self.tb = self.wb = None
        if is_main:
            os.makedirs(output_dir, exist_ok=True)
            if tensorboard:
                from torch.utils.tensorboard import SummaryWriter
                self.tb = SummaryWriter(os.path.join(output_dir, "tensorboard"))
            if wandb_project:
                import wandb
                mode = os.environ.get("WANDB_MODE", "offline")  # no network is assumed: runs are written to disk
                self.wb = wandb.init(project=wandb_project, name=run_name, dir=output_dir, mode=mode)
        self.t_last = time.perf_counter()
        self.t_start, self.first_step = self.t_last, None

    # -- start-up notes
    def log_config(self, args, extra: Optional[dict] = None) -> str:
        text = format_block("embodied training arguments", flatten_config(args))
        if extra:
            text += "\n" + format_block("model", flatten_config(extra))
        if self.is_main:
            print(text, flush=True)
            with open(os.path.join(self.output_dir, "config.json"), "w") as f:
                json.dump({k: (v if isinstance(v, (int, float, str, bool, type(None), list, dict)) else str(v))
                           for k, v in flatten_config(args).items()}, f, indent=1)
        return text

    def log_param_stats(self, model: torch.nn.Module) -> Dict[str, int]:
        total = sum(p.numel() for p in model.parameters())
        train = sum(p.numel() for p in model.parameters() if p.requires_grad)
        by_top: Dict[str, int] = collections.defaultdict(int)
        for n, p in model.named_parameters():
            parts = [x for x in n.split(".") if x not in ("module", "policy")]
            by_top[parts[0] if parts else n] += p.numel()
        if self.is_main:
            print(f" > parameters: {total:,d} total, {train:,d} trainable ({100.0 * train / max(total, 1):.2f}%) | "
                  + " | ".join(f"{k}: {v:,d}" for k, v in sorted(by_top.items(), key=lambda kv: -kv[1])), flush=True)
        return {"total": total, "trainable": train, **by_top}

    def note(self, message: str):
        if self.is_main:
            print(f" > {message}", flush=True)

    # -- per step
    def log(self, step: int, metrics: Dict[str, float], samples: int, stage_times: Optional[Dict[str, float]] = None) -> str:
        now = time.perf_counter()
        dt, self.t_last = now - self.t_last, now
        if self.first_step is None:
            self.first_step, self.t_start = step, now
        rec = {"step": step, "elapsed_ms": dt * 1e3, "samples_per_sec": samples / max(dt, 1e-9), **metrics}
        loss = metrics.get("loss")
        if isinstance(loss, float):
            if len(self.window) >= 5:
                mean = sum(self.window) / len(self.window)
                if loss > self.spike_factor * mean and mean > 0:
                    self.spikes += 1
                    rec["loss_spike"] = True
                    self.note(f"loss spike at step {step}: {loss:.4f} against a running mean of {mean:.4f}")
            self.window.append(loss)
            rec["loss_smoothed"] = sum(self.window) / len(self.window)
        if torch.cuda.is_available():
            rec["mem_allocated_gb"] = torch.cuda.max_memory_allocated() / 2 ** 30
            rec["mem_reserved_gb"] = torch.cuda.max_memory_reserved() / 2 ** 30
        if self.total and step > self.first_step:
            per = (now - self.t_start) / (step - self.first_step)
            rec["eta_s"] = per * (self.total - step)
        if stage_times:
            rec.update({f"time/{k}": v for k, v in stage_times.items()})
        shown = {k: v for k, v in metrics.items()}
        line = (f" iteration {step:8d}/{self.total or 0:8d} | elapsed time per iteration (ms): {dt * 1e3:.1f} | "
                + " | ".join(f"{k}: {v:.6E}" if isinstance(v, float) else f"{k}: {v}" for k, v in shown.items())
                + f" | samples/sec: {rec['samples_per_sec']:.2f} |"
                + (f" eta: {rec['eta_s'] / 60:.1f} min |" if "eta_s" in rec else ""))
        if self.is_main:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
            print(line, flush=True)
            if stage_times:
                print(StageTimers.line(stage_times), flush=True)
            scalars = {k: v for k, v in rec.items() if isinstance(v, (int, float)) and not isinstance(v, bool) and k != "step"}
            if self.tb is not None:
                for k, v in scalars.items():
                    self.tb.add_scalar(k if "/" in k else f"train/{k}", v, step)
            if self.wb is not None:
                self.wb.log(scalars, step=step)
        return line

    def finish(self):
        if self.tb is not None:
            self.tb.close()
        if self.wb is not None:
            self.wb.finish()
