"""Megatron-style console line plus ``metrics.jsonl`` (reference: loongforge/embodied/train/utils/logging.py)."""
from __future__ import annotations

import json
import os
import time
from typing import Dict, Optional


class MetricLogger:
    def __init__(self, output_dir: str, is_main: bool = True, total_steps: Optional[int] = None):
        self.is_main, self.total = is_main, total_steps
        self.path = os.path.join(output_dir, "metrics.jsonl")
        if is_main:
            os.makedirs(output_dir, exist_ok=True)
        self.t_last = time.perf_counter()

    def log(self, step: int, metrics: Dict[str, float], samples: int) -> str:
        now = time.perf_counter()
        dt, self.t_last = now - self.t_last, now
        rec = {"step": step, "elapsed_ms": dt * 1e3, "samples_per_sec": samples / max(dt, 1e-9), **metrics}
        line = (f" iteration {step:8d}/{self.total or 0:8d} | elapsed time per iteration (ms): {dt * 1e3:.1f} | "
                + " | ".join(f"{k}: {v:.6E}" if isinstance(v, float) else f"{k}: {v}" for k, v in metrics.items())
                + f" | samples/sec: {rec['samples_per_sec']:.2f} |")
        if self.is_main:
            with open(self.path, "a") as f:
                f.write(json.dumps(rec) + "\n")
            print(line, flush=True)
        return line
