"""Failure detection and recovery on the host side.

* ``RerunStateMachine``: validates the loss of every step (NaN / Inf / spike), can re-run the
  step from a saved RNG + data snapshot to tell a transient fault (result changes) from a
  persistent one (same bad result), and decides between continuing, skipping, or checkpoint-and-exit
  (the reference wires Megatron's rerun state machine at loongforge/train/initialize.py:213-233 and
  validates losses in loongforge/train/pretrain/pretrain_llm.py:98-127).
* ``ErrorInjector``: host-side fault injection (``--error-injection-rate/-type``): corrupts a loss
  value or raises inside the step at a chosen rate. Nothing is ever injected on the device.
* ``StragglerDetector``: per-rank step-time statistics exchanged over a CPU (gloo) group, flagging
  ranks slower than ``threshold`` x the median (loongforge/train/training_utils.py:162,2549-2560).
* ``Heartbeat``: rank liveness through the c10d store; a peer that stopped writing is reported
  before the next collective is launched.
* ``check_kernel_status``: surfaces bounded-wait timeouts of the native kernels as exceptions.
"""
from __future__ import annotations

import dataclasses
import math
import random
import time
from typing import Callable, Dict, List, Optional

import torch
import torch.distributed as dist


class TransientError(RuntimeError):
    pass


class PersistentError(RuntimeError):
    pass


@dataclasses.dataclass
class RerunDecision:
    action: str  # "continue" | "rerun" | "skip" | "exit"
    reason: str = ""


class RerunStateMachine:
    def __init__(self, mode: str = "validate_results", spiky_factor: float = 10.0, max_reruns: int = 1,
                 window: int = 50):
        assert mode in ("disabled", "validate_results", "report_stats")
        self.mode, self.spiky_factor, self.max_reruns = mode, spiky_factor, max_reruns
        self.history: List[float] = []
        self.window = window
        self.reruns = 0
        self.first_bad: Optional[float] = None
        self.stats = {"nan": 0, "inf": 0, "spiky": 0, "transient": 0, "persistent": 0}

    def classify(self, loss: float) -> Optional[str]:
        if math.isnan(loss):
            return "nan"
        if math.isinf(loss):
            return "inf"
        if len(self.history) >= 5:
            mean = sum(self.history) / len(self.history)
            if loss > self.spiky_factor * max(mean, 1e-12):
                return "spiky"
        return None

    def validate(self, loss: float) -> RerunDecision:
        """Call with the step's loss; on 'rerun' the caller restores its snapshot and calls again."""
        if self.mode == "disabled":
            return RerunDecision("continue")
        kind = self.classify(loss)
        if kind is None:
            if self.first_bad is not None:  # the re-run gave a good result: the fault was transient
                self.stats["transient"] += 1
                self.first_bad, self.reruns = None, 0
            self.history = (self.history + [loss])[-self.window:]
            return RerunDecision("continue")
        self.stats[kind] += 1
        if self.mode == "report_stats":
            return RerunDecision("continue", kind)
        if self.reruns < self.max_reruns:
            self.reruns += 1
            self.first_bad = loss
            return RerunDecision("rerun", kind)
        same = (self.first_bad is not None and
                ((math.isnan(loss) and math.isnan(self.first_bad)) or loss == self.first_bad))
        self.first_bad, self.reruns = None, 0
        if same:
            self.stats["persistent"] += 1
            return RerunDecision("exit", f"persistent {kind}: the same result was reproduced")
        self.stats["transient"] += 1
        return RerunDecision("skip", f"non-deterministic {kind}")

    def state_dict(self):
        return {"history": self.history, "stats": self.stats}

    def load_state_dict(self, sd):
        self.history, self.stats = list(sd["history"]), dict(sd["stats"])


class ErrorInjector:
    """Host-side fault injection. `rate` = one fault every `rate` calls on average (0 = never)."""

    def __init__(self, rate: int = 0, kind: str = "transient_error", seed: int = 0):
        assert kind in ("transient_error", "persistent_error", "exception", "correct_result")
        self.rate, self.kind = rate, kind
        self.rng = random.Random(seed)
        self.sticky = False

    def maybe_corrupt(self, loss: float, replay: bool = False) -> float:
        """``replay``: the value comes from the re-run of a step whose first result was rejected; a transient fault
        does not strike the same step twice."""
        if self.rate <= 0 or self.kind == "correct_result" or (replay and self.kind == "transient_error"):
            return loss
        if self.kind == "persistent_error" and self.sticky:
            return float("nan")
        if self.rng.randrange(self.rate) == 0:
            if self.kind == "exception":
                raise TransientError("injected host-side fault")
            self.sticky = self.kind == "persistent_error"
            return float("nan")
        return loss


class StragglerDetector:
    def __init__(self, group=None, threshold: float = 1.3):
        self.group, self.threshold = group, threshold
        self.times: List[float] = []
        self._t0 = None

    def start(self):
        self._t0 = time.perf_counter()

    def stop(self):
        self.times.append(time.perf_counter() - self._t0)

    def report(self) -> Dict[str, object]:
        mine = sum(self.times) / max(len(self.times), 1)
        self.times = []
        if dist.is_initialized() and dist.get_world_size(self.group) > 1:
            t = torch.tensor([mine], dtype=torch.float64)
            all_t = [torch.zeros_like(t) for _ in range(dist.get_world_size(self.group))]
            dist.all_gather(all_t, t, group=self.group)
            vals = [float(x) for x in all_t]
        else:
            vals = [mine]
        med = sorted(vals)[len(vals) // 2]
        slow = [i for i, v in enumerate(vals) if med > 0 and v > self.threshold * med]
        return {"mean_step_s": vals, "median": med, "stragglers": slow}


class Heartbeat:
    """Liveness over a key-value store (``dist.TCPStore`` / ``HashStore``): every rank bumps its counter
    between steps; ``dead_ranks`` lists peers whose counter has not moved for `timeout_s`."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0):
        self.store, self.rank, self.world, self.timeout_s = store, rank, world, timeout_s
        self.seen: Dict[int, tuple] = {}
        self.count = 0

    def beat(self):
        self.count += 1
        self.store.set(f"hb/{self.rank}", str(self.count))

    def dead_ranks(self, now: Optional[float] = None) -> List[int]:
        now = time.monotonic() if now is None else now
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            key = f"hb/{r}"
            try:
                # `get` blocks until the key exists: ask first, a rank that never wrote counts as silent
                v = int(self.store.get(key).decode()) if self.store.check([key]) else -1
            except Exception:  # noqa: BLE001 - store without `check`, or the key vanished
                v = -1
            last = self.seen.get(r)
            if last is None or last[0] != v:
                self.seen[r] = (v, now)
            elif now - last[1] > self.timeout_s:
                dead.append(r)
        return dead


def check_kernel_status():
    """Raise if a native kernel reported a wait that gave up (peer flag, TMA stage, accumulator)."""
    if torch.cuda.is_available():
        from ..ops import _ext
        _ext.check_status()


def run_step_with_recovery(step_fn: Callable[[], float], snapshot: Callable[[], object],
                           restore: Callable[[object], None], rsm: RerunStateMachine,
                           injector: Optional[ErrorInjector] = None) -> tuple:
    """Run one training step under the rerun state machine. Returns (loss, decision)."""
    snap = snapshot() if rsm.mode == "validate_results" else None
    while True:
        loss = step_fn()
        if injector is not None:
            loss = injector.maybe_corrupt(loss)
        d = rsm.validate(loss)
        if d.action == "rerun":
            restore(snap)
            continue
        return loss, d
