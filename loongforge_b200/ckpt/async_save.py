"""Checkpoint housekeeping around ``ckpt/checkpointing.py``: asynchronous saves (tensors staged to host memory, written
by a background thread), retention of every k-th checkpoint only, node-local non-persistent checkpoints, per-DP-rank
data-loader state files, and the decision to checkpoint-and-exit on a signal or a time limit (reference:
loongforge/train/checkpointing.py:729-738,1024-1030,1068-1123; training_utils.py:447-476,2926-2936)."""
from __future__ import annotations

import os
import shutil
import signal
import threading
import time
from typing import Callable, Dict, List, Optional

import torch


def stage_to_host(state: Dict) -> Dict:
    """Deep copy of a (nested) state dict with every tensor moved to host memory (pinned when it came from a GPU)."""
    if torch.is_tensor(state):
        if state.is_cuda:
            buf = torch.empty(state.shape, dtype=state.dtype, pin_memory=True)
            buf.copy_(state, non_blocking=True)
            return buf
        return state.detach().clone()
    if isinstance(state, dict):
        return {k: stage_to_host(v) for k, v in state.items()}
    if isinstance(state, (list, tuple)):
        return type(state)(stage_to_host(v) for v in state)
    return state


class AsyncSaver:
    """``save(path, state)`` returns once the tensors are staged; the file is written by a worker thread. The tracker
    file must only be updated from ``on_done`` (i.e. after the write finished)."""

    def __init__(self):
        self.thread: Optional[threading.Thread] = None
        self.error: Optional[BaseException] = None

    def wait(self) -> None:
        if self.thread is not None:
            self.thread.join()
            self.thread = None
        if self.error is not None:
            err, self.error = self.error, None
            raise err

    def save(self, path: str, state: Dict, on_done: Optional[Callable[[], None]] = None) -> None:
        self.wait()  # one save in flight at a time
        staged = stage_to_host(state)
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

        def work():
            try:
                os.makedirs(os.path.dirname(path), exist_ok=True)
                tmp = path + ".tmp"
                torch.save(staged, tmp)
                os.replace(tmp, path)
                if on_done is not None:
                    on_done()
            except BaseException as e:  # noqa: BLE001 - re-raised on the training thread by wait()
                self.error = e

        self.thread = threading.Thread(target=work, daemon=True)
        self.thread.start()


def list_iterations(root: str) -> List[int]:
    out = []
    for d in os.listdir(root) if os.path.isdir(root) else []:
        if d.startswith("iter_") and d[5:].isdigit():
            out.append(int(d[5:]))
    return sorted(out)


def apply_retention(root: str, keep_last: int = 1, retain_interval: Optional[int] = None) -> List[int]:
    """Deletes checkpoints except the newest `keep_last` and those whose iteration is a multiple of
    `retain_interval`. Returns the removed iterations."""
    its = list_iterations(root)
    keep = set(its[-keep_last:]) if keep_last > 0 else set()
    if retain_interval:
        keep |= {i for i in its if i % retain_interval == 0}
    removed = []
    for i in its:
        if i not in keep:
            shutil.rmtree(os.path.join(root, f"iter_{i:07d}"), ignore_errors=True)
            removed.append(i)
    return removed


class LocalCheckpointManager:
    """Frequent non-persistent checkpoints on node-local storage: only the newest is kept; ``find_latest`` compares it
    with the persistent tracker so that resume picks the more recent of the two."""

    def __init__(self, local_root: str, rank: int):
        self.root, self.rank = local_root, rank

    def path(self, iteration: int) -> str:
        return os.path.join(self.root, f"iter_{iteration:07d}", f"local_rank{self.rank:05d}.pt")

    def save(self, iteration: int, state: Dict) -> str:
        p = self.path(iteration)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        torch.save(stage_to_host(state), p + ".tmp")
        os.replace(p + ".tmp", p)
        for i in list_iterations(self.root):
            if i != iteration:
                shutil.rmtree(os.path.join(self.root, f"iter_{i:07d}"), ignore_errors=True)
        return p

    def find_latest(self, persistent_iteration: Optional[int]) -> Optional[int]:
        mine = [i for i in list_iterations(self.root) if os.path.isfile(self.path(i))]
        best = max(mine) if mine else None
        if best is not None and (persistent_iteration is None or best > persistent_iteration):
            return best
        return None

    def load(self, iteration: int) -> Dict:
        return torch.load(self.path(iteration), map_location="cpu", weights_only=False)


def dataloader_state_path(ckpt_dir: str, dp_rank: int) -> str:
    return os.path.join(ckpt_dir, f"train_dataloader_dprank{dp_rank:03d}.pt")


def save_dataloader_state(ckpt_dir: str, dp_rank: int, state: Dict) -> None:
    os.makedirs(ckpt_dir, exist_ok=True)
    torch.save(state, dataloader_state_path(ckpt_dir, dp_rank))


def load_dataloader_state(ckpt_dir: str, dp_rank: int) -> Optional[Dict]:
    p = dataloader_state_path(ckpt_dir, dp_rank)
    return torch.load(p, map_location="cpu", weights_only=False) if os.path.isfile(p) else None


class ExitDecider:
    """checkpoint-and-exit on SIGTERM / SIGINT, after `exit_duration_min` minutes, or at `exit_interval` iterations."""

    def __init__(self, exit_duration_min: Optional[float] = None, exit_interval: Optional[int] = None,
                 install_signal_handlers: bool = False):
        self.t0 = time.time()
        self.duration, self.interval = exit_duration_min, exit_interval
        self.signalled = False
        if install_signal_handlers:
            for s in (signal.SIGTERM, signal.SIGINT):
                signal.signal(s, self._on_signal)

    def _on_signal(self, signum, frame):
        self.signalled = True

    def should_exit(self, iteration: int) -> Optional[str]:
        if self.signalled:
            return "signal"
        if self.duration is not None and (time.time() - self.t0) / 60.0 >= self.duration:
            return "duration"
        if self.interval and iteration % self.interval == 0:
            return "interval"
        return None
