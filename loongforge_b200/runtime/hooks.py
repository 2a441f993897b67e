"""Per-step hooks of the training loop, built from the command-line flags: EMA (``--ema-decay``), profiler
(``--profile --profile-step-start/end --profile-ranks``), allocator history (``--record-memory-history``), tensor
inspector (``--enable-log-tensor --log-tensor-name-pattern``), scalar sinks (``--tensorboard-dir --wandb-project``),
manual garbage collection (``--manual-gc --manual-gc-interval``), checkpoint retention and exit decisions
(``--exit-interval --exit-duration-in-mins``, SIGTERM). The reference interleaves the same features in its train loop
(loongforge/train/training_utils.py:2431-2975)."""
from __future__ import annotations

import gc
from typing import List, Optional

import torch.distributed as dist


class TrainHook:
    def on_step_end(self, trainer, metrics, elapsed_ms) -> Optional[str]:
        """Return a non-empty reason string to request checkpoint-and-exit."""
        return None

    def on_train_end(self, trainer) -> None:
        pass


class EMAHook(TrainHook):
    def __init__(self, trainer, decay: float):
        from .ema import ModelEMA
        named = [(f"{i}.{n}", p) for i, m in enumerate(trainer.models) for n, p in m.named_parameters()]
        self.ema = ModelEMA(named, decay)

    def on_step_end(self, trainer, metrics, elapsed_ms):
        self.ema.update()

    def on_train_end(self, trainer):
        if trainer.tcfg.save:
            rank = dist.get_rank() if dist.is_initialized() else 0
            self.ema.save(trainer.tcfg.save, trainer.iteration, f"_rank{rank:05d}")


class ProfilerHook(TrainHook):
    def __init__(self, out_dir, start, end, ranks, rank):
        from .profiling import StepProfiler
        self.prof = StepProfiler(out_dir, start, end, ranks, rank)

    def on_step_end(self, trainer, metrics, elapsed_ms):
        self.prof.step(trainer.iteration)


class MemoryHistoryHook(TrainHook):
    def __init__(self, out_dir, rank, every: int = 0):
        from .profiling import MemoryHistory
        self.mh, self.every = MemoryHistory(out_dir, rank), every

    def on_step_end(self, trainer, metrics, elapsed_ms):
        if self.every and trainer.iteration % self.every == 0:
            self.mh.dump(f"it{trainer.iteration}")


class TensorInspectorHook(TrainHook):
    def __init__(self, trainer, patterns, out_path, rank):
        from .profiling import TensorInspector
        self.insp = [TensorInspector(m, patterns, out_path, rank=rank) for m in trainer.models]

    def on_step_end(self, trainer, metrics, elapsed_ms):
        for i in self.insp:
            i.step()

    def on_train_end(self, trainer):
        for i in self.insp:
            i.remove()


class ScalarHook(TrainHook):
    def __init__(self, out_dir, wandb_project, enabled, run_name=None):
        from .metrics_writers import ScalarWriter
        self.w = ScalarWriter(out_dir, wandb_project=wandb_project, enabled=enabled, run_name=run_name)

    def on_step_end(self, trainer, metrics, elapsed_ms):
        sc = {k: v for k, v in metrics.items() if isinstance(v, (int, float))}
        sc["iteration-time-ms"] = elapsed_ms
        self.w.add_scalars(sc, trainer.iteration)

    def on_train_end(self, trainer):
        self.w.close()


class ManualGCHook(TrainHook):
    def __init__(self, interval: int):
        self.interval = max(int(interval), 1)
        gc.disable()

    def on_step_end(self, trainer, metrics, elapsed_ms):
        if trainer.iteration % self.interval == 0:
            gc.collect()

    def on_train_end(self, trainer):
        gc.enable()


class DPBalanceWarmupHook(TrainHook):
    """Fits the cost model of the data-parallel load balancer from measured step times: during iterations
    [first, last] (``--vlm-dp-balance-warmup-iters first last``) every rank records the token counts of the micro-batches
    it ran with the step's forward + backward time; after `last` the observations of all ranks are pooled and the
    coefficients of ``a s^2 + b s + c`` replace the defaults."""

    def __init__(self, trainer, first: int, last: int):
        self.first, self.last, self.done = int(first), int(last), False

    def on_step_end(self, trainer, metrics, elapsed_ms):
        if self.done:
            return None
        it = next(iter(getattr(trainer, "_balanced_iterators", {}).values()), None)
        if it is None:
            return None
        if self.first <= trainer.iteration <= self.last and it.last_lengths:
            it.model.observe(it.last_lengths, elapsed_ms)
        if trainer.iteration >= self.last:
            from ..data.dp_balance import fit_cost_model_across_ranks
            coef = fit_cost_model_across_ranks(it.model, trainer.st.group("dp"))
            self.done = True
            metrics["dp_balance_cost_coefficients"] = [float(c) for c in coef]
        return None


class ExitHook(TrainHook):
    def __init__(self, duration_min, interval, signals: bool):
        from ..ckpt.async_save import ExitDecider
        self.d = ExitDecider(duration_min, interval, install_signal_handlers=signals)

    def on_step_end(self, trainer, metrics, elapsed_ms):
        return self.d.should_exit(trainer.iteration)


class RetentionHook(TrainHook):
    def __init__(self, keep_last: int, retain_interval):
        self.keep, self.retain = keep_last, retain_interval

    def on_step_end(self, trainer, metrics, elapsed_ms):
        t = trainer.tcfg
        is_main = (not dist.is_initialized()) or dist.get_rank() == 0
        if is_main and t.save and t.save_interval and trainer.iteration % t.save_interval == 0:
            from ..ckpt.async_save import apply_retention
            apply_retention(t.save, self.keep, self.retain)


class StragglerHook(TrainHook):
    """Per-rank step times exchanged every ``log_interval`` steps; ranks slower than the threshold x median are
    reported on the logging rank (``--log-straggler``, reference: loongforge/train/training_utils.py:162,2549-2560)."""

    def __init__(self, trainer, threshold: float = 1.3, sink=print):
        from .resilience import StragglerDetector
        self.det = StragglerDetector(None, threshold)
        self.sink, self.every = sink, max(1, trainer.tcfg.log_interval)
        self.reports: List[dict] = []

    def on_step_end(self, trainer, metrics, elapsed_ms):
        self.det.times.append(elapsed_ms / 1e3)
        if trainer.iteration % self.every == 0:
            rep = self.det.report()
            self.reports.append(rep)
            is_main = (not dist.is_initialized()) or dist.get_rank() == 0
            if rep["stragglers"] and is_main:
                self.sink(f" [straggler] iteration {trainer.iteration}: ranks {rep['stragglers']} are slower than "
                          f"{self.det.threshold:.2f} x median step time {rep['median'] * 1e3:.1f} ms")


class HeartbeatHook(TrainHook):
    """Rank liveness through the job's key-value store: every rank bumps its counter after each step; a peer whose
    counter stopped for ``timeout_s`` is reported BEFORE the next collective would hang on it, and the loop asks for
    checkpoint-and-exit."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 600.0):
        from .resilience import Heartbeat
        self.hb = Heartbeat(store, rank, world, timeout_s)
        self.dead: List[int] = []

    def on_step_end(self, trainer, metrics, elapsed_ms):
        self.hb.beat()
        self.dead = self.hb.dead_ranks()
        return f"ranks {self.dead} stopped sending heartbeats" if self.dead else None


def build_hooks(args, trainer) -> List[TrainHook]:
    rank = dist.get_rank() if dist.is_initialized() else 0
    world = dist.get_world_size() if dist.is_initialized() else 1
    out = getattr(args, "tensorboard_dir", None) or (trainer.tcfg.save or ".")
    hooks: List[TrainHook] = []
    if getattr(args, "ema_decay", None) or getattr(args, "enable_ema", False):
        # --enable-ema without a decay uses the reference's default of 0.9999
        hooks.append(EMAHook(trainer, getattr(args, "ema_decay", None) or 0.9999))
    if getattr(args, "profile", False) or getattr(args, "use_pytorch_profiler", False):
        hooks.append(ProfilerHook(out, args.profile_step_start, args.profile_step_end, args.profile_ranks, rank))
    if getattr(args, "record_memory_history", False):
        hooks.append(MemoryHistoryHook(out, rank))
    if getattr(args, "enable_log_tensor", False):
        pats = args.log_tensor_name_pattern or ["*"]
        pats = [pats] if isinstance(pats, str) else list(pats)
        hooks.append(TensorInspectorHook(trainer, pats, f"{out}/tensors_rank{rank}.jsonl", rank))
    if getattr(args, "tensorboard_dir", None) or getattr(args, "wandb_project", None):
        hooks.append(ScalarHook(out, getattr(args, "wandb_project", None), enabled=(rank == world - 1),
                                run_name=getattr(args, "wandb_exp_name", None)))
    if getattr(args, "manual_gc", False):
        hooks.append(ManualGCHook(getattr(args, "manual_gc_interval", 0) or 1))
    if getattr(args, "log_straggler", False):
        hooks.append(StragglerHook(trainer))
    if trainer.tcfg.dp_balance:
        w = list(getattr(args, "vlm_dp_balance_warmup_iters", None) or [2, 5])
        hooks.append(DPBalanceWarmupHook(trainer, int(w[0]), int(w[-1])))
    if getattr(args, "heartbeat_timeout_s", None) and dist.is_initialized() and world > 1:
        store = dist.distributed_c10d._get_default_store()
        hooks.append(HeartbeatHook(store, rank, world, float(args.heartbeat_timeout_s)))
    if getattr(args, "exit_interval", None) or getattr(args, "exit_duration_in_mins", None):
        hooks.append(ExitHook(getattr(args, "exit_duration_in_mins", None), getattr(args, "exit_interval", None), False))
    return hooks
