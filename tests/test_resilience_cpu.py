"""Failure detection without touching a GPU: injected host faults, a rank that stops, store heartbeats."""
import math

import pytest

import torch

from dist_utils import run_distributed


def test_rerun_state_machine_transient_vs_persistent():
    from loongforge_b200.runtime.resilience import ErrorInjector, RerunStateMachine, run_step_with_recovery

    rsm = RerunStateMachine()
    state = {"x": 0}
    calls = []

    def step():
        state["x"] += 1
        calls.append(state["x"])
        return 2.0

    # transient: first evaluation corrupted, the re-run is clean
    faults = iter([float("nan"), 2.0])

    class OneShot:
        def maybe_corrupt(self, loss):
            return next(faults, loss)

    loss, d = run_step_with_recovery(step, lambda: dict(state), lambda s: state.update(s), rsm, OneShot())
    assert d.action == "continue" and loss == 2.0 and rsm.stats["transient"] == 1
    assert calls == [1, 1]  # the step was re-run from the restored snapshot
    inj = ErrorInjector(rate=1, kind="persistent_error")
    loss, d = run_step_with_recovery(step, lambda: dict(state), lambda s: state.update(s), rsm, inj)
    assert d.action == "exit" and math.isnan(loss) and rsm.stats["persistent"] == 1


def test_spike_detection():
    from loongforge_b200.runtime.resilience import RerunStateMachine

    rsm = RerunStateMachine(mode="report_stats")
    for _ in range(10):
        assert rsm.validate(2.0).action == "continue"
    assert rsm.validate(50.0).reason == "spiky" and rsm.stats["spiky"] == 1


def _hb_worker(rank, world):
    import torch.distributed as dist
    from loongforge_b200.runtime.resilience import Heartbeat

    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, timeout_s=0.5)
    dead_seen = []
    for step in range(6):
        if not (rank == 1 and step >= 2):  # rank 1 stops beating after two steps (it "hangs" on the host)
            hb.beat()
        import time
        time.sleep(0.25)
        dead_seen.append(hb.dead_ranks())
    return dead_seen


def test_heartbeat_detects_silent_rank():
    res = run_distributed(_hb_worker, 2)
    assert res[0][-1] == [1] and res[0][0] == []
    assert res[1][-1] == []


def _straggler_worker(rank, world):
    import time
    from loongforge_b200.runtime.resilience import StragglerDetector

    sd = StragglerDetector()
    for _ in range(3):
        sd.start()
        time.sleep(0.15 if rank == 2 else 0.03)
        sd.stop()
    return sd.report()["stragglers"]


def test_straggler_detector():
    assert run_distributed(_straggler_worker, 3)[0] == [2]


def test_trainer_raises_on_kernel_status_word(monkeypatch):
    """The trainer reads the native kernels' status word every step and raises on a wait that gave up."""
    import types

    import torch

    from loongforge_b200.ops import _ext
    from loongforge_b200.runtime.trainer import Trainer

    word = torch.tensor([5], dtype=torch.int32)
    monkeypatch.setattr(_ext, "available", lambda: True)
    monkeypatch.setattr(_ext, "status_tensor", lambda device=None: word)
    stub = types.SimpleNamespace(device=types.SimpleNamespace(type="cuda"), iteration=7)
    with pytest.raises(RuntimeError, match="native kernel error 5"):
        Trainer._check_kernel_status(stub)
    assert int(word.item()) == 0
    Trainer._check_kernel_status(stub)  # a clean word passes


def test_tp_partial_grads_are_reduced_after_the_dp_sync():
    """The tensor-parallel partial-gradient all-reduce is the optimizer's FIRST post-sync hook, i.e. it runs after
    finish_grad_sync() and never while an overlapped data-parallel reduction is still in flight."""
    import torch

    from loongforge_b200.models.config import TransformerConfig
    from loongforge_b200.runtime.trainer import TrainConfig, Trainer

    cfg = TransformerConfig(num_layers=1, hidden_size=64, num_attention_heads=2, ffn_hidden_size=128, vocab_size=128)
    tc = TrainConfig(micro_batch_size=1, global_batch_size=1, seq_length=16, train_iters=1)
    tr = Trainer(cfg, tc, device=torch.device("cpu"))
    hooks = tr.optimizer.post_sync_hooks
    assert hooks and hooks[0].__func__ is Trainer._allreduce_sequence_parallel_grads
    order = []
    m = tr.models[0]
    orig_finish, orig_hook = m.finish_grad_sync, hooks[0]
    m.finish_grad_sync = lambda: (order.append("dp_sync"), orig_finish())[1]
    hooks[0] = lambda: (order.append("tp_partial"), orig_hook())[1]
    from loongforge_b200.data.synthetic import synthetic_batch_iterator

    tr.train_step(synthetic_batch_iterator(128, 16, 1))
    assert order.index("dp_sync") < order.index("tp_partial")
