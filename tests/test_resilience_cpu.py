"""Failure detection without touching a GPU: injected host faults, a rank that stops, store heartbeats."""
import math

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
