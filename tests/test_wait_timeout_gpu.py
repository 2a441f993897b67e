"""A device-side wait on a flag that nothing sets must run out of its budget, report through the status word
and leave the CUDA context usable. The budget is shortened to a few milliseconds for the test; no kernel
traps, faults or spins without a limit."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def short_budget():
    from loongforge_b200.ops import _ext

    old = _ext.peer_wait_budget_ms()
    _ext.set_peer_wait_budget_ms(5.0)
    st = _ext.status_tensor()
    st.zero_()
    yield _ext
    st.zero_()
    _ext.set_peer_wait_budget_ms(old)


def _expect_timeout(_ext, launch):
    st = _ext.status_tensor()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    launch(st)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert elapsed < 2.0, f"the wait took {elapsed:.2f} s with a 5 ms budget"
    assert int(st.item()) == 5  # LF_ERR_WAIT_PEER
    with pytest.raises(RuntimeError, match="peer GPU"):
        _ext.check_status()
    assert int(st.item()) == 0  # cleared by the check
    # the context survived: ordinary work still runs
    assert torch.ones(1024, device="cuda").sum().item() == 1024


def test_optimizer_peer_wait_runs_out(short_budget):
    _ext = short_budget
    mod = _ext.require()
    flags = torch.zeros(8, dtype=torch.int32, device="cuda")  # epoch 1 is never written
    _expect_timeout(_ext, lambda st: mod.peer_wait([flags.data_ptr(), flags.data_ptr()], 0, 1, st))


def test_moe_wait_runs_out(short_budget):
    _ext = short_budget
    mod = _ext.require()
    flags = torch.zeros(2 * 8, dtype=torch.int32, device="cuda")
    rows = torch.zeros(8, 8, dtype=torch.bfloat16, device="cuda")
    scal = torch.zeros(8, dtype=torch.float32, device="cuda")
    ptr = lambda t: [t.data_ptr(), t.data_ptr()]  # noqa: E731 - a "group" of two ranks that share this GPU's buffers
    _expect_timeout(_ext, lambda st: mod.moe_wait(ptr(rows), ptr(scal), ptr(flags), 0, 0, 1, st))


def test_budget_setter_round_trips(short_budget):
    _ext = short_budget
    assert abs(_ext.peer_wait_budget_ms() - 5.0) < 1e-6
    _ext.set_peer_wait_budget_ms(250.0)
    assert abs(_ext.peer_wait_budget_ms() - 250.0) < 1e-6
