import os
import sys

import pytest

if os.environ.get("PYTEST_XDIST_WORKER"):
    # several worker processes share the cores: keep each one's math library from spawning a thread per core
    os.environ.setdefault("OMP_NUM_THREADS", "2")
    os.environ.setdefault("MKL_NUM_THREADS", "2")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


@pytest.hookimpl(tryfirst=True)
def pytest_cmdline_main(config):
    """On a machine without a GPU the suite is dominated by multi-process (gloo) equivalence tests: spread the test
    files over a few worker processes when pytest-xdist is there and the caller did not choose a worker count. With a
    GPU everything stays in one process (tests must not share the device concurrently)."""
    if not hasattr(config.option, "numprocesses") or config.option.numprocesses is not None:
        return None
    if os.environ.get("LF_TEST_WORKERS", "") == "0" or os.environ.get("PYTEST_XDIST_WORKER") or hasattr(config, "workerinput"):
        return None  # switched off, or this process IS a worker
    import torch

    if torch.cuda.is_available():
        return None
    n = int(os.environ.get("LF_TEST_WORKERS", "0")) or max(1, min(4, (os.cpu_count() or 2) // 2))
    if n > 1:
        config.option.numprocesses = n
        config.option.dist = "loadfile"
    return None


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _reset_parallel_state():
    yield
    from loongforge_b200.parallel import state as ps

    ps.destroy_model_parallel()
