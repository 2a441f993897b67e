"""Build and load the in-tree sm_100a extension.

The shared object is built IN-TREE (``loongforge_b200/ops/_build``) so that it travels with
the source tree; it is never installed into site-packages. ``build()`` cross-compiles without a
GPU. On a machine with a GPU a missing or unloadable extension is an error (``require()``), not a
silent fallback to PyTorch ops.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import threading

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_CSRC = os.path.join(_HERE, "csrc")
_BUILD_DIR = os.path.join(_HERE, "_build")
_NAME = "lfb200_C"
_lock = threading.Lock()
_mod = None
_load_error: str | None = None

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17", "--use_fast_math",
    "-U__CUDA_NO_BFLOAT16_CONVERSIONS__", "-U__CUDA_NO_BFLOAT16_OPERATORS__",
    "-U__CUDA_NO_HALF_CONVERSIONS__", "-U__CUDA_NO_HALF_OPERATORS__",
]


def _sources() -> tuple[list[str], list[str]]:
    srcs = [os.path.join(_CSRC, "bindings.cpp")]
    defs = []
    for f in sorted(os.listdir(_CSRC)):
        if f.endswith(".cu"):
            srcs.append(os.path.join(_CSRC, f))
    if os.path.exists(os.path.join(_CSRC, "attention_sm100.cu")):
        defs.append("-DLF_HAVE_ATTN")
    if os.path.exists(os.path.join(_CSRC, "peer_gemm.cu")):
        defs.append("-DLF_HAVE_PEER")
    if os.path.exists(os.path.join(_CSRC, "peer_optim.cu")):
        defs.append("-DLF_HAVE_PEER_OPTIM")
    if os.path.exists(os.path.join(_CSRC, "fp8_sm100.cu")):
        defs.append("-DLF_HAVE_FP8")
    if os.path.exists(os.path.join(_CSRC, "moe_peer.cu")):
        defs.append("-DLF_HAVE_MOE_PEER")
    if os.path.exists(os.path.join(_CSRC, "grouped_gemm_sm100.cu")):
        defs.append("-DLF_HAVE_GROUPED")
    if os.path.exists(os.path.join(_CSRC, "dsa_sm100.cu")):
        defs.append("-DLF_HAVE_DSA")
    return srcs, defs


def _so_path() -> str:
    return os.path.join(_BUILD_DIR, _NAME + ".so")


def _stale() -> bool:
    so = _so_path()
    if not os.path.exists(so):
        return True
    t = os.path.getmtime(so)
    for f in os.listdir(_CSRC):
        if os.path.getmtime(os.path.join(_CSRC, f)) > t:
            return True
    return False


def build(verbose: bool = False, force: bool = False):
    """Compile every CUDA source for sm_100a into ``_build/lfb200_C.so`` and import it."""
    global _mod, _load_error
    with _lock:
        if _mod is not None and not force:
            return _mod
        if not force and not _stale():
            m = _import_prebuilt()
            if m is not None:
                _mod = m
                return m
        from torch.utils import cpp_extension

        os.makedirs(_BUILD_DIR, exist_ok=True)
        srcs, defs = _sources()
        # Keep torch from appending its own -gencode list: the arch is given explicitly.
        os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
        _mod = cpp_extension.load(
            name=_NAME,
            sources=srcs,
            extra_cflags=["-O3", "-std=c++17"] + defs,
            extra_cuda_cflags=NVCC_FLAGS + defs,
            extra_include_paths=[_CSRC],
            build_directory=_BUILD_DIR,
            verbose=verbose,
            with_cuda=True,
        )
        _load_error = None
        _apply_env_budget(_mod)
        return _mod


def _import_prebuilt():
    global _load_error
    so = _so_path()
    if not os.path.exists(so):
        _load_error = f"{so} does not exist"
        return None
    try:
        spec = importlib.util.spec_from_file_location(_NAME, so)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        sys.modules[_NAME] = mod
        _apply_env_budget(mod)
        return mod
    except Exception as e:  # noqa: BLE001 - reported through require()
        _load_error = f"{type(e).__name__}: {e}"
        return None


def get():
    """The extension module, or None when it cannot be loaded (CPU-only machine without a build)."""
    global _mod
    if _mod is not None:
        return _mod
    with _lock:
        if _mod is None and not _stale():
            _mod = _import_prebuilt()
    if _mod is None and torch.cuda.is_available():
        # A GPU box must run the native path: build it here rather than fall back.
        build()
    return _mod


def require():
    m = get()
    if m is None:
        raise RuntimeError(
            "loongforge_b200 native extension is not available "
            f"({_load_error}); run `python -c 'import __graft_entry__ as g; g.build()'`"
        )
    return m


def available() -> bool:
    return get() is not None


_status: dict[int, torch.Tensor] = {}


def status_tensor(device=None) -> torch.Tensor:
    """Per-device int32 word that kernels set when one of their bounded waits gives up."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = dev.index if dev.index is not None else torch.cuda.current_device()
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=torch.device("cuda", idx))
        _status[idx] = t
    return t


STATUS_NAMES = {
    1: "consumer timed out waiting for a TMA stage",
    2: "producer timed out waiting for a free stage",
    3: "epilogue timed out waiting for the accumulator",
    4: "MMA warp timed out waiting for a drained accumulator",
    5: "timed out waiting for a flag written by a peer GPU",
    6: "bad argument detected on the device",
    7: "an index read from device memory was out of range (access skipped)",
}


def check_status(device=None) -> None:
    """Synchronising check: raise if any kernel on `device` reported a wait that gave up."""
    t = status_tensor(device)
    code = int(t.item())
    if code != 0:
        t.zero_()
        raise RuntimeError(f"loongforge_b200 kernel error {code}: {STATUS_NAMES.get(code, 'unknown')}")


def set_peer_wait_budget_ms(ms: float) -> None:
    """Budget of the device-side waits on flags that another GPU writes (fused tensor-parallel GEMMs, expert
    exchange, peer-memory optimizer). Default two minutes, or ``LF_PEER_WAIT_MS`` from the environment; a wait
    that runs out sets the status word (code 5) and the kernel returns."""
    require().set_peer_wait_budget_ms(float(ms))


def peer_wait_budget_ms() -> float:
    return float(require().peer_wait_budget_ms())


def _apply_env_budget(mod) -> None:
    v = os.environ.get("LF_PEER_WAIT_MS")
    if v:
        mod.set_peer_wait_budget_ms(float(v))


def launch_count() -> int:
    m = get()
    return int(m.launch_count()) if m is not None else 0


def reset_launch_count() -> None:
    m = get()
    if m is not None:
        m.reset_launch_count()
