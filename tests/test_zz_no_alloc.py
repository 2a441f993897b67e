"""The allocation-free RMSNorm backward (``lf_rmsnorm_bwd_noalloc``) called through its exported
C symbol, the way a caller that cannot use the device allocator would: a C host program, or a
thread that runs while all device memory is already handed out. Checked against the regular
(allocating) backward on two consecutive calls, which share the library's built-in scratch array."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_noalloc_rmsnorm_bwd_matches_regular_entry_point():
    from loongforge_b200.ops import _ext

    mod = _ext.require()
    lib = ctypes.CDLL(mod.__file__)
    fn = lib.lf_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_float, ctypes.c_void_p]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.current_stream().cuda_stream
    # two calls in a row with different shapes: the second sees the first one's leftovers in the scratch
    for seed, (T, H) in enumerate([(777, 4096), (96, 1280)]):
        torch.manual_seed(seed)
        x = torch.randn(T, H, device=dev).bfloat16()
        w = (1 + 0.1 * torch.randn(H, device=dev)).bfloat16()
        dy = torch.randn(T, H, device=dev).bfloat16()
        _, rstd = mod.rmsnorm_fwd(x, w, 1e-5, 0.0)
        dx_ref, dw_ref = mod.rmsnorm_bwd(dy, x, w, rstd, None, 0.0)
        # outputs are allocated by the CALLER; the entry point itself allocates nothing
        dx = torch.empty_like(x)
        dw = torch.empty(H, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), T, H, 0.0,
                stream)
        torch.cuda.synchronize()
        assert rc == 0
        assert torch.cuda.memory_allocated() == before
        assert _rel(dx, dx_ref) < 1e-2
        assert _rel(dw, dw_ref) < 2e-2
    # sizes beyond the stated maximum are refused, nothing runs
    assert fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, 8192 + 8,
              0.0, stream) == 1
    assert fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, 100,
              0.0, stream) == 1
    # more rows than the kernels' 32-bit row counter can hold: refused, not narrowed
    assert fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 2 ** 31, 64,
              0.0, stream) == 1
    # a null or misaligned pointer is refused before anything is launched
    assert fn(None, x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, 64, 0.0,
              stream) == 2
    assert fn(dy.data_ptr() + 2, x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 4, 64,
              0.0, stream) == 2
    torch.cuda.synchronize()
