"""The tcgen05 flash-attention kernels (forward, dK/dV, dQ) against a plain fp32 PyTorch attention: full-size
sequences, ragged packed sequences, head dims below 128 (zero-filled inside the tile), bidirectional windows,
and query / key sides of different lengths with a bottom-right aligned causal mask."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


def _cu(lens, dev="cuda"):
    return torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)


def _check(Tq, Tk, Hq, Hkv, D, causal, lens_q=None, lens_k=None, seed=0, tol_o=2e-2, tol_g=3e-2):
    from loongforge_b200.ops import _ext
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(seed)
    dev = "cuda"
    q = torch.randn(Tq, Hq, D, device=dev).bfloat16().requires_grad_()
    k = torch.randn(Tk, Hkv, D, device=dev).bfloat16().requires_grad_()
    v = torch.randn(Tk, Hkv, D, device=dev).bfloat16().requires_grad_()
    cq = _cu(lens_q) if lens_q else None
    ck = _cu(lens_k) if lens_k else None
    OF.set_attention_impl("native")
    try:
        o, lse = OF.attention_with_lse(q, k, v, causal=causal, cu_seqlens=cq, cu_seqlens_k=ck)
        do = torch.randn_like(o)
        o.backward(do)
    finally:
        OF.set_attention_impl("auto")
    _ext.check_status()
    qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
    ref, lse_ref = OF.attention_ref(qr, kr, vr, causal, 1.0 / math.sqrt(D), cq, ck, return_lse=True)
    ref.backward(do.float())
    assert _rel(o, ref) < tol_o, f"o {_rel(o, ref)}"
    fin = torch.isfinite(lse_ref)
    assert torch.equal(torch.isfinite(lse), fin)
    assert (lse[fin] - lse_ref[fin]).abs().max().item() < 2e-2
    assert _rel(q.grad, qr.grad) < tol_g, f"dq {_rel(q.grad, qr.grad)}"
    assert _rel(k.grad, kr.grad) < tol_g, f"dk {_rel(k.grad, kr.grad)}"
    assert _rel(v.grad, vr.grad) < tol_g, f"dv {_rel(v.grad, vr.grad)}"


@pytest.mark.parametrize("T,Hq,Hkv,causal", [(128, 2, 2, True), (256, 4, 2, True), (384, 4, 1, False),
                                              (1000, 8, 2, True), (1024, 4, 4, False), (77, 2, 1, True)])
def test_square_small(T, Hq, Hkv, causal):
    _check(T, T, Hq, Hkv, 128, causal)


def test_full_size_sequence_gqa4():
    # the benchmark's sequence length and GQA ratio (fewer heads so that the fp32 reference fits comfortably)
    _check(8192, 8192, 8, 2, 128, True, seed=1)


def test_length_not_a_multiple_of_128_gqa4():
    _check(8192 - 37, 8192 - 37, 4, 1, 128, True, seed=2)


@pytest.mark.parametrize("causal", [True, False])
def test_ragged_packed_sequences(causal):
    lens = [130, 256, 77, 300, 1, 513, 128]
    _check(sum(lens), sum(lens), 6, 2, 128, causal, lens_q=lens, seed=3)


@pytest.mark.parametrize("D", [80, 64, 96, 32])
def test_head_dims_below_128(D):
    _check(700, 700, 4, 4, D, False, seed=4)
    _check(515, 515, 4, 2, D, True, seed=5)


def test_vit_windows_head_dim_80():
    # Qwen2.5-VL vision tower: 16 heads of 80, bidirectional attention inside windows of 64 merged units (and ragged
    # tails), all windows of a batch packed into one call
    lens = [64] * 20 + [48, 16, 64, 32, 8]
    _check(sum(lens), sum(lens), 16, 16, 80, False, lens_q=lens, seed=6)


@pytest.mark.parametrize("Tq,Tk", [(256, 1024), (300, 1324), (128, 128 + 512), (1024, 256)])
def test_bottom_right_causal_unequal_lengths(Tq, Tk):
    _check(Tq, Tk, 4, 2, 128, True, seed=7)
    _check(Tq, Tk, 4, 2, 128, False, seed=8)


def test_separate_query_and_key_boundaries():
    # chunks of packed sequences as the context-parallel schemes produce them: every sequence keeps its last rows on
    # the query side and its whole prefix on the key side
    lens_q = [100, 256, 31, 640]
    lens_k = [400, 256, 200, 1000]
    _check(sum(lens_q), sum(lens_k), 4, 2, 128, True, lens_q=lens_q, lens_k=lens_k, seed=9)
    _check(sum(lens_q), sum(lens_k), 4, 4, 128, False, lens_q=lens_q, lens_k=lens_k, seed=10)


def test_backward_from_merged_lse():
    """Two key blocks processed separately and merged by their log-sum-exp give the single-call result, forward and
    backward (what the context-parallel ring does per step)."""
    from loongforge_b200.ops import _ext
    from loongforge_b200.ops import functional as OF

    torch.manual_seed(12)
    dev = "cuda"
    T, H, D = 512, 4, 128
    q = torch.randn(T, H, D, device=dev).bfloat16()
    k = torch.randn(2 * T, H, D, device=dev).bfloat16()
    v = torch.randn(2 * T, H, D, device=dev).bfloat16()
    o1, l1 = OF.attention_with_lse(q, k[:T], v[:T], causal=False)
    o2, l2 = OF.attention_with_lse(q, k[T:], v[T:], causal=True)
    lse = torch.logaddexp(l1, l2)
    o = (o1.float() * torch.exp(l1 - lse).t().unsqueeze(-1) + o2.float() * torch.exp(l2 - lse).t().unsqueeze(-1))
    ref, lse_ref = OF.attention_ref(q.float(), k.float(), v.float(), True, 1.0 / math.sqrt(D), return_lse=True)
    assert _rel(o, ref) < 2e-2
    do = torch.randn_like(o1)
    ob = o.to(torch.bfloat16)
    dq1, dk1, dv1 = OF.attention_backward(do, q, k[:T].contiguous(), v[:T].contiguous(), ob, lse, None, None,
                                          1.0 / math.sqrt(D), False)
    dq2, dk2, dv2 = OF.attention_backward(do, q, k[T:].contiguous(), v[T:].contiguous(), ob, lse, None, None,
                                          1.0 / math.sqrt(D), True)
    _ext.check_status()
    qr, kr, vr = (t.float().requires_grad_() for t in (q, k, v))
    OF.attention_ref(qr, kr, vr, True, 1.0 / math.sqrt(D)).backward(do.float())
    assert _rel(dq1.float() + dq2.float(), qr.grad) < 3e-2
    assert _rel(torch.cat([dk1, dk2]), kr.grad) < 3e-2
    assert _rel(torch.cat([dv1, dv2]), vr.grad) < 3e-2
