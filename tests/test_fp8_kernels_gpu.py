"""FP8 block quantisers and the blockwise FP8 GEMM (csrc/fp8_sm100.cu) against the PyTorch formulation in ops/quant.py."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("pow2", [False, True])
def test_quant_1x128_matches_reference(pow2):
    from loongforge_b200.ops import _ext, quant as Q

    torch.manual_seed(0)
    x = (torch.randn(300, 512, device="cuda") * torch.logspace(-2, 2, 300, device="cuda")[:, None]).bfloat16()
    q, s = _ext.require().quant_1x128(x, pow2)
    qr, sr = Q.quantize_1x128_ref(x, pow2)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    # rounding of x / s to e4m3 may differ by one code at exact ties; compare de-quantised values
    assert (Q.dequantize_1x128(q, s) - Q.dequantize_1x128(qr, sr)).abs().max() <= s.max() * 32


def test_quant_128x128_matches_reference():
    from loongforge_b200.ops import _ext, quant as Q

    torch.manual_seed(1)
    w = torch.randn(384, 256, device="cuda").bfloat16()
    q, s = _ext.require().quant_128x128(w, False)
    qr, sr = Q.quantize_128x128_ref(w, False)
    assert torch.allclose(s, sr, rtol=1e-6, atol=0)
    assert (Q.dequantize_128x128(q, s) - Q.dequantize_128x128(qr, sr)).abs().max() <= s.max() * 32


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 256, 384), (1024, 512, 1024)])
def test_fp8_gemm_matches_dequantised_product(M, N, K):
    from loongforge_b200.ops import _ext, quant as Q

    torch.manual_seed(2)
    x = torch.randn(M, K, device="cuda").bfloat16()
    w = (torch.randn(N, K, device="cuda") * 0.05).bfloat16()
    qx, sx = Q.quantize_1x128_ref(x)
    qw, sw = Q.quantize_128x128_ref(w)
    y = _ext.require().gemm_fp8_blockwise(qx, sx.contiguous(), qw, sw.contiguous(), _ext.status_tensor(x.device))
    _ext.check_status()
    ref = Q.dequantize_1x128(qx, sx) @ Q.dequantize_128x128(qw, sw).t()
    err = ((y.float() - ref).norm() / ref.norm()).item()
    assert err < 5e-3, err
