"""FP8 (e4m3) block quantisation used by the DSA indexer and the blockwise-FP8 linear path: activations in 1 x 128
tiles, weights in 128 x 128 blocks, optional power-of-two scales, optional transposed copy for the wgrad GEMM
(reference kernels: loongforge/models/common/experimental_attention_variant/dsa_fused_kernels.py per-token-group
quantiser; TransformerEngine blockwise FP8 recipe).

The CUDA kernels live in ``csrc/quant.cu``; the functions here dispatch to them on the GPU and otherwise compute the
same numbers with PyTorch ops (also the oracle of the kernel tests)."""
from __future__ import annotations

import dataclasses
import os
from typing import Optional, Tuple

import torch

E4M3_MAX = 448.0


@dataclasses.dataclass
class QParams:
    power_2_scale: bool = False
    amax_epsilon: float = 0.0  # floor of the block maximum before the scale is derived


@dataclasses.dataclass
class BlockScalingRecipe:
    """Per-tensor-class settings of the blockwise FP8 linear: forward input (1 x 128 tiles), forward weight
    (128 x 128 blocks) and backward output gradient (1 x 128 tiles). Defaults come from the environment variables the
    reference's TransformerEngine patch introduces (patches/.../common/recipe/__init__.py.patch:9-31):
    ``NVTE_FP8_BLOCK_SCALING_FP32_SCALES`` (1 = plain fp32 scales, else powers of two), overridden per class by
    ``NVTE_FP8_BLOCK_SCALING_{FWD_INP,FWD_WEIGHT,BWD_GRAD}_POWER2`` and floored by
    ``FP8_QUANT_{FWD_INP,FWD_WEIGHT,BWD_GRAD}_AMAX_EPS``."""
    fwd_inp: QParams = dataclasses.field(default_factory=QParams)
    fwd_weight: QParams = dataclasses.field(default_factory=QParams)
    bwd_grad: QParams = dataclasses.field(default_factory=QParams)

    @staticmethod
    def from_env(env=None) -> "BlockScalingRecipe":
        env = os.environ if env is None else env
        f32 = env.get("NVTE_FP8_BLOCK_SCALING_FP32_SCALES", "0") == "1"

        def one(tag: str) -> QParams:
            v = env.get(f"NVTE_FP8_BLOCK_SCALING_{tag}_POWER2")
            return QParams((v == "1") if v is not None else (not f32), float(env.get(f"FP8_QUANT_{tag}_AMAX_EPS", "0.0")))

        return BlockScalingRecipe(one("FWD_INP"), one("FWD_WEIGHT"), one("BWD_GRAD"))


_RECIPE = {"r": None}


def get_recipe() -> BlockScalingRecipe:
    if _RECIPE["r"] is None:
        _RECIPE["r"] = BlockScalingRecipe.from_env()
    return _RECIPE["r"]


def set_recipe(r: Optional[BlockScalingRecipe]) -> None:
    """None re-reads the environment on the next use."""
    _RECIPE["r"] = r


def _scale(amax: torch.Tensor, pow2: bool, eps: float = 0.0) -> torch.Tensor:
    s = amax.clamp(min=max(eps, 1e-12)) / E4M3_MAX
    if pow2:
        # smallest power of two >= s, exactly (log2 / ceil is off by one binade at exact powers on some back ends)
        m, e = torch.frexp(s)  # s = m * 2^e, m in [0.5, 1)
        s = torch.ldexp(torch.ones_like(s), torch.where(m == 0.5, e - 1, e))
    return s


def quantize_1x128_ref(x: torch.Tensor, pow2: bool = False, eps: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """x [M, K] (K % 128 == 0) -> (q float8_e4m3fn [M, K], scales fp32 [M, K/128]); x ~= q * scale."""
    M, K = x.shape
    xb = x.float().view(M, K // 128, 128)
    s = _scale(xb.abs().amax(-1), pow2, eps)
    q = (xb / s.unsqueeze(-1)).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(M, K), s


def quantize_128x128_ref(w: torch.Tensor, pow2: bool = False, eps: float = 0.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """w [N, K] (both % 128 == 0) -> (q [N, K] e4m3, scales [N/128, K/128])."""
    N, K = w.shape
    wb = w.float().view(N // 128, 128, K // 128, 128)
    s = _scale(wb.abs().amax(dim=(1, 3)), pow2, eps)
    q = (wb / s[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q.view(N, K), s


def dequantize_1x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    M, K = q.shape
    return (q.float().view(M, K // 128, 128) * s.unsqueeze(-1)).view(M, K)


def dequantize_128x128(q: torch.Tensor, s: torch.Tensor) -> torch.Tensor:
    N, K = q.shape
    return (q.float().view(N // 128, 128, K // 128, 128) * s[:, None, :, None]).view(N, K)


_NATIVE = {"on": False}


def enable_native(flag: bool = True) -> None:
    """Route CUDA bf16 inputs to the kernels of ``csrc/fp8_sm100.cu``. Off by default: until their numerics tests
    have run on a GPU the PyTorch formulation stays the production path."""
    _NATIVE["on"] = bool(flag)


def _native(x: torch.Tensor) -> bool:
    return _NATIVE["on"] and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()


def quantize_1x128(x: torch.Tensor, pow2: bool = False, transpose: bool = False):
    """Returns (q, scales) or, with ``transpose``, (q, scales, q_t [K, M], scales_t [K, M/128]) where the transposed
    copy is quantised along M (what the wgrad GEMM contracts over)."""
    if _native(x) and x.shape[1] % 128 == 0:
        from . import _ext
        C = _ext.require()
        if hasattr(C, "quant_1x128"):
            q, s = C.quant_1x128(x, pow2)
            if not transpose:
                return q, s
            qt, st = C.quant_1x128(x.t().contiguous(), pow2) if x.shape[0] % 128 == 0 else quantize_1x128_ref(x.t(), pow2)
            return q, s, qt, st
    q, s = quantize_1x128_ref(x, pow2)
    if not transpose:
        return q, s
    qt, st = quantize_1x128_ref(x.t().contiguous(), pow2)
    return q, s, qt, st


def quantize_128x128(w: torch.Tensor, pow2: bool = False):
    if _native(w) and w.shape[0] % 128 == 0 and w.shape[1] % 128 == 0:
        from . import _ext
        C = _ext.require()
        if hasattr(C, "quant_128x128"):
            return C.quant_128x128(w, pow2)
    return quantize_128x128_ref(w, pow2)


def fp8_blockwise_linear_ref(x: torch.Tensor, w: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    """y = x @ w^T computed from the block-quantised operands (fp32 accumulate), bf16 out: the oracle of the FP8 GEMM."""
    qx, sx = quantize_1x128_ref(x, pow2)
    qw, sw = quantize_128x128_ref(w, pow2)
    return (dequantize_1x128(qx, sx) @ dequantize_128x128(qw, sw).t()).to(x.dtype)


def fp8_blockwise_linear(x: torch.Tensor, w: torch.Tensor, pow2: bool = False) -> torch.Tensor:
    if _native(x) and _native(w) and x.shape[1] % 128 == 0 and w.shape[0] % 128 == 0:
        from . import _ext
        C = _ext.require()
        if hasattr(C, "gemm_fp8_blockwise"):
            qx, sx = quantize_1x128(x, pow2)
            qw, sw = quantize_128x128(w, pow2)
            return C.gemm_fp8_blockwise(qx, sx, qw, sw, _ext.status_tensor(x.device))
    return fp8_blockwise_linear_ref(x, w, pow2)


# ----------------------------------------------------------------------------- FP8 linear for training
class _Fp8LinearFn(torch.autograd.Function):
    """y = x W^T with the forward GEMM and the input-gradient GEMM on block-quantised e4m3 operands (activations
    and output gradients in 1 x 128 tiles along the contraction, weights in 128 x 128 blocks), fp32 accumulation.
    The weight-gradient GEMM stays in the parameter dtype and accumulates into the fp32 ``main_grad`` buffer when
    there is one: its contraction runs over tokens, where both operands would need a second, transposed quantisation,
    and its result feeds an fp32 accumulator whose precision matters most."""

    @staticmethod
    def forward(ctx, x2, weight, pow2):
        ctx.save_for_backward(x2, weight)
        r = get_recipe()
        ctx.recipe = r
        return _recipe_linear(x2, weight, r.fwd_inp, r.fwd_weight, pow2)

    @staticmethod
    def backward(ctx, dy):
        from . import functional as OF

        x2, weight = ctx.saved_tensors
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dx [T, K] = dy [T, N] @ W [N, K]: contraction over N, so dy is tiled along N and W^T is the blocked operand
            dx = _recipe_linear(dy, weight.t().contiguous(), ctx.recipe.bwd_grad, ctx.recipe.fwd_weight, None)
        if ctx.needs_input_grad[1]:
            dw = OF._wgrad(dy, x2, weight)
        return dx, dw, None


def _recipe_linear(a: torch.Tensor, b: torch.Tensor, qa: QParams, qb: QParams, pow2_override) -> torch.Tensor:
    """a [M, K] (1 x 128 tiles) times b [N, K] (128 x 128 blocks) under the recipe's per-class settings. The native
    kernels implement the zero-epsilon case with one pow-2 switch; other settings use the PyTorch formulation."""
    pa = qa.power_2_scale if pow2_override is None else (pow2_override or qa.power_2_scale)
    pb = qb.power_2_scale if pow2_override is None else (pow2_override or qb.power_2_scale)
    if pa == pb and qa.amax_epsilon == 0.0 and qb.amax_epsilon == 0.0:
        return fp8_blockwise_linear(a, b, pa)
    qx, sx = quantize_1x128_ref(a, pa, qa.amax_epsilon)
    qw, sw = quantize_128x128_ref(b, pb, qb.amax_epsilon)
    return (dequantize_1x128(qx, sx) @ dequantize_128x128(qw, sw).t()).to(a.dtype)


def fp8_linear_supported(in_features: int, out_features: int) -> bool:
    return in_features % 128 == 0 and out_features % 128 == 0


def fp8_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
               residual: Optional[torch.Tensor] = None, pow2: bool = False) -> torch.Tensor:
    """Drop-in for ``functional.linear`` on shapes whose feature sizes are multiples of 128."""
    shape = x.shape
    y = _Fp8LinearFn.apply(x.reshape(-1, shape[-1]).contiguous(), weight, pow2).reshape(*shape[:-1], weight.shape[0])
    if bias is not None:
        y = y + bias
    if residual is not None:
        y = y + residual
    return y
