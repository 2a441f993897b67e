"""Quantised checkpoint formats the converter reads and writes (reference: tools/convert_checkpoint fp8 TE / pt
quant + dequant, INT4 compressed-tensors and MXFP4 dequantisation paths):

* FP8 block format of DeepSeek-V3 style HF checkpoints: ``weight`` in e4m3 with ``weight_scale_inv`` fp32 per
  128 x 128 block (ragged edge blocks allowed);
* INT4 "compressed-tensors" pack-quantised format: signed 4-bit values, eight per int32 along the input dim,
  group-wise scales (and optional zero points) per ``group_size`` input columns;
* MXFP4 (OCP microscaling): e2m1 values, two per byte, one shared e8m0 exponent per 32 values.
"""
from __future__ import annotations

import math
from typing import Dict, Optional, Tuple

import torch

E4M3_MAX = 448.0
_FP4_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0])


# ---- FP8 128x128 block format ------------------------------------------------------------------------------------
def fp8_block_quantize(w: torch.Tensor, block: int = 128) -> Tuple[torch.Tensor, torch.Tensor]:
    """-> (weight e4m3 [N, K], weight_scale_inv fp32 [ceil(N/b), ceil(K/b)]) with w ~= weight * scale_inv per block."""
    N, K = w.shape
    nb, kb = math.ceil(N / block), math.ceil(K / block)
    pad = torch.zeros(nb * block, kb * block, dtype=torch.float32)
    pad[:N, :K] = w.float()
    blocks = pad.view(nb, block, kb, block)
    scale = blocks.abs().amax(dim=(1, 3)).clamp(min=1e-12) / E4M3_MAX
    q = (blocks / scale[:, None, :, None]).clamp(-E4M3_MAX, E4M3_MAX).view(nb * block, kb * block)[:N, :K]
    return q.to(torch.float8_e4m3fn), scale


def fp8_block_dequantize(weight: torch.Tensor, scale_inv: torch.Tensor, block: int = 128,
                         dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
    N, K = weight.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return (weight.float() * s).to(dtype)


def dequantize_fp8_state_dict(sd: Dict[str, torch.Tensor], dtype=torch.bfloat16) -> Dict[str, torch.Tensor]:
    """Replaces every (``X.weight`` e4m3, ``X.weight_scale_inv``) pair by the de-quantised ``X.weight``."""
    out = {}
    for k, v in sd.items():
        if k.endswith(".weight_scale_inv"):
            continue
        s = sd.get(k + "_scale_inv") if k.endswith(".weight") else None
        out[k] = fp8_block_dequantize(v, s, dtype=dtype) if s is not None else v
    return out


def quantize_fp8_state_dict(sd: Dict[str, torch.Tensor], should_quantize=lambda k, v: v.dim() == 2 and "embed" not in k
                            and "lm_head" not in k and "norm" not in k) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        if k.endswith(".weight") and should_quantize(k, v):
            q, s = fp8_block_quantize(v)
            out[k], out[k + "_scale_inv"] = q, s
        else:
            out[k] = v
    return out


# ---- INT4 compressed-tensors (pack-quantised) -----------------------------------------------------------------------
def int4_pack(w: torch.Tensor, group_size: int = 128, symmetric: bool = True):
    """-> (weight_packed int32 [N, K/8], weight_scale [N, K/g], weight_zero_point int32 [N, K/g] or None)."""
    N, K = w.shape
    g = w.float().view(N, K // group_size, group_size)
    if symmetric:
        scale = g.abs().amax(-1).clamp(min=1e-12) / 7.0
        q = torch.round(g / scale.unsqueeze(-1)).clamp(-8, 7).to(torch.int32)
        zp = None
        u = q + 8  # stored as offset-binary nibbles
    else:
        lo, hi = g.amin(-1), g.amax(-1)
        scale = ((hi - lo) / 15.0).clamp(min=1e-12)
        zp = torch.round(-lo / scale).clamp(0, 15).to(torch.int32)
        u = (torch.round(g / scale.unsqueeze(-1)) + zp.unsqueeze(-1)).clamp(0, 15).to(torch.int32)
    u = u.view(N, K // 8, 8)
    packed = torch.zeros(N, K // 8, dtype=torch.int32)
    for i in range(8):
        packed |= u[..., i] << (4 * i)
    return packed, scale, zp


def int4_unpack(packed: torch.Tensor, scale: torch.Tensor, zero_point: Optional[torch.Tensor] = None,
                group_size: int = 128, dtype=torch.bfloat16) -> torch.Tensor:
    N = packed.shape[0]
    u = torch.stack([(packed >> (4 * i)) & 0xF for i in range(8)], dim=-1).view(N, -1)
    K = u.shape[1]
    g = u.view(N, K // group_size, group_size).float()
    g = g - (8.0 if zero_point is None else zero_point.unsqueeze(-1).float())
    return (g * scale.unsqueeze(-1).float()).view(N, K).to(dtype)


# ---- MXFP4 ------------------------------------------------------------------------------------------------------------
def mxfp4_dequantize(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
    """blocks uint8 [..., G, 16] (two e2m1 values per byte, low nibble first), scales uint8 [..., G] (e8m0, bias 127)
    -> [..., G * 32]."""
    lut = _FP4_VALUES.to(blocks.device)
    lo, hi = (blocks & 0xF).long(), (blocks >> 4).long()
    vals = torch.stack([lut[lo], lut[hi]], dim=-1).flatten(-2)  # [..., G, 32]
    out = vals * torch.exp2(scales.float() - 127.0).unsqueeze(-1)
    return out.flatten(-2).to(dtype)


def mxfp4_quantize(w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Inverse of :func:`mxfp4_dequantize` (nearest e2m1 value, shared power-of-two scale per 32 values)."""
    g = w.float().reshape(*w.shape[:-1], -1, 32)
    amax = g.abs().amax(-1).clamp(min=2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scaled = g / torch.exp2(e).unsqueeze(-1)
    idx = (scaled.unsqueeze(-1) - _FP4_VALUES).abs().argmin(-1)
    idx = idx.view(*g.shape[:-1], 16, 2)
    blocks = (idx[..., 0] | (idx[..., 1] << 4)).to(torch.uint8)
    return blocks, (e + 127).to(torch.uint8)
