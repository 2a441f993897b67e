"""Qwen2/2.5-VL style vision transformer and MLP projector.

Patch embedding (a Conv3d with kernel = stride, i.e. one GEMM over flattened
``C x t_patch x patch x patch`` pixel patches), 2-D rotary position ids, window attention expressed as
per-layer ``cu_seqlens`` over a window-major token order (full attention on the layers listed in
``fullatt_block_indexes``), and the 2x2 spatial-merge MLP projector that also restores the original
token order. Counterpart of loongforge/models/encoder/base_vision_models/base_vision_model.py:41-174,
loongforge/models/encoder/qwen2_vl_vision_models/vision_model.py:39-160 and adapter.py:16-91.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from ..ops import functional as OF
from ..parallel import layers as PL
from .config import TransformerConfig
from .transformer import Norm, PackedSeqParams, RotaryInputs, TransformerLayer


def rot_pos_ids(grid_thw: torch.Tensor, merge: int) -> torch.Tensor:
    """[n_patches, 2] (h, w) position of every patch, patches ordered in 2x2 merge units."""
    out = []
    for t, h, w in grid_thw.tolist():
        hp = torch.arange(h).unsqueeze(1).expand(-1, w)
        wp = torch.arange(w).unsqueeze(0).expand(h, -1)

        def unit_order(x):
            return x.reshape(h // merge, merge, w // merge, merge).permute(0, 2, 1, 3).flatten()

        ids = torch.stack([unit_order(hp), unit_order(wp)], dim=-1)
        out.append(ids.repeat(t, 1))
    return torch.cat(out, 0)


def window_index(grid_thw: torch.Tensor, window_px: int, patch: int, merge: int) -> Tuple[torch.Tensor, List[int]]:
    """Permutation of the merged units into window-major order and the cumulative window sizes
    (in PATCH tokens). Windows are ``window_px`` pixels square; ragged border windows are smaller."""
    win = window_px // patch // merge  # merged units per window side
    unit = merge * merge
    index, cu, base = [], [0], 0
    for t, h, w in grid_thw.tolist():
        gh, gw = h // merge, w // merge
        ids = torch.arange(t * gh * gw).reshape(t, gh, gw)
        ph, pw = (-gh) % win, (-gw) % win
        padded = torch.nn.functional.pad(ids, (0, pw, 0, ph), value=-100)
        nh, nw = (gh + ph) // win, (gw + pw) // win
        padded = padded.reshape(t, nh, win, nw, win).permute(0, 1, 3, 2, 4).reshape(t, nh * nw, win * win)
        counts = (padded != -100).sum(-1).reshape(-1)
        flat = padded.reshape(-1)
        index.append(flat[flat != -100] + base)
        for c in counts.tolist():
            if c > 0:
                cu.append(cu[-1] + c * unit)
        base += t * gh * gw
    return torch.cat(index), cu


class VisionRotary:
    def __init__(self, dim: int, theta: float = 10000.0):
        self.dim, self.theta = dim, theta  # dim = head_dim // 2 (half for h, half for w)

    def __call__(self, pos_hw: torch.Tensor) -> torch.Tensor:
        inv = 1.0 / (self.theta ** (torch.arange(0, self.dim, 2, dtype=torch.float32, device=pos_hw.device) / self.dim))
        fh = pos_hw[:, 0:1].float() * inv[None]
        fw = pos_hw[:, 1:2].float() * inv[None]
        return torch.cat([fh, fw], dim=-1).contiguous()  # [n, head_dim/2] angles


class PatchEmbed(nn.Module):
    def __init__(self, cfg: TransformerConfig, device=None):
        super().__init__()
        self.in_dim = cfg.in_channels * cfg.temporal_patch_size * cfg.patch_size * cfg.patch_size
        self.proj = nn.Module()
        w = PL.init_full_then_slice("vision.patch_embed.proj.weight", (cfg.hidden_size, self.in_dim),
                                    cfg.init_method_std, partition_dim=None, rank=0, world=1, device=device or "cpu",
                                    dtype=cfg.params_dtype)
        # stored with the Conv3d shape so that checkpoints interchange
        self.proj.weight = nn.Parameter(w.view(cfg.hidden_size, cfg.in_channels, cfg.temporal_patch_size,
                                               cfg.patch_size, cfg.patch_size))
        PL.mark_tp(self.proj.weight, None)

    def forward(self, pixels: torch.Tensor) -> torch.Tensor:
        w = self.proj.weight.view(self.proj.weight.shape[0], -1)
        x = pixels.to(w.dtype)
        pad = (-x.shape[1]) % 8
        if pad and x.is_cuda:  # the GEMM wants 16-byte rows
            x = torch.nn.functional.pad(x, (0, pad))
            w = torch.nn.functional.pad(w, (0, pad))
        return OF.linear(x, w)


class VisionModel(nn.Module):
    """ViT over flattened pixel patches ``[n_patches, C*t*p*p]`` with ``grid_thw [n_images, 3]``."""

    def __init__(self, cfg: TransformerConfig, *, device=None, parallel_state: Optional[str] = None):
        super().__init__()
        self.cfg = cfg
        self.patch_embed = PatchEmbed(cfg, device)
        self.rotary = VisionRotary(cfg.kv_channels // 2, cfg.rotary_base)
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList([TransformerLayer(cfg, i, device=device, parallel_state=parallel_state)
                                             for i in range(cfg.num_layers)])
        self.full_layers = set(cfg.fullatt_block_indexes or range(cfg.num_layers))

    def forward(self, pixels: torch.Tensor, grid_thw: torch.Tensor):
        cfg = self.cfg
        dev = pixels.device
        merge, unit = cfg.spatial_merge_size, cfg.spatial_merge_size ** 2
        x = self.patch_embed(pixels)
        n = x.shape[0]
        pos = rot_pos_ids(grid_thw.cpu(), merge).to(dev)
        widx, cu_win = window_index(grid_thw.cpu(), cfg.vision_window_size, cfg.patch_size, merge)
        widx = widx.to(dev)
        # window-major order of merge units (each unit = `unit` consecutive patch tokens)
        x = x.view(n // unit, unit, -1)[widx].reshape(n, -1)
        pos = pos.view(n // unit, unit, 2)[widx].reshape(n, 2)
        rotary = RotaryInputs(freqs=self.rotary(pos))
        cu_full = [0]
        for t, h, w in grid_thw.tolist():
            for _ in range(t):
                cu_full.append(cu_full[-1] + h * w)
        p_win = PackedSeqParams(torch.tensor(cu_win, dtype=torch.int32, device=dev), max(b - a for a, b in zip(cu_win, cu_win[1:])))
        p_full = PackedSeqParams(torch.tensor(cu_full, dtype=torch.int32, device=dev), max(b - a for a, b in zip(cu_full, cu_full[1:])))
        rec = cfg.recompute_granularity == "full" and torch.is_grad_enabled()
        for i, layer in enumerate(self.decoder.layers):
            packed = p_full if i in self.full_layers else p_win
            if rec:
                x = torch.utils.checkpoint.checkpoint(layer, x, rotary, packed, use_reentrant=False)
            else:
                x = layer(x, rotary, packed)
        return x, widx


class MLPAdapter(nn.Module):
    """RMSNorm -> merge 2x2 patch features -> fc1 -> GELU -> fc2 -> original (un-windowed) order."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, *, device=None, activation: str = "gelu"):
        super().__init__()
        unit = vit_cfg.spatial_merge_size ** 2
        self.unit = unit
        self.layernorm = Norm(vit_cfg.hidden_size, vit_cfg, device=device)
        hid = vit_cfg.hidden_size * unit
        self.linear_fc1 = PL.ColumnParallelLinear(hid, hid, bias=True, init_std=vit_cfg.init_method_std,
                                                  key="adapter.linear_fc1", gather_output=True,
                                                  params_dtype=vit_cfg.params_dtype, device=device)
        self.linear_fc2 = PL.ColumnParallelLinear(hid, out_hidden, bias=True, init_std=vit_cfg.init_method_std,
                                                  key="adapter.linear_fc2", gather_output=True,
                                                  params_dtype=vit_cfg.params_dtype, device=device)
        self.activation = activation

    def forward(self, x: torch.Tensor, window_idx: torch.Tensor) -> torch.Tensor:
        x = self.layernorm(x).view(x.shape[0] // self.unit, -1)
        x = self.linear_fc2(torch.nn.functional.gelu(self.linear_fc1(x)))
        return x[torch.argsort(window_idx)]
