"""Vision encoders and projectors beyond Qwen2/2.5-VL, built from one configurable ViT.

``GenericViT`` covers, by options:

* Qwen3-VL / Qwen3.5 ViT — learned position table bilinearly interpolated to each image grid, 2-D RoPE,
  DeepStack taps (features of chosen layers, each through its own merger, later added into early LLM
  layers) (loongforge/models/encoder/qwen3_vl_vision_models/vision_model.py:48-, qwen3_5_vision_models/);
* InternViT — class token + absolute position table, LayerScale on both residual branches, full-width
  TP-aware QK RMSNorm (loongforge/models/encoder/internvl_vision_models/intern_vision_attention.py:36-136,
  intern_vision_transformer_layer.py:21-49);
* RICE-ViT (LLaVA-OneVision-1.5) — 2-D RoPE, pre-norm ViT (llavaov1_5_vision_models/);
* MoonViT (Kimi) — interpolated learnable 2-D position table + 2-D RoPE (moon_vision_models/moon_vision_model.py:107-253);
* ERNIE-4.5-VL ViT — 2-D RoPE ViT feeding a variable-resolution resampler (ernie4_5_vl_vision_models/ernie_vision_model.py:103);
* MiniCPM-V 4.6 — ViT with a window-attention merger stage (minicpm_v_4_6_vision_models/vision_model.py:230).

Projectors: ``PixelShuffleAdapter`` (InternVL, adapter.py:25), ``PatchMergerAdapter`` (Moon,
patch_merger_adapter.py:13), ``ResamplerAdapter`` (ERNIE spatial 2x2 + temporal 2 fold), ``DownsampleMLPAdapter``
(MiniCPM-V merger.py:44). All take the packed patch sequence ``[n_patches, hidden]`` in raster order
per image and ``grid_thw``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..parallel import layers as PL
from .config import TransformerConfig
from .transformer import Norm, PackedSeqParams, RotaryInputs, TransformerLayer
from .vision import PatchEmbed, VisionRotary


def raster_pos_hw(grid_thw: torch.Tensor) -> torch.Tensor:
    """[n_patches, 2] (row, col) of every patch, raster order, repeated over time."""
    out = []
    for t, h, w in grid_thw.tolist():
        hh = torch.arange(h).unsqueeze(1).expand(h, w).reshape(-1)
        ww = torch.arange(w).unsqueeze(0).expand(h, w).reshape(-1)
        out.append(torch.stack([hh, ww], -1).repeat(t, 1))
    return torch.cat(out, 0)


def interpolate_pos_table(table: torch.Tensor, side: int, grid_thw: torch.Tensor) -> torch.Tensor:
    """Learned table [side*side, C] -> per-patch embeddings [n_patches, C], bilinear to every (h, w)."""
    C = table.shape[1]
    img = table.view(side, side, C).permute(2, 0, 1).unsqueeze(0).float()
    out = []
    for t, h, w in grid_thw.tolist():
        e = F.interpolate(img, size=(h, w), mode="bilinear", align_corners=False)[0].permute(1, 2, 0).reshape(h * w, C)
        out.append(e.repeat(t, 1))
    return torch.cat(out, 0).to(table.dtype)


class LayerScaleLayer(TransformerLayer):
    """x + ls1 * Attn(LN(x)); x + ls2 * MLP(LN(x)) with learned per-channel scales (InternViT)."""

    def __init__(self, cfg, layer_number, *, init_scale: float = 0.1, device=None, parallel_state=None):
        super().__init__(cfg, layer_number, device=device, parallel_state=parallel_state)
        self.ls1 = nn.Parameter(torch.full((cfg.hidden_size,), init_scale, device=device, dtype=cfg.params_dtype))
        self.ls2 = nn.Parameter(torch.full((cfg.hidden_size,), init_scale, device=device, dtype=cfg.params_dtype))
        for p in (self.ls1, self.ls2):
            PL.mark_tp(p, None, sequence_parallel=cfg.sequence_parallel)

    def forward(self, x, rotary=None, packed=None):
        h = self.input_layernorm(x) if self.input_layernorm is not None else x
        x = x + self.ls1 * self.self_attention(h, rotary, packed)
        h = self.pre_mlp_layernorm(x) if self.pre_mlp_layernorm is not None else x
        return x + self.ls2 * self.mlp(h)


class GenericViT(nn.Module):
    def __init__(self, cfg: TransformerConfig, *, pos_table_side: Optional[int] = None, rope_2d: bool = True,
                 cls_token: bool = False, layer_scale: bool = False, deepstack_indexes: Sequence[int] = (),
                 pre_norm: bool = False, post_norm: bool = False, patch_bias: bool = False, device=None,
                 parallel_state: Optional[str] = None):
        super().__init__()
        self.cfg, self.rope_2d, self.side = cfg, rope_2d, pos_table_side
        self.patch_embed = PatchEmbed(cfg, device)
        dt, dev = cfg.params_dtype, device or "cpu"
        if patch_bias:  # the patch convolution of InternViT / MoonViT / SigLIP-style towers has a bias
            self.patch_embed.proj.bias = nn.Parameter(torch.zeros(cfg.hidden_size, device=device, dtype=dt))
            PL.mark_tp(self.patch_embed.proj.bias, None)
        if pos_table_side:
            n = pos_table_side * pos_table_side + (1 if cls_token else 0)
            self.pos_embed = nn.Parameter(PL.init_full_then_slice("vision.pos_embed", (n, cfg.hidden_size), 0.02,
                                                                  partition_dim=None, rank=0, world=1, device=dev, dtype=dt))
            PL.mark_tp(self.pos_embed, None)
        else:
            self.pos_embed = None
        if cls_token:
            self.cls_token = nn.Parameter(torch.zeros(1, cfg.hidden_size, device=device, dtype=dt))
            PL.mark_tp(self.cls_token, None)
        else:
            self.cls_token = None
        self.rotary = VisionRotary(cfg.kv_channels // 2, cfg.rotary_base) if rope_2d else None
        Layer = LayerScaleLayer if layer_scale else TransformerLayer
        self.decoder = nn.Module()
        self.decoder.layers = nn.ModuleList([Layer(cfg, i, device=device, parallel_state=parallel_state)
                                             for i in range(cfg.num_layers)])
        self.pre_layernorm = Norm(cfg.hidden_size, cfg, device=device) if pre_norm else None
        self.post_layernorm = Norm(cfg.hidden_size, cfg, device=device) if post_norm else None
        self.deepstack_indexes = list(deepstack_indexes)

    def forward(self, pixels: torch.Tensor, grid_thw: torch.Tensor):
        """-> (features [n_tokens, hidden], list of DeepStack tap features). With a class token, one token per
        image/frame is prepended to that image's patches."""
        cfg, dev = self.cfg, pixels.device
        x = self.patch_embed(pixels)
        if getattr(self.patch_embed.proj, "bias", None) is not None:
            x = x + self.patch_embed.proj.bias.to(x.dtype)
        g = grid_thw.cpu()
        if self.pos_embed is not None:
            table = self.pos_embed[1:] if self.cls_token is not None else self.pos_embed
            x = x + interpolate_pos_table(table, self.side, g).to(dev)
        seq = [h * w for t, h, w in g.tolist() for _ in range(t)]
        pos = raster_pos_hw(g).to(dev)
        if self.cls_token is not None:
            parts, pparts, s = [], [], 0
            c = self.cls_token + self.pos_embed[:1]
            for n in seq:
                parts += [c, x[s:s + n]]
                pparts += [pos.new_zeros(1, 2), pos[s:s + n]]
                s += n
            x, pos = torch.cat(parts), torch.cat(pparts)
            seq = [n + 1 for n in seq]
        if self.pre_layernorm is not None:
            x = self.pre_layernorm(x)
        rotary = RotaryInputs(freqs=self.rotary(pos)) if self.rotary is not None else None
        cu = [0]
        for n in seq:
            cu.append(cu[-1] + n)
        packed = PackedSeqParams(torch.tensor(cu, dtype=torch.int32, device=dev), max(seq))
        taps: List[torch.Tensor] = []
        rec = cfg.recompute_granularity == "full" and torch.is_grad_enabled()
        for i, layer in enumerate(self.decoder.layers):
            if rec:
                x = torch.utils.checkpoint.checkpoint(layer, x, rotary, packed, use_reentrant=False)
            else:
                x = layer(x, rotary, packed)
            if i in self.deepstack_indexes:
                taps.append(x)
        if self.post_layernorm is not None:
            x = self.post_layernorm(x)
        return x, taps


def _linear(key: str, out_f: int, in_f: int, cfg: TransformerConfig, device, bias: bool = True) -> nn.Module:
    return PL.ColumnParallelLinear(in_f, out_f, bias=bias, init_std=cfg.init_method_std, key=key, gather_output=True,
                                   params_dtype=cfg.params_dtype, device=device)


def _merge_units(x: torch.Tensor, grid_thw: torch.Tensor, m: int) -> torch.Tensor:
    """Raster-ordered patches -> [n_units, m*m*C]: every m x m spatial neighbourhood concatenated."""
    out, s = [], 0
    for t, h, w in grid_thw.tolist():
        n = t * h * w
        seg = x[s:s + n].view(t, h // m, m, w // m, m, -1).permute(0, 1, 3, 2, 4, 5)
        out.append(seg.reshape(t * (h // m) * (w // m), -1))
        s += n
    return torch.cat(out, 0)


class PixelShuffleAdapter(nn.Module):
    """InternVL: drop the class token, fold every 2x2 neighbourhood into channels (pixel shuffle at scale 0.5),
    LayerNorm -> Linear -> GELU -> Linear."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, *, downsample: int = 2, device=None):
        super().__init__()
        self.m = downsample
        d = vit_cfg.hidden_size * downsample * downsample
        self.norm = nn.LayerNorm(d, device=device, dtype=vit_cfg.params_dtype)
        self.fc1 = _linear("adapter.pixel_shuffle.fc1", out_hidden, d, vit_cfg, device)
        self.fc2 = _linear("adapter.pixel_shuffle.fc2", out_hidden, out_hidden, vit_cfg, device)

    def forward(self, x, grid_thw, has_cls: bool = True):
        if has_cls:
            keep, s = [], 0
            for t, h, w in grid_thw.tolist():
                for _ in range(t):
                    keep.append(x[s + 1:s + 1 + h * w])
                    s += h * w + 1
            x = torch.cat(keep)
        u = _merge_units(x, grid_thw, self.m)
        return self.fc2(F.gelu(self.fc1(self.norm(u))))


class PatchMergerAdapter(nn.Module):
    """MoonViT: merge k x k patches, LayerNorm on the patch features, two-layer GELU MLP."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, *, merge: int = 2, device=None):
        super().__init__()
        self.m = merge
        d = vit_cfg.hidden_size * merge * merge
        self.pre_norm = nn.LayerNorm(vit_cfg.hidden_size, device=device, dtype=vit_cfg.params_dtype)
        self.fc1 = _linear("adapter.patch_merger.fc1", d, d, vit_cfg, device)
        self.fc2 = _linear("adapter.patch_merger.fc2", out_hidden, d, vit_cfg, device)

    def forward(self, x, grid_thw):
        return self.fc2(F.gelu(self.fc1(_merge_units(self.pre_norm(x), grid_thw, self.m))))


class ResamplerAdapter(nn.Module):
    """ERNIE-4.5-VL variable-resolution resampler: spatial m x m fold + MLP, then temporal fold of `tm`
    consecutive frames (a single frame is repeated) + MLP, projection to the LLM width, RMSNorm."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, *, spatial: int = 2, temporal: int = 2, device=None):
        super().__init__()
        self.m, self.tm = spatial, temporal
        d = vit_cfg.hidden_size * spatial * spatial
        self.spatial_fc1 = _linear("adapter.resampler.spatial_fc1", d, d, vit_cfg, device)
        self.spatial_fc2 = _linear("adapter.resampler.spatial_fc2", d, d, vit_cfg, device)
        self.spatial_norm = nn.LayerNorm(d, device=device, dtype=vit_cfg.params_dtype)
        self.temporal_fc1 = _linear("adapter.resampler.temporal_fc1", d, d * temporal, vit_cfg, device)
        self.temporal_fc2 = _linear("adapter.resampler.temporal_fc2", d, d, vit_cfg, device)
        self.temporal_norm = nn.LayerNorm(d, device=device, dtype=vit_cfg.params_dtype)
        self.proj = _linear("adapter.resampler.proj", out_hidden, d, vit_cfg, device)
        self.after_norm = Norm(out_hidden, vit_cfg, device=device)

    def forward(self, x, grid_thw):
        u = _merge_units(x, grid_thw, self.m)
        u = self.spatial_norm(self.spatial_fc2(F.gelu(self.spatial_fc1(u))))
        out, s = [], 0
        for t, h, w in grid_thw.tolist():
            per = (h // self.m) * (w // self.m)
            seg = u[s:s + t * per].view(t, per, -1)
            s += t * per
            if t % self.tm:
                seg = torch.cat([seg, seg[-1:].expand(self.tm - t % self.tm, -1, -1)], 0)
            seg = seg.view(-1, self.tm, per, seg.shape[-1]).permute(0, 2, 1, 3).reshape(-1, self.tm * seg.shape[-1])
            out.append(seg)
        v = torch.cat(out, 0)
        v = self.temporal_norm(self.temporal_fc2(F.gelu(self.temporal_fc1(v))))
        return self.after_norm(self.proj(v))


class DownsampleMLPAdapter(nn.Module):
    """MiniCPM-V 4.6: a window-attention merger stage (one non-causal layer over m x m windows) followed by the
    m x m fold and a two-layer MLP."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, *, merge: int = 2, device=None, parallel_state=None):
        super().__init__()
        self.m = merge
        self.window_layer = TransformerLayer(vit_cfg, vit_cfg.num_layers, device=device, parallel_state=parallel_state)
        d = vit_cfg.hidden_size * merge * merge
        self.norm = nn.LayerNorm(d, device=device, dtype=vit_cfg.params_dtype)
        self.fc1 = _linear("adapter.downsample.fc1", d, d, vit_cfg, device)
        self.fc2 = _linear("adapter.downsample.fc2", out_hidden, d, vit_cfg, device)

    def forward(self, x, grid_thw):
        # window-major order: each m x m window is one short sequence
        u = _merge_units(x, grid_thw, self.m)
        n_units, C = u.shape[0], x.shape[1]
        win = u.view(n_units * self.m * self.m, C)
        cu = torch.arange(0, n_units + 1, device=x.device, dtype=torch.int32) * (self.m * self.m)
        win = self.window_layer(win, None, PackedSeqParams(cu, self.m * self.m))
        return self.fc2(F.gelu(self.fc1(self.norm(win.view(n_units, -1)))))


class DeepStackMergers(nn.Module):
    """One 2x2 merger MLP per DeepStack tap (Qwen3-VL): tap features -> LLM width, to be added to the hidden
    states of the first LLM layers at the image-token positions."""

    def __init__(self, vit_cfg: TransformerConfig, out_hidden: int, n_taps: int, *, merge: int = 2, device=None):
        super().__init__()
        self.m = merge
        d = vit_cfg.hidden_size * merge * merge
        self.norms = nn.ModuleList([nn.LayerNorm(d, device=device, dtype=vit_cfg.params_dtype) for _ in range(n_taps)])
        self.fc1 = nn.ModuleList([_linear(f"adapter.deepstack.{i}.fc1", d, d, vit_cfg, device) for i in range(n_taps)])
        self.fc2 = nn.ModuleList([_linear(f"adapter.deepstack.{i}.fc2", out_hidden, d, vit_cfg, device)
                                  for i in range(n_taps)])

    def forward(self, taps: List[torch.Tensor], grid_thw) -> List[torch.Tensor]:
        return [f2(F.gelu(f1(n(_merge_units(t, grid_thw, self.m)))))
                for t, n, f1, f2 in zip(taps, self.norms, self.fc1, self.fc2)]


def make_deepstack_hook(features: List[torch.Tensor], image_mask: torch.Tensor):
    """Hook for ``TransformerBlock.deepstack_hook``: after LLM layer i (< number of taps) add tap i to the hidden
    states at image-token positions."""

    def hook(layer_idx: int, hidden: torch.Tensor) -> torch.Tensor:
        if layer_idx >= len(features):
            return hidden
        add = torch.zeros_like(hidden)
        add[image_mask] = features[layer_idx].to(hidden.dtype)
        return hidden + add

    return hook


VISION_FAMILIES = {
    # name: (GenericViT options, adapter class)
    "qwen3_vl_vit": (dict(pos_table_side=48, rope_2d=True, deepstack_indexes=(8, 16, 24)), None),
    "qwen3_5_vit": (dict(pos_table_side=48, rope_2d=True), None),
    "intern_vit": (dict(pos_table_side=32, rope_2d=False, cls_token=True, layer_scale=True, patch_bias=True), PixelShuffleAdapter),
    "rice_vit": (dict(rope_2d=True, pre_norm=True), None),
    "moon_vit": (dict(pos_table_side=64, rope_2d=True, post_norm=True, patch_bias=True), PatchMergerAdapter),
    "ernie_vit": (dict(rope_2d=True, post_norm=True), ResamplerAdapter),
    "minicpm_v_vit": (dict(pos_table_side=70, rope_2d=False, post_norm=True, patch_bias=True), DownsampleMLPAdapter),
}


def build_vision_encoder(family: str, cfg: TransformerConfig, *, device=None, parallel_state=None, **overrides):
    opts, _ = VISION_FAMILIES[family]
    return GenericViT(cfg, **{**opts, **overrides}, device=device, parallel_state=parallel_state)
