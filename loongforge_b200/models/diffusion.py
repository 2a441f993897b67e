"""Diffusion transformers: WAN 2.1/2.2 video DiT and Qwen-Image double-stream MMDiT, with flow-matching
and Gaussian-diffusion training objectives.

* ``WanModel``: 1x2x2 patch embedding of video latents, sinusoidal timestep embedding -> 6-way AdaLN
  modulation per block, self-attention with full-width QK RMSNorm and 3-D (frame, height, width) RoPE,
  cross-attention to text (and optional image) context, GELU-tanh FFN, modulated head, un-patchify
  (loongforge/models/diffusion/wan/wan_model.py, wan_layer.py:38-, wan_attention.py:87,365).
* ``QwenImageModel``: double-stream blocks — image and text tokens keep separate norms / QKV / MLP /
  modulation and attend JOINTLY over the concatenated sequence
  (loongforge/models/diffusion/qwen_image/qwen_image_layer.py:54,233, qwen_image_model.py:34,
  qwen_image_modules.py:47-260).
* ``FlowMatchScheduler`` (wan_flow_match.py:13) and ``GaussianDiffusion`` (gaussian_diffusion.py:186).

Sequence parallelism for long videos is Ulysses (all-to-all between sequence and head sharding,
``parallel/ulysses.py``), selected by passing ``ulysses_group``.
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF


@dataclasses.dataclass
class DiTConfig:
    hidden_size: int = 1536
    num_heads: int = 12
    num_layers: int = 30
    ffn_hidden_size: int = 8960
    in_channels: int = 16
    out_channels: int = 16
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    text_dim: int = 4096
    freq_dim: int = 256
    image_context_dim: Optional[int] = None  # WAN i2v: CLIP image tokens as extra cross-attention context
    eps: float = 1e-6
    rope_theta: float = 10000.0
    params_dtype: torch.dtype = torch.float32

    @property
    def head_dim(self) -> int:
        return self.hidden_size // self.num_heads


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


def rope_3d_inv(head_dim: int, theta: float, device):
    """Inverse frequencies [head_dim/2] and the axis (0 frame, 1 row, 2 column) each one follows: the head dim is
    split (d - 2*(d//3)) | d//3 | d//3 (rounded to even) over frame / row / column."""
    d_h = d_w = 2 * (head_dim // 6)
    d_f = head_dim - d_h - d_w
    inv, axis = [], []
    for a, d in enumerate((d_f, d_h, d_w)):
        inv.append(1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32, device=device) / d)))
        axis.append(torch.full((d // 2,), a, dtype=torch.long, device=device))
    return torch.cat(inv), torch.cat(axis)


def rope_3d_angles_at(pos: torch.Tensor, head_dim: int, theta: float) -> torch.Tensor:
    """pos [L, 3] (frame, row, column) -> angles [L, head_dim/2]."""
    inv, axis = rope_3d_inv(head_dim, theta, pos.device)
    return pos.float()[:, axis] * inv


def rope_3d_angles(grid: Tuple[int, int, int], head_dim: int, theta: float, device) -> torch.Tensor:
    """Angles [F*H*W, head_dim/2] of a raster-ordered (frame, row, column) grid."""
    f, h, w = grid
    pos = torch.stack(torch.meshgrid(torch.arange(f, device=device), torch.arange(h, device=device),
                                     torch.arange(w, device=device), indexing="ij"), dim=-1).reshape(-1, 3)
    return rope_3d_angles_at(pos, head_dim, theta)


def apply_rope_interleaved(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x [B, L, H, d], angles [L, d/2]; pairs (x0, x1), (x2, x3), ... rotate (complex multiplication)."""
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    cos, sin = angles.cos()[None, :, None, :], angles.sin()[None, :, None, :]
    a, b = xf[..., 0], xf[..., 1]
    return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2).to(x.dtype)


def _attention(q, k, v, ulysses_group=None):
    """q [B, Lq, H, d], k/v [B, Lk, H, d] -> [B, Lq, H*d]; non-causal."""
    if ulysses_group is not None:
        from ..parallel.ulysses import ulysses_attention
        return ulysses_attention(q, k, v, ulysses_group)
    B, Lq, H, d = q.shape
    if q.is_cuda and q.dtype == torch.bfloat16 and d == 128 and k.shape[1] == Lq:
        cu = torch.arange(0, B + 1, device=q.device, dtype=torch.int32) * Lq
        o = OF.attention(q.reshape(B * Lq, H, d), k.reshape(B * Lq, H, d), v.reshape(B * Lq, H, d), causal=False,
                         scale=d ** -0.5, cu_seqlens=cu)
        return o.reshape(B, Lq, H * d)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
    return o.transpose(1, 2).reshape(B, Lq, H * d)


class RMSNorm(nn.Module):
    def __init__(self, dim: int, eps: float, device=None, dtype=None):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[-1] % 8 == 0:
            return OF.rmsnorm(x.reshape(-1, x.shape[-1]), self.weight, self.eps).view(x.shape)
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()).to(x.dtype)


class _Linear(nn.Linear):
    """nn.Linear whose GEMM runs on the framework GEMM for bf16 CUDA inputs."""

    def forward(self, x):
        if x.is_cuda and x.dtype == torch.bfloat16 and self.in_features % 8 == 0 and self.out_features % 8 == 0:
            y = OF.linear(x.reshape(-1, x.shape[-1]), self.weight, self.bias)
            return y.view(*x.shape[:-1], self.out_features)
        return super().forward(x)


class WanSelfAttention(nn.Module):
    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        self.h, self.d = cfg.num_heads, cfg.head_dim
        self.q, self.k, self.v, self.o = (_Linear(C, C, **kw) for _ in range(4))
        self.norm_q, self.norm_k = RMSNorm(C, cfg.eps, **kw), RMSNorm(C, cfg.eps, **kw)

    def forward(self, x, angles, ulysses_group=None, cu_seqlens=None):
        B, L, C = x.shape
        q = self.norm_q(self.q(x)).view(B, L, self.h, self.d)
        k = self.norm_k(self.k(x)).view(B, L, self.h, self.d)
        v = self.v(x).view(B, L, self.h, self.d)
        q, k = apply_rope_interleaved(q, angles), apply_rope_interleaved(k, angles)
        if cu_seqlens is not None:
            # several samples packed into one token row: attention stays inside each sample
            o = OF.attention(q[0], k[0], v[0], causal=False, scale=self.d ** -0.5, cu_seqlens=cu_seqlens)
            return self.o(o.reshape(1, L, C))
        return self.o(_attention(q, k, v, ulysses_group))


class WanCrossAttention(nn.Module):
    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        self.h, self.d = cfg.num_heads, cfg.head_dim
        self.q, self.k, self.v, self.o = (_Linear(C, C, **kw) for _ in range(4))
        self.norm_q, self.norm_k = RMSNorm(C, cfg.eps, **kw), RMSNorm(C, cfg.eps, **kw)
        self.has_image = cfg.image_context_dim is not None
        if self.has_image:
            self.k_img, self.v_img = _Linear(C, C, **kw), _Linear(C, C, **kw)
            self.norm_k_img = RMSNorm(C, cfg.eps, **kw)

    def forward(self, x, context, image_context=None):
        B, L, C = x.shape
        q = self.norm_q(self.q(x)).view(B, L, self.h, self.d)
        k = self.norm_k(self.k(context)).view(B, -1, self.h, self.d)
        v = self.v(context).view(B, -1, self.h, self.d)
        o = _attention(q, k, v)
        if self.has_image and image_context is not None:
            ki = self.norm_k_img(self.k_img(image_context)).view(B, -1, self.h, self.d)
            vi = self.v_img(image_context).view(B, -1, self.h, self.d)
            o = o + _attention(q, ki, vi)
        return self.o(o)


class WanBlock(nn.Module):
    """x += g1 * SelfAttn(LN(x) * (1 + s1) + b1); x += CrossAttn(LN3(x)); x += g2 * FFN(LN(x) * (1 + s2) + b2),
    with (b1, s1, g1, b2, s2, g2) = learned table + timestep projection."""

    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        self.norm1 = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.norm2 = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.norm3 = nn.LayerNorm(C, eps=cfg.eps, **kw)
        self.self_attn = WanSelfAttention(cfg, device)
        self.cross_attn = WanCrossAttention(cfg, device)
        self.ffn = nn.Sequential(_Linear(C, cfg.ffn_hidden_size, **kw), nn.GELU(approximate="tanh"),
                                 _Linear(cfg.ffn_hidden_size, C, **kw))
        self.modulation = nn.Parameter(torch.randn(1, 6, C, **kw) / C ** 0.5)

    def forward(self, x, e, angles, context, image_context=None, ulysses_group=None, cu_seqlens=None):
        """``e`` is ``[B, 6, C]`` (one modulation per sample) or, for packed rows, ``[1, L, 6, C]`` (per token; then
        `context` / `image_context` are lists with one entry per packed sample and `cu_seqlens` their boundaries)."""
        per_token = e.dim() == 4
        b1, s1, g1, b2, s2, g2 = (self.modulation.float().unsqueeze(1) + e.float() if per_token
                                  else self.modulation.float() + e.float()).unbind(-2)
        up = (lambda t: t) if per_token else (lambda t: t[:, None])

        def mod(n, s, b):
            return (n.float() * (1 + up(s)) + up(b)).to(x.dtype)

        x = x + (self.self_attn(mod(self.norm1(x), s1, b1), angles, ulysses_group, cu_seqlens).float() * up(g1)).to(x.dtype)
        h = self.norm3(x)
        if cu_seqlens is not None:
            b = cu_seqlens.tolist()
            parts = [self.cross_attn(h[:, s_:e_], context[i], image_context[i] if image_context is not None else None)
                     for i, (s_, e_) in enumerate(zip(b, b[1:]))]
            x = x + torch.cat(parts, dim=1)
        else:
            x = x + self.cross_attn(h, context, image_context)
        return x + (self.ffn(mod(self.norm2(x), s2, b2)).float() * up(g2)).to(x.dtype)


class WanModel(nn.Module):
    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        self.cfg = cfg
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        pt, ph, pw = cfg.patch_size
        self.patch_embedding = _Linear(cfg.in_channels * pt * ph * pw, C, **kw)  # Conv3d with kernel = stride
        self.text_embedding = nn.Sequential(_Linear(cfg.text_dim, C, **kw), nn.GELU(approximate="tanh"), _Linear(C, C, **kw))
        self.time_embedding = nn.Sequential(_Linear(cfg.freq_dim, C, **kw), nn.SiLU(), _Linear(C, C, **kw))
        self.time_projection = nn.Sequential(nn.SiLU(), _Linear(C, 6 * C, **kw))
        if cfg.image_context_dim is not None:
            self.img_emb = nn.Sequential(nn.LayerNorm(cfg.image_context_dim, **kw), _Linear(cfg.image_context_dim, C, **kw),
                                         nn.GELU(), _Linear(C, C, **kw), nn.LayerNorm(C, **kw))
        self.blocks = nn.ModuleList([WanBlock(cfg, device) for _ in range(cfg.num_layers)])
        self.head_norm = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.head = _Linear(C, cfg.out_channels * pt * ph * pw, **kw)
        self.head_modulation = nn.Parameter(torch.randn(1, 2, C, **kw) / C ** 0.5)
        self.recompute = False

    def patchify(self, x: torch.Tensor):
        """[B, C, F, H, W] -> tokens [B, L, C*pt*ph*pw], grid (f, h, w)."""
        B, C, Fr, H, W = x.shape
        pt, ph, pw = self.cfg.patch_size
        f, h, w = Fr // pt, H // ph, W // pw
        x = x.view(B, C, f, pt, h, ph, w, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, f * h * w, C * pt * ph * pw), (f, h, w)

    def unpatchify(self, tok: torch.Tensor, grid):
        B = tok.shape[0]
        pt, ph, pw = self.cfg.patch_size
        f, h, w = grid
        x = tok.view(B, f, h, w, self.cfg.out_channels, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return x.reshape(B, self.cfg.out_channels, f * pt, h * ph, w * pw)

    def forward(self, latents, timesteps, text_context, image_context=None, ulysses_group=None):
        """latents [B, C, F, H, W], timesteps [B], text_context [B, Lt, text_dim] -> prediction like `latents`."""
        cfg = self.cfg
        tok, grid = self.patchify(latents)
        angles = rope_3d_angles(grid, cfg.head_dim, cfg.rope_theta, tok.device)
        if ulysses_group is not None:
            # Every token-wise computation (patch embedding ... head) runs on THIS rank's tokens only, so each
            # parameter's gradient is the partial sum over the local tokens and one rule holds for all of them: sum
            # over the sequence-parallel group.
            from ..parallel.ulysses import shard_sequence
            tok = shard_sequence(tok, ulysses_group, dim=1)
            angles = shard_sequence(angles, ulysses_group, dim=0)  # RoPE is applied to the local tokens
        x = self.patch_embedding(tok.to(cfg.params_dtype))
        e0 = self.time_embedding(timestep_embedding(timesteps, cfg.freq_dim).to(cfg.params_dtype))
        e = self.time_projection(e0).view(-1, 6, cfg.hidden_size)
        ctx = self.text_embedding(text_context.to(cfg.params_dtype))
        img = self.img_emb(image_context.to(cfg.params_dtype)) if image_context is not None else None
        for blk in self.blocks:
            if self.recompute and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, e, angles, ctx, img, ulysses_group, use_reentrant=False)
            else:
                x = blk(x, e, angles, ctx, img, ulysses_group)
        b, s = (self.head_modulation.float() + e0.float()[:, None]).unbind(1)
        x = self.head((self.head_norm(x).float() * (1 + s[:, None]) + b[:, None]).to(x.dtype))
        if ulysses_group is not None:
            from ..parallel.ulysses import gather_sequence
            x = gather_sequence(x, ulysses_group, dim=1)
        return self.unpatchify(x, grid)


    def forward_packed(self, latents, timesteps, text_contexts, image_contexts=None):
        """Samples of DIFFERENT sizes in one token row (the reference's WAN packing, wan_model.py:34-115): `latents` is
        a list of ``[C, F_i, H_i, W_i]``, `timesteps` ``[n]``, `text_contexts` a list of ``[Lt_i, text_dim]``. Tokens of
        all samples are concatenated; self-attention is confined to each sample through ``cu_seqlens``, rotary angles
        restart per sample, the timestep modulation is looked up per token, cross-attention pairs each sample with its
        own context. Returns the list of predictions."""
        cfg = self.cfg
        toks, grids, angs = [], [], []
        for lat in latents:
            t, g = self.patchify(lat[None])
            toks.append(t[0])
            grids.append(g)
            angs.append(rope_3d_angles(g, cfg.head_dim, cfg.rope_theta, lat.device))
        lens = [t.shape[0] for t in toks]
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=toks[0].device)
        sample = torch.repeat_interleave(torch.arange(len(lens), device=cu.device), torch.tensor(lens, device=cu.device))
        x = self.patch_embedding(torch.cat(toks)[None].to(cfg.params_dtype))
        angles = torch.cat(angs)
        e0 = self.time_embedding(timestep_embedding(timesteps, cfg.freq_dim).to(cfg.params_dtype))   # [n, C]
        e = self.time_projection(e0).view(-1, 6, cfg.hidden_size)[sample][None]                       # [1, L, 6, C]
        ctx = [self.text_embedding(c[None].to(cfg.params_dtype)) for c in text_contexts]
        img = ([self.img_emb(c[None].to(cfg.params_dtype)) for c in image_contexts]
               if image_contexts is not None else None)
        for blk in self.blocks:
            if self.recompute and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, e, angles, ctx, img, None, cu, use_reentrant=False)
            else:
                x = blk(x, e, angles, ctx, img, None, cu)
        b, s_ = (self.head_modulation.float() + e0.float()[:, None]).unbind(1)                        # [n, C] each
        x = self.head((self.head_norm(x).float() * (1 + s_[sample][None]) + b[sample][None]).to(x.dtype))
        return [self.unpatchify(x[:, a:z], g)[0] for a, z, g in zip(cu.tolist(), cu.tolist()[1:], grids)]


# ----------------------------------------------------------------------------- Qwen-Image MMDiT
class _StreamParams(nn.Module):
    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        self.mod = nn.Sequential(nn.SiLU(), _Linear(C, 6 * C, **kw))
        self.norm1 = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.norm2 = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.qkv = _Linear(C, 3 * C, **kw)
        self.norm_q, self.norm_k = RMSNorm(cfg.head_dim, cfg.eps, **kw), RMSNorm(cfg.head_dim, cfg.eps, **kw)
        self.out = _Linear(C, C, **kw)
        self.mlp = nn.Sequential(_Linear(C, cfg.ffn_hidden_size, **kw), nn.GELU(approximate="tanh"),
                                 _Linear(cfg.ffn_hidden_size, C, **kw))


class QwenImageBlock(nn.Module):
    """Double-stream block: per-stream modulation / QKV / MLP, one joint attention over [text ; image]."""

    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        self.cfg = cfg
        self.img, self.txt = _StreamParams(cfg, device), _StreamParams(cfg, device)

    def _qkv(self, sp: _StreamParams, x, m):
        B, L, C = x.shape
        h, d = self.cfg.num_heads, self.cfg.head_dim
        xin = (sp.norm1(x).float() * (1 + m[1][:, None]) + m[0][:, None]).to(x.dtype)
        q, k, v = sp.qkv(xin).view(B, L, 3, h, d).unbind(2)
        return sp.norm_q(q), sp.norm_k(k), v

    def forward(self, img, txt, temb, img_angles, txt_angles=None):
        mi = self.img.mod(temb).float().chunk(6, dim=-1)
        mt = self.txt.mod(temb).float().chunk(6, dim=-1)
        qi, ki, vi = self._qkv(self.img, img, mi)
        qt, kt, vt = self._qkv(self.txt, txt, mt)
        qi, ki = apply_rope_interleaved(qi, img_angles), apply_rope_interleaved(ki, img_angles)
        if txt_angles is not None:
            qt, kt = apply_rope_interleaved(qt, txt_angles), apply_rope_interleaved(kt, txt_angles)
        Lt = txt.shape[1]
        o = _attention(torch.cat([qt, qi], 1), torch.cat([kt, ki], 1), torch.cat([vt, vi], 1))
        ot, oi = o[:, :Lt], o[:, Lt:]
        outs = []
        for sp, x, o_, m in ((self.img, img, oi, mi), (self.txt, txt, ot, mt)):
            x = x + (sp.out(o_).float() * m[2][:, None]).to(x.dtype)
            h = (sp.norm2(x).float() * (1 + m[4][:, None]) + m[3][:, None]).to(x.dtype)
            outs.append(x + (sp.mlp(h).float() * m[5][:, None]).to(x.dtype))
        return outs[0], outs[1]


class QwenImageModel(nn.Module):
    def __init__(self, cfg: DiTConfig, device=None):
        super().__init__()
        self.cfg = cfg
        C, kw = cfg.hidden_size, dict(device=device, dtype=cfg.params_dtype)
        self.img_in = _Linear(cfg.in_channels * 4, C, **kw)  # 2x2 packed latents
        self.txt_norm = RMSNorm(cfg.text_dim, cfg.eps, **kw)
        self.txt_in = _Linear(cfg.text_dim, C, **kw)
        self.time_embed = nn.Sequential(_Linear(cfg.freq_dim, C, **kw), nn.SiLU(), _Linear(C, C, **kw))
        self.blocks = nn.ModuleList([QwenImageBlock(cfg, device) for _ in range(cfg.num_layers)])
        self.norm_out = nn.LayerNorm(C, eps=cfg.eps, elementwise_affine=False)
        self.mod_out = nn.Sequential(nn.SiLU(), _Linear(C, 2 * C, **kw))
        self.proj_out = _Linear(C, cfg.out_channels * 4, **kw)

    def forward(self, img_tokens, timesteps, txt_tokens, grid_hw: Tuple[int, int]):
        """img_tokens [B, h*w, 4*C_lat] (2x2 packed latents), txt_tokens [B, Lt, text_dim]."""
        cfg = self.cfg
        img = self.img_in(img_tokens.to(cfg.params_dtype))
        txt = self.txt_in(self.txt_norm(txt_tokens.to(cfg.params_dtype)))
        temb = self.time_embed(timestep_embedding(timesteps * 1000.0, cfg.freq_dim).to(cfg.params_dtype))
        angles = rope_3d_angles((1, grid_hw[0], grid_hw[1]), cfg.head_dim, cfg.rope_theta, img.device)
        Lt = txt.shape[1]
        # text tokens sit on the diagonal beyond the image grid
        t_pos = (torch.arange(Lt, device=img.device) + max(grid_hw))[:, None].expand(Lt, 3)
        txt_angles = rope_3d_angles_at(t_pos, cfg.head_dim, cfg.rope_theta)
        for blk in self.blocks:
            img, txt = blk(img, txt, temb, angles, txt_angles)
        s, b = self.mod_out(temb).float().chunk(2, dim=-1)
        return self.proj_out((self.norm_out(img).float() * (1 + s[:, None]) + b[:, None]).to(img.dtype))


# ----------------------------------------------------------------------------- objectives
class FlowMatchScheduler:
    """Rectified-flow training: x_t = (1 - s) x0 + s * noise, target = noise - x0, sigma shift
    ``s' = shift * s / (1 + (shift - 1) * s)`` and a bell-shaped timestep weighting."""

    def __init__(self, num_train_timesteps: int = 1000, shift: float = 3.0, sigma_min: float = 0.0):
        self.n = num_train_timesteps
        s = torch.linspace(1.0, sigma_min, num_train_timesteps)
        self.sigmas = shift * s / (1 + (shift - 1) * s)
        self.timesteps = self.sigmas * num_train_timesteps
        y = torch.exp(-2 * ((self.timesteps - num_train_timesteps / 2) / num_train_timesteps) ** 2)
        self.weights = (y - y.min()) / (y - y.min()).sum() * num_train_timesteps

    def sample_timestep_ids(self, batch: int, generator=None) -> torch.Tensor:
        return torch.randint(0, self.n, (batch,), generator=generator)

    def add_noise(self, x0, noise, ids):
        s = self.sigmas.to(x0.device)[ids].view(-1, *([1] * (x0.dim() - 1))).to(x0.dtype)
        return (1 - s) * x0 + s * noise

    def training_target(self, x0, noise):
        return noise - x0

    def loss(self, pred, x0, noise, ids):
        w = self.weights.to(pred.device)[ids]
        per = (pred.float() - self.training_target(x0, noise).float()).pow(2).flatten(1).mean(1)
        return (per * w).mean()

    def step(self, pred, ids, x_t):
        """One Euler step of the sampler from timestep id to id + 1 (towards sigma = sigma_min)."""
        s = self.sigmas.to(x_t.device)
        nxt = torch.where(ids + 1 < self.n, s[(ids + 1).clamp(max=self.n - 1)], torch.zeros_like(s[ids]))
        return x_t + pred * (nxt - s[ids]).view(-1, *([1] * (x_t.dim() - 1))).to(x_t.dtype)


class GaussianDiffusion:
    """DDPM forward process and epsilon-prediction MSE (linear or cosine betas)."""

    def __init__(self, num_timesteps: int = 1000, schedule: str = "linear"):
        if schedule == "linear":
            scale = 1000 / num_timesteps
            betas = torch.linspace(scale * 1e-4, scale * 0.02, num_timesteps, dtype=torch.float64)
        elif schedule == "cosine":
            f = lambda t: math.cos((t + 0.008) / 1.008 * math.pi / 2) ** 2  # noqa: E731
            betas = torch.tensor([min(1 - f((i + 1) / num_timesteps) / f(i / num_timesteps), 0.999)
                                  for i in range(num_timesteps)], dtype=torch.float64)
        else:
            raise ValueError(schedule)
        self.betas = betas
        self.alphas_cumprod = torch.cumprod(1 - betas, 0)
        self.n = num_timesteps

    def q_sample(self, x0, t, noise):
        a = self.alphas_cumprod.to(x0.device)[t].view(-1, *([1] * (x0.dim() - 1)))
        return (a.sqrt() * x0.double() + (1 - a).sqrt() * noise.double()).to(x0.dtype)

    def predict_x0_from_eps(self, x_t, t, eps):
        a = self.alphas_cumprod.to(x_t.device)[t].view(-1, *([1] * (x_t.dim() - 1)))
        return ((x_t.double() - (1 - a).sqrt() * eps.double()) / a.sqrt()).to(x_t.dtype)

    def training_loss(self, model_fn, x0, t, noise=None):
        noise = torch.randn_like(x0) if noise is None else noise
        return F.mse_loss(model_fn(self.q_sample(x0, t, noise), t).float(), noise.float())
