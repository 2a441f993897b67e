"""Parts shared by the world-model policies (LingBot-VA, FastWAM, DreamZero, Cosmos3): every one of them denoises video
latents and action chunks with a WAN-style transformer, and they differ in how the two token kinds meet (one sequence
with a teacher-forcing mask, two experts with joint attention, a block-causal model with action registers, a packed
two-tower language model).

* ``rope_angles`` / ``apply_rope``     — rotary angles from explicit (frame, row, column) positions, fractional frames
  allowed (actions sit between video frames);
* ``masked_attention``                 — attention over ``[B, L, H, d]`` heads with a boolean mask;
* ``Attention`` / ``DiTBlock`` / ``Head`` / ``TimeEmbedder`` — the WAN block (modulated self-attention, text
  cross-attention, modulated FFN) split into steps, so that mixture-of-transformers models can run the attention jointly
  over tokens that were projected by different experts; modulation per sample ``[B, 6, C]`` or per token ``[B, L, 6, C]``;
* ``FlowSchedule``                     — shifted rectified-flow schedule addressed by timestep ids of any shape;
* ``CausalVideoVAE``                   — causal 3-D convolutional auto-encoder (T frames -> 1 + (T - 1) / 4 latent frames,
  8x spatial), the frozen latent codec of these policies;
* ``TextEncoder``                      — bidirectional transformer over instruction tokens (the place of the frozen umT5
  encoder whose embeddings the reference caches).

(reference: loongforge/embodied/model/lingbot_va/modules/wan_model.py:52-128,362-545, fastwam/wan/dit.py, fastwam/wan/vae.py,
dreamzero/modules/wan_video_vae.py, lingbot_va/modules/flow_match.py)
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import RMSNorm, _Linear, rope_3d_inv, timestep_embedding


def rope_angles(pos: torch.Tensor, head_dim: int, theta: float = 10000.0) -> torch.Tensor:
    """pos ``[..., 3]`` (frame, row, column; any real values) -> angles ``[..., head_dim/2]``."""
    inv, axis = rope_3d_inv(head_dim, theta, pos.device)
    return pos.float()[..., axis] * inv


def grid_positions(f: int, h: int, w: int, device=None, frame_offset: float = 0.0) -> torch.Tensor:
    """Raster-ordered positions ``[f*h*w, 3]`` of a latent grid."""
    g = torch.stack(torch.meshgrid(torch.arange(f, device=device), torch.arange(h, device=device),
                                   torch.arange(w, device=device), indexing="ij"), dim=-1).reshape(-1, 3).float()
    g[:, 0] += frame_offset
    return g


def action_positions(frames: int, per_frame: int, device=None, frame_offset: float = 0.0) -> torch.Tensor:
    """Positions ``[frames*per_frame, 3]`` of action tokens: the i-th of the n actions of a frame sits at frame
    ``f + (i + 1) / (n + 1)``, outside the image plane (row = column = -1)."""
    f = torch.arange(frames, device=device, dtype=torch.float32)[:, None]
    frac = torch.arange(1, per_frame + 1, device=device, dtype=torch.float32)[None, :] / (per_frame + 1)
    t = (f + frac + frame_offset).reshape(-1)
    return torch.stack([t, torch.full_like(t, -1.0), torch.full_like(t, -1.0)], dim=-1)


def apply_rope(x: torch.Tensor, angles: Optional[torch.Tensor]) -> torch.Tensor:
    """x ``[B, L, H, d]``, angles ``[L, d/2]`` or ``[B, L, d/2]``: interleaved pairs rotate."""
    if angles is None:
        return x
    if angles.dim() == 2:
        angles = angles[None]
    xf = x.float().reshape(*x.shape[:-1], -1, 2)
    cos, sin = angles.cos()[:, :, None, :], angles.sin()[:, :, None, :]
    a, b = xf[..., 0], xf[..., 1]
    return torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1).flatten(-2).to(x.dtype)


def masked_attention(q, k, v, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q ``[B, Lq, H, d]``, k / v ``[B, Lk, Hk, d]`` (Hk divides H) -> ``[B, Lq, H*d]``. ``mask`` is boolean (True = may
    attend), ``[Lq, Lk]``, ``[B, Lk]`` (key padding) or ``[B, 1|H, Lq, Lk]``."""
    if isinstance(mask, SegmentMask):
        return segment_attention(q, k, v, mask.starts, mask.ends, mask.seg_mask, mask.causal)
    B, Lq, H, d = q.shape
    if k.shape[2] != H:
        rep = H // k.shape[2]
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    if mask is not None:
        if mask.dim() == 2 and mask.shape[0] == B and mask.shape[1] == k.shape[1] and mask.shape != (Lq, k.shape[1]):
            mask = mask[:, None, None, :]
        elif mask.dim() == 2:
            mask = mask[None, None]
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), attn_mask=mask)
    return o.transpose(1, 2).reshape(B, Lq, H * d)


def contiguous_runs(*attrs: torch.Tensor):
    """Tokens with equal attributes in a row form a run. Returns (starts, ends, representative token of each run)."""
    a = torch.stack([x.reshape(-1).to(torch.float64) for x in attrs], dim=-1)
    change = torch.ones(a.shape[0], dtype=torch.bool, device=a.device)
    change[1:] = (a[1:] != a[:-1]).any(-1)
    starts = torch.nonzero(change).flatten()
    ends = torch.cat([starts[1:], torch.tensor([a.shape[0]], device=a.device)])
    return starts.tolist(), ends.tolist(), starts


def segment_attention(q, k, v, starts, ends, seg_mask: torch.Tensor, causal=None) -> torch.Tensor:
    """Attention under a mask that is constant on blocks: query run i attends ALL tokens of the key runs j with
    ``seg_mask[i, j]`` and nothing else. Every query run is one un-masked attention call over the concatenation of its
    key runs (adjacent ones are taken as one slice), so no ``[L, L]`` mask or score matrix exists and cost follows the
    allowed area only. q ``[B, L, H, d]``, k / v ``[B, L, Hk, d]`` -> ``[B, L, H*d]``. Query runs with the same key set are
    batched into one call. A run i with ``causal[i]`` attends its own tokens causally (text inside a packed row): it is one
    call of its own with a ``[run, keys]`` mask."""
    B, L, H, d = q.shape
    if k.shape[2] != H:
        rep = H // k.shape[2]
        k, v = k.repeat_interleave(rep, dim=2), v.repeat_interleave(rep, dim=2)
    out = q.new_empty(B, L, H * d)
    rows = seg_mask.tolist()
    groups: dict = {}
    for i, row in enumerate(rows):                      # runs that see the same keys share one call
        keys = tuple(j for j, ok in enumerate(row) if ok)
        own_causal = bool(causal is not None and causal[i] and row[i])
        groups.setdefault((keys, i if own_causal else -1), []).append(i)
    for (keys, own), qs in groups.items():
        assert keys, "a run of queries attends nothing"
        spans, cur = [], None                            # merge adjacent key runs into slices
        for j in keys:
            if cur is not None and starts[j] == cur[1]:
                cur[1] = ends[j]
            else:
                cur = [starts[j], ends[j]]
                spans.append(cur)
        kk = k[:, spans[0][0]:spans[0][1]] if len(spans) == 1 else torch.cat([k[:, a:b] for a, b in spans], dim=1)
        vv = v[:, spans[0][0]:spans[0][1]] if len(spans) == 1 else torch.cat([v[:, a:b] for a, b in spans], dim=1)
        qq = torch.cat([q[:, starts[i]:ends[i]] for i in qs], dim=1) if len(qs) > 1 else q[:, starts[qs[0]]:ends[qs[0]]]
        am = None
        if own >= 0:                                     # all of the other runs, the lower triangle of its own
            n = ends[own] - starts[own]
            am = torch.cat([torch.ones(n, ends[j] - starts[j], dtype=torch.bool, device=q.device) if j != own else
                            torch.ones(n, n, dtype=torch.bool, device=q.device).tril() for j in keys], dim=1)
        o = F.scaled_dot_product_attention(qq.transpose(1, 2), kk.transpose(1, 2), vv.transpose(1, 2), attn_mask=am).transpose(1, 2)
        o = o.reshape(B, -1, H * d)
        at = 0
        for i in qs:
            n = ends[i] - starts[i]
            out[:, starts[i]:ends[i]] = o[:, at:at + n]
            at += n
    return out


class SegmentMask:
    """A block-constant mask in run form; ``Attention`` / ``masked_attention`` callers pass it instead of a dense mask."""

    def __init__(self, starts, ends, seg_mask: torch.Tensor, causal=None):
        self.starts, self.ends, self.seg_mask, self.causal = starts, ends, seg_mask, causal

    def dense(self, device=None) -> torch.Tensor:
        L = self.ends[-1]
        owner = torch.zeros(L, dtype=torch.long)
        for i, (a, b) in enumerate(zip(self.starts, self.ends)):
            owner[a:b] = i
        m = self.seg_mask.cpu()[owner][:, owner]
        if self.causal is not None:
            idx = torch.arange(L)
            own_causal = torch.tensor([bool(c) for c in self.causal])[owner]
            m = m & ~(own_causal[:, None] & (owner[:, None] == owner[None, :]) & (idx[None, :] > idx[:, None]))
        return m.to(device)


class Attention(nn.Module):
    """WAN attention: q / k / v / o projections, RMS norm over the whole q and k rows, rotary on q and k."""

    def __init__(self, dim: int, heads: int, kv_dim: Optional[int] = None, eps: float = 1e-6, inner: Optional[int] = None,
                 qk_norm: bool = True):
        super().__init__()
        inner = inner or dim
        self.h, self.d = heads, inner // heads
        self.q, self.k, self.v = _Linear(dim, inner), _Linear(kv_dim or dim, inner), _Linear(kv_dim or dim, inner)
        self.o = _Linear(inner, dim)
        self.norm_q = RMSNorm(inner, eps) if qk_norm else nn.Identity()
        self.norm_k = RMSNorm(inner, eps) if qk_norm else nn.Identity()

    def project(self, x, angles=None, ctx=None, ctx_angles=None):
        src = x if ctx is None else ctx
        B = x.shape[0]
        q = apply_rope(self.norm_q(self.q(x)).view(B, -1, self.h, self.d), angles)
        k = apply_rope(self.norm_k(self.k(src)).view(B, -1, self.h, self.d), angles if ctx is None else ctx_angles)
        return q, k, self.v(src).view(B, -1, self.h, self.d)

    def forward(self, x, angles=None, mask=None, ctx=None):
        q, k, v = self.project(x, angles, ctx)
        return self.o(masked_attention(q, k, v, mask))


def _mod(e: torch.Tensor, table: torch.Tensor):
    """Learned table ``[1, n, C]`` + timestep projection ``[B, n, C]`` (per sample) or ``[B, L, n, C]`` (per token) -> n
    tensors that broadcast against ``[B, L, C]``."""
    if e.dim() == 4:
        return (table.float()[:, None] + e.float()).unbind(-2)
    return tuple(t[:, None] for t in (table.float() + e.float()).unbind(-2))


class DiTBlock(nn.Module):
    """x += g1 * SelfAttn(LN(x) (1 + s1) + b1); x += CrossAttn(LN(x), text); x += g2 * FFN(LN(x) (1 + s2) + b2). The three
    steps are separate methods: a mixture-of-transformers model calls ``attn_input`` / ``after_attention`` of each
    expert's block around ONE joint attention."""

    def __init__(self, dim: int, ffn_dim: int, heads: int, eps: float = 1e-6, cross_attn_norm: bool = True,
                 inner: Optional[int] = None, cross: bool = True):
        super().__init__()
        self.norm1 = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.attn1 = Attention(dim, heads, eps=eps, inner=inner)
        self.cross = cross
        if cross:
            self.norm2 = nn.LayerNorm(dim, eps=eps) if cross_attn_norm else nn.Identity()
            self.attn2 = Attention(dim, heads, eps=eps, inner=inner)
        self.norm3 = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.ffn = nn.Sequential(_Linear(dim, ffn_dim), nn.GELU(approximate="tanh"), _Linear(ffn_dim, dim))
        self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / dim ** 0.5)

    def attn_input(self, x, e):
        b1, s1, g1, b2, s2, g2 = _mod(e, self.scale_shift_table)
        return (self.norm1(x).float() * (1 + s1) + b1).to(x.dtype), (g1, b2, s2, g2)

    def after_attention(self, x, attn_out, rest, ctx=None, ctx_mask=None):
        g1, b2, s2, g2 = rest
        x = (x.float() + attn_out.float() * g1).to(x.dtype)
        if self.cross and ctx is not None:
            x = x + self.attn2(self.norm2(x), mask=ctx_mask, ctx=ctx)
        h = (self.norm3(x).float() * (1 + s2) + b2).to(x.dtype)
        return (x.float() + self.ffn(h).float() * g2).to(x.dtype)

    def forward(self, x, e, angles=None, ctx=None, mask=None, ctx_mask=None):
        h, rest = self.attn_input(x, e)
        return self.after_attention(x, self.attn1(h, angles, mask), rest, ctx, ctx_mask)


class TimeEmbedder(nn.Module):
    """Sinusoidal features -> MLP -> (embedding ``[..., C]``, modulation ``[..., n, C]``)."""

    def __init__(self, dim: int, freq_dim: int = 256, n_mod: int = 6):
        super().__init__()
        self.freq_dim, self.n = freq_dim, n_mod
        self.time_embedding = nn.Sequential(_Linear(freq_dim, dim), nn.SiLU(), _Linear(dim, dim))
        self.time_projection = nn.Sequential(nn.SiLU(), _Linear(dim, n_mod * dim))

    def forward(self, t: torch.Tensor, dtype=None) -> Tuple[torch.Tensor, torch.Tensor]:
        w = self.time_embedding[0].weight
        f = timestep_embedding(t.reshape(-1), self.freq_dim).to(w.dtype)
        emb = self.time_embedding(f)
        mod = self.time_projection(emb)
        return emb.view(*t.shape, -1), mod.view(*t.shape, self.n, -1)


class Head(nn.Module):
    """Final modulated LayerNorm + projection; ``temb`` is ``[B, C]`` or per token ``[B, L, C]``."""

    def __init__(self, dim: int, out_dim: int, eps: float = 1e-6):
        super().__init__()
        self.norm = nn.LayerNorm(dim, eps=eps, elementwise_affine=False)
        self.proj = _Linear(dim, out_dim)
        self.scale_shift_table = nn.Parameter(torch.randn(1, 2, dim) / dim ** 0.5)

    def forward(self, x, temb):
        t = temb.float()
        t = t[:, None] if t.dim() == 2 else t
        b, s = (self.scale_shift_table.float()[:, None] + t[:, :, None]).unbind(-2)
        return self.proj((self.norm(x).float() * (1 + s) + b).to(x.dtype))


class FlowSchedule:
    """x_t = (1 - s) x0 + s noise with s from a table of ``n`` shifted sigmas (id 0 = pure noise), target noise - x0, a
    bell-shaped weight per timestep. Ids may have any shape that broadcasts against the sample once ``expand`` unit
    axes are appended (per sample, per frame, ...)."""

    def __init__(self, n: int = 1000, shift: float = 3.0, sigma_min: float = 0.0, extra_one_step: bool = True):
        self.n, self.shift = n, shift
        s = torch.linspace(1.0, sigma_min, n + 1)[:-1] if extra_one_step else torch.linspace(1.0, sigma_min, n)
        self.sigmas = shift * s / (1 + (shift - 1) * s)
        self.timesteps = self.sigmas * n
        y = torch.exp(-2 * ((self.timesteps - n / 2) / n) ** 2)
        self.weights = (y - y.min()) * (n / (y - y.min()).sum())

    def sample_ids(self, shape, lo: float = 0.0, hi: float = 1.0, generator=None, beta: Optional[Tuple[float, float]] = None):
        """Uniform ids in ``[lo, hi) * n``; with ``beta = (a, b)`` the NOISE RATIO follows Beta(a, b) instead (high-noise
        emphasis), id = (1 - ratio) * n."""
        if beta is not None:
            r = torch.distributions.Beta(beta[0], beta[1]).sample(tuple(shape))
            return ((1 - r) * self.n).long().clamp(0, self.n - 1)
        u = torch.rand(tuple(shape), generator=generator) * (hi - lo) + lo
        return (u * self.n).long().clamp(0, self.n - 1)

    def _at(self, table, ids, ref, expand):
        v = table.to(ref.device)[ids.to(ref.device)]
        return v.view(*v.shape, *([1] * expand)).to(ref.dtype)

    def sigma(self, ids, ref, expand: int = 0):
        return self._at(self.sigmas, ids, ref, expand)

    def timestep(self, ids, ref):
        return self._at(self.timesteps, ids, ref, 0)

    def weight(self, ids, ref):
        return self._at(self.weights, ids, ref, 0)

    def add_noise(self, x0, noise, ids, expand: int):
        s = self.sigma(ids, x0, expand)
        return (1 - s) * x0 + s * noise

    def inference_sigmas(self, steps: int, device=None) -> torch.Tensor:
        """``steps + 1`` sigmas from 1 to 0 along the same shift."""
        s = torch.linspace(1.0, 0.0, steps + 1, device=device)
        return self.shift * s / (1 + (self.shift - 1) * s)


# ------------------------------------------------------------------------------------------------ latent codec
class CausalConv3d(nn.Conv3d):
    """3-D convolution that pads only the PAST side of the time axis (frame t never sees frame t + 1)."""

    def __init__(self, cin, cout, kernel=3, stride=(1, 1, 1)):
        k = (kernel,) * 3 if isinstance(kernel, int) else kernel
        super().__init__(cin, cout, k, stride=stride, padding=(0, k[1] // 2, k[2] // 2))
        self._tpad = k[0] - 1

    def forward(self, x):
        return super().forward(F.pad(x, (0, 0, 0, 0, self._tpad, 0)))


class _ChannelNorm(nn.Module):
    """RMS norm over the channels of every (frame, row, column) position: no statistics cross the time axis, so the
    codec stays causal (a group norm over the clip would not)."""

    def __init__(self, ch: int):
        super().__init__()
        self.gamma = nn.Parameter(torch.ones(1, ch, 1, 1, 1))

    def forward(self, x):
        return F.normalize(x.float(), dim=1).to(x.dtype) * (x.shape[1] ** 0.5) * self.gamma


class _Res3d(nn.Module):
    def __init__(self, cin, cout):
        super().__init__()
        self.n1, self.c1 = _ChannelNorm(cin), CausalConv3d(cin, cout)
        self.n2, self.c2 = _ChannelNorm(cout), CausalConv3d(cout, cout)
        self.skip = nn.Conv3d(cin, cout, 1) if cin != cout else nn.Identity()

    def forward(self, x):
        h = self.c1(F.silu(self.n1(x)))
        return self.skip(x) + self.c2(F.silu(self.n2(h)))


class CausalVideoVAE(nn.Module):
    """Video ``[B, 3, T, H, W]`` (T = 1 + 4k) <-> latents ``[B, z, 1 + k, H/8, W/8]``. Three spatial halvings, the last two
    also halve time with a stride-2 causal convolution (an odd number of frames 2m + 1 becomes m + 1: the first frame
    keeps a latent of its own, as WAN's codec does). The decoder mirrors it: a convolution doubles the channels, they
    are interleaved into twice the frames and the first (duplicate of nothing) frame is dropped. Latents are normalised
    with per-channel ``mean`` / ``std`` buffers."""

    def __init__(self, z_dim: int = 16, base: int = 32, spatial_stages: int = 3, temporal_stages: int = 2):
        super().__init__()
        self.z, self.ss, self.ts = z_dim, spatial_stages, temporal_stages
        ch = [base * 2 ** i for i in range(spatial_stages + 1)]
        enc = [CausalConv3d(3, ch[0])]
        for i in range(spatial_stages):
            t = 2 if i >= spatial_stages - temporal_stages else 1
            enc += [_Res3d(ch[i], ch[i]), CausalConv3d(ch[i], ch[i + 1], 3, stride=(t, 2, 2))]
        enc += [_Res3d(ch[-1], ch[-1]), _ChannelNorm(ch[-1]), nn.SiLU(), CausalConv3d(ch[-1], 2 * z_dim)]
        self.encoder = nn.Sequential(*enc)
        self.dec_in = CausalConv3d(z_dim, ch[-1])
        self.dec_res = nn.ModuleList([_Res3d(ch[i + 1], ch[i + 1]) for i in reversed(range(spatial_stages))])
        self.dec_up = nn.ModuleList([CausalConv3d(ch[i + 1], ch[i] * (2 if i >= spatial_stages - temporal_stages else 1))
                                     for i in reversed(range(spatial_stages))])
        self.dec_out = nn.Sequential(_ChannelNorm(ch[0]), nn.SiLU(), CausalConv3d(ch[0], 3))
        self.register_buffer("mean", torch.zeros(z_dim))
        self.register_buffer("std", torch.ones(z_dim))

    @property
    def temporal_factor(self) -> int:
        return 2 ** self.ts

    @property
    def spatial_factor(self) -> int:
        return 2 ** self.ss

    def latent_frames(self, frames: int) -> int:
        return 1 + (frames - 1) // self.temporal_factor

    def encode(self, video: torch.Tensor, sample: bool = False) -> torch.Tensor:
        assert (video.shape[2] - 1) % self.temporal_factor == 0, "the codec takes 1 + 4k frames"
        mu, logvar = self.encoder(video.to(self.mean.dtype)).chunk(2, dim=1)   # (the buffers follow the module's dtype)
        z = mu + torch.randn_like(mu) * (0.5 * logvar.clamp(-30, 20)).exp() if sample else mu
        return (z - self.mean.view(1, -1, 1, 1, 1)) / self.std.view(1, -1, 1, 1, 1)

    def decode(self, z: torch.Tensor) -> torch.Tensor:
        x = self.dec_in(z.to(self.mean.dtype) * self.std.view(1, -1, 1, 1, 1) + self.mean.view(1, -1, 1, 1, 1))
        for j, (res, up) in enumerate(zip(self.dec_res, self.dec_up)):
            i = self.ss - 1 - j
            x = up(res(x))
            if i >= self.ss - self.ts:  # time x2: channel halves interleave into frames, the first one is dropped
                B, C2, T, H, W = x.shape
                x = x.view(B, 2, C2 // 2, T, H, W).permute(0, 2, 3, 1, 4, 5).reshape(B, C2 // 2, 2 * T, H, W)[:, :, 1:]
            B, C, T, H, W = x.shape
            x = F.interpolate(x.transpose(1, 2).reshape(B * T, C, H, W), scale_factor=2.0, mode="nearest") \
                .view(B, T, C, 2 * H, 2 * W).transpose(1, 2)
        return self.dec_out(x)


class TextEncoder(nn.Module):
    """Instruction tokens ``[B, L]`` (0 = padding) -> ``[B, L, dim]`` with a few bidirectional pre-norm layers."""

    def __init__(self, vocab_size: int, dim: int, layers: int = 2, heads: int = 4, max_len: int = 512):
        super().__init__()
        self.embed = nn.Embedding(vocab_size, dim)
        self.pos = nn.Embedding(max_len, dim)
        self.layers = nn.ModuleList([nn.ModuleDict(dict(n1=RMSNorm(dim, 1e-6), attn=Attention(dim, heads, qk_norm=False),
                                                        n2=RMSNorm(dim, 1e-6),
                                                        ffn=nn.Sequential(_Linear(dim, 4 * dim), nn.GELU(), _Linear(4 * dim, dim))))
                                     for _ in range(layers)])
        self.norm = RMSNorm(dim, 1e-6)

    def forward(self, tokens: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
        mask = (tokens != 0) if mask is None else mask.bool()
        keep = mask.clone()
        keep[:, 0] = True  # an empty instruction still has one key
        x = self.embed(tokens) + self.pos(torch.arange(tokens.shape[1], device=tokens.device))[None]
        for l in self.layers:
            x = x + l["attn"](l["n1"](x), mask=keep)
            x = x + l["ffn"](l["n2"](x))
        return self.norm(x) * mask[..., None].to(x.dtype)


def video_from_batch(batch: dict, frames: int, multiple: int = 16) -> torch.Tensor:
    """``[B, 3, T, H, W]`` in [-1, 1] from a trainer batch: ``video`` (``[B, T, 3, H, W]`` or ``[B, 3, T, H, W]``, values in
    [0, 1]) when the data set provides future frames, otherwise the current camera-0 image repeated (a still video:
    enough for shape checks and action-only training, not for learning dynamics). Height and width are resized up to
    the next multiple of ``multiple`` (codec stride x patch size)."""
    if "video" in batch:
        v = batch["video"]
        v = v if v.shape[1] == 3 and v.shape[2] != 3 else v.transpose(1, 2)
        v = v.float() * 2 - 1
    else:
        img = batch["images"][:, 0].float() * 2 - 1
        v = img[:, :, None].expand(-1, -1, frames, -1, -1)
    B, C, T, H, W = v.shape
    Hn, Wn = -(-H // multiple) * multiple, -(-W // multiple) * multiple
    if (Hn, Wn) != (H, W):
        v = F.interpolate(v.transpose(1, 2).reshape(B * T, C, H, W), size=(Hn, Wn), mode="bilinear", align_corners=False) \
            .view(B, T, C, Hn, Wn).transpose(1, 2)
    return v.contiguous()
