"""FastWAM: a WAN video expert and a narrower action expert as a mixture of transformers. Every layer projects each
expert's tokens with that expert's own weights to heads of ONE shared geometry (heads x head_dim), runs a single joint
attention over ``[video tokens | action tokens]`` under a mask, and hands each slice back to its expert's output
projection, text cross-attention and FFN. The experts have their own timestep (video and actions are noised
independently) and their own text embedding; the proprioceptive state is one more context token.

The first latent frame is the observation: it stays clean (its tokens are modulated with timestep 0 and get no loss).

Mask variants (``variant``):

* ``fastwam``  actions attend actions and the FIRST video frame only; video never attends actions. At test time the
  first frame's keys / values are computed once (``prefill_video_cache``) and only the action expert is denoised — no
  video is generated, which is what makes the policy fast;
* ``joint``    actions attend the whole video (video and actions are denoised together at test time);
* ``idm``      inverse-dynamics teacher forcing: ``[noisy video | condition video | actions]`` where the condition copy is
  clean (or, half of the time, lightly noised) and actions attend only it.

Video-to-video masks (``video_mask_mode``): ``bidirectional``, ``per_frame_causal``, ``first_frame_causal`` (the first frame
does not look at later frames, so its keys / values do not depend on them).

(reference: loongforge/embodied/model/fastwam/mot/fastwam.py:36-108,322-632,697-790,973-1120, mot/model.py:56-609,
mot/joint.py:28-62, mot/idm.py:29-254, action/dit.py:57-350, action/schedulers.py:51-80, wan/dit.py:693-728)
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import _Linear
from .wan_blocks import (CausalVideoVAE, DiTBlock, Head, SegmentMask, TextEncoder, TimeEmbedder, grid_positions, masked_attention,
                         rope_angles, video_from_batch)


@dataclasses.dataclass
class FastWAMConfig:
    # video expert (WAN 2.2 TI2V-5B geometry)
    hidden_size: int = 3072
    ffn_hidden_size: int = 14336
    num_heads: int = 24
    head_dim: int = 128
    num_layers: int = 30
    latent_channels: int = 48
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    # action expert: narrower, same heads / head_dim / depth
    action_hidden_size: int = 1024
    action_ffn_hidden_size: int = 4096
    action_dim: int = 7
    action_horizon: int = 16
    state_dim: Optional[int] = 8          # None: no proprioception token
    text_dim: int = 4096
    freq_dim: int = 256
    eps: float = 1e-6
    variant: str = "fastwam"              # fastwam | joint | idm
    video_mask_mode: str = "first_frame_causal"
    video_shift: float = 5.0
    action_shift: float = 1.0
    num_train_timesteps: int = 1000
    loss_lambda_video: float = 1.0
    loss_lambda_action: float = 1.0
    video_cond_noise_prob: float = 0.5    # idm: how often the condition video is noised
    video_frames: int = 9
    image_size: int = 224
    vocab_size: int = 32000
    text_layers: int = 2
    vae_base: int = 32
    freeze_text_encoder: bool = True
    recompute: bool = False
    segment_attention: bool = True        # evaluate the joint mask run by run (no [L, L] mask)

    @classmethod
    def tiny(cls, **kw) -> "FastWAMConfig":
        base = dict(hidden_size=48, ffn_hidden_size=96, num_heads=4, head_dim=8, num_layers=2, latent_channels=8,
                    action_hidden_size=24, action_ffn_hidden_size=48, text_dim=32, freq_dim=32, video_frames=5,
                    image_size=32, vae_base=8, action_horizon=4, text_layers=1)
        base.update(kw)
        return cls(**base)


def video_to_video_mask(frames: int, per_frame: int, mode: str, device=None) -> torch.Tensor:
    L = frames * per_frame
    if mode == "bidirectional":
        return torch.ones(L, L, dtype=torch.bool, device=device)
    if mode == "per_frame_causal":
        return torch.tril(torch.ones(frames, frames, dtype=torch.bool, device=device)) \
            .repeat_interleave(per_frame, 0).repeat_interleave(per_frame, 1)
    if mode == "first_frame_causal":
        m = torch.ones(L, L, dtype=torch.bool, device=device)
        m[:per_frame, per_frame:] = False
        return m
    raise ValueError(f"unknown video mask mode {mode!r}")


def mot_mask(variant: str, frames: int, per_frame: int, n_action: int, mode: str, device=None) -> torch.Tensor:
    """Joint mask over ``[video | action]`` (``idm``: ``[noisy video | condition video | action]``)."""
    vv = video_to_video_mask(frames, per_frame, mode, device)
    Lv = frames * per_frame
    if variant == "idm":
        L = 2 * Lv + n_action
        m = torch.zeros(L, L, dtype=torch.bool, device=device)
        m[:Lv, :Lv] = vv
        m[Lv:2 * Lv, Lv:2 * Lv] = vv
        m[2 * Lv:, 2 * Lv:] = True
        m[2 * Lv:, Lv:2 * Lv] = True
        return m
    L = Lv + n_action
    m = torch.zeros(L, L, dtype=torch.bool, device=device)
    m[:Lv, :Lv] = vv
    m[Lv:, Lv:] = True
    m[Lv:, :(Lv if variant == "joint" else per_frame)] = True
    return m


def mot_segment_mask(variant: str, frames: int, per_frame: int, n_action: int, mode: str, device=None) -> SegmentMask:
    """``mot_mask`` in run form: the mask is constant on frames and on the action block, so the rule evaluated with one token
    per frame and one action token is the run-level mask."""
    n_video = (2 if variant == "idm" else 1) * frames
    starts = [f * per_frame for f in range(n_video)] + [n_video * per_frame]
    ends = starts[1:] + [n_video * per_frame + n_action]
    return SegmentMask(starts, ends, mot_mask(variant, frames, 1, 1, mode, device))


class _Expert(nn.Module):
    """Blocks, timestep embedder and text embedding of one expert; ``inner`` = heads x head_dim is shared."""

    def __init__(self, dim: int, ffn: int, c: FastWAMConfig):
        super().__init__()
        inner = c.num_heads * c.head_dim
        self.time = TimeEmbedder(dim, c.freq_dim)
        self.text_embedding = nn.Sequential(_Linear(c.text_dim, dim), nn.GELU(approximate="tanh"), _Linear(dim, dim))
        self.blocks = nn.ModuleList([DiTBlock(dim, ffn, c.num_heads, c.eps, inner=inner) for _ in range(c.num_layers)])


class FastWAMModel(nn.Module):
    # the joint attention reaches into both experts' blocks and their attention projections
    FSDP_NO_WRAP = ("_Expert", "DiTBlock", "Attention", "FastWAMModel")

    def __init__(self, c: FastWAMConfig):
        super().__init__()
        self.c = c
        p = c.patch_size
        self.video = _Expert(c.hidden_size, c.ffn_hidden_size, c)
        self.action = _Expert(c.action_hidden_size, c.action_ffn_hidden_size, c)
        self.patch_embedding = _Linear(c.latent_channels * p[0] * p[1] * p[2], c.hidden_size)
        self.video_head = Head(c.hidden_size, c.latent_channels * p[0] * p[1] * p[2], c.eps)
        self.action_encoder = _Linear(c.action_dim, c.action_hidden_size)
        self.action_head = _Linear(c.action_hidden_size, c.action_dim)
        for lin in (self.action_encoder, self.action_head):
            nn.init.normal_(lin.weight, std=0.02)
            nn.init.zeros_(lin.bias)
        self.proprio_encoder = _Linear(c.state_dim, c.text_dim) if c.state_dim else None

    def patchify(self, lat):
        B, Cc, Fr, H, W = lat.shape
        pt, ph, pw = self.c.patch_size
        x = lat.view(B, Cc, Fr // pt, pt, H // ph, ph, W // pw, pw).permute(0, 2, 4, 6, 1, 3, 5, 7)
        return x.reshape(B, -1, Cc * pt * ph * pw), (Fr // pt, H // ph, W // pw)

    def unpatchify(self, tok, grid):
        B = tok.shape[0]
        pt, ph, pw = self.c.patch_size
        f, h, w = grid
        x = tok.view(B, f, h, w, self.c.latent_channels, pt, ph, pw).permute(0, 4, 1, 5, 2, 6, 3, 7)
        return x.reshape(B, self.c.latent_channels, f * pt, h * ph, w * pw)

    def context(self, text, text_mask, state):
        """Text (+ one proprioception token) for both experts; returns the raw context and its key mask."""
        if self.proprio_encoder is not None and state is not None:
            tok = self.proprio_encoder(state.to(text.dtype))[:, None]
            text = torch.cat([text, tok], dim=1)
            if text_mask is not None:
                text_mask = torch.cat([text_mask, torch.ones_like(text_mask[:, :1])], dim=1)
        return text, text_mask

    def embed_video(self, lat, t_video, first_frame_clean: bool = True):
        """Tokens, per-token modulation (first-frame tokens at timestep 0), per-token embedding, angles, grid."""
        tok, (f, h, w) = self.patchify(lat)
        x = self.patch_embedding(tok.to(self.patch_embedding.weight.dtype))
        t = t_video[:, None].expand(-1, f).clone()
        if first_frame_clean:
            t[:, 0] = 0
        temb, mod = self.video.time(t.repeat_interleave(h * w, dim=1))
        return x, mod, temb, rope_angles(grid_positions(f, h, w, lat.device), self.c.head_dim), (f, h, w)

    def embed_action(self, act, t_action):
        x = self.action_encoder(act.to(self.action_encoder.weight.dtype))
        _, mod = self.action.time(t_action)                                # [B, 6, Ca]
        n = act.shape[1]
        pos = torch.zeros(n, 3, device=act.device)
        pos[:, 0] = torch.arange(n, device=act.device)
        return x, mod, rope_angles(pos, self.c.head_dim)

    def layers(self, streams: List[dict], mask: torch.Tensor, cache: Optional[List] = None, store: Optional[List] = None):
        """``streams``: dicts with ``expert`` (the ``_Expert``), ``x``, ``mod``, ``angles``, ``ctx``, ``ctx_mask``. One joint
        attention per layer. ``cache`` (per layer (k, v)) is prepended to the keys (queries are the streams' tokens only; the
        mask then is ``[L_streams, L_cache + L_streams]``); ``store`` collects the per-layer (k, v) of the first stream."""
        xs = [s["x"] for s in streams]
        for li in range(self.c.num_layers):
            qs, ks, vs, rests = [], [], [], []
            for s, x in zip(streams, xs):
                blk = s["expert"].blocks[li]
                h, rest = blk.attn_input(x, s["mod"])
                q, k, v = blk.attn1.project(h, s["angles"])
                qs.append(q), ks.append(k), vs.append(v), rests.append(rest)
            if store is not None:
                store.append((ks[0], vs[0]))
            k_all, v_all = torch.cat(ks, 1), torch.cat(vs, 1)
            if cache is not None:
                k_all, v_all = torch.cat([cache[li][0], k_all], 1), torch.cat([cache[li][1], v_all], 1)
            o = masked_attention(torch.cat(qs, 1), k_all, v_all, mask)
            at, new = 0, []
            for s, x, rest in zip(streams, xs, rests):
                blk, n = s["expert"].blocks[li], x.shape[1]

                def post(x_, o_, *rest_, blk=blk, s=s):
                    return blk.after_attention(x_, blk.attn1.o(o_), rest_, s["ctx"], s["ctx_mask"])

                if self.c.recompute and torch.is_grad_enabled():
                    new.append(torch.utils.checkpoint.checkpoint(post, x, o[:, at:at + n], *rest, use_reentrant=False))
                else:
                    new.append(post(x, o[:, at:at + n], *rest))
                at += n
            xs = new
        return xs


class FastWAMPolicy(nn.Module):

    def default_lora_targets(self):
        """Attention and FFN projections of the transformer blocks; codec, text encoder and heads stay as they are."""
        return [f"*model.*.blocks.*.{n}" for n in ("q", "k", "v", "o", "k_img", "v_img", "ffn.0", "ffn.2")]

    def __init__(self, c: FastWAMConfig):
        super().__init__()
        assert c.variant in ("fastwam", "joint", "idm")
        self.c = c
        self.vae = CausalVideoVAE(c.latent_channels, c.vae_base).requires_grad_(False)
        self.text_encoder = TextEncoder(c.vocab_size, c.text_dim, c.text_layers)
        if c.freeze_text_encoder:
            self.text_encoder.requires_grad_(False)
        self.model = FastWAMModel(c)

    def train(self, mode: bool = True):
        super().train(mode)
        self.vae.eval()
        return self

    # -- continuous shifted schedule: sigma = shift u / (1 + (shift - 1) u), u ~ U(0, 1)
    def _sample_t(self, B, shift, device):
        u = torch.rand(B, device=device)
        return shift * u / (1 + (shift - 1) * u) * self.c.num_train_timesteps

    def _weight(self, t):
        n = float(self.c.num_train_timesteps)
        grid = torch.linspace(0, n, 1001, device=t.device)
        y = lambda v: torch.exp(-2.0 * ((v - n / 2) / n) ** 2)  # noqa: E731
        y_min = y(grid).min()
        return (y(t.float()) - y_min) / ((y(grid) - y_min).mean() + 1e-8)

    def _text(self, batch):
        if "text_emb" in batch:
            return batch["text_emb"], batch.get("text_emb_mask")
        tok = batch["tokens"] if "tokens" in batch else batch["text"]
        mask = batch.get("token_mask", tok != 0)
        keep = mask.clone()
        keep[:, 0] = True
        return self.text_encoder(tok, mask), keep

    def _latents(self, batch):
        if "latents" in batch:
            return batch["latents"]
        with torch.no_grad():
            return self.vae.encode(video_from_batch(batch, self.c.video_frames))

    def _streams(self, text, text_mask, state, video_parts, action_part):
        m = self.model
        ctx, ctx_mask = m.context(text, text_mask, state)
        vctx, actx = m.video.text_embedding(ctx), m.action.text_embedding(ctx)
        streams = [dict(expert=m.video, x=x, mod=mod, angles=ang, ctx=vctx, ctx_mask=ctx_mask) for x, mod, ang in video_parts]
        if action_part is not None:
            x, mod, ang = action_part
            streams.append(dict(expert=m.action, x=x, mod=mod, angles=ang, ctx=actx, ctx_mask=ctx_mask))
        return streams

    def forward(self, batch: Dict[str, torch.Tensor], noise=None, t=None):
        c, m = self.c, self.model
        lat = self._latents(batch)
        B, dev = lat.shape[0], lat.device
        act = batch["actions"]
        text, text_mask = self._text(batch)
        n = float(c.num_train_timesteps)
        t_v, t_a = self._sample_t(B, c.video_shift, dev), self._sample_t(B, c.action_shift, dev)
        sv, sa = (t_v / n).view(B, 1, 1, 1, 1).to(lat.dtype), (t_a / n).view(B, 1, 1).to(act.dtype)
        noise_v, noise_a = torch.randn_like(lat), (torch.randn_like(act) if noise is None else noise)
        noisy_v = (1 - sv) * lat + sv * noise_v
        noisy_v[:, :, :1] = lat[:, :, :1]                                   # the observed frame stays clean
        noisy_a = (1 - sa) * act + sa * noise_a
        xv, modv, tembv, angv, grid = m.embed_video(noisy_v, t_v)
        video_parts = [(xv, modv, angv)]
        if c.variant == "idm":
            cond, t_c = lat, torch.zeros(B, device=dev)
            if torch.rand(()).item() < c.video_cond_noise_prob:
                t_c = self._sample_t(B, c.video_shift, dev)
                sc = (t_c / n).view(B, 1, 1, 1, 1).to(lat.dtype)
                cond = (1 - sc) * lat + sc * torch.randn_like(lat)
                cond[:, :, :1] = lat[:, :, :1]
            xc, modc, _, angc, _ = m.embed_video(cond, t_c)
            video_parts.append((xc, modc, angc))
        streams = self._streams(text, text_mask, batch.get("state"), video_parts, m.embed_action(noisy_a, t_a))
        mask = (mot_segment_mask if c.segment_attention else mot_mask)(
            c.variant, grid[0], grid[1] * grid[2], act.shape[1], c.video_mask_mode, dev)
        out = m.layers(streams, mask)
        pred_v = m.unpatchify(m.video_head(out[0], tembv), grid)[:, :, 1:]
        tgt_v = (noise_v - lat)[:, :, 1:]
        per_frame = (pred_v.float() - tgt_v.float()).pow(2).mean(dim=(1, 3, 4))               # [B, F - 1]
        if "image_is_pad" in batch:  # [B, T] raw frames: a latent step is padding when all its raw frames are
            pad = batch["image_is_pad"][:, 1:].view(B, -1, self.vae.temporal_factor).all(-1)
            valid = (~pad).float()
            per_sample = (per_frame * valid).sum(1) / valid.sum(1).clamp(min=1)
        else:
            per_sample = per_frame.mean(1)
        loss_v = (per_sample * self._weight(t_v)).mean()
        pred_a = m.action_head(out[-1])
        err = (pred_a.float() - (noise_a - act).float()).pow(2).mean(-1)                       # [B, T]
        am = batch.get("action_mask")
        per_sample_a = (err * am).sum(1) / am.sum(1).clamp(min=1) if am is not None else err.mean(1)
        loss_a = (per_sample_a * self._weight(t_a)).mean()
        self.last_losses = {"video loss": loss_v.detach(), "action loss": loss_a.detach()}
        return c.loss_lambda_video * loss_v + c.loss_lambda_action * loss_a

    @torch.no_grad()
    def prefill_video_cache(self, first_latent, text, text_mask, state):
        """Keys / values of the observed frame's tokens in every layer (valid because under ``first_frame_causal`` that
        frame attends nothing else): the action expert is then denoised against them alone."""
        m = self.model
        xv, modv, _, angv, grid = m.embed_video(first_latent, torch.zeros(first_latent.shape[0], device=first_latent.device))
        store: List = []
        streams = self._streams(text, text_mask, state, [(xv, modv, angv)], None)
        m.layers(streams, torch.ones(xv.shape[1], xv.shape[1], dtype=torch.bool, device=xv.device), store=store)
        return store

    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: Optional[int] = None, generator=None) -> torch.Tensor:
        """``fastwam``: actions only, against the cached first frame. ``joint`` / ``idm``: video latents and actions are
        denoised together (the imagined video is kept in ``last_rollout_latents``)."""
        c, m = self.c, self.model
        steps = steps or 10
        first = obs["latents"][:, :, :1] if "latents" in obs else self.vae.encode(video_from_batch(obs, 1)[:, :, :1])
        B, dev = first.shape[0], first.device
        text, text_mask = self._text(obs)
        state = obs.get("state")
        u = torch.linspace(1.0, 0.0, steps + 1, device=dev)
        sig_a = c.action_shift * u / (1 + (c.action_shift - 1) * u)
        a = torch.randn(B, c.action_horizon, c.action_dim, device=dev, generator=generator)
        n = float(c.num_train_timesteps)
        if c.variant == "fastwam":
            assert c.video_mask_mode == "first_frame_causal", "action-only inference caches the first frame alone"
            cache = self.prefill_video_cache(first, text, text_mask, state)
            Lc = cache[0][0].shape[1]
            mask = torch.ones(c.action_horizon, Lc + c.action_horizon, dtype=torch.bool, device=dev)
            ctx, ctx_mask = m.context(text, text_mask, state)
            actx = m.action.text_embedding(ctx)
            for i in range(steps):
                x, mod, ang = m.embed_action(a, (sig_a[i] * n).expand(B))
                out = m.layers([dict(expert=m.action, x=x, mod=mod, angles=ang, ctx=actx, ctx_mask=ctx_mask)], mask, cache=cache)
                a = a + m.action_head(out[0]) * (sig_a[i + 1] - sig_a[i])
            return a
        frames = self.vae.latent_frames(c.video_frames)
        sig_v = c.video_shift * u / (1 + (c.video_shift - 1) * u)
        lat = torch.randn(B, first.shape[1], frames, *first.shape[3:], device=dev, generator=generator)
        lat[:, :, :1] = first
        for i in range(steps):
            xv, modv, tembv, angv, grid = m.embed_video(lat, (sig_v[i] * n).expand(B))
            parts = [(xv, modv, angv)] * (2 if c.variant == "idm" else 1)  # idm: the evolving video is its own condition
            streams = self._streams(text, text_mask, state, parts, m.embed_action(a, (sig_a[i] * n).expand(B)))
            mask = (mot_segment_mask if c.segment_attention else mot_mask)(
                c.variant, grid[0], grid[1] * grid[2], c.action_horizon, c.video_mask_mode, dev)
            out = m.layers(streams, mask)
            v = m.unpatchify(m.video_head(out[0], tembv), grid)
            lat = lat + v * (sig_v[i + 1] - sig_v[i])
            lat[:, :, :1] = first
            a = a + m.action_head(out[-1]) * (sig_a[i + 1] - sig_a[i])
        self.last_rollout_latents = lat
        return a
