"""LingBot-VA: ONE WAN-style transformer denoises video latents and action chunks in the same token sequence, trained
with teacher forcing.

Sequence of a sample: ``[noisy latents | clean latents | noisy actions | clean actions]``. Latent frame f and the n
actions that follow it (rotary frame position ``f + (i + 1) / (n + 1)``, outside the image plane) form step f; steps are
grouped into chunks of a randomly drawn size, a latent chunk c has order 2c and its action chunk 2c + 1. Attention:

* clean tokens attend clean tokens of the same or an earlier order (causal history);
* noisy tokens attend clean tokens of STRICTLY earlier order and the noisy tokens of their own order;
* nothing attends further back than a randomly drawn window of orders.

So the actions of chunk c are denoised given the video up to chunk c and the video of chunk c + 1 given the actions of
chunk c: policy and world model in one network. Every frame has a noise level of its own; with some probability the
"clean" copy is itself lightly noised (robustness to the model's own roll-outs) and its level is told to the network.
Modulation is per token, with separate timestep embedders for latents and actions; each kind has its output projection.

``predict_action`` rolls the model out: actions of step 0 from the observed frame, then latent frame 1 from those
actions, and so on, re-using the training mask rules.

(reference: loongforge/embodied/model/lingbot_va/modeling_lingbot_va.py:78-257, modules/wan_model.py:232-353,545-755,
modules/flow_match.py:12-135, modeling_lingbot_va_infer.py)
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import _Linear
from .wan_blocks import (CausalVideoVAE, DiTBlock, FlowSchedule, SegmentMask, TextEncoder, TimeEmbedder, action_positions,
                         contiguous_runs, grid_positions, rope_angles, video_from_batch)


@dataclasses.dataclass
class LingBotVAConfig:
    hidden_size: int = 3072
    num_heads: int = 24
    num_layers: int = 30
    ffn_hidden_size: int = 14336
    latent_channels: int = 48
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    action_dim: int = 7            # channels of the robot at hand
    max_action_dim: int = 30       # width of the action embedder (robots are padded to it)
    action_horizon: int = 16
    text_dim: int = 4096
    freq_dim: int = 256
    eps: float = 1e-6
    cross_attn_norm: bool = True
    chunk_size: int = 4            # chunk size is drawn from 1..chunk_size per step
    window_size: int = 64          # attention window (in chunk orders) is drawn from 4..window_size
    latent_shift: float = 5.0
    action_shift: float = 1.0
    noisy_cond_prob: float = 0.5
    action_noisy_cond_prob: float = 0.0
    video_loss_weight: float = 1.0
    action_loss_weight: float = 1.0
    num_train_timesteps: int = 1000
    video_frames: int = 9          # raw frames per sample (1 + 4k); the codec turns them into 1 + k latent frames
    image_size: int = 224
    vocab_size: int = 32000
    text_layers: int = 2
    vae_base: int = 32
    freeze_text_encoder: bool = True
    recompute: bool = False
    segment_attention: bool = True  # evaluate the block-constant mask run by run (no [L, L] mask); False: dense boolean mask

    @classmethod
    def tiny(cls, **kw) -> "LingBotVAConfig":
        base = dict(hidden_size=48, num_heads=4, num_layers=2, ffn_hidden_size=96, latent_channels=8, max_action_dim=8,
                    text_dim=32, freq_dim=32, video_frames=5, image_size=32, vae_base=8, action_horizon=4, text_layers=1)
        base.update(kw)
        return cls(**base)


@dataclasses.dataclass
class _Part:
    """One run of tokens of the sequence."""
    x: torch.Tensor          # [B, n, C] embedded tokens
    pos: torch.Tensor        # [n, 3] rotary positions
    order: torch.Tensor      # [n] chunk order (2c latents, 2c + 1 actions)
    noisy: bool
    t: torch.Tensor          # [B, n] timesteps
    action: bool


def teacher_forcing_mask(order: torch.Tensor, noisy: torch.Tensor, window: int) -> torch.Tensor:
    """``[L, L]`` boolean mask (True = query row may attend key column) from per-token chunk orders and noise flags."""
    oq, ok = order[:, None], order[None, :]
    nq, nk = noisy[:, None], noisy[None, :]
    clean_causal = ~nq & ~nk & (ok <= oq)
    noise_to_clean = nq & ~nk & (ok < oq)
    noise_self = nq & nk & (ok == oq)
    return (clean_causal | noise_to_clean | noise_self) & ((oq - ok).abs() <= window)


class LingBotVAModel(nn.Module):
    """The transformer: embedders, blocks with per-token modulation, two output projections."""

    def __init__(self, c: LingBotVAConfig):
        super().__init__()
        self.c = c
        C, p = c.hidden_size, c.patch_size
        self.patch_embedding = _Linear(c.latent_channels * p[0] * p[1] * p[2], C)
        self.action_embedder = _Linear(c.max_action_dim, C)
        self.text_embedding = nn.Sequential(_Linear(c.text_dim, C), nn.GELU(approximate="tanh"), _Linear(C, C))
        self.time, self.time_action = TimeEmbedder(C, c.freq_dim), TimeEmbedder(C, c.freq_dim)
        self.blocks = nn.ModuleList([DiTBlock(C, c.ffn_hidden_size, c.num_heads, c.eps, c.cross_attn_norm)
                                     for _ in range(c.num_layers)])
        self.norm_out = nn.LayerNorm(C, eps=c.eps, elementwise_affine=False)
        self.scale_shift_table = nn.Parameter(torch.randn(1, 2, C) / C ** 0.5)
        self.proj_out = _Linear(C, c.latent_channels * p[0] * p[1] * p[2])
        self.action_proj_out = _Linear(C, c.max_action_dim)

    # -- token <-> tensor
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

    def latent_part(self, lat, t_frame, noisy: bool, chunk: int, first_frame: int = 0) -> _Part:
        """lat ``[B, C, F, H, W]``, t_frame ``[B, F]``; frames are numbered from ``first_frame``."""
        tok, (f, h, w) = self.patchify(lat)
        frames = torch.arange(first_frame, first_frame + f, device=lat.device)
        return _Part(self.patch_embedding(tok.to(self.patch_embedding.weight.dtype)),
                     grid_positions(f, h, w, lat.device, frame_offset=float(first_frame)),
                     ((frames // chunk) * 2).repeat_interleave(h * w), noisy, t_frame.repeat_interleave(h * w, dim=1), False)

    def action_part(self, act, t_frame, noisy: bool, chunk: int, first_frame: int = 0) -> _Part:
        """act ``[B, F, n, A]`` (n actions follow each latent frame), t_frame ``[B, F]``."""
        B, f, n, A = act.shape
        frames = torch.arange(first_frame, first_frame + f, device=act.device)
        return _Part(self.action_embedder(act.reshape(B, f * n, A).to(self.action_embedder.weight.dtype)),
                     action_positions(f, n, act.device, frame_offset=float(first_frame)),
                     ((frames // chunk) * 2 + 1).repeat_interleave(n), noisy, t_frame.repeat_interleave(n, dim=1), True)

    def forward(self, parts: List[_Part], text_emb: torch.Tensor, window: int, text_mask=None) -> List[torch.Tensor]:
        """Runs the sequence made of ``parts``; returns, per part, the latent-patch or action prediction of its tokens."""
        c = self.c
        x = torch.cat([p.x for p in parts], dim=1)
        angles = rope_angles(torch.cat([p.pos for p in parts]), c.hidden_size // c.num_heads)
        order = torch.cat([p.order for p in parts])
        noisy = torch.cat([torch.full_like(p.order, p.noisy, dtype=torch.bool) for p in parts])
        if c.segment_attention:  # the mask is constant on (part, order) runs: one un-masked attention per run
            starts, ends, rep = contiguous_runs(order, noisy.long())
            mask = SegmentMask(starts, ends, teacher_forcing_mask(order[rep], noisy[rep], window))
        else:
            mask = teacher_forcing_mask(order, noisy, window)
        temb, mod = [], []
        for p in parts:
            e, m = (self.time_action if p.action else self.time)(p.t)
            temb.append(e)
            mod.append(m)
        temb, mod = torch.cat(temb, dim=1), torch.cat(mod, dim=1)           # [B, L, C], [B, L, 6, C]
        ctx = self.text_embedding(text_emb.to(x.dtype))
        for blk in self.blocks:
            if c.recompute and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, mod, angles, ctx, mask, text_mask, use_reentrant=False)
            else:
                x = blk(x, mod, angles, ctx, mask, text_mask)
        b, s = (self.scale_shift_table.float()[:, None] + temb.float()[:, :, None]).unbind(-2)
        x = (self.norm_out(x).float() * (1 + s) + b).to(x.dtype)
        outs, at = [], 0
        for p in parts:
            h = x[:, at:at + p.x.shape[1]]
            at += p.x.shape[1]
            outs.append(self.action_proj_out(h) if p.action else self.proj_out(h))
        return outs


class LingBotVAPolicy(nn.Module):
    """Codec + text encoder + transformer, the training loss and the roll-out."""

    def default_lora_targets(self):
        """Attention and FFN projections of the transformer blocks; codec, text encoder and heads stay as they are."""
        return [f"*model.blocks.*.{n}" for n in ("q", "k", "v", "o", "k_img", "v_img", "ffn.0", "ffn.2")]


    def __init__(self, c: LingBotVAConfig):
        super().__init__()
        self.c = c
        self.vae = CausalVideoVAE(c.latent_channels, c.vae_base).requires_grad_(False)
        self.text_encoder = TextEncoder(c.vocab_size, c.text_dim, c.text_layers)
        if c.freeze_text_encoder:
            self.text_encoder.requires_grad_(False)
        self.model = LingBotVAModel(c)
        self.latent_schedule = FlowSchedule(c.num_train_timesteps, c.latent_shift)
        self.action_schedule = FlowSchedule(c.num_train_timesteps, c.action_shift)

    def train(self, mode: bool = True):
        super().train(mode)
        self.vae.eval()
        return self

    # -- inputs
    def _latents(self, batch) -> torch.Tensor:
        if "latents" in batch:
            return batch["latents"]
        with torch.no_grad():
            return self.vae.encode(video_from_batch(batch, self.c.video_frames))

    def _text(self, batch):
        if "text_emb" in batch:
            return batch["text_emb"], batch.get("text_emb_mask")
        tok = batch["tokens"] if "tokens" in batch else batch["text"]
        mask = batch.get("token_mask", tok != 0)
        keep = mask.clone()
        keep[:, 0] = True
        return self.text_encoder(tok, mask), keep

    def _actions(self, batch, frames: int):
        """``[B, F, n, Amax]`` actions and their mask: the horizon is divided over the latent frames (padded up when it does
        not divide), channels beyond the robot's own are zero and masked."""
        c = self.c
        a = batch["actions"]
        B, Hn, A = a.shape
        m = batch.get("action_mask")
        m = torch.ones(B, Hn, device=a.device) if m is None else m.float()
        n = -(-Hn // frames)
        pad = n * frames - Hn
        a = F.pad(a, (0, c.max_action_dim - A, 0, pad))
        m = F.pad(m, (0, pad))[..., None] * (torch.arange(c.max_action_dim, device=a.device) < A).float()
        return a.view(B, frames, n, -1), m.view(B, frames, n, -1)

    def _noised(self, x0, schedule: FlowSchedule, cond_prob: float, frame_dim: int):
        """Per-frame noise levels; returns (noisy, target, condition copy, ids, condition timesteps)."""
        B, Fr = x0.shape[0], x0.shape[frame_dim]
        shape = [B] + [1] * (x0.dim() - 1)
        shape[frame_dim] = Fr
        ids = schedule.sample_ids((B, Fr))
        noise = torch.randn_like(x0)
        sig = schedule.sigma(ids, x0).view(shape)
        noisy = (1 - sig) * x0 + sig * noise
        cond, t_cond = x0, torch.zeros(B, Fr, device=x0.device, dtype=x0.dtype)
        if cond_prob > 0 and torch.rand(()).item() < cond_prob:
            cid = schedule.sample_ids((B, Fr), 0.5, 1.0)               # the low-noise half of the table
            cs = schedule.sigma(cid, x0).view(shape)
            cond, t_cond = (1 - cs) * x0 + cs * torch.randn_like(x0), schedule.timestep(cid, x0)
        return noisy, noise - x0, cond, ids, t_cond

    def forward(self, batch: Dict[str, torch.Tensor], noise=None, t=None):
        c = self.c
        lat = self._latents(batch)                                        # [B, C, F, h, w]
        Fr = lat.shape[2]
        act, amask = self._actions(batch, Fr)                             # [B, F, n, A]
        text, text_mask = self._text(batch)
        n_lat, tgt_lat, c_lat, id_lat, tc_lat = self._noised(lat, self.latent_schedule, c.noisy_cond_prob, 2)
        n_act, tgt_act, c_act, id_act, tc_act = self._noised(act, self.action_schedule, c.action_noisy_cond_prob, 1)
        n_act, tgt_act, c_act = n_act * amask, tgt_act * amask, c_act * amask
        chunk = int(torch.randint(1, c.chunk_size + 1, ()).item())
        window = int(torch.randint(min(4, c.window_size), c.window_size + 1, ()).item())
        m = self.model
        parts = [m.latent_part(n_lat, self.latent_schedule.timestep(id_lat, lat), True, chunk),
                 m.latent_part(c_lat, tc_lat, False, chunk),
                 m.action_part(n_act, self.action_schedule.timestep(id_act, act), True, chunk),
                 m.action_part(c_act, tc_act, False, chunk)]
        out = m(parts, text, window, text_mask)
        _, grid = m.patchify(lat)
        pred_lat = m.unpatchify(out[0], grid)
        w_lat = self.latent_schedule.weight(id_lat, lat).float()          # [B, F]
        video_loss = ((pred_lat.float() - tgt_lat.float()).pow(2).mean(dim=(1, 3, 4)) * w_lat).mean()
        pred_act = out[2].view_as(act)
        w_act = self.action_schedule.weight(id_act, act).float()[:, :, None, None]
        err = (pred_act.float() - tgt_act.float()).pow(2) * w_act * amask
        per_frame = err.flatten(2).sum(-1) / (amask.flatten(2).sum(-1) + 1e-6)
        action_loss = per_frame.mean()
        self.last_losses = {"video loss": video_loss.detach(), "action loss": action_loss.detach()}
        return c.video_loss_weight * video_loss + c.action_loss_weight * action_loss

    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: Optional[int] = None, generator=None) -> torch.Tensor:
        """Roll-out from the observed frame: for step f = 0, 1, ... denoise the n actions of step f given the clean
        history, then latent frame f + 1 given those actions; returns ``[B, horizon, action_dim]``."""
        c, m = self.c, self.model
        steps = steps or 10
        lat0 = obs["latents"][:, :, :1] if "latents" in obs else self.vae.encode(video_from_batch(obs, 1)[:, :, :1])
        B, dev = lat0.shape[0], lat0.device
        text, text_mask = self._text(obs)
        frames = self.vae.latent_frames(c.video_frames)
        n = -(-c.action_horizon // frames)
        clean_lat, clean_act = lat0, None
        zeros = lambda f: torch.zeros(B, f, device=dev)  # noqa: E731  clean tokens carry timestep 0

        def denoise(kind: str, f: int):
            sched = self.action_schedule if kind == "act" else self.latent_schedule
            x = (torch.randn(B, 1, n, c.max_action_dim, device=dev, generator=generator) if kind == "act"
                 else torch.randn(B, *lat0.shape[1:], device=dev, generator=generator))
            sig = sched.inference_sigmas(steps, dev)
            for i in range(steps):
                tt = (sig[i] * c.num_train_timesteps).expand(B, 1)
                parts = [m.latent_part(clean_lat, zeros(clean_lat.shape[2]), False, 1)]
                if clean_act is not None:
                    parts.append(m.action_part(clean_act, zeros(clean_act.shape[1]), False, 1))
                parts.append(m.action_part(x, tt, True, 1, f) if kind == "act" else m.latent_part(x, tt, True, 1, f))
                v = m(parts, text, c.window_size, text_mask)[-1]
                v = v.view_as(x) if kind == "act" else m.unpatchify(v, m.patchify(x)[1])
                x = x + v * (sig[i + 1] - sig[i])
            return x

        for f in range(frames):
            a = denoise("act", f)
            clean_act = a if clean_act is None else torch.cat([clean_act, a], dim=1)
            if f + 1 < frames:
                clean_lat = torch.cat([clean_lat, denoise("lat", f + 1)], dim=2)
        self.last_rollout_latents = clean_lat
        return clean_act.reshape(B, frames * n, -1)[:, :c.action_horizon, :c.action_dim]
