"""DreamZero: a block-causal WAN image-to-video world model whose sequence also carries the robot's action chunk and
proprioceptive state of every block ("action registers"), so the policy is read off the world model.

Sequence (teacher forcing): ``[clean video | noisy video | noisy actions | states]``. Latent frame 0 is the observation;
frames 1.. are grouped into blocks of ``num_frame_per_block`` frames, each with ``num_action_per_block`` action tokens
and ``num_state_per_block`` state tokens. Attention rules (plus the diagonal):

* clean video of block b   -> the observation and clean blocks <= b;
* noisy video of block b   -> clean blocks < b (observation included), the noisy block itself, actions and states of b;
* noisy actions of block b -> clean blocks < b, noisy video block b, actions and states of b;
* the observation         -> its own tokens only; states -> themselves only (pure conditioning);
* optionally only the last ``local_attn_blocks`` blocks of history (the observation always).

Without teacher forcing (roll-out) the clean history is the already denoised frames inside the video stream itself,
carried at timestep 0. All frames of a block share a noise level, the observation has one of its own; the action tokens
share their block's level unless ``decouple_video_action_noise``. Modulation is per token. Actions are embedded by an
embodiment-specific encoder together with their noise level, states by an embodiment-specific MLP, and action
velocities are read by an embodiment-specific decoder. Text goes through cross-attention; image features of the
observation (CLIP tower) are a second key / value set of the same cross-attention; the observation's latent is also
concatenated channel-wise to the video input (``concat_first_frame_latent``).

(reference: loongforge/embodied/model/dreamzero/modules/causal_wan_model.py:417-487,2180-2366,2368-2581,2894-3082,
modules/action_head_tf.py:157-352,793-1038,1111-1457, modules/wan_video_image_encoder.py)
"""
from __future__ import annotations

import dataclasses
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import RMSNorm, _Linear
from .groot import CategoryLinear, CategoryMLP, _sincos
from .wan_blocks import (Attention, CausalVideoVAE, DiTBlock, FlowSchedule, Head, SegmentMask, TextEncoder, TimeEmbedder,
                         contiguous_runs, grid_positions, masked_attention, rope_angles, video_from_batch)


@dataclasses.dataclass
class DreamZeroConfig:
    hidden_size: int = 5120
    ffn_hidden_size: int = 13824
    num_heads: int = 40
    num_layers: int = 40
    latent_channels: int = 16
    patch_size: Tuple[int, int, int] = (1, 2, 2)
    text_dim: int = 4096
    image_dim: int = 1280                 # width of the image tower's tokens
    freq_dim: int = 256
    eps: float = 1e-6
    concat_first_frame_latent: bool = True
    num_frame_per_block: int = 2
    num_action_per_block: int = 8
    num_state_per_block: int = 1
    local_attn_blocks: int = -1           # -1: the whole history
    max_num_embodiments: int = 32
    action_dim: int = 7
    max_action_dim: int = 32
    state_dim: int = 8
    max_state_dim: int = 64
    action_horizon: int = 16
    shift: float = 5.0
    num_train_timesteps: int = 1000
    decouple_video_action_noise: bool = False
    high_noise_beta: Optional[Tuple[float, float]] = None   # e.g. (3.0, 1.0): noise ratio ~ Beta, emphasis on high noise
    video_frames: int = 9
    image_size: int = 224
    image_tower_layers: int = 2
    image_tower_patch: int = 14
    vocab_size: int = 32000
    text_layers: int = 2
    vae_base: int = 32
    freeze_text_encoder: bool = True
    tune_diffusion_model: bool = True
    tune_projector: bool = True
    recompute: bool = False
    segment_attention: bool = True        # run-by-run evaluation of the block-causal mask (no [L, L] mask)

    @classmethod
    def tiny(cls, **kw) -> "DreamZeroConfig":
        base = dict(hidden_size=48, ffn_hidden_size=96, num_heads=4, num_layers=2, latent_channels=8, text_dim=32,
                    image_dim=24, freq_dim=32, num_frame_per_block=1, num_action_per_block=2, max_num_embodiments=3,
                    max_action_dim=8, max_state_dim=8, action_horizon=4, video_frames=9, image_size=32,
                    image_tower_layers=1, image_tower_patch=8, vae_base=8, text_layers=1)
        base.update(kw)
        return cls(**base)


# token kinds
CLEAN, NOISY, ACT, STATE = 0, 1, 2, 3


def block_token_attributes(frames: int, per_frame: int, nfb: int, n_act: int, apb: int, n_state: int, spb: int,
                           teacher_forcing: bool, device=None, register_block_offset: int = 0):
    """Per token of ``[clean video (teacher forcing only) | video | actions | states]``: kind, block (frame 0 = -1; the
    registers belong to blocks ``register_block_offset, ...``) and, for state tokens, a number of their own (they attend
    themselves only)."""
    fb = (torch.arange(frames, device=device) - 1).div(nfb, rounding_mode="floor")   # frame 0 -> block -1
    vb = fb.repeat_interleave(per_frame)
    kinds, blocks = [], []
    if teacher_forcing:
        kinds.append(torch.full_like(vb, CLEAN)), blocks.append(vb)
    kinds.append(torch.full_like(vb, NOISY)), blocks.append(vb)
    ab = torch.arange(n_act, device=device) // apb + register_block_offset
    sb = torch.arange(n_state, device=device) // spb + register_block_offset
    kinds += [torch.full_like(ab, ACT), torch.full_like(sb, STATE)]
    blocks += [ab, sb]
    kind, blk = torch.cat(kinds), torch.cat(blocks)
    own = torch.where(kind == STATE, torch.arange(kind.numel(), device=device), torch.full_like(kind, -1))
    return kind, blk, own


def block_causal_rule(kind, blk, own, teacher_forcing: bool, local_blocks: int = -1) -> torch.Tensor:
    """The attention rule on token attributes (or on one representative per run of equal attributes)."""
    kq, kk, bq, bk = kind[:, None], kind[None, :], blk[:, None], blk[None, :]
    hist = CLEAN if teacher_forcing else NOISY                    # where a block's history lives
    in_window = (bk == -1) | (bq - bk <= local_blocks) if local_blocks > 0 else torch.ones_like(bq == bk)
    history = (kk == hist) & (bk < bq) & in_window
    same = bk == bq
    m = (own[:, None] == own[None, :]) & (own[:, None] >= 0)      # a state token sees itself
    if teacher_forcing:
        m = m | ((kq == CLEAN) & (kk == CLEAN) & (bk <= bq) & in_window)
    m = m | ((kq == NOISY) & (kk == NOISY) & same)                # a frame / block sees all of itself (observation too)
    generated = (kq == NOISY) & (bq >= 0)
    m = m | (generated & (history | (same & ((kk == NOISY) | (kk == ACT) | (kk == STATE)))))
    m = m | ((kq == ACT) & (history | (same & ((kk == NOISY) | (kk == ACT) | (kk == STATE)))))
    return m


def block_causal_mask(frames: int, per_frame: int, nfb: int, n_act: int, apb: int, n_state: int, spb: int,
                      teacher_forcing: bool, local_blocks: int = -1, device=None, register_block_offset: int = 0,
                      segments: bool = False):
    """``[L, L]`` boolean mask, or with ``segments`` the same mask in run form (``wan_blocks.SegmentMask``): it is constant on
    runs of equal (kind, block), so attention can be evaluated run by run without the dense mask."""
    kind, blk, own = block_token_attributes(frames, per_frame, nfb, n_act, apb, n_state, spb, teacher_forcing, device,
                                            register_block_offset)
    if not segments:
        return block_causal_rule(kind, blk, own, teacher_forcing, local_blocks)
    starts, ends, rep = contiguous_runs(kind, blk, own)
    return SegmentMask(starts, ends, block_causal_rule(kind[rep], blk[rep], own[rep], teacher_forcing, local_blocks))


class ImageTower(nn.Module):
    """ViT over the observed frame -> ``[B, 1 + patches, image_dim]`` (class token first); frozen, the place of the CLIP
    vision tower of WAN image-to-video models."""

    def __init__(self, c: DreamZeroConfig):
        super().__init__()
        d, p = c.image_dim, c.image_tower_patch
        self.p = p
        self.patch = nn.Conv2d(3, d, p, stride=p)
        self.cls = nn.Parameter(torch.zeros(1, 1, d))
        self.pos = nn.Parameter(0.02 * torch.randn(1, 1 + (c.image_size // p) ** 2, d))
        heads = max(1, d // 64) if d % 64 == 0 else 4
        self.layers = nn.ModuleList([nn.ModuleDict(dict(n1=nn.LayerNorm(d), attn=Attention(d, heads, qk_norm=False), n2=nn.LayerNorm(d),
                                                        ffn=nn.Sequential(_Linear(d, 4 * d), nn.GELU(), _Linear(4 * d, d))))
                                     for _ in range(c.image_tower_layers)])

    def forward(self, image):
        x = self.patch(image.to(self.patch.weight.dtype)).flatten(2).transpose(1, 2)
        x = torch.cat([self.cls.expand(x.shape[0], -1, -1), x], dim=1)
        x = x + F.interpolate(self.pos.transpose(1, 2), size=x.shape[1], mode="linear").transpose(1, 2) \
            if x.shape[1] != self.pos.shape[1] else x + self.pos
        for l in self.layers:
            x = x + l["attn"](l["n1"](x))
            x = x + l["ffn"](l["n2"](x))
        return x


class I2VCrossAttention(nn.Module):
    """One query projection, two key / value sets (text, image tokens); the two attention results add."""

    def __init__(self, dim: int, heads: int, eps: float):
        super().__init__()
        self.h, self.d = heads, dim // heads
        self.q, self.k, self.v, self.o = (_Linear(dim, dim) for _ in range(4))
        self.k_img, self.v_img = _Linear(dim, dim), _Linear(dim, dim)
        self.norm_q, self.norm_k, self.norm_k_img = RMSNorm(dim, eps), RMSNorm(dim, eps), RMSNorm(dim, eps)

    def forward(self, x, angles=None, mask=None, ctx=None):
        text, img = ctx
        B = x.shape[0]
        q = self.norm_q(self.q(x)).view(B, -1, self.h, self.d)
        o = masked_attention(q, self.norm_k(self.k(text)).view(B, -1, self.h, self.d), self.v(text).view(B, -1, self.h, self.d), mask)
        if img is not None:
            o = o + masked_attention(q, self.norm_k_img(self.k_img(img)).view(B, -1, self.h, self.d),
                                     self.v_img(img).view(B, -1, self.h, self.d))
        return self.o(o)


class PerTokenActionEncoder(nn.Module):
    """``W3 swish(W2 [W1 a | sincos(t)])`` with embodiment-specific weights and a noise level per action token."""

    def __init__(self, n: int, action_dim: int, width: int):
        super().__init__()
        self.width = width
        self.W1, self.W2, self.W3 = CategoryLinear(n, action_dim, width), CategoryLinear(n, 2 * width, width), \
            CategoryLinear(n, width, width)

    def forward(self, actions, t, ids):
        a = self.W1(actions, ids)
        return self.W3(F.silu(self.W2(torch.cat([a, _sincos(t, self.width).to(a.dtype)], dim=-1), ids)), ids)


class CausalWanModel(nn.Module):
    def __init__(self, c: DreamZeroConfig):
        super().__init__()
        self.c = c
        C, p = c.hidden_size, c.patch_size
        cin = (2 * c.latent_channels + 1) if c.concat_first_frame_latent else c.latent_channels
        self.patch_embedding = _Linear(cin * p[0] * p[1] * p[2], C)
        self.text_embedding = nn.Sequential(_Linear(c.text_dim, C), nn.GELU(approximate="tanh"), _Linear(C, C))
        self.img_emb = nn.Sequential(nn.LayerNorm(c.image_dim), _Linear(c.image_dim, C), nn.GELU(), _Linear(C, C), nn.LayerNorm(C))
        self.time = TimeEmbedder(C, c.freq_dim)
        self.blocks = nn.ModuleList([DiTBlock(C, c.ffn_hidden_size, c.num_heads, c.eps) for _ in range(c.num_layers)])
        for b in self.blocks:
            b.attn2 = I2VCrossAttention(C, c.num_heads, c.eps)
        self.head = Head(C, c.latent_channels * p[0] * p[1] * p[2], c.eps)
        n = c.max_num_embodiments
        self.action_encoder = PerTokenActionEncoder(n, c.max_action_dim, C)
        self.state_encoder = CategoryMLP(n, c.max_state_dim, C, C)
        self.action_decoder = CategoryMLP(n, C, C, c.max_action_dim)

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

    def _video_tokens(self, lat, first):
        if self.c.concat_first_frame_latent:
            y = torch.zeros_like(lat)
            y[:, :, :1] = first
            flag = torch.zeros_like(lat[:, :1])
            flag[:, :, :1] = 1
            lat = torch.cat([lat, y, flag], dim=1)
        tok, grid = self.patchify(lat)
        return self.patch_embedding(tok.to(self.patch_embedding.weight.dtype)), grid

    def forward(self, video, t_frame, first, text_emb, image_tokens, action=None, t_action=None, state=None,
                embodiment_id=None, clean_video=None, text_mask=None, register_block_offset: int = 0):
        """video ``[B, C, F, h, w]`` with per-frame timesteps ``t_frame [B, F]``; ``clean_video`` switches teacher forcing on;
        action ``[B, Na, max_action_dim]`` with ``t_action [B, Na]``, state ``[B, Ns, max_state_dim]``. Returns the video
        velocity ``[B, C, F, h, w]`` and the action velocity ``[B, Na, max_action_dim]`` (None without actions)."""
        c = self.c
        B, dev = video.shape[0], video.device
        x, (f, h, w) = self._video_tokens(video, first)
        per_frame = h * w
        pos = grid_positions(f, h, w, dev)
        t_tok = t_frame.repeat_interleave(per_frame, dim=1)
        xs, ts, poss = [x], [t_tok], [pos]
        tf = clean_video is not None
        if tf:
            xs.insert(0, self._video_tokens(clean_video, first)[0])
            ts.insert(0, torch.zeros_like(t_tok))
            poss.insert(0, pos)
        na = ns = 0
        if action is not None:
            ids = embodiment_id if embodiment_id is not None else torch.zeros(B, dtype=torch.long, device=dev)
            a_tok = self.action_encoder(action.to(x.dtype), t_action, ids)
            s_tok = self.state_encoder(state.to(x.dtype), ids)
            na, ns = a_tok.shape[1], s_tok.shape[1]
            stride = max(na // max(ns, 1), 1)
            xs += [a_tok, s_tok]
            ts += [t_action, t_action[:, ::stride][:, :ns]]
            # action i of block b sits after the block's last frame; registers live outside the image plane
            apb, spb = c.num_action_per_block, c.num_state_per_block
            off_b = register_block_offset
            fa = (torch.arange(na, device=dev) // apb + off_b + 1) * c.num_frame_per_block \
                + (torch.arange(na, device=dev) % apb + 1).float() / (apb + 1)
            fs = (torch.arange(ns, device=dev) // spb + off_b) * c.num_frame_per_block + 0.5
            off = lambda t: torch.stack([t, torch.full_like(t, -1.0), torch.full_like(t, -1.0)], -1)  # noqa: E731
            poss += [off(fa.float()), off(fs.float())]
        x, t_all = torch.cat(xs, dim=1), torch.cat(ts, dim=1)
        angles = rope_angles(torch.cat(poss), c.hidden_size // c.num_heads)
        temb, mod = self.time(t_all)
        mask = block_causal_mask(f, per_frame, c.num_frame_per_block, na, c.num_action_per_block, ns,
                                 c.num_state_per_block, tf, c.local_attn_blocks, dev, register_block_offset,
                                 segments=c.segment_attention)
        ctx = (self.text_embedding(text_emb.to(x.dtype)), self.img_emb(image_tokens.to(x.dtype)) if image_tokens is not None else None)
        for blk in self.blocks:
            if c.recompute and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(blk, x, mod, angles, ctx, mask, text_mask, use_reentrant=False)
            else:
                x = blk(x, mod, angles, ctx, mask, text_mask)
        v0 = f * per_frame if tf else 0
        Lv = f * per_frame
        video_v = self.unpatchify(self.head(x[:, v0:v0 + Lv], temb[:, v0:v0 + Lv]), (f, h, w))
        action_v = self.action_decoder(x[:, v0 + Lv:v0 + Lv + na], ids) if action is not None else None
        return video_v, action_v


class DreamZeroPolicy(nn.Module):

    def default_lora_targets(self):
        """Attention and FFN projections of the transformer blocks; codec, text encoder and heads stay as they are."""
        return [f"*model.blocks.*.{n}" for n in ("q", "k", "v", "o", "k_img", "v_img", "ffn.0", "ffn.2")]

    def __init__(self, c: DreamZeroConfig):
        super().__init__()
        self.c = c
        self.vae = CausalVideoVAE(c.latent_channels, c.vae_base).requires_grad_(False)
        self.image_tower = ImageTower(c).requires_grad_(False)
        self.text_encoder = TextEncoder(c.vocab_size, c.text_dim, c.text_layers)
        if c.freeze_text_encoder:
            self.text_encoder.requires_grad_(False)
        self.model = CausalWanModel(c)
        self.schedule = FlowSchedule(c.num_train_timesteps, c.shift)
        self.set_trainable_parameters(c.tune_projector, c.tune_diffusion_model)
        self._history = None

    def set_trainable_parameters(self, tune_projector: bool, tune_diffusion_model: bool):
        """Projector = the embodiment-specific action / state encoders and the action decoder; the rest is the DiT."""
        proj = ("action_encoder.", "state_encoder.", "action_decoder.")
        for n, p in self.model.named_parameters():
            p.requires_grad_(tune_projector if n.startswith(proj) else tune_diffusion_model)

    def train(self, mode: bool = True):
        super().train(mode)
        self.vae.eval(), self.image_tower.eval()
        return self

    def _text(self, batch):
        if "text_emb" in batch:
            return batch["text_emb"], batch.get("text_emb_mask")
        tok = batch["tokens"] if "tokens" in batch else batch["text"]
        mask = batch.get("token_mask", tok != 0)
        keep = mask.clone()
        keep[:, 0] = True
        return self.text_encoder(tok, mask), keep

    def _registers(self, batch, blocks: int):
        """Actions ``[B, blocks * apb, Amax]`` (resampled from the batch's horizon by index), their mask, the states
        ``[B, blocks * spb, Smax]``."""
        c = self.c
        a = batch["actions"]
        B, Hn, A = a.shape
        na = blocks * c.num_action_per_block
        idx = torch.arange(na, device=a.device).clamp(max=Hn - 1)
        m = batch.get("action_mask")
        m = torch.ones(B, Hn, device=a.device) if m is None else m.float()
        valid = (torch.arange(na, device=a.device) < Hn).float()
        act = F.pad(a[:, idx], (0, c.max_action_dim - A))
        amask = (m[:, idx] * valid)[..., None] * (torch.arange(c.max_action_dim, device=a.device) < A).float()
        s = batch["state"]
        s = s[:, None].expand(-1, blocks * c.num_state_per_block, -1) if s.dim() == 2 else s
        return act, amask, F.pad(s, (0, c.max_state_dim - s.shape[-1]))

    def forward(self, batch: Dict[str, torch.Tensor], noise=None, t=None):
        c, m, sch = self.c, self.model, self.schedule
        with torch.no_grad():
            video = video_from_batch(batch, c.video_frames) if not ("latents" in batch and "image_tokens" in batch) else None
            lat = batch["latents"] if "latents" in batch else self.vae.encode(video)
            img = batch["image_tokens"] if "image_tokens" in batch else self.image_tower(video[:, :, 0])
        B, _, Fr, _, _ = lat.shape
        nfb = c.num_frame_per_block
        assert (Fr - 1) % nfb == 0, "latent frames after the observation must fill whole blocks"
        blocks = (Fr - 1) // nfb
        text, text_mask = self._text(batch)
        act, amask, state = self._registers(batch, blocks)
        ids = sch.sample_ids((B, 1 + blocks), beta=c.high_noise_beta)                 # observation + one per block
        id_frame = torch.cat([ids[:, :1], ids[:, 1:].repeat_interleave(nfb, dim=1)], dim=1)
        id_act = (sch.sample_ids((B, act.shape[1])) if c.decouple_video_action_noise
                  else ids[:, 1:].repeat_interleave(c.num_action_per_block, dim=1))
        noise_v, noise_a = torch.randn_like(lat), torch.randn_like(act)
        noisy_v = sch.add_noise(lat.transpose(1, 2), noise_v.transpose(1, 2), id_frame, 3).transpose(1, 2)
        noisy_a = sch.add_noise(act, noise_a, id_act, 1)
        vv, av = m(noisy_v, sch.timestep(id_frame, lat), lat[:, :, :1], text, img, noisy_a, sch.timestep(id_act, act), state,
                   batch.get("embodiment_id"), clean_video=lat, text_mask=text_mask)
        w_v = sch.weight(id_frame, lat).float()
        dyn = ((vv.float() - (noise_v - lat).float()).pow(2).mean(dim=(1, 3, 4)) * w_v).mean()
        w_a = sch.weight(id_act, act).float()[..., None]
        real = batch.get("has_real_action")
        if real is not None:
            amask = amask * real.float().view(B, 1, 1)
        act_loss = ((av.float() - (noise_a - act).float()).pow(2) * w_a * amask).sum() / amask.sum().clamp(min=1)
        self.last_losses = {"dynamics loss": dyn.detach(), "action loss": act_loss.detach()}
        return dyn + act_loss

    # -- closed-loop inference
    def reset(self):
        """Forget the frames generated / observed so far (start of an episode)."""
        self._history = None

    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: Optional[int] = None, generator=None,
                       keep_history: bool = False) -> torch.Tensor:
        """Block-by-block roll-out from the observation: each block's frames and actions are denoised jointly given the
        frames so far (kept at timestep 0 inside the video stream), then become history. ``keep_history`` keeps the
        generated frames for the next call (until ``reset``)."""
        c, m, sch = self.c, self.model, self.schedule
        steps = steps or 8
        frame0 = video_from_batch(obs, 1)[:, :, :1]
        first = obs["latents"][:, :, :1] if "latents" in obs else self.vae.encode(frame0)
        img = self.image_tower(frame0[:, :, 0])
        B, dev = first.shape[0], first.device
        text, text_mask = self._text(obs)
        nfb, apb = c.num_frame_per_block, c.num_action_per_block
        blocks = -(-c.action_horizon // apb)
        s = obs["state"]
        s = F.pad(s[:, None] if s.dim() == 2 else s[:, :1], (0, c.max_state_dim - s.shape[-1]))
        hist = first if (self._history is None or not keep_history) else self._history
        sig = sch.inference_sigmas(steps, dev)
        n = float(c.num_train_timesteps)
        out = []
        for _ in range(blocks):
            x = torch.randn(B, first.shape[1], nfb, *first.shape[3:], device=dev, generator=generator)
            a = torch.randn(B, apb, c.max_action_dim, device=dev, generator=generator)
            nh = hist.shape[2]
            assert (nh - 1) % nfb == 0
            done = (nh - 1) // nfb
            # registers of earlier blocks are not in the sequence: only this block's actions and state, numbered `done`
            for i in range(steps):
                t_frame = torch.cat([torch.zeros(B, nh, device=dev), (sig[i] * n).expand(B, nfb)], dim=1)
                vv, av = m(torch.cat([hist, x], dim=2), t_frame, first, text, img, a, (sig[i] * n).expand(B, apb),
                           s.expand(-1, c.num_state_per_block, -1), obs.get("embodiment_id"), text_mask=text_mask,
                           register_block_offset=done)
                x = x + vv[:, :, nh:] * (sig[i + 1] - sig[i])
                a = a + av * (sig[i + 1] - sig[i])
            hist = torch.cat([hist, x], dim=2)
            out.append(a)
        self._history = hist if keep_history else None
        self.last_rollout_latents = hist
        return torch.cat(out, dim=1)[:, :c.action_horizon, :c.action_dim]
