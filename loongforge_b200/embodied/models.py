"""Vision-language-action and world-model policies of the embodied stack.

All eight reference policies share one skeleton — observation encoders -> a token backbone -> an action head trained
with flow matching — and differ in which parts they use; ``POLICY_PRESETS`` records the differences:

=============  =======================================================================================
pi05           own architecture in ``embodied/pi05.py`` (PaliGemma-style prefix + Gemma action expert with
               shared attention and adaptive RMSNorm); the skeleton below only with ``architecture: skeleton``
groot_n1_6     own architecture in ``embodied/groot.py`` (Eagle backbone + alternating vision / language DiT
               action head with embodiment-specific encoders)
groot_n1_7     ``embodied/groot.py`` with the N1.7 additions (self-attention over the backbone features, state dropout)
xvla           own architecture in ``embodied/xvla.py`` (DaViT-style tower + BART-style fusion encoder, domain-aware
               soft-prompted transformer, action spaces with regressed and gripper-logit channels)
lingbot_va     ``embodied/lingbot_va.py``: one WAN transformer over noisy / clean video latents and action chunks
               with a teacher-forcing mask, roll-out at test time
fastwam        ``embodied/fastwam.py``: WAN video expert + narrow action expert with joint attention (variants
               fastwam / joint / idm), action-only inference against the cached first frame
dreamzero      ``embodied/dreamzero.py``: block-causal WAN image-to-video model with embodiment-specific action and
               state registers in the sequence
cosmos3        ``embodied/cosmos3.py``: Qwen3-VL-style decoder with understanding / generation pathways over
               packed sequences, unified 3-D M-RoPE, domain-aware action projections
=============  =======================================================================================

Every policy has an architecture of its own; the skeleton below (one backbone + a flow-matching action head) remains
for ``model_overrides: {architecture: skeleton}`` (quick experiments, tests of the trainer).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import DiTConfig, WanModel, timestep_embedding


@dataclasses.dataclass
class PolicyConfig:
    name: str = "pi05"
    backbone: str = "vlm"  # vlm | wan
    hidden: int = 256
    layers: int = 4
    heads: int = 4
    expert_hidden: int = 128  # action expert width (pi05) / DiT width
    expert_layers: int = 4
    patch: int = 14
    vocab: int = 32000
    adaln: bool = True  # DiT-style timestep modulation in the action head (False: time token, pi0 style)
    action_dim: int = 7
    state_dim: int = 8
    action_horizon: int = 16
    image_size: int = 56
    num_cameras: int = 1
    wan_latent_channels: int = 4


POLICY_PRESETS: Dict[str, dict] = {
    "pi05": dict(backbone="vlm", adaln=True),
    "groot_n1_6": dict(backbone="vlm", adaln=True, expert_layers=6),
    "groot_n1_7": dict(backbone="vlm", adaln=True, expert_layers=6, layers=6),
    "xvla": dict(backbone="vlm", adaln=False),
    "lingbot_va": dict(backbone="wan", adaln=True),
    "fastwam": dict(backbone="wan", adaln=True, expert_layers=2),
    "dreamzero": dict(backbone="wan", adaln=True),
    "cosmos3": dict(backbone="wan", adaln=True, layers=6),
}


class Block(nn.Module):
    """Pre-norm transformer block with optional cross-attention to a context and optional AdaLN modulation."""

    def __init__(self, dim: int, heads: int, ctx_dim: Optional[int] = None, adaln: bool = False):
        super().__init__()
        self.h = heads
        self.n1, self.n2 = nn.LayerNorm(dim, elementwise_affine=not adaln), nn.LayerNorm(dim, elementwise_affine=not adaln)
        self.qkv, self.o = nn.Linear(dim, 3 * dim), nn.Linear(dim, dim)
        self.mlp = nn.Sequential(nn.Linear(dim, 4 * dim), nn.GELU(approximate="tanh"), nn.Linear(4 * dim, dim))
        if ctx_dim is not None:
            self.nc = nn.LayerNorm(dim)
            self.cq, self.ckv, self.co = nn.Linear(dim, dim), nn.Linear(ctx_dim, 2 * dim), nn.Linear(dim, dim)
        self.has_ctx = ctx_dim is not None
        self.mod = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim)) if adaln else None

    def _attn(self, q, k, v, causal=False):
        B, L, C = q.shape
        sp = lambda t: t.view(B, -1, self.h, C // self.h).transpose(1, 2)  # noqa: E731
        o = F.scaled_dot_product_attention(sp(q), sp(k), sp(v), is_causal=causal)
        return o.transpose(1, 2).reshape(B, L, C)

    def forward(self, x, ctx=None, temb=None, causal=False):
        if self.mod is not None:
            b1, s1, g1, b2, s2, g2 = self.mod(temb).unsqueeze(1).chunk(6, dim=-1)
        else:
            b1 = b2 = 0.0
            s1 = s2 = 0.0
            g1 = g2 = 1.0
        h = self.n1(x) * (1 + s1) + b1
        q, k, v = self.qkv(h).chunk(3, dim=-1)
        x = x + g1 * self.o(self._attn(q, k, v, causal))
        if self.has_ctx and ctx is not None:
            k, v = self.ckv(ctx).chunk(2, dim=-1)
            x = x + self.co(self._attn(self.cq(self.nc(x)), k, v))
        return x + g2 * self.mlp(self.n2(x) * (1 + s2) + b2)


class VLMBackbone(nn.Module):
    """Patch-embedded camera images + instruction tokens + state token through a bidirectional transformer."""

    def __init__(self, c: PolicyConfig):
        super().__init__()
        self.c = c
        self.patch = nn.Linear(3 * c.patch * c.patch, c.hidden)
        n_patch = (c.image_size // c.patch) ** 2 * c.num_cameras
        self.pos = nn.Parameter(torch.zeros(1, n_patch, c.hidden))
        self.tok = nn.Embedding(c.vocab, c.hidden)
        self.state = nn.Linear(c.state_dim, c.hidden)
        self.blocks = nn.ModuleList([Block(c.hidden, c.heads) for _ in range(c.layers)])
        self.norm = nn.LayerNorm(c.hidden)

    def forward(self, images, text, state):
        B, cams, C, H, W = images.shape
        p = self.c.patch
        x = images.reshape(B * cams, C, H // p, p, W // p, p).permute(0, 2, 4, 1, 3, 5).reshape(B, -1, C * p * p)
        x = self.patch(x.to(self.patch.weight.dtype)) + self.pos
        seq = torch.cat([x, self.tok(text), self.state(state.to(x.dtype)).unsqueeze(1)], dim=1)
        for b in self.blocks:
            seq = b(seq)
        return self.norm(seq)


class WanBackbone(nn.Module):
    """Camera frames as (tiny) video latents through the WAN DiT; its output tokens are the action head's context."""

    def __init__(self, c: PolicyConfig):
        super().__init__()
        self.c = c
        self.to_latent = nn.Conv2d(3, c.wan_latent_channels, kernel_size=c.patch // 2, stride=c.patch // 2)
        self.tok = nn.Embedding(c.vocab, c.hidden)
        self.state = nn.Linear(c.state_dim, c.hidden)
        self.wan = WanModel(DiTConfig(hidden_size=c.hidden, num_heads=c.heads, num_layers=c.layers,
                                      ffn_hidden_size=4 * c.hidden, in_channels=c.wan_latent_channels,
                                      out_channels=c.hidden // 4, text_dim=c.hidden, freq_dim=64))

    def forward(self, images, text, state):
        B, cams, C, H, W = images.shape
        lat = self.to_latent(images.reshape(B * cams, C, H, W).to(self.to_latent.weight.dtype))
        lat = lat.view(B, cams, *lat.shape[1:]).transpose(1, 2)  # cameras act as frames: [B, C, F, h, w]
        h, w = lat.shape[-2] // 2 * 2, lat.shape[-1] // 2 * 2
        ctx = torch.cat([self.tok(text), self.state(state.to(lat.dtype)).unsqueeze(1)], dim=1)
        out = self.wan(lat[..., :h, :w], torch.zeros(B, device=lat.device), ctx)  # [B, hidden/4, F, h, w]
        tokens, _ = self.wan.patchify(out)
        return tokens  # [B, L, hidden]


class ActionHead(nn.Module):
    """Flow-matching action expert: noisy action chunk tokens attend to the backbone tokens."""

    def __init__(self, c: PolicyConfig):
        super().__init__()
        self.c, d = c, c.expert_hidden
        self.inp = nn.Linear(c.action_dim, d)
        self.pos = nn.Parameter(torch.zeros(1, c.action_horizon, d))
        self.time = nn.Sequential(nn.Linear(64, d), nn.SiLU(), nn.Linear(d, d))
        self.blocks = nn.ModuleList([Block(d, c.heads, ctx_dim=c.hidden, adaln=c.adaln) for _ in range(c.expert_layers)])
        self.norm = nn.LayerNorm(d)
        self.out = nn.Linear(d, c.action_dim)

    def forward(self, noisy_actions, t, context):
        temb = self.time(timestep_embedding(t * 1000.0, 64).to(noisy_actions.dtype))
        x = self.inp(noisy_actions) + self.pos
        if not self.c.adaln:
            x = x + temb.unsqueeze(1)
        for b in self.blocks:
            x = b(x, ctx=context, temb=temb)
        return self.out(self.norm(x))


class FlowMatchingPolicy(nn.Module):
    def __init__(self, c: PolicyConfig):
        super().__init__()
        self.c = c
        self.backbone = VLMBackbone(c) if c.backbone == "vlm" else WanBackbone(c)
        self.head = ActionHead(c)

    def forward(self, batch: Dict[str, torch.Tensor], noise: Optional[torch.Tensor] = None,
                t: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Flow-matching loss: x_t = t * noise + (1 - t) * actions, target velocity = noise - actions, masked MSE."""
        actions = batch["actions"]
        B = actions.shape[0]
        noise = torch.randn_like(actions) if noise is None else noise
        if t is None:  # Beta(1.5, 1) skewed towards noisy samples, as pi0 does
            t = torch.distributions.Beta(1.5, 1.0).sample((B,)).to(actions.device) * 0.999 + 0.001
        ctx = self.backbone(batch["images"], batch["text"], batch["state"])
        tt = t.view(B, 1, 1).to(actions.dtype)
        v = self.head(tt * noise + (1 - tt) * actions, t, ctx)
        err = (v.float() - (noise - actions).float()).pow(2).mean(-1)
        m = batch.get("action_mask")
        return (err * m).sum() / m.sum().clamp(min=1) if m is not None else err.mean()

    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: int = 10, generator=None) -> torch.Tensor:
        """Euler integration of the learned velocity field from noise (t = 1) to actions (t = 0)."""
        B = obs["state"].shape[0]
        ctx = self.backbone(obs["images"], obs["text"], obs["state"])
        x = torch.randn(B, self.c.action_horizon, self.c.action_dim, device=ctx.device, dtype=ctx.dtype, generator=generator)
        dt = -1.0 / steps
        t = torch.ones(B, device=ctx.device)
        for _ in range(steps):
            x = x + dt * self.head(x, t, ctx)
            t = t + dt
        return x


class _BatchAdapter(nn.Module):
    """Lets the dedicated architectures (embodied/pi05.py, embodied/groot.py) take the trainer's batch layout:
    ``text`` is their ``tokens``; the padded part of the instruction (token id 0) is masked."""

    def __init__(self, policy: nn.Module):
        super().__init__()
        self.policy = policy
        self.c = policy.c

    @staticmethod
    def _adapt(batch):
        b = dict(batch)
        if "tokens" not in b:
            b["tokens"] = b["text"]
            b.setdefault("token_mask", b["text"] != 0)
        return b

    def forward(self, batch, noise=None, t=None):
        return self.policy(self._adapt(batch), noise=noise, t=t)

    @torch.no_grad()
    def predict_action(self, obs, steps=None, generator=None):
        return self.policy.predict_action(self._adapt(obs), steps=steps)


def _dedicated_policy(name: str, args, overrides: dict) -> Optional[nn.Module]:
    """Every named policy has an architecture of its own. ``model_overrides: {size: tiny}`` selects the small test
    geometry, any other key overrides a field of the architecture's configuration."""
    if name not in ("pi05", "groot_n1_6", "groot_n1_7", "xvla", "lingbot_va", "fastwam", "dreamzero", "cosmos3"):
        return None
    kw = dict(getattr(args, "model_overrides", None) or {}) if args is not None else {}
    kw.update(overrides)
    size = kw.pop("size", "full")
    if size == "tiny":
        kw.setdefault("vocab_size", 32000)  # the hash tokenizer of the synthetic / npz data sets
    if args is not None:
        kw.setdefault("action_dim", args.action_dim)
        kw.setdefault("action_horizon", args.action_horizon)
        kw.setdefault("image_size", args.image_size)
    if name in ("lingbot_va", "fastwam", "dreamzero", "cosmos3"):
        import importlib
        mod = importlib.import_module(f".{name}", __package__)
        cfg_cls, pol_cls = {"lingbot_va": ("LingBotVAConfig", "LingBotVAPolicy"), "fastwam": ("FastWAMConfig", "FastWAMPolicy"),
                            "dreamzero": ("DreamZeroConfig", "DreamZeroPolicy"), "cosmos3": ("Cosmos3Config", "Cosmos3Policy")}[name]
        cfg_cls, pol_cls = getattr(mod, cfg_cls), getattr(mod, pol_cls)
        fields = {f.name for f in dataclasses.fields(cfg_cls)}
        if args is not None:
            kw.setdefault("state_dim", args.state_dim)
            if getattr(args, "video_frames", 0):
                kw.setdefault("video_frames", args.video_frames)
        kw = {k: v for k, v in kw.items() if k in fields}
        return _BatchAdapter(pol_cls(cfg_cls.tiny(**kw) if size == "tiny" else cfg_cls(**kw)))
    if name == "pi05":
        from .pi05 import Pi05Config, Pi05Policy
        if args is not None:
            kw.setdefault("num_cameras", args.num_cameras)
        fields = {f.name for f in dataclasses.fields(Pi05Config)}
        kw = {k: v for k, v in kw.items() if k in fields}
        cfg = Pi05Config.tiny(**kw) if size == "tiny" else Pi05Config(**kw)
        return _BatchAdapter(Pi05Policy(cfg))
    if name == "xvla":
        from .xvla import XVLAConfig, XVLAPolicy
        kw["num_actions"] = kw.pop("action_horizon", kw.get("num_actions", 30))
        if args is not None:
            kw.setdefault("num_views", args.num_cameras)
        if "action_space" not in kw:  # any robot: regress the real channels, pad to the model's width
            kw["action_space"] = "auto"
            kw["max_action_dim"] = max(kw.get("max_action_dim", 20 if size != "tiny" else 8), kw.get("action_dim", 7))
        fields = {f.name for f in dataclasses.fields(XVLAConfig)}
        kw = {k: v for k, v in kw.items() if k in fields}
        cfg = XVLAConfig.tiny(**kw) if size == "tiny" else XVLAConfig(**kw)
        return _BatchAdapter(XVLAPolicy(cfg))
    from .groot import GrootConfig, GrootPolicy
    if args is not None:
        kw.setdefault("state_dim", args.state_dim)
    fields = {f.name for f in dataclasses.fields(GrootConfig)}
    kw = {k: v for k, v in kw.items() if k in fields}
    if name == "groot_n1_7":
        extra = dict(vl_self_attention_layers=2, vl_self_attention_heads=4, state_dropout_prob=0.2) if size == "tiny" else {}
        cfg = GrootConfig.tiny(**{**extra, **kw}) if size == "tiny" else GrootConfig.n1_7(**kw)
    else:
        cfg = GrootConfig.tiny(**kw) if size == "tiny" else GrootConfig(**kw)
    return _BatchAdapter(GrootPolicy(cfg))


def build_policy(name: str, args=None, **overrides) -> nn.Module:
    if name not in POLICY_PRESETS:
        raise KeyError(f"unknown policy {name!r}; known: {sorted(POLICY_PRESETS)}")
    if (getattr(args, "model_overrides", None) or {}).get("architecture", overrides.get("architecture")) != "skeleton":
        dedicated = _dedicated_policy(name, args, {k: v for k, v in overrides.items() if k != "architecture"})
        if dedicated is not None:
            return dedicated
    overrides = {k: v for k, v in overrides.items() if k != "architecture"}
    skeleton_fields = {f.name for f in dataclasses.fields(PolicyConfig)}
    kw = dict(POLICY_PRESETS[name], name=name)
    if args is not None:
        kw.update(action_dim=args.action_dim, state_dim=args.state_dim, action_horizon=args.action_horizon,
                  image_size=args.image_size, num_cameras=args.num_cameras)
        kw.update({k: v for k, v in (args.model_overrides or {}).items() if k in skeleton_fields})
    kw.update({k: v for k, v in overrides.items() if k in skeleton_fields})
    return FlowMatchingPolicy(PolicyConfig(**kw))
