"""GR00T N1.6 / N1.7 vision-language-action policy (reference: loongforge/embodied/model/groot_n1_6/modeling_groot_n1_6.py
:74-896, modules/dit.py:35-420, modules/embodiment_mlp.py:67-250, eagle3_model/).

Two parts.
* Backbone ("Eagle"): a SigLIP-style ViT per image, a 2 x 2 pixel-shuffle + MLP connector, and the first `select_layer`
  layers of a Qwen3-style causal decoder over [image tokens | instruction tokens]. Its output is the feature sequence,
  its padding mask and a mask of which positions are image tokens.
* Action head: the state goes through an embodiment-specific MLP (one weight set per robot embodiment, picked by
  `embodiment_id`), the noisy action chunk through an embodiment-specific encoder that mixes in a sinusoidal encoding of
  the flow time; [state | actions] tokens (+ learned positions) run through a DiT whose even blocks cross-attend to the
  backbone features and whose odd blocks self-attend. The cross-attending blocks alternate between the NON-image
  tokens and the image tokens of the backbone (every `attend_text_every_n_blocks`-th one reads text). Every block is
  modulated by the time embedding (AdaLayerNorm: scale / shift), as is the output layer; an embodiment-specific MLP
  decodes the last `action_horizon` tokens to action velocities.

Flow matching (note the direction, opposite to Pi0.5): ``x_t = (1 - t) * noise + t * actions``, target
``actions - noise``, ``t = (1 - Beta(1.5, 1)) * 0.999`` discretised into 1000 buckets for the time embedding; sampling
integrates from noise (t = 0) with `num_inference_timesteps` Euler steps.

N1.7 (``GrootConfig.n1_7``; reference loongforge/embodied/model/groot_n1_7/modeling_groot_n1_7.py:45-290) adds a 4-layer
self-attention transformer over the backbone features before the DiT reads them, state dropout with a learned mask
token, and larger state / action paddings (132) with a 40-step horizon.

`GROOT_HEAD_NAME_MAP` / `convert_groot_state_dict` translate the public GR00T checkpoints' parameter names
(``action_head.model.transformer_blocks.N.attn1.to_q`` ...) to the names used here."""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class GrootConfig:
    # backbone
    vocab_size: int = 151680
    image_size: int = 224
    patch_size: int = 14
    vit_width: int = 1152
    vit_depth: int = 27
    vit_heads: int = 16
    vit_mlp: int = 4304
    llm_width: int = 2048
    llm_layers: int = 28
    select_layer: int = 16        # features are taken after this many decoder layers
    llm_heads: int = 16
    llm_kv_heads: int = 8
    llm_head_dim: int = 128
    llm_mlp: int = 6144
    rope_theta: float = 1e6
    # action head
    hidden_size: int = 1024       # width of the state encoder / decoder MLPs and the DiT output
    input_embedding_dim: int = 1536  # DiT token width (= heads * head_dim)
    dit_layers: int = 32
    dit_heads: int = 32
    dit_head_dim: int = 48
    attend_text_every_n_blocks: int = 2
    dropout: float = 0.2
    max_seq_len: int = 1024
    max_num_embodiments: int = 32
    max_state_dim: int = 128
    max_action_dim: int = 128
    action_dim: int = 7
    state_dim: int = 7
    action_horizon: int = 50
    num_inference_timesteps: int = 4
    noise_beta: Tuple[float, float] = (1.5, 1.0)
    noise_s: float = 0.999
    num_timestep_buckets: int = 1000
    tune_llm: bool = False
    tune_visual: bool = False
    # GR00T N1.7 additions: a small self-attention transformer over the backbone features before the DiT reads them,
    # and state dropout (the state token is replaced by a learned mask token with this probability while training)
    vl_self_attention_layers: int = 0
    vl_self_attention_heads: int = 32
    state_dropout_prob: float = 0.0

    @staticmethod
    def n1_7(**kw) -> "GrootConfig":
        """GR00T N1.7 geometry (reference: loongforge/embodied/model/groot_n1_7/model_configuration_groot_n1_7.py:30-95)."""
        base = dict(max_state_dim=132, max_action_dim=132, action_horizon=40, vl_self_attention_layers=4,
                    vl_self_attention_heads=32, state_dropout_prob=0.2)
        base.update(kw)
        return GrootConfig(**base)

    @staticmethod
    def tiny(**kw) -> "GrootConfig":
        base = dict(vocab_size=256, image_size=28, patch_size=7, vit_width=32, vit_depth=2, vit_heads=4, vit_mlp=64,
                    llm_width=48, llm_layers=3, select_layer=2, llm_heads=4, llm_kv_heads=2, llm_head_dim=12, llm_mlp=96,
                    hidden_size=40, input_embedding_dim=32, dit_layers=4, dit_heads=4, dit_head_dim=8, dropout=0.0,
                    max_seq_len=64, max_num_embodiments=4, max_state_dim=16, max_action_dim=16, action_horizon=5,
                    tune_llm=True, tune_visual=True)
        base.update(kw)
        return GrootConfig(**base)


# ------------------------------------------------------------------------------------------------ backbone
class _ViT(nn.Module):
    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        n = (c.image_size // c.patch_size) ** 2
        self.patch_embedding = nn.Conv2d(3, c.vit_width, c.patch_size, c.patch_size)
        self.position_embedding = nn.Embedding(n, c.vit_width)
        self.layers = nn.ModuleList([nn.ModuleDict(dict(
            ln1=nn.LayerNorm(c.vit_width, eps=1e-6), qkv=nn.Linear(c.vit_width, 3 * c.vit_width),
            out=nn.Linear(c.vit_width, c.vit_width), ln2=nn.LayerNorm(c.vit_width, eps=1e-6),
            fc1=nn.Linear(c.vit_width, c.vit_mlp), fc2=nn.Linear(c.vit_mlp, c.vit_width))) for _ in range(c.vit_depth)])
        self.post_layernorm = nn.LayerNorm(c.vit_width, eps=1e-6)

    def forward(self, images):
        x = self.patch_embedding(images.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = x + self.position_embedding.weight
        B, L, C = x.shape
        h = self.c.vit_heads
        for blk in self.layers:
            q, k, v = blk["qkv"](blk["ln1"](x)).view(B, L, 3, h, C // h).permute(2, 0, 3, 1, 4)
            x = x + blk["out"](F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, C))
            x = x + blk["fc2"](F.gelu(blk["fc1"](blk["ln2"](x)), approximate="tanh"))
        return self.post_layernorm(x)


class _Rms(nn.Module):
    def __init__(self, d, eps=1e-6):
        super().__init__()
        self.weight, self.eps = nn.Parameter(torch.ones(d)), eps

    def forward(self, x):
        xf = x.float()
        return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)).to(x.dtype) * self.weight


class _QwenLayer(nn.Module):
    """Qwen3 decoder layer: GQA with per-head RMS norm of q and k, rotary positions, SwiGLU."""

    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        self.input_norm, self.post_norm = _Rms(c.llm_width), _Rms(c.llm_width)
        self.qkv = nn.Linear(c.llm_width, (c.llm_heads + 2 * c.llm_kv_heads) * c.llm_head_dim, bias=False)
        self.q_norm, self.k_norm = _Rms(c.llm_head_dim), _Rms(c.llm_head_dim)
        self.o = nn.Linear(c.llm_heads * c.llm_head_dim, c.llm_width, bias=False)
        self.gate_up = nn.Linear(c.llm_width, 2 * c.llm_mlp, bias=False)
        self.down = nn.Linear(c.llm_mlp, c.llm_width, bias=False)

    def forward(self, x, mask, positions):
        c = self.c
        B, L, _ = x.shape
        qkv = self.qkv(self.input_norm(x)).view(B, L, c.llm_heads + 2 * c.llm_kv_heads, c.llm_head_dim).transpose(1, 2)
        q, k, v = qkv.split([c.llm_heads, c.llm_kv_heads, c.llm_kv_heads], dim=1)
        from .pi05 import rope
        q, k = rope(self.q_norm(q), positions, c.rope_theta), rope(self.k_norm(k), positions, c.rope_theta)
        rep = c.llm_heads // c.llm_kv_heads
        o = F.scaled_dot_product_attention(q, k.repeat_interleave(rep, 1), v.repeat_interleave(rep, 1), attn_mask=mask)
        x = x + self.o(o.transpose(1, 2).reshape(B, L, -1))
        g, u = self.gate_up(self.post_norm(x)).chunk(2, dim=-1)
        return x + self.down(F.silu(g) * u)


class EagleBackbone(nn.Module):
    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        self.vision = _ViT(c)
        # connector: LayerNorm + 2-layer MLP over 2 x 2 pixel-shuffled patches
        self.connector = nn.Sequential(nn.LayerNorm(4 * c.vit_width), nn.Linear(4 * c.vit_width, c.llm_width), nn.GELU(),
                                       nn.Linear(c.llm_width, c.llm_width))
        self.embed_tokens = nn.Embedding(c.vocab_size, c.llm_width)
        self.layers = nn.ModuleList([_QwenLayer(c) for _ in range(min(c.select_layer, c.llm_layers))])
        if not c.tune_visual:
            self.vision.requires_grad_(False)
            self.connector.requires_grad_(False)
        if not c.tune_llm:
            self.embed_tokens.requires_grad_(False)
            self.layers.requires_grad_(False)

    def image_tokens(self, images):
        x = self.vision(images)  # [N, g*g, C]
        N, L, C = x.shape
        g = int(math.isqrt(L))
        x = x.view(N, g // 2, 2, g // 2, 2, C).permute(0, 1, 3, 2, 4, 5).reshape(N, (g // 2) ** 2, 4 * C)
        return self.connector(x)

    def forward(self, images, image_masks, tokens, token_mask):
        """images [B, cams, 3, H, W] -> (features [B, S, W], valid [B, S], is_image [B, S])."""
        B, cams = images.shape[:2]
        img = self.image_tokens(images.flatten(0, 1))
        n = img.shape[1]
        img = img.view(B, cams * n, -1)
        tok = self.embed_tokens(tokens)
        x = torch.cat([img.to(tok.dtype), tok], dim=1)
        iv = torch.ones(B, cams, dtype=torch.bool, device=x.device) if image_masks is None else image_masks.bool()
        tv = torch.ones_like(tokens, dtype=torch.bool) if token_mask is None else token_mask.bool()
        valid = torch.cat([iv.repeat_interleave(n, 1), tv], dim=1)
        is_image = torch.cat([torch.ones(B, cams * n, dtype=torch.bool, device=x.device), torch.zeros_like(tv)], dim=1)
        S = x.shape[1]
        causal = torch.ones(S, S, dtype=torch.bool, device=x.device).tril()
        mask = (causal[None] & valid[:, None, :])[:, None]
        pos = (valid.long().cumsum(1) - 1).clamp(min=0)
        for layer in self.layers:
            x = layer(x, mask, pos)
        return x, valid, is_image


# ------------------------------------------------------------------------------------------------ action head
class CategoryLinear(nn.Module):
    """One (W, b) per embodiment: ``y = x W[id] + b[id]``."""

    def __init__(self, n: int, din: int, dout: int):
        super().__init__()
        self.W = nn.Parameter(0.02 * torch.randn(n, din, dout))
        self.b = nn.Parameter(torch.zeros(n, dout))

    def forward(self, x, ids):
        return torch.bmm(x, self.W[ids].to(x.dtype)) + self.b[ids].to(x.dtype).unsqueeze(1)


class CategoryMLP(nn.Module):
    def __init__(self, n, din, dh, dout):
        super().__init__()
        self.layer1, self.layer2 = CategoryLinear(n, din, dh), CategoryLinear(n, dh, dout)

    def forward(self, x, ids):
        return self.layer2(F.relu(self.layer1(x, ids)), ids)


def _sincos(t: torch.Tensor, dim: int) -> torch.Tensor:
    """t [B, T] -> [B, T, dim] (sin | cos, base 10000)."""
    half = dim // 2
    freq = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
    ang = t.float().unsqueeze(-1) * freq
    return torch.cat([ang.sin(), ang.cos()], dim=-1)


class ActionEncoder(nn.Module):
    """``W3 swish(W2 [W1 a | sincos(t)])``, all three embodiment-specific."""

    def __init__(self, n, action_dim, width):
        super().__init__()
        self.width = width
        self.W1, self.W2, self.W3 = CategoryLinear(n, action_dim, width), CategoryLinear(n, 2 * width, width), \
            CategoryLinear(n, width, width)

    def forward(self, actions, t_bucket, ids):
        B, T, _ = actions.shape
        a = self.W1(actions, ids)
        tau = _sincos(t_bucket.view(B, 1).expand(B, T), self.width).to(a.dtype)
        return self.W3(F.silu(self.W2(torch.cat([a, tau], dim=-1), ids)), ids)


class TimestepEncoder(nn.Module):
    """256 sinusoid channels (cos | sin order, frequency exponent over half - 1) -> 2-layer SiLU MLP."""

    def __init__(self, dim):
        super().__init__()
        self.linear_1, self.linear_2 = nn.Linear(256, dim), nn.Linear(dim, dim)

    def forward(self, t):
        half = 128
        freq = torch.exp(-math.log(10000.0) * torch.arange(half, device=t.device, dtype=torch.float32) / (half - 1))
        ang = t.float()[:, None] * freq
        emb = torch.cat([ang.cos(), ang.sin()], dim=-1).to(self.linear_1.weight.dtype)
        return self.linear_2(F.silu(self.linear_1(emb)))


class DiTBlock(nn.Module):
    def __init__(self, c: GrootConfig, cross_dim: Optional[int]):
        super().__init__()
        d = c.input_embedding_dim
        self.h = c.dit_heads
        self.norm1 = nn.LayerNorm(d, elementwise_affine=False, eps=1e-5)
        self.ada = nn.Linear(d, 2 * d)  # scale, shift from silu(temb)
        kv_in = cross_dim if cross_dim is not None else d
        self.to_q, self.to_k, self.to_v = nn.Linear(d, d), nn.Linear(kv_in, d), nn.Linear(kv_in, d)
        self.to_out = nn.Linear(d, d)
        self.norm3 = nn.LayerNorm(d, eps=1e-5)
        self.ff_in, self.ff_out = nn.Linear(d, 4 * d), nn.Linear(4 * d, d)
        self.drop = nn.Dropout(c.dropout)

    def forward(self, x, temb, ctx=None, ctx_mask=None):
        B, L, D = x.shape
        scale, shift = self.ada(F.silu(temb)).unsqueeze(1).chunk(2, dim=-1)
        h = self.norm1(x) * (1 + scale) + shift
        src = h if ctx is None else ctx.to(h.dtype)
        sp = lambda t: t.view(B, -1, self.h, D // self.h).transpose(1, 2)  # noqa: E731
        m = None if ctx_mask is None else ctx_mask[:, None, None, :]
        o = F.scaled_dot_product_attention(sp(self.to_q(h)), sp(self.to_k(src)), sp(self.to_v(src)), attn_mask=m)
        x = x + self.drop(self.to_out(o.transpose(1, 2).reshape(B, L, D)))
        return x + self.drop(self.ff_out(self.drop(F.gelu(self.ff_in(self.norm3(x)), approximate="tanh"))))


class AlternateVLDiT(nn.Module):
    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        d = c.input_embedding_dim
        assert d == c.dit_heads * c.dit_head_dim
        self.timestep_encoder = TimestepEncoder(d)
        self.blocks = nn.ModuleList([DiTBlock(c, c.llm_width if i % 2 == 0 else None) for i in range(c.dit_layers)])
        self.norm_out = nn.LayerNorm(d, elementwise_affine=False, eps=1e-6)
        self.proj_out_1, self.proj_out_2 = nn.Linear(d, 2 * d), nn.Linear(d, c.hidden_size)

    def forward(self, x, ctx, t_bucket, valid, is_image):
        temb = self.timestep_encoder(t_bucket)
        img_mask, txt_mask = is_image & valid, (~is_image) & valid
        # a row that may attend to nothing would produce NaNs: let it see every valid token instead
        img_mask = torch.where(img_mask.any(1, keepdim=True), img_mask, valid)
        txt_mask = torch.where(txt_mask.any(1, keepdim=True), txt_mask, valid)
        n = self.c.attend_text_every_n_blocks
        for i, blk in enumerate(self.blocks):
            if i % 2 == 1:
                x = blk(x, temb)
            else:
                x = blk(x, temb, ctx, txt_mask if i % (2 * n) == 0 else img_mask)
        shift, scale = self.proj_out_1(F.silu(temb)).chunk(2, dim=1)
        return self.proj_out_2(self.norm_out(x) * (1 + scale[:, None]) + shift[:, None])


class VLSelfAttention(nn.Module):
    """Pre-norm self-attention + feed-forward blocks over the backbone features (padded positions masked as keys)."""

    def __init__(self, c: GrootConfig):
        super().__init__()
        d, self.h = c.llm_width, c.vl_self_attention_heads
        self.blocks = nn.ModuleList([nn.ModuleDict(dict(
            norm1=nn.LayerNorm(d), to_q=nn.Linear(d, d), to_k=nn.Linear(d, d), to_v=nn.Linear(d, d), to_out=nn.Linear(d, d),
            norm3=nn.LayerNorm(d), ff_in=nn.Linear(d, 4 * d), ff_out=nn.Linear(4 * d, d)))
            for _ in range(c.vl_self_attention_layers)])
        self.drop = nn.Dropout(c.dropout)

    def forward(self, x, valid):
        B, L, D = x.shape
        sp = lambda t: t.view(B, L, self.h, D // self.h).transpose(1, 2)  # noqa: E731
        m = valid[:, None, None, :]
        for b in self.blocks:
            h = b["norm1"](x)
            o = F.scaled_dot_product_attention(sp(b["to_q"](h)), sp(b["to_k"](h)), sp(b["to_v"](h)), attn_mask=m)
            x = x + self.drop(b["to_out"](o.transpose(1, 2).reshape(B, L, D)))
            x = x + self.drop(b["ff_out"](F.gelu(b["ff_in"](b["norm3"](x)), approximate="tanh")))
        return x


class GrootActionHead(nn.Module):
    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        n = c.max_num_embodiments
        self.model = AlternateVLDiT(c)
        self.vl_self_attention = VLSelfAttention(c) if c.vl_self_attention_layers > 0 else None
        self.mask_token = nn.Parameter(0.02 * torch.randn(1, 1, c.input_embedding_dim)) if c.state_dropout_prob > 0 else None
        self.state_encoder = CategoryMLP(n, c.max_state_dim, c.hidden_size, c.input_embedding_dim)
        self.action_encoder = ActionEncoder(n, c.max_action_dim, c.input_embedding_dim)
        self.action_decoder = CategoryMLP(n, c.hidden_size, c.hidden_size, c.max_action_dim)
        self.vlln = nn.LayerNorm(c.llm_width)
        self.position_embedding = nn.Embedding(c.max_seq_len, c.input_embedding_dim)
        nn.init.normal_(self.position_embedding.weight, std=0.02)

    def velocity(self, feats, valid, is_image, state, x_t, t_bucket, ids):
        c = self.c
        s = self.state_encoder(F.pad(state, (0, c.max_state_dim - state.shape[-1])).unsqueeze(1), ids)
        if self.mask_token is not None and self.training:
            drop = torch.rand(s.shape[0], 1, 1, device=s.device) < c.state_dropout_prob
            s = torch.where(drop, self.mask_token.to(s.dtype), s)
        feats = self.vlln(feats)
        if self.vl_self_attention is not None:
            feats = self.vl_self_attention(feats, valid)
        a = self.action_encoder(F.pad(x_t, (0, c.max_action_dim - x_t.shape[-1])), t_bucket, ids)
        a = a + self.position_embedding(torch.arange(a.shape[1], device=a.device)).to(a.dtype)
        out = self.model(torch.cat([s, a], dim=1), feats, t_bucket, valid, is_image)
        return self.action_decoder(out, ids)[:, -x_t.shape[1]:, : x_t.shape[-1]]


class GrootPolicy(nn.Module):
    """batch: ``images`` [B, cams, 3, H, W], ``image_masks``, ``tokens`` [B, L], ``token_mask``, ``state`` [B, state_dim],
    ``embodiment_id`` [B], ``actions`` [B, horizon, action_dim], ``action_mask`` (optional)."""

    def default_lora_targets(self):
        """Attention projections of the backbone's language layers and of the DiT head."""
        return ["qkv", "o", "to_q", "to_k", "to_v", "to_out"]


    def __init__(self, c: GrootConfig):
        super().__init__()
        self.c = c
        self.backbone = EagleBackbone(c)
        self.action_head = GrootActionHead(c)

    def _ids(self, batch, B, device):
        ids = batch.get("embodiment_id")
        if ids is None:
            return torch.zeros(B, dtype=torch.long, device=device)
        ids = torch.as_tensor(ids, device=device).long().reshape(-1)
        return ids.expand(B) if ids.numel() == 1 else ids

    def forward(self, batch, noise=None, t=None):
        c = self.c
        actions = batch["actions"]
        B = actions.shape[0]
        feats, valid, is_image = self.backbone(batch["images"], batch.get("image_masks"), batch["tokens"],
                                               batch.get("token_mask"))
        noise = torch.randn_like(actions) if noise is None else noise
        if t is None:
            t = (1 - torch.distributions.Beta(*c.noise_beta).sample((B,)).to(actions.device)) * c.noise_s
        tt = t.view(B, 1, 1).to(actions.dtype)
        x_t, target = (1 - tt) * noise + tt * actions, actions - noise
        t_bucket = (t * c.num_timestep_buckets).long()
        v = self.action_head.velocity(feats, valid, is_image, batch["state"].to(feats.dtype), x_t.to(feats.dtype),
                                      t_bucket, self._ids(batch, B, actions.device))
        err = (v.float() - target.float()).pow(2)
        m = batch.get("action_mask")
        if m is not None:
            m = m.float() if m.dim() == 3 else m.float().unsqueeze(-1).expand_as(err)
            return (err * m).sum() / m.sum().clamp(min=1)
        return err.mean()

    @torch.no_grad()
    def predict_action(self, obs, steps: Optional[int] = None, noise=None):
        c = self.c
        steps = steps or c.num_inference_timesteps
        feats, valid, is_image = self.backbone(obs["images"], obs.get("image_masks"), obs["tokens"], obs.get("token_mask"))
        B = feats.shape[0]
        ids = self._ids(obs, B, feats.device)
        x = torch.randn(B, c.action_horizon, c.action_dim, device=feats.device, dtype=feats.dtype) if noise is None \
            else noise.clone().to(feats.dtype)
        for k in range(steps):
            t_bucket = torch.full((B,), int(k / steps * c.num_timestep_buckets), device=feats.device, dtype=torch.long)
            x = x + self.action_head.velocity(feats, valid, is_image, obs["state"].to(feats.dtype), x, t_bucket, ids) / steps
        return x


# ------------------------------------------------------------------------------------------------ checkpoints
_AH = "action_head."
GROOT_HEAD_NAME_MAP: List[Tuple[str, str]] = [
    (_AH + "model.timestep_encoder.timestep_embedder.linear_1.{wb}", "action_head.model.timestep_encoder.linear_1.{wb}"),
    (_AH + "model.timestep_encoder.timestep_embedder.linear_2.{wb}", "action_head.model.timestep_encoder.linear_2.{wb}"),
    (_AH + "model.transformer_blocks.{i}.norm1.linear.{wb}", "action_head.model.blocks.{i}.ada.{wb}"),
    (_AH + "model.transformer_blocks.{i}.attn1.to_q.{wb}", "action_head.model.blocks.{i}.to_q.{wb}"),
    (_AH + "model.transformer_blocks.{i}.attn1.to_k.{wb}", "action_head.model.blocks.{i}.to_k.{wb}"),
    (_AH + "model.transformer_blocks.{i}.attn1.to_v.{wb}", "action_head.model.blocks.{i}.to_v.{wb}"),
    (_AH + "model.transformer_blocks.{i}.attn1.to_out.0.{wb}", "action_head.model.blocks.{i}.to_out.{wb}"),
    (_AH + "model.transformer_blocks.{i}.norm3.{wb}", "action_head.model.blocks.{i}.norm3.{wb}"),
    (_AH + "model.transformer_blocks.{i}.ff.net.0.proj.{wb}", "action_head.model.blocks.{i}.ff_in.{wb}"),
    (_AH + "model.transformer_blocks.{i}.ff.net.2.{wb}", "action_head.model.blocks.{i}.ff_out.{wb}"),
    (_AH + "model.proj_out_1.{wb}", "action_head.model.proj_out_1.{wb}"),
    (_AH + "model.proj_out_2.{wb}", "action_head.model.proj_out_2.{wb}"),
    (_AH + "vlln.{wb}", "action_head.vlln.{wb}"),
    (_AH + "position_embedding.weight", "action_head.position_embedding.weight"),
    (_AH + "mask_token", "action_head.mask_token"),
] + [(_AH + f"vl_self_attention.transformer_blocks.{{i}}.{there}.{{wb}}", f"action_head.vl_self_attention.blocks.{{i}}.{here}.{{wb}}")
     for there, here in (("norm1", "norm1"), ("attn1.to_q", "to_q"), ("attn1.to_k", "to_k"), ("attn1.to_v", "to_v"),
                         ("attn1.to_out.0", "to_out"), ("norm3", "norm3"), ("ff.net.0.proj", "ff_in"), ("ff.net.2", "ff_out"))
] + [(_AH + f"{m}.{l}.{p}", f"action_head.{m}.{l}.{p}") for m, ls in (("state_encoder", ("layer1", "layer2")),
                                                                     ("action_decoder", ("layer1", "layer2")),
                                                                     ("action_encoder", ("W1", "W2", "W3")))
     for l in ls for p in ("W", "b")]


def convert_groot_state_dict(sd: Dict[str, torch.Tensor], cfg: GrootConfig, to_public: bool = False,
                             head_only: bool = True) -> Dict[str, torch.Tensor]:
    """Action-head tensors of a public GR00T N1.6 checkpoint -> names here (or back). Backbone tensors
    (``backbone.*``) are passed over when `head_only`; otherwise any tensor without a place raises."""
    out, used = {}, set()
    for there, here in GROOT_HEAD_NAME_MAP:
        a, b = (here, there) if to_public else (there, here)
        depth = cfg.vl_self_attention_layers if "vl_self_attention" in there else cfg.dit_layers
        for i in (range(depth) if "{i}" in there else [None]):
            for wb in (("weight", "bias") if "{wb}" in there else (None,)):
                ka = a.replace("{i}", str(i)).replace("{wb}", wb or "")
                if ka in sd and ka not in used:
                    out[b.replace("{i}", str(i)).replace("{wb}", wb or "")] = sd[ka]
                    used.add(ka)
    left = [k for k in sd if k not in used and not (head_only and k.startswith("backbone."))]
    if left:
        raise KeyError(f"{len(left)} tensors have no counterpart, e.g. {sorted(left)[:4]}")
    return out
