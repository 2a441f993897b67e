"""X-VLA policy (reference: loongforge/embodied/model/xvla/modeling_xvla.py:42-232, transformer.py:230-459,
action_hub.py:60-479; the Florence-2 backbone there is a 3,200-line Hugging Face port).

Three parts, all built here from plain modules:
* Backbone (Florence-2 used as an ENCODER): a hierarchical vision tower in the DaViT style (four stages; every block
  pairs a spatial WINDOW attention with a CHANNEL-group attention, each followed by an MLP; a strided convolution
  between stages) turns the main camera image into tokens; they are projected, get 2-D position and a learned
  "visual temporal" embedding, are concatenated with the instruction's token embeddings and run through a BART-style
  encoder (post-LayerNorm, learned positions). Further camera views go through the vision tower and the projection
  only ("auxiliary visual inputs").
* Soft-prompted transformer: the noisy action chunk, the proprioceptive state and a sinusoidal time embedding are fused
  per action step by a DOMAIN-AWARE linear layer (one weight matrix per robot domain, stored in an embedding table);
  [action tokens | backbone features | auxiliary features] + learned positions, followed by that domain's soft prompt
  tokens, run through pre-LayerNorm transformer blocks; a domain-aware linear layer decodes the action tokens.
* Action space: which action channels are regressed (MSE, scaled per group) and which are gripper logits (BCE), what
  is zeroed in the inputs, what the sampler post-processes (sigmoid on grippers).

The head predicts the clean ACTION (not a velocity): training mixes ``x_t = t * noise + (1 - t) * action`` with one
uniformly spread t per sample; sampling starts from noise and, for t = 1, 1 - 1/steps, ..., re-mixes the noise with
the latest prediction."""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class XVLAConfig:
    # vision tower (DaViT-style)
    image_size: int = 224
    stage_dims: Sequence[int] = (128, 256, 512, 1024)
    stage_depths: Sequence[int] = (1, 1, 9, 1)
    stage_heads: Sequence[int] = (4, 8, 16, 32)
    window: int = 12
    # language / fusion encoder (BART-style)
    vocab_size: int = 51289
    d_model: int = 768
    encoder_layers: int = 6
    encoder_heads: int = 12
    encoder_ffn: int = 3072
    max_text_len: int = 64
    # soft-prompted transformer
    hidden_size: int = 1024
    depth: int = 24
    num_heads: int = 16
    num_domains: int = 20
    len_soft_prompts: int = 32
    max_len_seq: int = 1024
    dim_time: int = 32
    use_hetero_proj: bool = False
    dropout: float = 0.1
    # task
    action_space: str = "ee6d"      # ee6d | joint | auto
    action_dim: int = 20            # real width (auto space pads it to max_action_dim)
    max_action_dim: int = 20
    num_actions: int = 30
    num_views: int = 3
    num_steps: int = 10

    @staticmethod
    def tiny(**kw) -> "XVLAConfig":
        base = dict(image_size=32, stage_dims=(8, 16, 16, 32), stage_depths=(1, 1, 1, 1), stage_heads=(2, 2, 2, 4), window=4,
                    vocab_size=32000, d_model=32, encoder_layers=1, encoder_heads=4, encoder_ffn=64, max_text_len=32,
                    hidden_size=32, depth=2, num_heads=4, num_domains=4, len_soft_prompts=3, max_len_seq=256, dim_time=8,
                    dropout=0.0, action_space="auto", action_dim=7, max_action_dim=8, num_actions=4, num_views=2)
        base.update(kw)
        return XVLAConfig(**base)


# ------------------------------------------------------------------------------------------------ vision tower
class _Mlp(nn.Module):
    def __init__(self, d, ratio=4.0, drop=0.0):
        super().__init__()
        self.fc1, self.fc2, self.drop = nn.Linear(d, int(d * ratio)), nn.Linear(int(d * ratio), d), nn.Dropout(drop)

    def forward(self, x):
        return self.drop(self.fc2(self.drop(F.gelu(self.fc1(x)))))


class _DualBlock(nn.Module):
    """Spatial window attention + MLP, then channel-group attention + MLP (tokens [B, H*W, C] on an H x W grid)."""

    def __init__(self, dim, heads, window):
        super().__init__()
        self.h, self.win = heads, window
        self.n1, self.qkv1, self.o1, self.n2, self.m1 = nn.LayerNorm(dim), nn.Linear(dim, 3 * dim), nn.Linear(dim, dim), \
            nn.LayerNorm(dim), _Mlp(dim)
        self.n3, self.qkv2, self.o2, self.n4, self.m2 = nn.LayerNorm(dim), nn.Linear(dim, 3 * dim), nn.Linear(dim, dim), \
            nn.LayerNorm(dim), _Mlp(dim)

    def _window_attention(self, x, H, W):
        B, _, C = x.shape
        w = self.win
        ph, pw = (-H) % w, (-W) % w
        g = F.pad(x.view(B, H, W, C), (0, 0, 0, pw, 0, ph))
        Hp, Wp = H + ph, W + pw
        g = g.view(B, Hp // w, w, Wp // w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(-1, w * w, C)
        q, k, v = self.qkv1(g).view(g.shape[0], w * w, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(-1, w * w, C)
        o = self.o1(o).view(B, Hp // w, Wp // w, w, w, C).permute(0, 1, 3, 2, 4, 5).reshape(B, Hp, Wp, C)
        return o[:, :H, :W].reshape(B, H * W, C)

    def _channel_attention(self, x):
        """Attention ACROSS channel groups: every head's channels are the 'tokens', the spatial positions the feature
        axis (scores are C/h x C/h, scaled by the token count)."""
        B, N, C = x.shape
        q, k, v = self.qkv2(x).view(B, N, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)  # [B, h, N, c]
        att = torch.softmax((q.transpose(-1, -2) * (N ** -0.5)) @ k, dim=-1)                 # [B, h, c, c]
        o = (att @ v.transpose(-1, -2)).transpose(-1, -2)                                     # [B, h, N, c]
        return self.o2(o.transpose(1, 2).reshape(B, N, C))

    def forward(self, x, H, W):
        x = x + self._window_attention(self.n1(x), H, W)
        x = x + self.m1(self.n2(x))
        x = x + self._channel_attention(self.n3(x))
        return x + self.m2(self.n4(x))


class DaViTTower(nn.Module):
    def __init__(self, c: XVLAConfig):
        super().__init__()
        dims = list(c.stage_dims)
        self.embeds = nn.ModuleList([nn.Conv2d(3 if i == 0 else dims[i - 1], d, 7 if i == 0 else 3, 4 if i == 0 else 2,
                                               3 if i == 0 else 1) for i, d in enumerate(dims)])
        self.embed_norms = nn.ModuleList([nn.LayerNorm(d) for d in dims])
        self.stages = nn.ModuleList([nn.ModuleList([_DualBlock(d, h, c.window) for _ in range(n)])
                                     for d, h, n in zip(dims, c.stage_heads, c.stage_depths)])
        self.out_dim = dims[-1]

    def forward(self, images):
        """[N, 3, S, S] -> (tokens [N, h*w, C_last], (h, w))."""
        x = images
        for conv, norm, blocks in zip(self.embeds, self.embed_norms, self.stages):
            x = conv(x.to(conv.weight.dtype))
            N, C, H, W = x.shape
            t = norm(x.flatten(2).transpose(1, 2))
            for b in blocks:
                t = b(t, H, W)
            x = t.transpose(1, 2).reshape(N, C, H, W)
        return x.flatten(2).transpose(1, 2), (x.shape[2], x.shape[3])


# ------------------------------------------------------------------------------------------------ fusion encoder
class _BartLayer(nn.Module):
    def __init__(self, d, heads, ffn, drop):
        super().__init__()
        self.h = heads
        self.qkv, self.o, self.ln1 = nn.Linear(d, 3 * d), nn.Linear(d, d), nn.LayerNorm(d)
        self.fc1, self.fc2, self.ln2, self.drop = nn.Linear(d, ffn), nn.Linear(ffn, d), nn.LayerNorm(d), nn.Dropout(drop)

    def forward(self, x, key_valid):
        B, L, D = x.shape
        q, k, v = self.qkv(x).view(B, L, 3, self.h, D // self.h).permute(2, 0, 3, 1, 4)
        o = F.scaled_dot_product_attention(q, k, v, attn_mask=key_valid[:, None, None, :])
        x = self.ln1(x + self.drop(self.o(o.transpose(1, 2).reshape(B, L, D))))       # post-LayerNorm, as BART
        return self.ln2(x + self.drop(self.fc2(self.drop(F.gelu(self.fc1(x))))))


class FlorenceEncoder(nn.Module):
    def __init__(self, c: XVLAConfig):
        super().__init__()
        self.c = c
        self.tower = DaViTTower(c)
        grid = max(c.image_size // 32, 1)
        self.image_proj = nn.Linear(self.tower.out_dim, c.d_model)
        self.image_proj_norm = nn.LayerNorm(c.d_model)
        self.row_embed = nn.Embedding(max(grid, 50), c.d_model - c.d_model // 2)
        self.col_embed = nn.Embedding(max(grid, 50), c.d_model // 2)
        self.temporal_embed = nn.Parameter(torch.zeros(1, 1, c.d_model))
        self.embed_tokens = nn.Embedding(c.vocab_size, c.d_model)
        self.embed_positions = nn.Embedding(4096, c.d_model)
        self.embed_norm = nn.LayerNorm(c.d_model)
        self.layers = nn.ModuleList([_BartLayer(c.d_model, c.encoder_heads, c.encoder_ffn, c.dropout)
                                     for _ in range(c.encoder_layers)])

    def image_features(self, images):
        t, (h, w) = self.tower(images)
        # tables are read through the modules' forward (under FSDP their weights are shards outside it)
        col, row = self.col_embed(torch.arange(w, device=t.device)), self.row_embed(torch.arange(h, device=t.device))
        pos = torch.cat([col.unsqueeze(0).expand(h, -1, -1), row.unsqueeze(1).expand(-1, w, -1)], dim=-1).reshape(1, h * w, -1)
        f = self.image_proj(t)
        f = self.image_proj_norm(f + pos.to(f.dtype))
        return f + self.temporal_embed.to(f.dtype)

    def forward(self, tokens, token_mask, images, image_mask):
        """images [B, V, 3, S, S], image_mask [B, V]: view 0 is fused with the text, the other views are auxiliary."""
        B, V = images.shape[:2]
        feats = self.image_features(images.flatten(0, 1))
        n = feats.shape[1]
        feats = feats.view(B, V, n, -1) * image_mask.view(B, V, 1, 1).to(feats.dtype)
        text = self.embed_tokens(tokens) * math.sqrt(self.c.d_model)
        x = torch.cat([feats[:, 0], text.to(feats.dtype)], dim=1)
        valid = torch.cat([torch.ones(B, n, dtype=torch.bool, device=x.device), token_mask.bool()], dim=1)
        x = self.embed_norm(x + self.embed_positions(torch.arange(x.shape[1], device=x.device)).to(x.dtype))
        for layer in self.layers:
            x = layer(x, valid)
        aux = feats[:, 1:].reshape(B, (V - 1) * n, feats.shape[-1])  # one camera: no auxiliary tokens
        return x, aux


# ------------------------------------------------------------------------------------------------ action head
class DomainAwareLinear(nn.Module):
    """Per-domain (W, b), stored as rows of two embedding tables: ``y = x W[d] + b[d]``."""

    def __init__(self, din, dout, num_domains):
        super().__init__()
        self.din, self.dout = din, dout
        self.fc, self.bias = nn.Embedding(num_domains, din * dout), nn.Embedding(num_domains, dout)
        nn.init.xavier_uniform_(self.fc.weight.view(num_domains, din, dout))
        nn.init.zeros_(self.bias.weight)

    def forward(self, x, domain_id):
        B = domain_id.shape[0]
        W = self.fc(domain_id).view(B, self.din, self.dout).to(x.dtype)
        return torch.matmul(x, W) + self.bias(domain_id).view(B, 1, self.dout).to(x.dtype)


def _time_embedding(t: torch.Tensor, dim: int) -> torch.Tensor:
    half = dim // 2
    freq = torch.exp(-math.log(100.0) * torch.arange(half, device=t.device, dtype=torch.float32) / max(half, 1))
    ang = t.float()[:, None] * 100.0 * freq
    return torch.cat([ang.cos(), ang.sin()], dim=-1)


class SoftPromptedTransformer(nn.Module):
    def __init__(self, c: XVLAConfig, dim_action: int, dim_proprio: int):
        super().__init__()
        self.c, d = c, c.hidden_size
        self.blocks = nn.ModuleList([nn.ModuleDict(dict(
            n1=nn.LayerNorm(d), qkv=nn.Linear(d, 3 * d), o=nn.Linear(d, d), n2=nn.LayerNorm(d), mlp=_Mlp(d, 4.0, c.dropout)))
            for _ in range(c.depth)])
        if c.use_hetero_proj:
            self.vlm_proj, self.aux_proj = DomainAwareLinear(c.d_model, d, c.num_domains), DomainAwareLinear(c.d_model, d, c.num_domains)
        else:
            self.vlm_proj, self.aux_proj = nn.Linear(c.d_model, d), nn.Linear(c.d_model, d)
        self.pos_emb = nn.Parameter(torch.zeros(1, c.max_len_seq, d))
        nn.init.normal_(self.pos_emb, std=0.02)
        self.norm = nn.LayerNorm(d)
        self.action_encoder = DomainAwareLinear(dim_action + c.dim_time + dim_proprio, d, c.num_domains)
        self.action_decoder = DomainAwareLinear(d, dim_action, c.num_domains)
        self.soft_prompt_hub = nn.Embedding(c.num_domains, c.len_soft_prompts * d) if c.len_soft_prompts > 0 else None
        if self.soft_prompt_hub is not None:
            nn.init.normal_(self.soft_prompt_hub.weight, std=0.02)

    def forward(self, domain_id, vlm, aux, noisy_action, proprio, t):
        c = self.c
        B, T, _ = noisy_action.shape
        time_tok = _time_embedding(t, c.dim_time).to(noisy_action.dtype).unsqueeze(1).expand(B, T, -1)
        prop_tok = proprio.unsqueeze(1).expand(B, T, -1)
        x = self.action_encoder(torch.cat([noisy_action, prop_tok, time_tok], dim=-1), domain_id)
        pv = self.vlm_proj(vlm, domain_id) if c.use_hetero_proj else self.vlm_proj(vlm)
        pa = self.aux_proj(aux, domain_id) if c.use_hetero_proj else self.aux_proj(aux)
        x = torch.cat([x, pv.to(x.dtype), pa.to(x.dtype)], dim=1)
        if x.shape[1] > self.pos_emb.shape[1]:
            raise ValueError(f"sequence length {x.shape[1]} exceeds max_len_seq = {self.pos_emb.shape[1]}")
        x = x + self.pos_emb[:, : x.shape[1]].to(x.dtype)
        if self.soft_prompt_hub is not None:
            x = torch.cat([x, self.soft_prompt_hub(domain_id).view(B, c.len_soft_prompts, -1).to(x.dtype)], dim=1)
        h = c.num_heads
        for b in self.blocks:
            L, D = x.shape[1], x.shape[2]
            q, k, v = b["qkv"](b["n1"](x)).view(B, L, 3, h, D // h).permute(2, 0, 3, 1, 4)
            x = x + b["o"](F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, D))
            x = x + b["mlp"](b["n2"](x))
        return self.action_decoder(self.norm(x[:, :T]), domain_id)


# ------------------------------------------------------------------------------------------------ action spaces
class ActionSpace(nn.Module):
    """`regress`: (start, end, scale) channel groups under MSE; `gripper`: channels that are logits under BCE."""
    dim_action = 0
    regress: List[Tuple[int, int, float]] = []
    gripper: Tuple[int, ...] = ()

    def compute_loss(self, pred, target, valid: Optional[torch.Tensor] = None) -> Dict[str, torch.Tensor]:
        B, T, _ = pred.shape
        v = torch.ones(B, device=pred.device, dtype=pred.dtype) if valid is None else valid.to(pred.dtype)
        nv = v.sum().clamp(min=1)
        out = {}
        for i, (s, e, scale) in enumerate(self.regress):
            sq = ((pred[..., s:e] - target[..., s:e]).float().pow(2) * v.view(B, 1, 1)).sum()
            out[f"regress_{i}"] = sq / (T * (e - s)) / nv * scale
        if self.gripper:
            g = list(self.gripper)
            l, y = pred[..., g].float(), target[..., g].float()
            per = l.clamp(min=0) - l * y + torch.log1p(torch.exp(-l.abs()))
            out["gripper"] = (per * v.view(B, 1, 1)).sum() / (T * len(g)) / nv
        return out

    def preprocess(self, proprio, action):
        if not self.gripper:
            return proprio, action
        g = list(self.gripper)
        p, a = proprio.clone(), action.clone()
        p[..., [i for i in g if i < p.shape[-1]]] = 0.0
        a[..., g] = 0.0
        return p, a

    def postprocess(self, action):
        if self.gripper:
            action = action.clone()
            g = list(self.gripper)
            action[..., g] = torch.sigmoid(action[..., g])
        return action


class EE6DSpace(ActionSpace):
    """Two arms x (xyz, 6-D rotation, gripper): 20 channels; positions weighted 500, rotations 10."""
    dim_action = 20
    regress = [(0, 3, 500.0), (10, 13, 500.0), (3, 9, 10.0), (13, 19, 10.0)]
    gripper = (9, 19)


class JointSpace(ActionSpace):
    """Two arms x (7 joints + gripper): joints regressed, grippers as logits."""
    dim_action = 16
    regress = [(0, 7, 1.0), (8, 15, 1.0)]
    gripper = (7, 15)


class AutoSpace(ActionSpace):
    """Any robot: `real_dim` channels regressed, padded with zeros to the model's width."""

    def __init__(self, real_dim: int, max_dim: int):
        super().__init__()
        self.real_dim, self.dim_action = real_dim, max_dim
        self.regress = [(0, real_dim, 1.0)]

    def pad(self, x):
        return F.pad(x, (0, self.dim_action - x.shape[-1])) if x.shape[-1] < self.dim_action else x

    def preprocess(self, proprio, action):
        return self.pad(proprio), self.pad(action)

    def postprocess(self, action):
        return action[..., : self.real_dim]


def build_action_space(c: XVLAConfig) -> ActionSpace:
    if c.action_space == "ee6d":
        return EE6DSpace()
    if c.action_space == "joint":
        return JointSpace()
    if c.action_space == "auto":
        return AutoSpace(c.action_dim, c.max_action_dim)
    raise KeyError(f"unknown action space {c.action_space!r}")


# ------------------------------------------------------------------------------------------------ the policy
class XVLAPolicy(nn.Module):
    """batch: ``images`` [B, views, 3, S, S], ``image_masks`` [B, views], ``tokens`` [B, L], ``token_mask``, ``state``
    [B, d], ``domain_id`` [B], ``actions`` [B, num_actions, action_dim]."""

    def default_lora_targets(self):
        return ["qkv", "o", "qkv1", "qkv2", "o1", "o2"]


    def __init__(self, c: XVLAConfig):
        super().__init__()
        self.c = c
        self.space = build_action_space(c)
        self.encoder = FlorenceEncoder(c)
        self.transformer = SoftPromptedTransformer(c, self.space.dim_action, self.space.dim_action)

    def _domain(self, batch, B, device):
        d = batch.get("domain_id", batch.get("embodiment_id"))
        if d is None:
            return torch.zeros(B, dtype=torch.long, device=device)
        d = torch.as_tensor(d, device=device).long().reshape(-1)
        return d.expand(B) if d.numel() == 1 else d

    def _encode(self, batch):
        imgs = batch["images"]
        B, V = imgs.shape[:2]
        im = batch.get("image_masks")
        im = torch.ones(B, V, dtype=torch.bool, device=imgs.device) if im is None else im.bool()
        tm = batch.get("token_mask")
        tm = torch.ones_like(batch["tokens"], dtype=torch.bool) if tm is None else tm.bool()
        return self.encoder(batch["tokens"], tm, imgs, im)

    def _proprio(self, batch, dtype):
        s = batch["state"].to(dtype)
        d = self.space.dim_action
        return F.pad(s, (0, d - s.shape[-1])) if s.shape[-1] < d else s[..., :d]

    def forward(self, batch, noise=None, t=None):
        action = batch["actions"]
        B = action.shape[0]
        vlm, aux = self._encode(batch)
        if t is None:  # one random offset, samples spread evenly over [0, 1)
            t = (torch.rand(1, device=action.device) + torch.arange(B, device=action.device) / B) % (1 - 1e-5)
        noise = torch.randn_like(action) if noise is None else noise
        tt = t.view(B, 1, 1).to(action.dtype)
        proprio, noisy = self.space.preprocess(self._proprio(batch, vlm.dtype), (noise * tt + action * (1 - tt)).to(vlm.dtype))
        pred = self.transformer(self._domain(batch, B, action.device), vlm, aux, noisy, proprio, t)
        target = self.space.pad(action) if isinstance(self.space, AutoSpace) else action
        losses = self.space.compute_loss(pred, target.to(pred.dtype), batch.get("valid_mask"))
        return sum(losses.values())

    @torch.no_grad()
    def predict_action(self, obs, steps: Optional[int] = None, noise=None):
        c = self.c
        steps = max(1, int(steps or c.num_steps))
        vlm, aux = self._encode(obs)
        B = vlm.shape[0]
        dom = self._domain(obs, B, vlm.device)
        D = self.space.dim_action
        x1 = torch.randn(B, c.num_actions, D, device=vlm.device, dtype=vlm.dtype) if noise is None else \
            F.pad(noise, (0, D - noise.shape[-1])).to(vlm.dtype)
        action = torch.zeros_like(x1)
        prop = self._proprio(obs, vlm.dtype)
        for i in range(steps, 0, -1):
            t = torch.full((B,), i / steps, device=vlm.device)
            tt = t.view(B, 1, 1).to(x1.dtype)
            p_m, x_m = self.space.preprocess(prop, x1 * tt + action * (1 - tt))
            action = self.transformer(dom, vlm, aux, x_m, p_m, t)
        return self.space.postprocess(action)
