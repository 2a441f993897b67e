"""Pi0.5 vision-language-action policy (reference: loongforge/embodied/model/pi05/modeling_pi05.py:259-1064, which
wraps the Hugging Face PaliGemma classes; this file builds the network from plain modules).

Architecture. A *prefix* of image tokens (SigLIP-style ViT, one image per camera, projected to the language width) and
instruction tokens (the discretised robot state is part of the instruction text in Pi0.5) runs through a Gemma-style
decoder; a *suffix* of `action_horizon` noisy-action tokens runs through a narrower Gemma-style "action expert" with the
same depth and head geometry. The two stacks share attention layer by layer: queries / keys / values of both streams are
concatenated, every stream keeps its own weights for everything else (mixture of transformers). Mask: the prefix is
bidirectional within itself and never looks at the suffix; the suffix sees the prefix and itself. The flow-matching
time enters the expert through adaptive RMSNorm: ``cond = swish(W2 swish(W1 sincos(t)))`` gives every norm of the expert
a (scale, shift, gate) triple; the language stack uses plain RMSNorm (``x * (1 + w)``).

Training: ``x_t = t * noise + (1 - t) * actions``, target ``noise - actions``, t ~ 0.001 + 0.999 * Beta(1.5, 1), MSE
over the real action dims. Sampling: the prefix runs once (its keys / values are cached), then `num_steps` Euler steps
from t = 1 to 0 re-run only the expert.

Checkpoints: `PI05_NAME_MAP` maps the parameter names of the public lerobot / openpi Pi0.5 checkpoints
(``paligemma_with_expert.paligemma...``, ``paligemma_with_expert.gemma_expert...``) to the names used here;
`convert_pi05_state_dict` applies it (both directions) and fuses / splits the q, k, v and gate, up projections."""
from __future__ import annotations

import dataclasses
import math
import re
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F


@dataclasses.dataclass
class GemmaDims:
    width: int
    depth: int
    mlp_dim: int
    num_heads: int = 8
    num_kv_heads: int = 1
    head_dim: int = 256


GEMMA_VARIANTS = {"gemma_2b": GemmaDims(2048, 18, 16384), "gemma_300m": GemmaDims(1024, 18, 4096),
                  "tiny": GemmaDims(64, 2, 128, 4, 1, 16), "tiny_expert": GemmaDims(32, 2, 64, 4, 1, 16)}


@dataclasses.dataclass
class Pi05Config:
    vlm: str = "gemma_2b"
    expert: str = "gemma_300m"
    vocab_size: int = 257152
    # vision tower (SigLIP So400m/14 at 224 px by default)
    image_size: int = 224
    patch_size: int = 14
    vit_width: int = 1152
    vit_depth: int = 27
    vit_heads: int = 16
    vit_mlp: int = 4304
    num_cameras: int = 3
    # task
    action_dim: int = 7
    max_action_dim: int = 32
    action_horizon: int = 50
    max_token_len: int = 200
    # flow matching
    time_beta: Tuple[float, float] = (1.5, 1.0)
    min_period: float = 4e-3
    max_period: float = 4.0
    num_steps: int = 10
    rope_theta: float = 10000.0
    freeze_vision_encoder: bool = False
    train_expert_only: bool = False

    @staticmethod
    def tiny(**kw) -> "Pi05Config":
        base = dict(vlm="tiny", expert="tiny_expert", vocab_size=512, image_size=28, patch_size=14, vit_width=32,
                    vit_depth=2, vit_heads=4, vit_mlp=64, num_cameras=2, action_dim=7, max_action_dim=8,
                    action_horizon=6, max_token_len=12)
        base.update(kw)
        return Pi05Config(**base)


# ------------------------------------------------------------------------------------------------ building blocks
class RMSNorm(nn.Module):
    """Gemma RMSNorm ``x / rms * (1 + w)``; with `cond_dim` the adaptive form: a linear map of the condition gives
    (scale, shift, gate) and the norm has no weight of its own."""

    def __init__(self, dim: int, cond_dim: Optional[int] = None, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        if cond_dim is None:
            self.weight = nn.Parameter(torch.zeros(dim))
            self.dense = None
        else:
            self.weight = None
            self.dense = nn.Linear(cond_dim, 3 * dim)
            nn.init.zeros_(self.dense.weight)
            nn.init.zeros_(self.dense.bias)

    def forward(self, x, cond=None):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps)
        if self.dense is None:
            return (y * (1.0 + self.weight.float())).to(x.dtype), None
        scale, shift, gate = self.dense(cond).float().unsqueeze(1).chunk(3, dim=-1)
        return (y * (1.0 + scale) + shift).to(x.dtype), gate.to(x.dtype)


def _residual(x, y, gate):
    return x + y if gate is None else x + y * gate


def rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """x [B, H, L, D], positions [B, L]: rotate-half rotary embedding."""
    d = x.shape[-1]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = positions.float()[:, None, :, None] * inv
    cos, sin = ang.cos(), ang.sin()
    x1, x2 = x.float()[..., : d // 2], x.float()[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], dim=-1).to(x.dtype)


class GemmaLayer(nn.Module):
    """One stream's weights of a joint layer: fused QKV, output projection, GeGLU MLP, two (adaptive) norms."""

    def __init__(self, d: GemmaDims, cond_dim: Optional[int]):
        super().__init__()
        self.d = d
        self.input_norm = RMSNorm(d.width, cond_dim)
        self.qkv = nn.Linear(d.width, (d.num_heads + 2 * d.num_kv_heads) * d.head_dim, bias=False)
        self.o = nn.Linear(d.num_heads * d.head_dim, d.width, bias=False)
        self.post_norm = RMSNorm(d.width, cond_dim)
        self.gate_up = nn.Linear(d.width, 2 * d.mlp_dim, bias=False)
        self.down = nn.Linear(d.mlp_dim, d.width, bias=False)

    def project_qkv(self, x, cond):
        h, gate = self.input_norm(x, cond)
        B, L, _ = h.shape
        d = self.d
        qkv = self.qkv(h).view(B, L, d.num_heads + 2 * d.num_kv_heads, d.head_dim).transpose(1, 2)
        q, k, v = qkv.split([d.num_heads, d.num_kv_heads, d.num_kv_heads], dim=1)
        return q, k, v, gate

    def finish(self, x, attn, gate, cond):
        x = _residual(x, self.o(attn), gate)
        h, gate2 = self.post_norm(x, cond)
        g, u = self.gate_up(h).chunk(2, dim=-1)
        return _residual(x, self.down(F.gelu(g, approximate="tanh") * u), gate2)


class JointDecoder(nn.Module):
    """Language stack + action expert with shared attention. ``forward`` takes one or both streams; a cache of the
    prefix keys / values lets the expert run alone during sampling."""

    FSDP_NO_WRAP = ("GemmaLayer",)  # the decoder calls the layers' projection / finish methods, not their forward

    def __init__(self, c: Pi05Config):
        super().__init__()
        self.c = c
        self.vd, self.ed = GEMMA_VARIANTS[c.vlm], GEMMA_VARIANTS[c.expert]
        assert (self.vd.depth, self.vd.num_heads, self.vd.num_kv_heads, self.vd.head_dim) == \
            (self.ed.depth, self.ed.num_heads, self.ed.num_kv_heads, self.ed.head_dim), "streams must share head geometry"
        self.embed_tokens = nn.Embedding(c.vocab_size, self.vd.width)
        self.lang = nn.ModuleList([GemmaLayer(self.vd, None) for _ in range(self.vd.depth)])
        self.expert = nn.ModuleList([GemmaLayer(self.ed, self.ed.width) for _ in range(self.ed.depth)])
        self.lang_norm = RMSNorm(self.vd.width)
        self.expert_norm = RMSNorm(self.ed.width, self.ed.width)

    def forward(self, prefix, suffix, mask, positions, cond=None, cache: Optional[List] = None, fill_cache=False):
        """prefix [B, P, Wv] or None (then `cache` holds its keys / values), suffix [B, S, We] or None; `mask`
        [B, Lq, Lk] boolean over the concatenated (prefix, suffix) keys; `positions` [B, Lq]."""
        streams = [(prefix, self.lang, None), (suffix, self.expert, cond)]
        new_cache = [] if fill_cache else None
        rep = self.vd.num_heads // self.vd.num_kv_heads
        for li in range(self.vd.depth):
            qs, ks, vs, gates = [], [], [], []
            for x, layers, cnd in streams:
                if x is None:
                    continue
                q, k, v, g = layers[li].project_qkv(x, cnd)
                qs.append(q), ks.append(k), vs.append(v), gates.append(g)
            q = rope(torch.cat(qs, dim=2), positions, self.c.rope_theta)
            k_new, v_new = torch.cat(ks, dim=2), torch.cat(vs, dim=2)
            k_new = rope(k_new, positions, self.c.rope_theta)
            if fill_cache:
                new_cache.append((k_new, v_new))
            if cache is not None:  # the expert alone: its keys follow the cached prefix keys
                k_all, v_all = torch.cat([cache[li][0], k_new], dim=2), torch.cat([cache[li][1], v_new], dim=2)
            else:
                k_all, v_all = k_new, v_new
            o = F.scaled_dot_product_attention(q, k_all.repeat_interleave(rep, dim=1), v_all.repeat_interleave(rep, dim=1),
                                               attn_mask=mask[:, None])
            o = o.transpose(1, 2).reshape(q.shape[0], q.shape[2], -1)
            outs, start, gi = [], 0, 0
            new_streams = []
            for x, layers, cnd in streams:
                if x is None:
                    new_streams.append((None, layers, cnd))
                    continue
                n = x.shape[1]
                y = layers[li].finish(x, o[:, start:start + n].to(x.dtype), gates[gi], cnd)
                start, gi = start + n, gi + 1
                new_streams.append((y, layers, cnd))
            streams = new_streams
        pre = self.lang_norm(streams[0][0])[0] if streams[0][0] is not None else None
        suf = self.expert_norm(streams[1][0], cond)[0] if streams[1][0] is not None else None
        return pre, suf, new_cache


class SiglipTower(nn.Module):
    """ViT encoder: conv patch embedding + learned positions, pre-LayerNorm blocks with biased projections and a
    tanh-GELU MLP, final LayerNorm; a linear projector maps to the language width."""

    def __init__(self, c: Pi05Config, out_dim: int):
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
        self.projector = nn.Linear(c.vit_width, out_dim)

    def forward(self, images: torch.Tensor) -> torch.Tensor:
        """images [B, 3, H, W] in [-1, 1] -> [B, n_patches, out_dim]."""
        x = self.patch_embedding(images.to(self.patch_embedding.weight.dtype)).flatten(2).transpose(1, 2)
        x = x + self.position_embedding.weight
        B, L, C = x.shape
        h = self.c.vit_heads
        for blk in self.layers:
            q, k, v = blk["qkv"](blk["ln1"](x)).view(B, L, 3, h, C // h).permute(2, 0, 3, 1, 4)
            x = x + blk["out"](F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, C))
            x = x + blk["fc2"](F.gelu(blk["fc1"](blk["ln2"](x)), approximate="tanh"))
        return self.projector(self.post_layernorm(x))


def sincos_time_embedding(t: torch.Tensor, dim: int, min_period: float, max_period: float) -> torch.Tensor:
    """t [B] in [0, 1] -> [B, dim]: sin | cos over log-spaced periods in [min_period, max_period]."""
    frac = torch.linspace(0.0, 1.0, dim // 2, dtype=torch.float64, device=t.device)
    period = min_period * (max_period / min_period) ** frac
    ang = (2 * math.pi / period)[None, :] * t.double()[:, None]
    return torch.cat([ang.sin(), ang.cos()], dim=-1).float()


# ------------------------------------------------------------------------------------------------ the policy
class Pi05Policy(nn.Module):
    """batch: ``images`` [B, cams, 3, H, W], ``image_masks`` [B, cams] (False = camera absent), ``tokens`` [B, L],
    ``token_mask`` [B, L], ``actions`` [B, horizon, action_dim] (training)."""

    def default_lora_targets(self):
        """Attention and MLP projections of the language stack and the action expert (the vision tower stays exact)."""
        return ["policy.decoder.*.qkv", "policy.decoder.*.o", "policy.decoder.*.gate_up", "policy.decoder.*.down",
                "decoder.*.qkv", "decoder.*.o", "decoder.*.gate_up", "decoder.*.down"]


    def __init__(self, c: Pi05Config):
        super().__init__()
        self.c = c
        self.decoder = JointDecoder(c)
        we = self.decoder.ed.width
        self.vision = SiglipTower(c, self.decoder.vd.width)
        self.action_in_proj = nn.Linear(c.max_action_dim, we)
        self.action_out_proj = nn.Linear(we, c.max_action_dim)
        self.time_mlp_in = nn.Linear(we, we)
        self.time_mlp_out = nn.Linear(we, we)
        if c.freeze_vision_encoder or c.train_expert_only:
            self.vision.requires_grad_(False)
        if c.train_expert_only:
            self.decoder.lang.requires_grad_(False)
            self.decoder.embed_tokens.requires_grad_(False)
            self.decoder.lang_norm.requires_grad_(False)

    # ---- embedding of the two streams
    def embed_prefix(self, batch) -> Tuple[torch.Tensor, torch.Tensor]:
        imgs = batch["images"]
        B, cams = imgs.shape[:2]
        emb = self.vision(imgs.flatten(0, 1))  # [B * cams, n, W]
        n = emb.shape[1]
        emb = emb.view(B, cams * n, -1)
        img_valid = batch.get("image_masks")
        img_valid = torch.ones(B, cams, dtype=torch.bool, device=imgs.device) if img_valid is None else img_valid.bool()
        tok = self.decoder.embed_tokens(batch["tokens"]) * math.sqrt(self.decoder.vd.width)
        tmask = batch.get("token_mask")
        tmask = torch.ones_like(batch["tokens"], dtype=torch.bool) if tmask is None else tmask.bool()
        valid = torch.cat([img_valid.repeat_interleave(n, dim=1), tmask], dim=1)
        return torch.cat([emb.to(tok.dtype), tok], dim=1), valid

    def embed_suffix(self, noisy_actions, t):
        c = self.c
        a = F.pad(noisy_actions, (0, c.max_action_dim - noisy_actions.shape[-1]))
        x = self.action_in_proj(a.to(self.action_in_proj.weight.dtype))
        te = sincos_time_embedding(t, x.shape[-1], c.min_period, c.max_period).to(x.dtype)
        cond = F.silu(self.time_mlp_out(F.silu(self.time_mlp_in(te))))
        return x, cond

    @staticmethod
    def _masks(valid_prefix, n_suffix):
        """-> (joint mask [B, P + S, P + S], positions [B, P + S]): padded keys are masked; positions count valid tokens."""
        B, P = valid_prefix.shape
        dev = valid_prefix.device
        key_valid = torch.cat([valid_prefix, torch.ones(B, n_suffix, dtype=torch.bool, device=dev)], dim=1)
        is_suffix = torch.cat([torch.zeros(P, dtype=torch.bool, device=dev), torch.ones(n_suffix, dtype=torch.bool, device=dev)])
        allowed = is_suffix[:, None] | ~is_suffix[None, :]  # query row sees key column unless (prefix row, suffix column)
        mask = allowed[None] & key_valid[:, None, :]
        pos = key_valid.long().cumsum(1) - 1
        return mask, pos.clamp(min=0)

    # ---- training
    def sample_time(self, B, device):
        a, b = self.c.time_beta
        return torch.distributions.Beta(a, b).sample((B,)).to(device) * 0.999 + 0.001

    def forward(self, batch: Dict[str, torch.Tensor], noise: Optional[torch.Tensor] = None,
                t: Optional[torch.Tensor] = None) -> torch.Tensor:
        actions = batch["actions"]
        B, Hn, A = actions.shape
        noise = torch.randn_like(actions) if noise is None else noise
        t = self.sample_time(B, actions.device) if t is None else t
        tt = t.view(B, 1, 1).to(actions.dtype)
        x_t, u_t = tt * noise + (1 - tt) * actions, noise - actions
        prefix, valid = self.embed_prefix(batch)
        suffix, cond = self.embed_suffix(x_t, t)
        mask, pos = self._masks(valid, Hn)
        _, suf, _ = self.decoder(prefix, suffix.to(prefix.dtype), mask, pos, cond.to(prefix.dtype))
        v = self.action_out_proj(suf.to(self.action_out_proj.weight.dtype))[..., :A]
        err = (v.float() - u_t.float()).pow(2)
        m = batch.get("action_mask")
        if m is not None:
            m = m.float() if m.dim() == 3 else m.float().unsqueeze(-1).expand_as(err)
            return (err * m).sum() / m.sum().clamp(min=1)
        return err.mean()

    # ---- sampling
    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: Optional[int] = None, noise=None) -> torch.Tensor:
        c = self.c
        steps = steps or c.num_steps
        prefix, valid = self.embed_prefix(obs)
        B, P = valid.shape
        mask, pos = self._masks(valid, c.action_horizon)
        # the prefix alone, once: its rows of the joint mask never look at suffix columns
        _, _, cache = self.decoder(prefix, None, mask[:, :P, :P], pos[:, :P], fill_cache=True)
        x = torch.randn(B, c.action_horizon, c.action_dim, device=prefix.device) if noise is None else noise.clone()
        dt = -1.0 / steps
        t = torch.ones(B, device=prefix.device)
        for _ in range(steps):
            suffix, cond = self.embed_suffix(x, t)
            _, suf, _ = self.decoder(None, suffix.to(prefix.dtype), mask[:, P:], pos[:, P:], cond.to(prefix.dtype), cache=cache)
            v = self.action_out_proj(suf.to(self.action_out_proj.weight.dtype))[..., :c.action_dim]
            x = x + dt * v.to(x.dtype)
            t = t + dt
        return x


# ------------------------------------------------------------------------------------------------ checkpoints
_PG = "paligemma_with_expert.paligemma.model"
_EX = "paligemma_with_expert.gemma_expert.model"
_VT = _PG + ".vision_tower.vision_model"
# (public checkpoint name pattern, name here); {i} is the layer index. Fused tensors are handled in the converter.
PI05_NAME_MAP: List[Tuple[str, str]] = [
    (_VT + ".embeddings.patch_embedding.{wb}", "vision.patch_embedding.{wb}"),
    (_VT + ".embeddings.position_embedding.weight", "vision.position_embedding.weight"),
    (_VT + ".encoder.layers.{i}.layer_norm1.{wb}", "vision.layers.{i}.ln1.{wb}"),
    (_VT + ".encoder.layers.{i}.layer_norm2.{wb}", "vision.layers.{i}.ln2.{wb}"),
    (_VT + ".encoder.layers.{i}.self_attn.out_proj.{wb}", "vision.layers.{i}.out.{wb}"),
    (_VT + ".encoder.layers.{i}.mlp.fc1.{wb}", "vision.layers.{i}.fc1.{wb}"),
    (_VT + ".encoder.layers.{i}.mlp.fc2.{wb}", "vision.layers.{i}.fc2.{wb}"),
    (_VT + ".post_layernorm.{wb}", "vision.post_layernorm.{wb}"),
    (_PG + ".multi_modal_projector.linear.{wb}", "vision.projector.{wb}"),
    (_PG + ".language_model.embed_tokens.weight", "decoder.embed_tokens.weight"),
    (_PG + ".language_model.norm.weight", "decoder.lang_norm.weight"),
    (_PG + ".language_model.layers.{i}.input_layernorm.weight", "decoder.lang.{i}.input_norm.weight"),
    (_PG + ".language_model.layers.{i}.post_attention_layernorm.weight", "decoder.lang.{i}.post_norm.weight"),
    (_PG + ".language_model.layers.{i}.self_attn.o_proj.weight", "decoder.lang.{i}.o.weight"),
    (_PG + ".language_model.layers.{i}.mlp.down_proj.weight", "decoder.lang.{i}.down.weight"),
    (_EX + ".norm.dense.{wb}", "decoder.expert_norm.dense.{wb}"),
    (_EX + ".layers.{i}.input_layernorm.dense.{wb}", "decoder.expert.{i}.input_norm.dense.{wb}"),
    (_EX + ".layers.{i}.post_attention_layernorm.dense.{wb}", "decoder.expert.{i}.post_norm.dense.{wb}"),
    (_EX + ".layers.{i}.self_attn.o_proj.weight", "decoder.expert.{i}.o.weight"),
    (_EX + ".layers.{i}.mlp.down_proj.weight", "decoder.expert.{i}.down.weight"),
    ("action_in_proj.{wb}", "action_in_proj.{wb}"), ("action_out_proj.{wb}", "action_out_proj.{wb}"),
    ("time_mlp_in.{wb}", "time_mlp_in.{wb}"), ("time_mlp_out.{wb}", "time_mlp_out.{wb}"),
]
# fused here, separate in the public checkpoints: (prefix there, parts there, fused name here)
_FUSED = [(_VT + ".encoder.layers.{i}.self_attn", ("q_proj", "k_proj", "v_proj"), "vision.layers.{i}.qkv", ("weight", "bias")),
          (_PG + ".language_model.layers.{i}.self_attn", ("q_proj", "k_proj", "v_proj"), "decoder.lang.{i}.qkv", ("weight",)),
          (_PG + ".language_model.layers.{i}.mlp", ("gate_proj", "up_proj"), "decoder.lang.{i}.gate_up", ("weight",)),
          (_EX + ".layers.{i}.self_attn", ("q_proj", "k_proj", "v_proj"), "decoder.expert.{i}.qkv", ("weight",)),
          (_EX + ".layers.{i}.mlp", ("gate_proj", "up_proj"), "decoder.expert.{i}.gate_up", ("weight",))]
_STRIP = ("model.architecture.pi05_model.", "architecture.pi05_model.", "model.")
_RENAME = (("action_time_mlp_in.", "time_mlp_in."), ("action_time_mlp_out.", "time_mlp_out."))


def _expand(pattern: str, i: Optional[int], wb: Optional[str]) -> str:
    return pattern.replace("{i}", str(i) if i is not None else "{i}").replace("{wb}", wb or "{wb}")


def convert_pi05_state_dict(sd: Dict[str, torch.Tensor], cfg: Pi05Config, to_public: bool = False
                            ) -> Dict[str, torch.Tensor]:
    """Public checkpoint -> this module's ``state_dict`` (or back with ``to_public``). Unknown keys raise: a silent
    skip would leave weights at their random initialisation."""
    vd, ed = GEMMA_VARIANTS[cfg.vlm], GEMMA_VARIANTS[cfg.expert]
    depth = {"vision": cfg.vit_depth, "lang": vd.depth, "expert": ed.depth}

    def layer_range(name_here: str):
        return range(depth["vision"] if name_here.startswith("vision") else depth["lang"]) if "{i}" in name_here else [None]

    if not to_public:
        src = {}
        for k, v in sd.items():
            for p in _STRIP:  # longest wrapper prefix first
                if k.startswith(p):
                    k = k[len(p):]
                    break
            for a, b in _RENAME:
                k = k.replace(a, b)
            if k.startswith("state_proj."):
                continue  # Pi0 leftover: Pi0.5 feeds the state as text
            src[k] = v
        lm_head = src.pop("paligemma_with_expert.paligemma.lm_head.weight", None)
        if lm_head is not None:  # tied: the head weight is the embedding table
            src.setdefault(_PG + ".language_model.embed_tokens.weight", lm_head)
        out: Dict[str, torch.Tensor] = {}
        used = set()
        for there, here in PI05_NAME_MAP:
            for i in layer_range(here):
                for wb in (("weight", "bias") if "{wb}" in there else (None,)):
                    k = _expand(there, i, wb)
                    if k in src:
                        out[_expand(here, i, wb)] = src[k]
                        used.add(k)
        for prefix, parts, here, wbs in _FUSED:
            for i in layer_range(here):
                for wb in wbs:
                    ks = [f"{_expand(prefix, i, None)}.{p}.{wb}" for p in parts]
                    if all(k in src for k in ks):
                        out[f"{_expand(here, i, None)}.{wb}"] = torch.cat([src[k] for k in ks], dim=0)
                        used.update(ks)
        left = sorted(set(src) - used)
        if left:
            raise KeyError(f"{len(left)} checkpoint tensors have no place in the model, e.g. {left[:4]}")
        return out
    out = {}
    sizes_qkv = {"vision": [cfg.vit_width] * 3,
                 "lang": [vd.num_heads * vd.head_dim, vd.num_kv_heads * vd.head_dim, vd.num_kv_heads * vd.head_dim]}
    used = set()
    for there, here in PI05_NAME_MAP:
        for i in layer_range(here):
            for wb in (("weight", "bias") if "{wb}" in there else (None,)):
                k = _expand(here, i, wb)
                if k in sd:
                    out[_expand(there, i, wb)] = sd[k]
                    used.add(k)
    for prefix, parts, here, wbs in _FUSED:
        for i in layer_range(here):
            for wb in wbs:
                k = f"{_expand(here, i, None)}.{wb}"
                if k not in sd:
                    continue
                t = sd[k]
                if len(parts) == 3:
                    pieces = t.split(sizes_qkv["vision" if here.startswith("vision") else "lang"], dim=0)
                else:
                    pieces = t.chunk(2, dim=0)
                for p, piece in zip(parts, pieces):
                    out[f"{_expand(prefix, i, None)}.{p}.{wb}"] = piece
                used.add(k)
    left = sorted(set(sd) - used)
    if left:
        raise KeyError(f"{len(left)} model tensors have no public name, e.g. {left[:4]}")
    return out


def load_pi05_checkpoint(model: Pi05Policy, path: str, strict: bool = True) -> None:
    """``model.safetensors`` (file or directory) of a public Pi0.5 checkpoint into `model`."""
    import os

    from safetensors.torch import load_file
    f = os.path.join(path, "model.safetensors") if os.path.isdir(path) else path
    missing, unexpected = model.load_state_dict(convert_pi05_state_dict(load_file(f), model.c), strict=False)
    if strict and (missing or unexpected):
        raise KeyError(f"missing {missing[:4]} unexpected {unexpected[:4]}")
