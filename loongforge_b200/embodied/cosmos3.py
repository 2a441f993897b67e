"""Cosmos3: a Qwen3-VL-style decoder turned into a mixture of transformers with an UNDERSTANDING pathway (text tokens,
causal) and a GENERATION pathway (video-latent and action tokens, flow matching), over PACKED sequences.

* Packing: the samples of a micro-batch, each ``[text | video latent patches | action tokens]`` of its own length, are laid
  end to end in one token row; attention never crosses samples. Text attends text causally; generation tokens attend the
  sample's text and generation tokens (all of them, or — ``video_temporal_causal`` — only frames up to their own, an action
  belonging to the frame it leads to).
* Every layer has two sets of weights (norms, q / k / v / o with per-head q / k RMS norm, SwiGLU MLP); a token is processed
  by the set of its pathway, ONE attention runs over the whole packed row (grouped-query heads).
* Unified 3-D M-RoPE: text positions advance all three axes together; a video's patches keep (row, column) from 0 and a
  frame axis that continues after the text; action tokens sit on the frame axis between the frames they connect, so the
  two modalities are aligned in time; the rotary frequencies are dealt to the axes in the interleaved t, h, w pattern.
* Latent patches enter through ``vae2llm`` (+ a modality embedding), actions through a DOMAIN-aware linear (one weight set
  per robot / data domain); the timestep embedding is added to the NOISY tokens only — conditioning frames (the observed
  first frame) stay clean, carry no timestep and no loss. ``llm2vae`` / a domain-aware ``llm2action`` read velocities.
* Optional next-token loss on the text (``predict_text_tokens``).

(reference: loongforge/embodied/model/cosmos3/unified_mot.py:170-475, cosmos3_vfm_network.py:132-252,325-500,566-830,930-1144,
unified_3dmrope_utils.py:45-198, modeling_cosmos3.py:284-467, sequence_packing.py)
"""
from __future__ import annotations

import dataclasses
import math
from typing import Dict, List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..models.diffusion import RMSNorm, _Linear, timestep_embedding
from .wan_blocks import CausalVideoVAE, SegmentMask, contiguous_runs, masked_attention, video_from_batch
from .xvla import DomainAwareLinear


@dataclasses.dataclass
class Cosmos3Config:
    hidden_size: int = 2048
    ffn_hidden_size: int = 6144
    num_layers: int = 28
    num_heads: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    vocab_size: int = 151936
    rms_eps: float = 1e-6
    rope_theta: float = 5_000_000.0
    mrope_section: Tuple[int, int, int] = (24, 20, 20)
    qk_norm_text: bool = True
    qk_norm_diffusion: bool = True
    latent_channels: int = 48
    latent_patch: int = 2
    action_dim: int = 7
    max_action_dim: int = 32
    num_domains: int = 32
    action_horizon: int = 16
    timestep_scale: float = 0.001
    freq_dim: int = 256
    shift: float = 3.0
    video_temporal_causal: bool = False
    condition_frames: Tuple[int, ...] = (0,)
    predict_text_tokens: bool = False
    action_loss_weight: float = 1.0
    vision_loss_weight: float = 1.0
    num_train_timesteps: int = 1000
    video_frames: int = 9
    image_size: int = 224
    vae_base: int = 32
    vae_spatial_stages: int = 3
    recompute: bool = False
    segment_attention: bool = True       # evaluate the packed mask run by run (no [L, L] mask)

    @classmethod
    def tiny(cls, **kw) -> "Cosmos3Config":
        base = dict(hidden_size=48, ffn_hidden_size=96, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=12,
                    vocab_size=32000, mrope_section=(2, 2, 2), latent_channels=8, max_action_dim=8, num_domains=3,
                    action_horizon=4, freq_dim=32, video_frames=5, image_size=32, vae_base=8)
        base.update(kw)
        return cls(**base)


UND, GEN = 0, 1


@dataclasses.dataclass
class PackedSequence:
    """One packed row. All index tensors address the row's ``L`` tokens."""
    text_ids: torch.Tensor            # [n_text] token ids, in row order
    text_index: torch.Tensor          # [n_text] row positions of text tokens
    vision_index: torch.Tensor        # [n_vision] row positions of latent patches (sample-major, raster order)
    action_index: torch.Tensor        # [n_action]
    sample: torch.Tensor              # [L] sample id of every token
    frame: torch.Tensor               # [L] latent frame a generation token belongs to (text: -1)
    position: torch.Tensor            # [L, 3] M-RoPE positions (float: action tokens sit between frames)
    grids: List[Tuple[int, int, int]]  # per sample (frames, rows, columns) of latent patches
    n_action: List[int]               # per sample number of action tokens
    length: int

    @property
    def pathway(self) -> torch.Tensor:
        p = torch.full((self.length,), GEN, dtype=torch.long, device=self.sample.device)
        p[self.text_index] = UND
        return p


def pack_samples(text_tokens: List[torch.Tensor], grids: List[Tuple[int, int, int]], n_action: List[int], device=None) -> PackedSequence:
    """Lays samples end to end and derives indices, frames and positions. Actions are spread over the frames after the
    first: action i of n leads to latent frame ``1 + floor(i * (F - 1) / n)`` and sits at time
    ``first frame + 1 + i * (F - 1) / n - 0.5`` on the frame axis (between the frame before and the frame it leads to)."""
    ids, t_idx, v_idx, a_idx, sample, frame, pos = [], [], [], [], [], [], []
    at = 0
    for s, (tok, (f, h, w), na) in enumerate(zip(text_tokens, grids, n_action)):
        lt, lv = tok.numel(), f * h * w
        ids.append(tok)
        t_idx.append(torch.arange(at, at + lt))
        tp = torch.arange(lt, dtype=torch.float32)
        pos.append(torch.stack([tp, tp, tp], dim=-1))
        frame.append(torch.full((lt,), -1))
        g = torch.stack(torch.meshgrid(torch.arange(f), torch.arange(h), torch.arange(w), indexing="ij"), dim=-1).reshape(-1, 3).float()
        frame.append(g[:, 0].long())
        g[:, 0] += lt                                          # the frame axis continues after the text
        pos.append(g)
        v_idx.append(torch.arange(at + lt, at + lt + lv))
        span = max(f - 1, 1)
        i = torch.arange(na, dtype=torch.float32)
        frame.append((1 + (i * span / max(na, 1)).floor().long()).clamp(max=max(f - 1, 0)))
        ta = lt + 1 + i * span / max(na, 1) - 0.5
        pos.append(torch.stack([ta, torch.zeros(na), torch.zeros(na)], dim=-1))
        a_idx.append(torch.arange(at + lt + lv, at + lt + lv + na))
        n = lt + lv + na
        sample.append(torch.full((n,), s))
        at += n
    cat = lambda xs: torch.cat(xs).to(device)  # noqa: E731
    return PackedSequence(cat(ids), cat(t_idx), cat(v_idx), cat(a_idx), cat(sample), cat(frame), cat(pos), list(grids),
                          list(n_action), at)


def packed_attention_mask(seq: PackedSequence, temporal_causal: bool) -> torch.Tensor:
    """``[L, L]``: same sample; text -> earlier text; generation -> the sample's text and generation tokens (frames <= own
    when ``temporal_causal``)."""
    L = seq.length
    idx = torch.arange(L, device=seq.sample.device)
    same = seq.sample[:, None] == seq.sample[None, :]
    path = seq.pathway
    q_und, k_und = (path == UND)[:, None], (path == UND)[None, :]
    m = same & q_und & k_und & (idx[None, :] <= idx[:, None])
    gen = same & ~q_und
    if temporal_causal:
        gen = gen & (k_und | (seq.frame[None, :] <= seq.frame[:, None]))
    return m | gen


def packed_segment_mask(seq: PackedSequence, temporal_causal: bool) -> SegmentMask:
    """``packed_attention_mask`` in run form: runs of equal (sample, pathway, frame); a text run attends itself causally,
    everything else is constant on runs, so attention is evaluated run by run without the ``[L, L]`` mask."""
    path = seq.pathway
    starts, ends, rep = contiguous_runs(seq.sample, path, seq.frame)
    sample, und, frame = seq.sample[rep], path[rep] == UND, seq.frame[rep]
    same = sample[:, None] == sample[None, :]
    m = same & und[:, None] & und[None, :] & (rep[None, :] <= rep[:, None])
    gen = same & ~und[:, None]
    if temporal_causal:
        gen = gen & (und[None, :] | (frame[None, :] <= frame[:, None]))
    return SegmentMask(starts, ends, m | gen, causal=und.tolist())


def mrope_angles(pos: torch.Tensor, head_dim: int, theta: float, section: Tuple[int, int, int]) -> torch.Tensor:
    """pos ``[L, 3]`` -> ``[L, head_dim/2]``: frequency i follows the row axis when ``i % 3 == 1`` and ``i < 3 * section[1]``,
    the column axis when ``i % 3 == 2`` and ``i < 3 * section[2]``, the time axis otherwise (interleaved M-RoPE)."""
    half = head_dim // 2
    inv = theta ** (-torch.arange(half, device=pos.device, dtype=torch.float32) / half)
    i = torch.arange(half, device=pos.device)
    axis = torch.zeros(half, dtype=torch.long, device=pos.device)
    axis[(i % 3 == 1) & (i < 3 * section[1])] = 1
    axis[(i % 3 == 2) & (i < 3 * section[2])] = 2
    return pos.float()[:, axis] * inv


def _rope_half(x: torch.Tensor, angles: torch.Tensor) -> torch.Tensor:
    """x ``[L, H, d]``, angles ``[L, d/2]``; pairs are (i, i + d/2)."""
    cos, sin = angles.cos()[:, None, :], angles.sin()[:, None, :]
    a, b = x.float().chunk(2, dim=-1)
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1).to(x.dtype)


class _Pathway(nn.Module):
    """One pathway's weights of a layer."""

    def __init__(self, c: Cosmos3Config, qk_norm: bool):
        super().__init__()
        C, H, Hk, d = c.hidden_size, c.num_heads, c.num_kv_heads, c.head_dim
        self.input_layernorm, self.post_attention_layernorm = RMSNorm(C, c.rms_eps), RMSNorm(C, c.rms_eps)
        self.q_proj, self.k_proj, self.v_proj = _Linear(C, H * d, bias=False), _Linear(C, Hk * d, bias=False), _Linear(C, Hk * d, bias=False)
        self.o_proj = _Linear(H * d, C, bias=False)
        self.q_norm = RMSNorm(d, c.rms_eps) if qk_norm else nn.Identity()
        self.k_norm = RMSNorm(d, c.rms_eps) if qk_norm else nn.Identity()
        self.gate_proj, self.up_proj = _Linear(C, c.ffn_hidden_size, bias=False), _Linear(C, c.ffn_hidden_size, bias=False)
        self.down_proj = _Linear(c.ffn_hidden_size, C, bias=False)

    def qkv(self, x, angles, c: Cosmos3Config):
        h = self.input_layernorm(x)
        q = self.q_norm(self.q_proj(h).view(-1, c.num_heads, c.head_dim))
        k = self.k_norm(self.k_proj(h).view(-1, c.num_kv_heads, c.head_dim))
        return _rope_half(q, angles), _rope_half(k, angles), self.v_proj(h).view(-1, c.num_kv_heads, c.head_dim)

    def finish(self, x, attn):
        x = x + self.o_proj(attn)
        h = self.post_attention_layernorm(x)
        return x + self.down_proj(F.silu(self.gate_proj(h)) * self.up_proj(h))


class MoTDecoderLayer(nn.Module):
    def __init__(self, c: Cosmos3Config):
        super().__init__()
        self.c = c
        self.und, self.gen = _Pathway(c, c.qk_norm_text), _Pathway(c, c.qk_norm_diffusion)

    def forward(self, x, und_idx, gen_idx, angles, mask):
        """x ``[L, C]``; tokens at ``und_idx`` / ``gen_idx`` go through their pathway, one attention over the row."""
        c, L = self.c, x.shape[0]
        xu, xg = x[und_idx], x[gen_idx]
        qu, ku, vu = self.und.qkv(xu, angles[und_idx], c)
        qg, kg, vg = self.gen.qkv(xg, angles[gen_idx], c)
        q = x.new_empty(L, c.num_heads, c.head_dim)
        k, v = x.new_empty(L, c.num_kv_heads, c.head_dim), x.new_empty(L, c.num_kv_heads, c.head_dim)
        q = q.index_copy(0, und_idx, qu.to(q.dtype)).index_copy(0, gen_idx, qg.to(q.dtype))
        k = k.index_copy(0, und_idx, ku.to(k.dtype)).index_copy(0, gen_idx, kg.to(k.dtype))
        v = v.index_copy(0, und_idx, vu.to(v.dtype)).index_copy(0, gen_idx, vg.to(v.dtype))
        o = masked_attention(q[None], k[None], v[None], mask)[0]
        out = torch.empty_like(x)
        out = out.index_copy(0, und_idx, self.und.finish(xu, o[und_idx]))
        return out.index_copy(0, gen_idx, self.gen.finish(xg, o[gen_idx]))


class Cosmos3Network(nn.Module):
    def __init__(self, c: Cosmos3Config):
        super().__init__()
        self.c = c
        C, p = c.hidden_size, c.latent_patch
        self.embed_tokens = nn.Embedding(c.vocab_size, C)
        self.layers = nn.ModuleList([MoTDecoderLayer(c) for _ in range(c.num_layers)])
        self.norm, self.norm_moe_gen = RMSNorm(C, c.rms_eps), RMSNorm(C, c.rms_eps)
        self.vae2llm, self.llm2vae = _Linear(c.latent_channels * p * p, C), _Linear(C, c.latent_channels * p * p)
        self.vision_modality_embed = nn.Parameter(torch.zeros(C))
        self.action2llm = DomainAwareLinear(c.max_action_dim, C, c.num_domains)
        self.llm2action = DomainAwareLinear(C, c.max_action_dim, c.num_domains)
        self.action_modality_embed = nn.Parameter(torch.zeros(C))
        self.time_embedder = nn.Sequential(_Linear(c.freq_dim, C), nn.SiLU(), _Linear(C, C))
        if c.predict_text_tokens:
            self.lm_head = _Linear(C, c.vocab_size, bias=False)

    def patchify(self, lat):
        """``[C, F, H, W]`` -> ``[F*h*w, C*p*p]``."""
        Cc, Fr, H, W = lat.shape
        p = self.c.latent_patch
        return lat.view(Cc, Fr, H // p, p, W // p, p).permute(1, 2, 4, 0, 3, 5).reshape(Fr * (H // p) * (W // p), Cc * p * p)

    def unpatchify(self, tok, grid):
        f, h, w = grid
        p, Cc = self.c.latent_patch, self.c.latent_channels
        return tok.view(f, h, w, Cc, p, p).permute(3, 0, 1, 4, 2, 5).reshape(Cc, f, h * p, w * p)

    def time_embed(self, t):
        f = timestep_embedding(t.float() * self.c.timestep_scale * self.c.num_train_timesteps, self.c.freq_dim)
        return self.time_embedder(f.to(self.time_embedder[0].weight.dtype))

    def forward(self, seq: PackedSequence, latents: List[torch.Tensor], actions: List[torch.Tensor], timesteps: torch.Tensor,
                domain_id: torch.Tensor, noisy_vision: torch.Tensor, noisy_action: torch.Tensor):
        """latents: per sample ``[C, F, H, W]`` (already noised), actions: per sample ``[n, max_action_dim]``; timesteps ``[B]``
        in [0, 1]; ``noisy_vision`` / ``noisy_action``: boolean per vision / action token (False = conditioning, clean).
        Returns per-sample velocity predictions for the latents and the actions, and the final hidden states."""
        c = self.c
        t_emb = self.embed_tokens(seq.text_ids)   # (through the module's forward: its weight may be a shard outside it)
        x = t_emb.new_zeros(seq.length, c.hidden_size).index_copy(0, seq.text_index, t_emb)
        temb = self.time_embed(timesteps)                                             # [B, C]
        v_tok = self.vae2llm(torch.cat([self.patchify(l) for l in latents]).to(x.dtype)) + self.vision_modality_embed
        v_tok = v_tok + temb[seq.sample[seq.vision_index]] * noisy_vision[:, None].to(x.dtype)
        x = x.index_copy(0, seq.vision_index, v_tok)
        if seq.action_index.numel():
            a_sample = seq.sample[seq.action_index]
            a_tok = torch.cat([self.action2llm(a[None].to(x.dtype), domain_id[i:i + 1])[0] for i, a in enumerate(actions)])
            a_tok = a_tok + self.action_modality_embed + temb[a_sample] * noisy_action[:, None].to(x.dtype)
            x = x.index_copy(0, seq.action_index, a_tok)
        gen_idx = torch.cat([seq.vision_index, seq.action_index]).sort().values
        und_idx = seq.text_index
        angles = mrope_angles(seq.position, c.head_dim, c.rope_theta, c.mrope_section)
        mask = (packed_segment_mask if c.segment_attention else packed_attention_mask)(seq, c.video_temporal_causal)
        for layer in self.layers:
            if c.recompute and torch.is_grad_enabled():
                x = torch.utils.checkpoint.checkpoint(layer, x, und_idx, gen_idx, angles, mask, use_reentrant=False)
            else:
                x = layer(x, und_idx, gen_idx, angles, mask)
        h = torch.empty_like(x)
        h = h.index_copy(0, und_idx, self.norm(x[und_idx])).index_copy(0, gen_idx, self.norm_moe_gen(x[gen_idx]))
        v_out = self.llm2vae(h[seq.vision_index])
        preds_v, at = [], 0
        for g in seq.grids:
            n = g[0] * g[1] * g[2]
            preds_v.append(self.unpatchify(v_out[at:at + n], g))
            at += n
        preds_a, at = [], 0
        for i, n in enumerate(seq.n_action):
            preds_a.append(self.llm2action(h[seq.action_index[at:at + n]][None], domain_id[i:i + 1])[0])
            at += n
        return preds_v, preds_a, h


class Cosmos3Policy(nn.Module):

    def default_lora_targets(self):
        """Every projection of both pathways of the decoder layers."""
        return ["*net.layers.*_proj"]

    def __init__(self, c: Cosmos3Config):
        super().__init__()
        self.c = c
        self.vae = CausalVideoVAE(c.latent_channels, c.vae_base, c.vae_spatial_stages).requires_grad_(False)
        self.net = Cosmos3Network(c)

    def train(self, mode: bool = True):
        super().train(mode)
        self.vae.eval()
        return self

    def _sigma(self, u):
        return self.c.shift * u / (1 + (self.c.shift - 1) * u)

    def _prepare(self, batch, with_actions: bool = True):
        c = self.c
        tok = batch["tokens"] if "tokens" in batch else batch["text"]
        tmask = batch.get("token_mask", tok != 0)
        texts = []
        for t, m in zip(tok, tmask):
            t = t[m]
            texts.append(t if t.numel() else tok.new_zeros(1))           # an empty instruction keeps one token
        B = tok.shape[0]
        domain = batch.get("domain_id", batch.get("embodiment_id"))
        domain = torch.zeros(B, dtype=torch.long, device=tok.device) if domain is None else domain.long()
        return texts, domain

    def _latents(self, batch, frames):
        if "latents" in batch:
            return batch["latents"]
        with torch.no_grad():
            return self.vae.encode(video_from_batch(batch, frames))

    def forward(self, batch: Dict[str, torch.Tensor], noise=None, t=None):
        c, net = self.c, self.net
        lat = self._latents(batch, c.video_frames)                                     # [B, C, F, H, W]
        B, _, Fr, H, W = lat.shape
        dev = lat.device
        texts, domain = self._prepare(batch)
        act = batch["actions"]
        A = act.shape[-1]
        act = F.pad(act, (0, c.max_action_dim - A))
        amask = batch.get("action_mask")
        amask = torch.ones(act.shape[:2], device=dev) if amask is None else amask.float()
        chan = (torch.arange(c.max_action_dim, device=dev) < A).float()
        sig = self._sigma(torch.rand(B, device=dev)) if t is None else t
        p = c.latent_patch
        grid = (Fr, H // p, W // p)
        cond = torch.zeros(Fr, dtype=torch.bool, device=dev)
        cond[[f for f in c.condition_frames if f < Fr]] = True
        sv = sig.view(B, 1, 1, 1, 1) * (~cond).float().view(1, 1, Fr, 1, 1)            # conditioning frames stay clean
        noise_v = torch.randn_like(lat)
        noisy_v = (sv * noise_v + (1 - sv) * lat)
        noise_a = torch.randn_like(act) if noise is None else F.pad(noise, (0, c.max_action_dim - A))
        sa = sig.view(B, 1, 1)
        noisy_a = (sa * noise_a + (1 - sa) * act) * chan                               # padded channels enter as zeros
        seq = pack_samples(texts, [grid] * B, [act.shape[1]] * B, dev)
        noisy_tok_v = (~cond).repeat_interleave(grid[1] * grid[2]).repeat(B)
        noisy_tok_a = torch.ones(seq.action_index.numel(), dtype=torch.bool, device=dev)
        preds_v, preds_a, h = net(seq, list(noisy_v), list(noisy_a), sig, domain, noisy_tok_v, noisy_tok_a)
        pv, pa = torch.stack(preds_v), torch.stack(preds_a)
        err_v = (pv.float() - (noise_v - lat).float()).pow(2).mean(dim=(1, 3, 4))      # [B, F]
        keep = (~cond).float()[None]
        loss_v = (err_v * keep).sum() / (keep.sum() * B).clamp(min=1)
        w = amask[..., None] * chan
        loss_a = ((pa.float() - (noise_a - act).float()).pow(2) * w).sum() / w.sum().clamp(min=1)
        loss = c.vision_loss_weight * loss_v + c.action_loss_weight * loss_a
        self.last_losses = {"vision loss": loss_v.detach(), "action loss": loss_a.detach()}
        if c.predict_text_tokens:
            logits = net.lm_head(h[seq.text_index])
            nxt_same = seq.sample[seq.text_index][1:] == seq.sample[seq.text_index][:-1]
            ce = F.cross_entropy(logits[:-1][nxt_same].float(), seq.text_ids[1:][nxt_same]) if nxt_same.any() else logits.sum() * 0
            self.last_losses["text loss"] = ce.detach()
            loss = loss + ce
        return loss

    @torch.no_grad()
    def predict_action(self, obs: Dict[str, torch.Tensor], steps: Optional[int] = None, generator=None) -> torch.Tensor:
        """Joint Euler integration of the video latents (first frame = observation, kept clean) and the action chunk."""
        c, net = self.c, self.net
        steps = steps or 10
        first = obs["latents"][:, :, :1] if "latents" in obs else self.vae.encode(video_from_batch(obs, 1)[:, :, :1])
        B, dev = first.shape[0], first.device
        Fr = self.vae.latent_frames(c.video_frames)
        texts, domain = self._prepare(obs)
        p = c.latent_patch
        grid = (Fr, first.shape[3] // p, first.shape[4] // p)
        lat = torch.randn(B, first.shape[1], Fr, *first.shape[3:], device=dev, generator=generator)
        lat[:, :, :1] = first
        a = torch.randn(B, c.action_horizon, c.max_action_dim, device=dev, generator=generator)
        chan = (torch.arange(c.max_action_dim, device=dev) < c.action_dim).float()
        seq = pack_samples(texts, [grid] * B, [c.action_horizon] * B, dev)
        cond = torch.zeros(Fr, dtype=torch.bool, device=dev)
        cond[0] = True
        noisy_tok_v = (~cond).repeat_interleave(grid[1] * grid[2]).repeat(B)
        noisy_tok_a = torch.ones(seq.action_index.numel(), dtype=torch.bool, device=dev)
        sig = self._sigma(torch.linspace(1.0, 0.0, steps + 1, device=dev))
        for i in range(steps):
            pv, pa, _ = net(seq, list(lat), list(a * chan), sig[i].expand(B), domain, noisy_tok_v, noisy_tok_a)
            lat = lat + torch.stack(pv) * (sig[i + 1] - sig[i])
            lat[:, :, :1] = first
            a = a + torch.stack(pa) * (sig[i + 1] - sig[i])
        self.last_rollout_latents = lat
        return a[..., :c.action_dim]
