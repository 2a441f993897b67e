"""GPT-style language model: vocab-parallel embedding, rotary tables (RoPE / YaRN / M-RoPE),
the decoder layers of this pipeline stage, final norm, and the output layer fused with the
cross-entropy loss.

Counterpart of the reference's BaseGPTModel (loongforge/models/foundation/base/base_gpt_model.py:
51-1018): `_preprocess` (:309-453), decoder, `_postprocess` with the fused output layer + CE
(:709-720, :864-898). State-dict keys follow Megatron: ``embedding.word_embeddings.weight``,
``decoder.layers.N...``, ``decoder.final_layernorm.weight``, ``output_layer.weight``.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence

import torch
import torch.nn as nn

from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import mappings as M
from ..parallel import state as ps
from .config import TransformerConfig
from .transformer import PackedSeqParams, RotaryInputs, TransformerBlock


def yarn_inv_freq(cfg: TransformerConfig, rot_dim: int, device) -> tuple[torch.Tensor, float]:
    """YaRN frequency blend and attention mscale (DeepSeek-V2/V3 convention)."""
    base, factor = cfg.rotary_base, cfg.yarn_scaling_factor
    pos_freqs = base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim)
    extra, inter = 1.0 / pos_freqs, 1.0 / (factor * pos_freqs)

    def corr_dim(n_rot):
        return (rot_dim * math.log(cfg.yarn_original_max_position / (n_rot * 2 * math.pi))) / (2 * math.log(base))

    low = max(math.floor(corr_dim(cfg.yarn_beta_fast)), 0)
    high = min(math.ceil(corr_dim(cfg.yarn_beta_slow)), rot_dim - 1)
    if low == high:
        high += 0.001
    ramp = ((torch.arange(rot_dim // 2, dtype=torch.float32, device=device) - low) / (high - low)).clamp(0, 1)
    mask = 1.0 - ramp
    inv = inter * (1 - mask) + extra * mask

    def get_mscale(scale, m):
        return 1.0 if scale <= 1 else 0.1 * m * math.log(scale) + 1.0

    mscale = get_mscale(factor, cfg.yarn_mscale) / get_mscale(factor, cfg.yarn_mscale_all_dim)
    return inv, float(mscale)


class RotaryEmbedding:
    """Angle tables for RoPE, YaRN and M-RoPE (loongforge/models/foundation/base/base_gpt_model.py:184-227,
    loongforge/models/foundation/qwen2/qwen_model.py:127-165)."""

    def __init__(self, cfg: TransformerConfig, rot_dim: int):
        self.cfg, self.rot_dim = cfg, rot_dim
        self._cache = {}

    def _inv_freq(self, device, n_pos: Optional[int] = None):
        cfg = self.cfg
        if cfg.position_embedding_type == "yarn":
            return yarn_inv_freq(cfg, self.rot_dim, device)
        base = cfg.rotary_base
        if cfg.rotary_dynamic_ntk and n_pos is not None and n_pos > cfg.max_position_embeddings:
            # dynamic NTK: the base grows with the sequence length beyond the trained context (Qwen2 / InternLM,
            # loongforge/models/foundation/qwen2/qwen_model.py:56-126)
            f, d = cfg.rotary_dynamic_ntk_factor, self.rot_dim
            base = base * ((f * n_pos / cfg.max_position_embeddings) - (f - 1)) ** (d / (d - 2))
        inv = 1.0 / (base ** (torch.arange(0, self.rot_dim, 2, dtype=torch.float32, device=device) / self.rot_dim))
        return inv / cfg.rotary_scaling_factor if cfg.rotary_scaling_factor != 1.0 else inv, 1.0

    def table(self, n_pos: int, device) -> RotaryInputs:
        key = (n_pos, str(device))
        if key not in self._cache:
            inv, mscale = self._inv_freq(device, n_pos)
            t = torch.arange(n_pos, dtype=torch.float32, device=device)
            self._cache = {key: (torch.outer(t, inv).contiguous(), mscale)}
        f, m = self._cache[key]
        return RotaryInputs(freqs=f, mscale=m)

    def mrope(self, position_ids: torch.Tensor) -> RotaryInputs:
        """position_ids [3, T] (t/h/w streams). Frequencies take sections ``mrope_section`` of the
        half-dim from the three streams in turn (A.4: [16,24,24] for head_dim 128), half-rotation."""
        cfg = self.cfg
        inv, mscale = self._inv_freq(position_ids.device)
        ang = position_ids.float()[:, :, None] * inv[None, None, :]  # [3, T, rot/2]
        sec = cfg.mrope_section or [self.rot_dim // 2]
        if cfg.mrope_interleaved:
            idx = torch.arange(self.rot_dim // 2, device=ang.device) % 3
            limit = torch.tensor([sec[0] * 3, sec[1] * 3, sec[2] * 3], device=ang.device)
            pos = torch.arange(self.rot_dim // 2, device=ang.device)
            stream = torch.where(pos < limit[idx], idx, torch.zeros_like(idx))
            mixed = ang.gather(0, stream[None, None, :].expand(1, ang.shape[1], -1))[0]
        else:
            parts, start = [], 0
            for i, n in enumerate(sec):
                parts.append(ang[i % 3, :, start:start + n])
                start += n
            mixed = torch.cat(parts, dim=-1)
        return RotaryInputs(freqs=mixed.contiguous(), mscale=mscale)


def pipeline_layer_split(num_layers: int, pp: int, custom: Optional[Sequence[int]] = None) -> List[List[int]]:
    """Layer indices per pipeline stage; `custom` = explicit counts per stage
    (--custom-pipeline-layers, loongforge/train/arguments.py:1334)."""
    if custom:
        assert len(custom) == pp and sum(custom) == num_layers
        counts = list(custom)
    else:
        assert num_layers % pp == 0, "num_layers must divide by pipeline size (or give custom layers)"
        counts = [num_layers // pp] * pp
    out, s = [], 0
    for c in counts:
        out.append(list(range(s, s + c)))
        s += c
    return out


class GPTModel(nn.Module):
    def __init__(self, cfg: TransformerConfig, *, pre_process: bool = True, post_process: bool = True,
                 layer_numbers: Optional[Sequence[int]] = None, device=None, parallel_state: Optional[str] = None):
        super().__init__()
        self.cfg = cfg
        self.pre_process, self.post_process = pre_process, post_process
        self.state_name = parallel_state
        st = ps.get_state(parallel_state)
        cfg.pad_vocab(st.dims.tp)
        if layer_numbers is None:
            layer_numbers = list(range(cfg.num_layers))
        # With pipeline parallelism the last stage needs the word embedding too when it is tied to the output layer or
        # feeds the multi-token-prediction layers. Both stages then hold a copy ("shared_embedding"); their gradients are
        # summed over the embedding group after every backward, so the copies stay identical (reference: Megatron
        # LanguageModule.setup_embeddings_and_output_layer, used through base_gpt_model.py:709-720).
        needs_copy = post_process and (not cfg.untie_embeddings_and_output_weights or cfg.mtp_num_layers > 0)
        shared = st.dims.pp > 1 and (not cfg.untie_embeddings_and_output_weights or cfg.mtp_num_layers > 0)
        if pre_process or (shared and needs_copy):
            self.embedding = nn.Module()
            self.embedding.word_embeddings = PL.VocabParallelEmbedding(
                cfg.padded_vocab_size, cfg.hidden_size, init_std=cfg.init_method_std,
                sequence_parallel=cfg.sequence_parallel, params_dtype=cfg.params_dtype, device=device,
                parallel_state=parallel_state)
            if shared:
                self.embedding.word_embeddings.weight.shared_embedding = True
                if not pre_process:
                    self.embedding.word_embeddings.weight.shared_embedding_replica = True
        self.decoder = TransformerBlock(cfg, layer_numbers, post_process=post_process, device=device,
                                        parallel_state=parallel_state)
        if post_process:
            if cfg.untie_embeddings_and_output_weights:
                self.output_layer = PL.ColumnParallelLinear(
                    cfg.hidden_size, cfg.padded_vocab_size, bias=False, init_std=cfg.output_layer_init_std,
                    key="output_layer", params_dtype=cfg.params_dtype, device=device, parallel_state=parallel_state)
            else:
                self.output_layer = None
            if cfg.mtp_num_layers > 0:
                from .mtp import MultiTokenPredictionBlock
                self.mtp = MultiTokenPredictionBlock(cfg, device=device, parallel_state=parallel_state)
            else:
                self.mtp = None
            # weights that collect gradients from several places of one backward pass (output layer + embedding lookup
            # when tied, one more loss head per MTP depth) must not start their data-parallel reduction at the first
            multi = [self.embedding.word_embeddings.weight] if hasattr(self, "embedding") else []
            if self.output_layer is not None and cfg.mtp_num_layers > 0:
                multi.append(self.output_layer.weight)
            if not cfg.untie_embeddings_and_output_weights or cfg.mtp_num_layers > 0:
                for w in multi:
                    w.defer_grad_sync = True
        rot_dim = cfg.qk_pos_emb_head_dim if (cfg.multi_latent_attention or cfg.csa_compress_ratios is not None) else int(cfg.kv_channels * cfg.rotary_percent)
        self.rotary = RotaryEmbedding(cfg, rot_dim) if cfg.position_embedding_type in ("rope", "yarn", "mrope") else None
        self.input_tensor = None  # set by the pipeline schedule on non-first stages

    # ------------------------------------------------------------------ pipeline plumbing
    def set_input_tensor(self, t):
        self.input_tensor = t

    def shared_embedding_weight(self):
        if self.cfg.untie_embeddings_and_output_weights:
            return self.output_layer.weight
        return self.embedding.word_embeddings.weight

    # ------------------------------------------------------------------ forward
    def build_rotary(self, position_ids: torch.Tensor, n_tokens: int, device) -> Optional[RotaryInputs]:
        if self.rotary is None:
            return None
        if self.cfg.rope_3d_freq_allocation and position_ids.dim() == 2:
            from .ernie import ernie_3d_angles
            return ernie_3d_angles(position_ids, self.rotary.rot_dim, self.cfg.rotary_base,
                                   self.cfg.rope_3d_freq_allocation)
        if self.cfg.position_embedding_type == "mrope" or position_ids.dim() == 2 and position_ids.shape[0] == 3:
            return self.rotary.mrope(position_ids)
        # position ids index the table: under context parallelism a rank holds n_tokens of a row that is cp times as
        # long, so its ids run up to cp * n_tokens - 1 (an index past the table would be read as garbage on a GPU)
        cp = max(ps.get_state(self.state_name).dims.cp, 1) if ps.model_parallel_is_initialized() else 1
        n_pos = max(self.cfg.max_position_embeddings, n_tokens * cp)
        r = self.rotary.table(n_pos, device)
        return RotaryInputs(freqs=r.freqs, pos_ids=position_ids.to(torch.int32), mscale=r.mscale)

    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        x = self.embedding.word_embeddings(tokens)
        if self.cfg.params_dtype != x.dtype:
            x = x.to(self.cfg.params_dtype)
        return x

    def forward(self, tokens: Optional[torch.Tensor], position_ids: torch.Tensor, *,
                labels: Optional[torch.Tensor] = None, loss_mask: Optional[torch.Tensor] = None,
                packed: Optional[PackedSeqParams] = None, decoder_input: Optional[torch.Tensor] = None,
                loss_scale: Optional[float] = None, token_type: Optional[torch.Tensor] = None,
                full_batch: Optional[dict] = None):
        """tokens / labels / loss_mask are flat ``[T]``; position_ids ``[T]`` or ``[3, T]`` (M-RoPE).

        Returns per-token losses ``[T]`` when `labels` is given on the last stage, logits
        ``[T, V/tp]`` when not, and the hidden state ``[T(/tp), h]`` on other stages.
        `loss_scale` is the scalar the masked loss sum will be multiplied with (lets the fused
        linear+CE write weight gradients straight into ``main_grad``)."""
        cfg = self.cfg
        if self.pre_process:
            x = decoder_input if decoder_input is not None else self.embed(tokens)
        else:
            x = self.input_tensor
        n_tok = position_ids.shape[-1]
        rotary = self.build_rotary(position_ids, n_tok, x.device)
        if cfg.moe_multi_type:
            for layer in self.decoder.layers:
                if hasattr(layer.mlp, "set_token_type"):
                    layer.mlp.set_token_type(token_type)
        if cfg.moe_n_hash_layers:
            from .moe import set_current_token_ids
            set_current_token_ids(tokens)
        x = self.decoder(x, rotary, packed)
        if not self.post_process:
            return x
        return self.postprocess(x, labels, loss_mask, loss_scale, tokens=tokens, position_ids=position_ids,
                                rotary=rotary, packed=packed, full_batch=full_batch)

    def postprocess(self, hidden, labels, loss_mask, loss_scale, **mtp_kw):
        cfg = self.cfg
        st = ps.get_state(self.state_name)
        g = st.group("tp")
        hidden_local = hidden  # what the MTP layers continue from: the sequence shard under sequence parallelism
        if cfg.sequence_parallel and st.dims.tp > 1:
            hidden = M.gather_from_sequence_parallel_region(hidden, g, True)
        elif st.dims.tp > 1:
            hidden = M.copy_to_tensor_model_parallel_region(hidden, g)
        w = self.shared_embedding_weight()
        if labels is None:
            return OF.linear(hidden, w)
        per = cfg.padded_vocab_size // st.dims.tp
        v0 = st.tp_rank * per
        valid = max(0, min(per, cfg.vocab_size - v0))
        losses = OF.linear_cross_entropy(hidden, w, labels, loss_mask, vocab_start=v0, valid_vocab=valid,
                                         tp_group=g if st.dims.tp > 1 else None,
                                         chunk_tokens=cfg.cross_entropy_chunk_tokens, fused_scale=loss_scale)
        if self.mtp is not None and self.training:
            losses = self.mtp.attach(self, hidden_local, losses, labels, loss_mask, loss_scale, **mtp_kw)
        return losses
