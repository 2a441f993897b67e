"""Multi-token prediction (DeepSeek-V3 style): extra depth-k modules that predict token t+1+k from
the main model's hidden state at t and the embedding of token t+k.

Counterpart of Megatron's ``MultiTokenPredictionBlock`` as used by the reference
(loongforge/models/foundation/base/base_gpt_model.py:34-41,650-664,782-794) with the checkpoint
names ``mtp.layers.{k}.{enorm,hnorm,eh_proj,transformer_layer.*,final_layernorm}``
(configs/models/deepseek3/ckpt_convert/deepseek_v3_2_convert.yaml:70-150). The MTP loss is scaled by
``mtp_loss_scaling_factor / mtp_num_layers`` and attached to the main loss through the same
autograd scaler as the MoE auxiliary losses. This implementation requires the MTP block to live
on the last pipeline stage together with a copy of the embedding when pipeline parallelism is on
(single-stage models share the embedding module directly).
"""
from __future__ import annotations

import copy

import torch
import torch.nn as nn

from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import state as ps
from .config import TransformerConfig
from .moe import AuxLossScaler, track_aux_loss
from .transformer import Norm, TransformerLayer


class MTPLayer(nn.Module):
    def __init__(self, cfg: TransformerConfig, k: int, device=None, parallel_state=None):
        super().__init__()
        self.cfg = cfg
        sp = cfg.sequence_parallel
        self.state_name = parallel_state
        self.enorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=sp)
        self.hnorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=sp)
        self.eh_proj = PL.ColumnParallelLinear(2 * cfg.hidden_size, cfg.hidden_size, gather_output=True,
                                               init_std=cfg.init_method_std, key=f"mtp.layers.{k}.eh_proj",
                                               params_dtype=cfg.params_dtype, device=device,
                                               parallel_state=parallel_state, sequence_parallel=sp)
        self.transformer_layer = TransformerLayer(cfg, cfg.num_layers - 1, device=device, parallel_state=parallel_state)
        self.final_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=sp)

    def forward(self, hidden, emb_next, rotary, packed):
        """hidden / emb_next are sequence shards ``[T/tp, H]`` under sequence parallelism (full otherwise)."""
        parts = [self.enorm(emb_next), self.hnorm(hidden)]
        if self.cfg.mtp_hidden_first:  # MiMo concatenates [hidden, embedding]
            parts.reverse()
        x = self.eh_proj(torch.cat(parts, dim=-1))  # all-gathers tokens, gathers features: [T, H] on every rank
        st = ps.get_state(self.state_name)
        if self.cfg.sequence_parallel and st.dims.tp > 1:
            from ..parallel import mappings as M
            x = M.scatter_to_sequence_parallel_region(x, st.group("tp"))
        x = self.transformer_layer(x, rotary, packed)
        return self.final_layernorm(x)


class MultiTokenPredictionBlock(nn.Module):
    def __init__(self, cfg: TransformerConfig, device=None, parallel_state=None):
        super().__init__()
        self.cfg = cfg
        lcfg = copy.copy(cfg)
        lcfg.tp_comm_overlap = False  # the fused TP kernels are sized for the trunk's shapes
        self.layers = nn.ModuleList([MTPLayer(lcfg, k, device, parallel_state) for k in range(cfg.mtp_num_layers)])

    def attach(self, model, hidden, losses, labels, loss_mask, loss_scale, *, tokens, position_ids, rotary, packed,
               full_batch=None):
        """Adds the MTP losses to the autograd graph of `losses` and returns `losses`.

        ``full_batch`` (context parallelism): flat ``tokens`` / ``labels`` / ``loss_mask`` of the micro-batch BEFORE it
        was cut into this rank's chunks. The token that follows the last position of a chunk lives on another rank, so
        the shifts run on the full rows and this rank's positions are selected afterwards."""
        cfg = self.cfg
        st = ps.get_state(model.state_name)
        T = tokens.shape[0]
        h = hidden
        sp = cfg.sequence_parallel and st.dims.tp > 1
        g = st.group("tp")
        tok, lab = tokens, labels
        mask = loss_mask.float() if loss_mask is not None else torch.ones(T, device=tokens.device)
        local_idx = None
        if full_batch is not None and st.dims.cp > 1:
            from ..parallel.context_parallel import _positions
            local_idx, _ = _positions(T, st.dims.cp, st.cp_rank, tokens.device, None,
                                      packed.row_length if packed is not None else None)
            tok, lab = full_batch["tokens"].reshape(-1), full_batch["labels"].reshape(-1)
            mask = full_batch["loss_mask"].reshape(-1).float()
        w = model.shared_embedding_weight()
        per = cfg.padded_vocab_size // st.dims.tp
        v0 = st.tp_rank * per
        valid = max(0, min(per, cfg.vocab_size - v0))
        total = losses.new_zeros(())
        for k, layer in enumerate(self.layers):
            # shift left by one: position t now sees token t+1+k and predicts label t+1+k
            tok = torch.cat([tok[1:], tok[-1:]])
            lab = torch.cat([lab[1:], lab[-1:]])
            mask = torch.cat([mask[1:], mask.new_zeros(1)])
            if packed is not None and packed.cu_seqlens is not None:
                ends = (packed.cu_seqlens[1:].long() - 1).clamp_min(0)
                mask = mask.clone()
                mask[ends] = 0  # never predict across a packed-sequence boundary
            tok_k, lab_k, mask_k, denom = tok, lab, mask, mask.sum().clamp_min(1)
            if local_idx is not None:
                # this rank's positions of the shifted full rows; the mean runs over the whole micro-batch: gradients are
                # averaged over the context-parallel ranks, hence the factor cp
                tok_k, lab_k, mask_k = tok[local_idx], lab[local_idx], mask[local_idx]
                denom = denom / st.dims.cp
            emb = model.embed(tok_k)  # a sequence shard under sequence parallelism
            h = layer(h, emb, rotary, packed)
            # the vocab-parallel loss needs the full sequence and sums partial hidden-state gradients over TP
            from ..parallel import mappings as M
            h_full = M.gather_from_sequence_parallel_region(h, g, True) if sp else (
                M.copy_to_tensor_model_parallel_region(h, g) if st.dims.tp > 1 else h)
            l_k = OF.linear_cross_entropy(h_full, w, lab_k, mask_k, vocab_start=v0, valid_vocab=valid,
                                          tp_group=st.group("tp") if st.dims.tp > 1 else None,
                                          chunk_tokens=cfg.cross_entropy_chunk_tokens)
            mtp_loss = (l_k * mask_k).sum() / denom
            track_aux_loss("mtp_loss", mtp_loss, k, max(cfg.mtp_num_layers, 1))
            total = total + mtp_loss * (cfg.mtp_loss_scaling_factor / cfg.mtp_num_layers)
        return AuxLossScaler.apply(losses, total)
