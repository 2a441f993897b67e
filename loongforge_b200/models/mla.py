"""Multi-latent attention (DeepSeek-V2/V3) and its sparse variant with the lightning indexer (V3.2).

Counterpart of the reference's ``MLASelfAttentionFused`` / ``DSAIndexerFused`` / ``DSAttentionFused``
(loongforge/models/common/experimental_attention_variant/multi_latent_attention.py:66-1338,
dsa_fused.py:111-971). Parameter names follow the converter map
(configs/models/deepseek3/ckpt_convert/deepseek_v3_2_convert.yaml:70-150):
``linear_q_down_proj``, ``q_layernorm``, ``linear_q_up_proj``, ``linear_kv_down_proj``,
``kv_layernorm``, ``linear_kv_up_proj``, ``linear_proj`` and
``core_attention.indexer.{linear_wq_b,linear_wk,k_norm,linear_weights_proj}``.

Dense MLA materialises per-head K/V from the latent (192-dim keys, 128-dim values). DSA runs the
ABSORBED form: queries are projected into the 512-dim latent space with W_uk, attention runs
against the shared ``[kv_c | k_pe]`` (576-dim) rows selected by the indexer, and the 512-dim result
is projected with W_uv. Down projections are replicated across TP ranks; heads are TP-sharded.
Under context parallelism the compressed KV (576 values per token) is all-gathered, which is cheap
for MLA, and each rank attends from its own query chunk.

Sequence-first mode (``cfg.dsa_sp_first``, ``--use-dsa-sp-first``; reference multi_latent_attention.py:260-368): under
TP + SP the sparse attention does not split heads. Every rank keeps its T / tp tokens, the up projections and the
output projection are replicated (full heads), and only the compressed keys and the indexer keys are gathered over
the TP group, exactly as under context parallelism. The absorbed query tile then has all 128 heads (a full 128-row
tensor-core tile) instead of 128 / tp, the hidden states are never gathered, and the output needs no reduce-scatter.
All parameters of the block see a token shard, so their gradients are partial sums over the TP group.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn as nn

from ..ops import dsa_ops
from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import mappings as M
from ..parallel import state as ps
from .config import TransformerConfig
from .moe import AuxLossScaler, track_aux_loss


class _ReplicatedLinear(nn.Module):
    """[out, in] weight held by every TP rank (TP-duplicated down projections)."""

    def __init__(self, in_f, out_f, key, cfg, device=None, bias=False):
        super().__init__()
        w = PL.init_full_then_slice(key + ".weight", (out_f, in_f), cfg.init_method_std, partition_dim=None, rank=0,
                                    world=1, device=device or "cpu", dtype=cfg.params_dtype)
        self.weight = nn.Parameter(w)
        PL.mark_tp(self.weight, None, sequence_parallel=cfg.sequence_parallel)
        if bias:
            self.bias = nn.Parameter(torch.zeros(out_f, dtype=cfg.params_dtype, device=device))
            PL.mark_tp(self.bias, None, sequence_parallel=cfg.sequence_parallel)
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        return OF.linear(x, self.weight, self.bias)


def _rope_pe(t: torch.Tensor, rotary, interleaved: bool = True) -> torch.Tensor:
    """RoPE on a [T, heads, d_pe] tensor (DeepSeek stores the rotary pairs interleaved)."""
    return OF.rope(t, rotary.freqs, pos_ids=rotary.pos_ids, interleaved=interleaved, mscale=1.0)


class DSAIndexer(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, device=None):
        super().__init__()
        self.cfg = cfg
        self.nh, self.d = cfg.dsa_indexer_n_heads, cfg.dsa_indexer_head_dim
        q_in = cfg.q_lora_rank or cfg.hidden_size
        self.linear_wq_b = _ReplicatedLinear(q_in, self.nh * self.d, key + ".linear_wq_b", cfg, device)
        self.linear_wk = _ReplicatedLinear(cfg.hidden_size, self.d, key + ".linear_wk", cfg, device)
        self.k_norm = nn.LayerNorm(self.d, eps=cfg.dsa_indexer_k_norm_epsilon, device=device, dtype=cfg.params_dtype)
        self.linear_weights_proj = _ReplicatedLinear(cfg.hidden_size, self.nh, key + ".linear_weights_proj", cfg, device)
        self.rope_dim = cfg.qk_pos_emb_head_dim
        self.softmax_scale = self.d ** -0.5

    def project(self, x, q_c, rotary):
        """x [T, h], q_c [T, q_lora] (both detached by the caller) -> q [T, Hi, D], k [T, D], w [T, Hi]."""
        T = x.shape[0]
        q = self.linear_wq_b(q_c).view(T, self.nh, self.d)
        k = self.k_norm(self.linear_wk(x))
        # rotary part comes FIRST in the indexer's head layout (half-split pairs; GLM-5.x: interleaved pairs)
        il = self.cfg.dsa_indexer_rope_interleaved
        q = OF.rope(q, rotary.freqs, pos_ids=rotary.pos_ids, rot_dim=self.rope_dim, rot_offset=0, interleaved=il)
        k = OF.rope(k.view(T, 1, self.d), rotary.freqs, pos_ids=rotary.pos_ids, rot_dim=self.rope_dim, rot_offset=0,
                    interleaved=il).view(T, self.d)
        if self.cfg.dsa_indexer_rotate_activation:
            q = dsa_ops.hadamard_transform(q)
            k = dsa_ops.hadamard_transform(k)
        w = self.linear_weights_proj(x).float() * (self.nh ** -0.5) * self.softmax_scale
        return q, k, w


class MLASelfAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, layer_number: int, *, device=None, parallel_state=None):
        super().__init__()
        self.cfg, self.layer_number, self.state_name = cfg, layer_number, parallel_state
        st = ps.get_state(parallel_state)
        tp = st.dims.tp
        nh = cfg.num_attention_heads
        assert nh % tp == 0
        self.sp_first = bool(cfg.use_dsa and getattr(cfg, "dsa_sp_first", False) and tp > 1 and cfg.sequence_parallel)
        if self.sp_first and st.dims.cp > 1:
            raise ValueError("sequence-first sparse attention does not combine with context parallelism")
        self.nh_local = nh if self.sp_first else nh // tp
        self.dn, self.dr, self.dv, self.dc = cfg.qk_head_dim, cfg.qk_pos_emb_head_dim, cfg.v_head_dim, cfg.kv_lora_rank
        qd = self.dn + self.dr
        common = dict(init_std=cfg.init_method_std, params_dtype=cfg.params_dtype, device=device,
                      parallel_state=parallel_state)

        def column(in_f, out_f, name):
            if self.sp_first:  # replicated, full heads; its gradient is a partial sum over the ranks' token shards
                return _ReplicatedLinear(in_f, out_f, key + "." + name, cfg, device)
            return PL.ColumnParallelLinear(in_f, out_f, key=key + "." + name, **common)

        if cfg.q_lora_rank:
            self.linear_q_down_proj = _ReplicatedLinear(cfg.hidden_size, cfg.q_lora_rank, key + ".linear_q_down_proj",
                                                        cfg, device)
            from .transformer import Norm
            self.q_layernorm = Norm(cfg.q_lora_rank, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.linear_q_up_proj = column(cfg.q_lora_rank, nh * qd, "linear_q_up_proj")
        else:
            self.linear_q_proj = column(cfg.hidden_size, nh * qd, "linear_q_proj")
        self.linear_kv_down_proj = _ReplicatedLinear(cfg.hidden_size, self.dc + self.dr, key + ".linear_kv_down_proj",
                                                     cfg, device)
        from .transformer import Norm
        self.kv_layernorm = Norm(self.dc, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
        self.linear_kv_up_proj = column(self.dc, nh * (self.dn + self.dv), "linear_kv_up_proj")
        common["init_std"] = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        if self.sp_first:
            import dataclasses
            self.linear_proj = _ReplicatedLinear(nh * self.dv, cfg.hidden_size, key + ".linear_proj",
                                                 dataclasses.replace(cfg, init_method_std=common["init_std"]), device)
        else:
            self.linear_proj = PL.RowParallelLinear(nh * self.dv, cfg.hidden_size, key=key + ".linear_proj",
                                                    sequence_parallel=cfg.sequence_parallel, **common)
        if cfg.use_dsa:
            self.core_attention = nn.Module()
            # IndexShare: a layer without an indexer receives the top-k indices of its source layer
            self.computes_topk = cfg.dsa_computes_topk(layer_number)
            if self.computes_topk:
                self.core_attention.indexer = DSAIndexer(cfg, key + ".core_attention.indexer", device)
            self.last_topk_indices = None  # what this layer selected (or was given) in its latest forward
            self.shared_topk_indices = None  # set by the layer loop before calling a layer that reuses indices
            if self.sp_first and self.computes_topk:
                for p in self.core_attention.indexer.k_norm.parameters():
                    p.sequence_parallel = True  # sees a token shard here: partial gradient
        self.mscale = 1.0  # set from the rotary inputs (YaRN)

    def _softmax_scale(self, rotary) -> float:
        m = rotary.mscale if rotary is not None else 1.0
        return (m * m) / math.sqrt(self.dn + self.dr)

    def forward(self, x, rotary, packed, residual=None):
        cfg = self.cfg
        st = ps.get_state(self.state_name)
        g_tp = st.group("tp")
        if self.sp_first:
            # this rank's tokens are rows [r T, (r + 1) T) of the micro-batch: rotary angles of exactly those rows
            T = x.shape[0]
            lo = st.tp_rank * T
            if rotary is not None:
                from .transformer import RotaryInputs
                ids = rotary.pos_ids[lo:lo + T] if rotary.pos_ids is not None else \
                    torch.arange(lo, lo + T, device=x.device, dtype=torch.int32)
                rotary = RotaryInputs(freqs=rotary.freqs, pos_ids=ids, mscale=rotary.mscale)
        elif cfg.sequence_parallel and st.dims.tp > 1:
            x = M.gather_from_sequence_parallel_region(x, g_tp, True)
        T = x.shape[0]
        H = self.nh_local
        # ---- latents
        if cfg.q_lora_rank:
            q_c = self.q_layernorm(self.linear_q_down_proj(x))
            q = self.linear_q_up_proj(q_c)
        else:
            q_c = x
            q = self.linear_q_proj(x)
        q = q.view(T, H, self.dn + self.dr)
        kv = self.linear_kv_down_proj(x)
        kv_c = self.kv_layernorm(kv[:, : self.dc].contiguous())
        k_pe = kv[:, self.dc:].contiguous().view(T, 1, self.dr)
        q_nope, q_pe = q[..., : self.dn], q[..., self.dn:]
        if rotary is not None:
            q_pe = _rope_pe(q_pe.contiguous(), rotary)
            k_pe = _rope_pe(k_pe, rotary)
        scale = self._softmax_scale(rotary)
        cu = packed.cu_seqlens if packed is not None else None
        self._row_length = packed.row_length if packed is not None else None
        w_up = self.linear_kv_up_proj.weight.view(H, self.dn + self.dv, self.dc)
        if not cfg.use_dsa:
            kvu = self.linear_kv_up_proj(kv_c).view(T, H, self.dn + self.dv)
            k = torch.cat([kvu[..., : self.dn], k_pe.expand(T, H, self.dr)], dim=-1)
            v = kvu[..., self.dn:]
            qq = torch.cat([q_nope, q_pe], dim=-1)
            from .transformer import core_attention  # ring / all-gather attention under context parallelism
            o = core_attention(qq.contiguous(), k.contiguous(), v.contiguous(), causal=True, scale=scale, cu_seqlens=cu,
                               cfg=cfg, row_length=packed.row_length if packed is not None else None,
                               training=self.training)
        else:
            o = self._dsa(x, q_c, q_nope, q_pe, kv_c, k_pe, w_up, rotary, cu, scale)
        if self.sp_first:
            out = self.linear_proj(o.reshape(T, H * self.dv))  # already this rank's sequence shard: nothing to reduce
            return out if residual is None else out + residual
        return self.linear_proj(o.reshape(T, H * self.dv), residual)

    # ------------------------------------------------------------------ sparse path
    def _dsa(self, x, q_c, q_nope, q_pe, kv_c, k_pe, w_up, rotary, cu, scale):
        cfg = self.cfg
        st = ps.get_state(self.state_name)
        T, H = q_nope.shape[0], self.nh_local
        w_uk, w_uv = w_up[:, : self.dn, :], w_up[:, self.dn:, :]  # [H, dn, dc], [H, dv, dc]
        # absorbed query: q_nope @ W_uk -> latent space; key = [kv_c | k_pe] shared by all heads
        q_abs = torch.einsum("thd,hdc->thc", q_nope, w_uk.to(q_nope.dtype))
        query = torch.cat([q_abs, q_pe], dim=-1)  # [T, H, dc + dr]
        key = torch.cat([kv_c, k_pe.view(T, self.dr)], dim=-1)  # [T, dc + dr]
        seq_group = st.group("cp") if st.dims.cp > 1 else (st.group("tp") if self.sp_first else None)
        if st.dims.cp > 1:
            # this rank holds two chunks of the packed row: causal order and sequence membership follow the ROW position
            from ..parallel.context_parallel import _positions
            pos, seg = _positions(T, st.dims.cp, st.cp_rank, x.device, cu, self._row_length)
        elif self.sp_first:
            # this rank holds rows [r T, (r + 1) T) of a micro-batch of tp * T tokens
            lo = st.tp_rank * T
            pos = torch.arange(lo, lo + T, device=x.device)
            seg = None
            if cu is not None:
                seg = torch.bucketize(pos, cu[1:].long().to(x.device), right=True)
                # causal order inside a packed sequence is the row order, so row positions serve as positions
        else:
            pos = rotary.pos_ids.long() if (rotary is not None and rotary.pos_ids is not None) \
                else torch.arange(T, device=x.device)
            seg = None
            if cu is not None:
                seg = torch.bucketize(torch.arange(T, device=x.device), cu[1:].long().to(x.device), right=True)
        key_all, pos_k, seg_k = key, pos, seg
        from .transformer import CHUNK_PREFIX
        chunked = CHUNK_PREFIX["active"]
        if chunked:
            # sequence-chunk pipelining: the compressed keys (and the indexer keys) of the sequence's earlier chunks are
            # the prefix; this chunk's tokens sit behind them
            assert cu is None and seq_group is None, "chunk pipelining runs one unpacked sequence, without cp / sp-first"
            past = CHUNK_PREFIX["past"]
            n_past = past[0].shape[0] if past is not None else 0
            pos = torch.arange(n_past, n_past + T, device=x.device)
            key_all = torch.cat([past[0], key]) if past is not None else key
            pos_k = torch.arange(n_past + T, device=x.device)
        if seq_group is not None:
            g = seq_group
            key_all = M.gather_from_sequence_parallel_region(key, g, True)
            pos_k = M._all_gather_dim0(pos, g)
            seg_k = M._all_gather_dim0(seg, g) if seg is not None else None
        if self.computes_topk:
            idxr = self.core_attention.indexer
            qi, ki, wi = idxr.project(x.detach(), q_c.detach(), rotary)
            # index keys of the other context-parallel ranks; their gradient (indexer loss) flows back by reduce-scatter
            ki_all = M.gather_from_sequence_parallel_region(ki, seq_group, True) if seq_group is not None else ki
            if chunked:
                CHUNK_PREFIX["out"] = (key, ki)
                ki_all = torch.cat([past[1], ki]) if past is not None else ki
            with torch.no_grad():
                qq, _ = dsa_ops.quant_fp8_rowwise_pow2(qi) if cfg.fp8 else (qi, None)
                kq, _ = dsa_ops.quant_fp8_rowwise_pow2(ki_all) if cfg.fp8 else (ki_all, None)
                if self.sp_first or chunked:
                    # keys are in row order (contiguous shards / prefix then chunk): one index range per query
                    indices, _ = dsa_ops.indexer_topk(qq, kq, wi, cfg.dsa_indexer_topk, pos, pos_k, seg, seg_k,
                                                      keys_in_order=True)
                elif st.dims.cp > 1:
                    # gathered keys arrive rank-major: put them into row order so that every query's candidates are
                    # one contiguous index range (what the native kernels want), and map the selection back
                    order = torch.argsort(pos_k)
                    sel, _ = dsa_ops.indexer_topk(qq, kq.index_select(0, order), wi, cfg.dsa_indexer_topk, pos,
                                                  pos_k.index_select(0, order), seg,
                                                  seg_k.index_select(0, order) if seg_k is not None else None,
                                                  keys_in_order=True)
                    indices = torch.where(sel >= 0, order[sel.clamp_min(0)], sel)
                else:
                    # one rank holds the row(s) in order: causal order is index order inside every sequence
                    ar = torch.arange(T, device=x.device)
                    indices, _ = dsa_ops.indexer_topk(qq, kq, wi, cfg.dsa_indexer_topk, ar, ar, seg, seg_k,
                                                      keys_in_order=True)
        else:
            if chunked:
                CHUNK_PREFIX["out"] = (key, key.new_zeros(T, 0))  # no indexer here: nothing but the keys to cache
            indices = self.shared_topk_indices
            if indices is None:
                raise RuntimeError(f"layer {self.layer_number} reuses top-k indices (IndexShare) but received none; "
                                   "a pipeline stage must start on a layer that computes them")
        self.last_topk_indices = indices
        want_loss = self.training and cfg.dsa_indexer_loss_coeff > 0 and self.computes_topk
        out = dsa_ops.sparse_mla_attention(query, key_all, indices, scale, d_v=self.dc,
                                           return_head_mean_probs=want_loss)
        if want_loss:
            o_c, pmean = out
            # index scores at the selected slots, differentiable w.r.t. the indexer weights only
            sc = dsa_ops.indexer_scores_at(qi, wi, ki_all, indices)
            loss = dsa_ops.indexer_kl_loss(sc, pmean, indices, cfg.dsa_indexer_loss_coeff)
            if st.dims.tp > 1:
                loss = M.reduce_from_tensor_model_parallel_region(loss, st.group("tp")) / st.dims.tp
            track_aux_loss("indexer_loss", loss / cfg.dsa_indexer_loss_coeff, self.layer_number, cfg.num_layers)
            o_c = AuxLossScaler.apply(o_c, loss)
        else:
            o_c = out
        return torch.einsum("thc,hvc->thv", o_c, w_uv.to(o_c.dtype))
