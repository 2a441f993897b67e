"""Compressed sparse attention (DeepSeek-V4 hybrid attention).

Every query attends, through ONE shared key/value latent head (MQA with K = V), to

* the last ``window`` tokens of its own sequence (sliding window over the original tokens), and
* the ``topk`` most relevant COMPRESSED entries, where a learned compressor folds every ``ratio``
  consecutive tokens into one entry and an indexer scores entries per query
  (``ratio`` 0 disables compression for the layer: window + sink only),

with a learnable per-head attention sink in the softmax denominator.

Reference: loongforge/models/foundation/deepseek_v4/deepseek_v4_csa.py — unfused attention math
``:506-598``, window / compressed top-k index builders ``:221-270,722-830``, ``Compressor :945-1318``,
indexer ``:1319-1524``, ``CompressedSparseAttention :1947-``; the reference runs the indexer logits
on DeepGEMM, the top-k on flashinfer and the backward in closed kernels. Here the whole path is
PyTorch ops over gathered entries, with the selection itself non-differentiable as in the reference.
"""
from __future__ import annotations

import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import state as ps
from .config import TransformerConfig
from .transformer import Norm, PackedSeqParams, RotaryInputs


def sparse_mqa_attention_with_sink(q: torch.Tensor, kv: torch.Tensor, idx: torch.Tensor, sink: torch.Tensor,
                                   scale: float) -> torch.Tensor:
    """q [T, H, d]; kv [N, d] (keys == values); idx [T, K] int64 rows of ``kv`` (-1 = empty slot);
    sink [H]. Returns [T, H, d]. Softmax over the K gathered entries plus the sink logit."""
    safe = idx.clamp(min=0)
    g = kv[safe].float()  # [T, K, d]
    s = torch.einsum("thd,tkd->thk", q.float(), g) * scale
    s = s.masked_fill((idx < 0).unsqueeze(1), float("-inf"))
    sk = sink.float().view(1, -1, 1)
    m = torch.maximum(s.max(-1, keepdim=True).values, sk)
    e = torch.exp(s - m)
    w = e / (e.sum(-1, keepdim=True) + torch.exp(sk - m))
    return torch.einsum("thk,tkd->thd", w, g).to(q.dtype)


def _bounds(T: int, cu_seqlens) -> List[int]:
    if cu_seqlens is None:
        return [0, T]
    return [int(b) for b in (cu_seqlens.tolist() if torch.is_tensor(cu_seqlens) else cu_seqlens)]


def window_indices(T: int, window: int, cu_seqlens, device) -> torch.Tensor:
    """[T, window] indices of the last `window` tokens (self included) of each token's own sequence."""
    pos = torch.arange(T, device=device)
    start = torch.zeros(T, dtype=torch.long, device=device)
    b = _bounds(T, cu_seqlens)
    for s, e in zip(b, b[1:]):
        start[s:e] = s
    cand = pos.unsqueeze(1) - torch.arange(window, device=device).unsqueeze(0)
    return torch.where(cand >= start.unsqueeze(1), cand, torch.full_like(cand, -1))


class Compressor(nn.Module):
    """Folds every `ratio` consecutive tokens of a sequence into one entry:
    ``c_j = sum_t softmax_t(score(x_t) + pos_bias[t mod ratio]) * kv_t`` over the block's tokens.
    A trailing partial block is dropped (it is still covered by the sliding window)."""

    def __init__(self, cfg: TransformerConfig, key: str, ratio: int, dim: int, device=None):
        super().__init__()
        self.ratio, self.dim = ratio, dim
        w = PL.init_full_then_slice(key + ".score.weight", (1, cfg.hidden_size), cfg.init_method_std, partition_dim=None,
                                    rank=0, world=1, device=device or "cpu", dtype=cfg.params_dtype)
        self.score_weight = nn.Parameter(w)
        self.pos_bias = nn.Parameter(torch.zeros(ratio, device=device, dtype=torch.float32))
        for p in (self.score_weight, self.pos_bias):
            PL.mark_tp(p, None)
            p.tp_partial_grad = True  # entries feed this rank's heads only

    def forward(self, x: torch.Tensor, kv: torch.Tensor, cu_seqlens) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """x [T, hidden], kv [T, dim] -> (entries [M, dim], last token index of each entry [M], sequence
        start of each entry [M])."""
        T, c = x.shape[0], self.ratio
        score = F.linear(x, self.score_weight).float().squeeze(-1)
        outs, ends, starts = [], [], []
        b = _bounds(T, cu_seqlens)
        for s, e in zip(b, b[1:]):
            n = (e - s) // c
            if n == 0:
                continue
            sc = score[s:s + n * c].view(n, c) + self.pos_bias
            w = torch.softmax(sc, dim=-1).to(kv.dtype)
            outs.append((w.unsqueeze(-1) * kv[s:s + n * c].view(n, c, -1)).sum(1))
            ends.append(s + (torch.arange(n, device=x.device) + 1) * c - 1)
            starts.append(torch.full((n,), s, device=x.device, dtype=torch.long))
        if not outs:
            z = torch.zeros(0, dtype=torch.long, device=x.device)
            return kv.new_zeros(0, kv.shape[1]), z, z
        return torch.cat(outs), torch.cat(ends), torch.cat(starts)


class CSAIndexer(nn.Module):
    """Scores compressed entries per query: ``I[t, j] = sum_h w[t, h] * relu(q_idx[t, h] . k_idx[j])``
    and keeps the `topk` best entries that lie entirely in the query's past and sequence."""

    def __init__(self, cfg: TransformerConfig, key: str, kv_dim: int, device=None):
        super().__init__()
        self.h, self.d, self.topk = cfg.dsa_indexer_n_heads, cfg.dsa_indexer_head_dim, cfg.dsa_indexer_topk
        kw = dict(partition_dim=None, rank=0, world=1, device=device or "cpu", dtype=cfg.params_dtype)
        self.wq = nn.Parameter(PL.init_full_then_slice(key + ".wq", (self.h * self.d, cfg.hidden_size),
                                                       cfg.init_method_std, **kw))
        self.wk = nn.Parameter(PL.init_full_then_slice(key + ".wk", (self.d, kv_dim), cfg.init_method_std, **kw))
        self.ww = nn.Parameter(PL.init_full_then_slice(key + ".weights", (self.h, cfg.hidden_size),
                                                       cfg.init_method_std, **kw))
        for p in (self.wq, self.wk, self.ww):
            PL.mark_tp(p, None, sequence_parallel=cfg.sequence_parallel)

    @torch.no_grad()
    def forward(self, x, entries, entry_end, entry_start, token_start) -> torch.Tensor:
        """-> [T, min(topk, M)] indices into `entries` (-1 = none)."""
        T, M = x.shape[0], entries.shape[0]
        k = min(self.topk, M)
        if k == 0:
            return torch.full((T, 0), -1, dtype=torch.long, device=x.device)
        q = F.linear(x, self.wq).view(T, self.h, self.d).float()
        kk = F.linear(entries, self.wk).float()
        w = F.linear(x, self.ww).float() * (self.h ** -0.5) * (self.d ** -0.5)
        s = (torch.relu(torch.einsum("thd,md->thm", q, kk)) * w.unsqueeze(-1)).sum(1)
        pos = torch.arange(T, device=x.device)
        ok = (entry_end.unsqueeze(0) <= pos.unsqueeze(1)) & (entry_start.unsqueeze(0) == token_start.unsqueeze(1))
        s = s.masked_fill(~ok, float("-inf"))
        v, i = s.topk(k, dim=-1)
        return torch.where(torch.isfinite(v), i, torch.full_like(i, -1))


class CompressedSparseAttention(nn.Module):
    """Low-rank query path, one shared KV latent head with partial RoPE, sliding window + top-k compressed
    entries, attention sink. Query heads are split over tensor-parallel ranks; the KV latent is replicated."""

    def __init__(self, cfg: TransformerConfig, key: str, layer_number: int, *, device=None, parallel_state=None):
        super().__init__()
        st = ps.get_state(parallel_state)
        tp = st.dims.tp
        self.cfg = cfg
        self.ratio = (cfg.csa_compress_ratios or [0] * (layer_number + 1))[layer_number]
        self.window = cfg.csa_window_size
        self.d = cfg.v_head_dim  # latent dim of q heads and the shared kv head
        self.rope_d = cfg.qk_pos_emb_head_dim
        self.nq = cfg.num_attention_heads
        assert self.nq % tp == 0
        self.nq_l = self.nq // tp
        common = dict(sequence_parallel=cfg.sequence_parallel, params_dtype=cfg.params_dtype, device=device,
                      parallel_state=parallel_state)
        rep = dict(partition_dim=None, rank=0, world=1, device=device or "cpu", dtype=cfg.params_dtype)
        qr = cfg.q_lora_rank or cfg.hidden_size
        self.linear_q_down = nn.Parameter(PL.init_full_then_slice(key + ".linear_q_down_proj.weight",
                                                                  (qr, cfg.hidden_size), cfg.init_method_std, **rep))
        self.linear_kv = nn.Parameter(PL.init_full_then_slice(key + ".linear_kv_proj.weight", (self.d, cfg.hidden_size),
                                                              cfg.init_method_std, **rep))
        for p in (self.linear_q_down, self.linear_kv):
            PL.mark_tp(p, None)
        self.q_layernorm = Norm(qr, cfg, device=device)
        self.kv_layernorm = Norm(self.d, cfg, device=device)
        for p in (self.linear_q_down, self.linear_kv, *self.q_layernorm.parameters(), *self.kv_layernorm.parameters()):
            p.tp_partial_grad = True  # whole-sequence input, this rank's heads downstream
        self.linear_q_up = PL.ColumnParallelLinear(qr, self.nq * self.d, bias=False, init_std=cfg.init_method_std,
                                                   key=key + ".linear_q_up_proj", **{**common, "sequence_parallel": False})
        self.linear_proj = PL.RowParallelLinear(self.nq * self.d, cfg.hidden_size, bias=False,
                                                init_std=cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers),
                                                key=key + ".linear_proj", **common)
        self.attn_sink = nn.Parameter(torch.zeros(self.nq_l, device=device, dtype=torch.float32))
        PL.mark_tp(self.attn_sink, 0 if tp > 1 else None)
        if self.ratio:
            self.compressor = Compressor(cfg, key + ".compressor", self.ratio, self.d, device=device)
            self.indexer = CSAIndexer(cfg, key + ".indexer", self.d, device=device)
        self.scale = cfg.attention_softmax_scale or 1.0 / math.sqrt(self.d)

    def _rope(self, t, rotary: Optional[RotaryInputs]):
        if rotary is None or self.rope_d == 0:
            return t
        f = rotary.freqs[:, 0] if rotary.freqs.dim() == 3 else rotary.freqs
        return OF.rope(t, f, pos_ids=rotary.pos_ids, rot_dim=self.rope_d, rot_offset=self.d - self.rope_d,
                       interleaved=self.cfg.rotary_interleaved, mscale=rotary.mscale)

    def forward(self, x, rotary: Optional[RotaryInputs], packed: Optional[PackedSeqParams], residual=None):
        from ..parallel import mappings as M

        cfg = self.cfg
        st = ps.get_state()
        # Every rank works on the WHOLE sequence with its own heads: the shared projections (q down, kv, compressor)
        # are replicated and each rank's gradient for them, and for x, is the partial sum over its heads. The region
        # mapping below sums the x gradients over the TP ranks in backward; the trainer sums the parameter gradients.
        if st.dims.tp > 1:
            x = M.gather_from_sequence_parallel_region(x, st.group("tp"), True) if cfg.sequence_parallel \
                else M.copy_to_tensor_model_parallel_region(x, st.group("tp"))
        own = None
        if st.dims.cp > 1:
            # The window and the compressed entries of a query reach into tokens of other context-parallel ranks: the
            # layer runs on the gathered sequence (redundantly on every rank) and keeps this rank's outputs. Rotary
            # angles follow the gathered positions.
            from ..parallel.context_parallel import gather_full_sequence
            extra = [rotary.pos_ids] if (rotary is not None and rotary.pos_ids is not None) else (
                [rotary.freqs] if (rotary is not None and rotary.freqs.shape[0] == x.shape[0]) else [])
            gathered, own = gather_full_sequence([x] + extra, packed.row_length if packed is not None else None)
            x = gathered[0]
            if extra and rotary.pos_ids is not None:
                rotary = RotaryInputs(freqs=rotary.freqs, pos_ids=gathered[1], mscale=rotary.mscale)
            elif extra:
                rotary = RotaryInputs(freqs=gathered[1], pos_ids=None, mscale=rotary.mscale)
        T = x.shape[0]
        cu = packed.cu_seqlens if packed is not None else None
        ql = self.q_layernorm(F.linear(x, self.linear_q_down))
        # column-parallel weight applied WITHOUT the module's own input mapping: its backward all-reduce would hand
        # every rank the full gradient of ql, which the sums above would then count once per rank
        q = OF.linear(ql, self.linear_q_up.weight).view(T, self.nq_l, self.d)
        kv = self.kv_layernorm(F.linear(x, self.linear_kv))
        q = self._rope(q, rotary)
        kv = self._rope(kv.unsqueeze(1), rotary).squeeze(1)
        idx = window_indices(T, min(self.window, T), cu, x.device)
        kv_all = kv
        if self.ratio:
            token_start = torch.zeros(T, dtype=torch.long, device=x.device)
            b = _bounds(T, cu)
            for s, e in zip(b, b[1:]):
                token_start[s:e] = s
            entries, ends, starts = self.compressor(x, kv, cu)
            sel = self.indexer(x, entries, ends, starts, token_start)
            if sel.shape[1] > 0:
                idx = torch.cat([idx, torch.where(sel >= 0, sel + T, sel)], dim=1)
                kv_all = torch.cat([kv, entries], 0)
        from ..ops.blockwise import blockwise_apply
        scale = self.scale
        o = blockwise_apply(lambda qb, ib, kvv, sk: sparse_mqa_attention_with_sink(qb, kvv, ib, sk, scale),
                            [q, idx], [kv_all, self.attn_sink], block=256)
        o = o.reshape(T, self.nq_l * self.d)
        if own is not None:
            o = o.index_select(0, own)
        return self.linear_proj(o, residual)
