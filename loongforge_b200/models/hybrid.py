"""Hybrid-attention layers of Qwen3-Next / Qwen3.5: output-gated softmax attention and GatedDeltaNet
linear attention, mixed by ``cfg.layer_types``.

* ``GatedAttention``: the query projection is twice as wide; the second half is a per-element gate,
  ``out = attn(q, k, v) * sigmoid(gate)`` before the output projection; per-head QK RMSNorm
  (zero-centred weight), partial rotary (reference: loongforge/models/foundation/qwen3_next/gated_attention.py:53-).
* ``GatedDeltaNet``: in-projections to (q, k, v, z) and (b, a); depthwise causal conv + SiLU over
  q|k|v; ``beta = sigmoid(b)``, log-decay ``g = -exp(A_log) * softplus(a + dt_bias)``; gated delta rule;
  RMSNorm gated by ``silu(z)``; out-projection (reference: .../qwen3_next/gated_deltanet.py:129-420).
  Heads are split over tensor parallel ranks (value heads, with their share of key heads).
"""
from __future__ import annotations

import math
import zlib
from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..ops import linear_attn as LA
from ..parallel import layers as PL
from ..parallel import state as ps
from .config import TransformerConfig
from .transformer import Norm, PackedSeqParams, RotaryInputs, core_attention


class GatedAttention(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, *, device=None, parallel_state=None):
        super().__init__()
        st = ps.get_state(parallel_state)
        tp = st.dims.tp
        self.cfg, self.d = cfg, cfg.kv_channels
        self.nq, self.ng = cfg.num_attention_heads, cfg.num_query_groups
        assert self.nq % tp == 0 and self.ng % tp == 0
        self.nq_l, self.ng_l = self.nq // tp, self.ng // tp
        common = dict(sequence_parallel=cfg.sequence_parallel, params_dtype=cfg.params_dtype, device=device,
                      parallel_state=parallel_state)
        # per query group: [q heads | gate heads | k | v], so a TP shard keeps whole groups
        self.r = self.nq // self.ng
        out = (2 * self.nq + 2 * self.ng) * self.d
        self.linear_qgkv = PL.ColumnParallelLinear(cfg.hidden_size, out, bias=False, init_std=cfg.init_method_std,
                                                   key=key + ".linear_qgkv", **common)
        self.q_layernorm = Norm(self.d, cfg, device=device)
        self.k_layernorm = Norm(self.d, cfg, device=device)
        if tp > 1:
            PL.mark_tp_partial_grad(self.q_layernorm)
            PL.mark_tp_partial_grad(self.k_layernorm)
        self.linear_proj = PL.RowParallelLinear(self.nq * self.d, cfg.hidden_size, bias=False,
                                                init_std=cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers),
                                                key=key + ".linear_proj", **common)
        self.scale = cfg.attention_softmax_scale or 1.0 / math.sqrt(self.d)
        self.rot_dim = int(self.d * cfg.rotary_percent)

    def forward(self, x, rotary: Optional[RotaryInputs], packed: Optional[PackedSeqParams], residual=None):
        T = x.shape[0] * (ps.get_state().dims.tp if self.cfg.sequence_parallel else 1)
        y = self.linear_qgkv(x).view(-1, self.ng_l, 2 * self.r + 2, self.d)
        T = y.shape[0]
        q = self.q_layernorm(y[:, :, :self.r].reshape(T, self.nq_l, self.d))
        gate = y[:, :, self.r:2 * self.r].reshape(T, self.nq_l * self.d)
        k = self.k_layernorm(y[:, :, 2 * self.r].contiguous())
        v = y[:, :, 2 * self.r + 1]
        if rotary is not None:
            kw = dict(pos_ids=rotary.pos_ids, rot_dim=self.rot_dim, interleaved=self.cfg.rotary_interleaved,
                      mscale=rotary.mscale)
            f = rotary.freqs
            if f.dim() == 3:
                f, kw = f[:, 0], {**kw, "pos_ids": None, "interleaved": False}
            q, k = OF.rope(q, f, **kw), OF.rope(k, f, **kw)
        cu = packed.cu_seqlens if packed is not None else None
        o = core_attention(q, k, v, causal=True, scale=self.scale, cu_seqlens=cu, cfg=self.cfg,
                           row_length=packed.row_length if packed is not None else None)
        o = o.reshape(T, self.nq_l * self.d) * torch.sigmoid(gate.float()).to(o.dtype)
        return self.linear_proj(o, residual)


class GatedRMSNorm(nn.Module):
    """y = rmsnorm(x) * w * silu(z), over the value head dim."""

    def __init__(self, dim: int, eps: float, device=None, dtype=torch.float32):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(dim, device=device, dtype=dtype))
        self.eps = eps

    def forward(self, x, z):
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight.float()
        return (y * F.silu(z.float())).to(x.dtype)


class GatedDeltaNet(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, *, device=None, parallel_state=None):
        super().__init__()
        st = ps.get_state(parallel_state)
        self.cp = st.dims.cp  # > 1: convolution and recurrence run on the gathered sequence (see forward)
        tp = st.dims.tp
        self.cfg = cfg
        self.dk, self.dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
        self.hk, self.hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
        assert self.hk % tp == 0 and self.hv % self.hk == 0
        self.hk_l, self.hv_l = self.hk // tp, self.hv // tp
        self.ratio = self.hv // self.hk
        self.K = cfg.linear_conv_kernel_dim
        common = dict(sequence_parallel=cfg.sequence_parallel, params_dtype=cfg.params_dtype, device=device,
                      parallel_state=parallel_state)
        # per key head: [q | k | v (ratio heads) | z (ratio heads)] and [b (ratio) | a (ratio)]
        per_head = 2 * self.dk + 2 * self.ratio * self.dv
        self.in_proj_qkvz = PL.ColumnParallelLinear(cfg.hidden_size, self.hk * per_head, bias=False,
                                                    init_std=cfg.init_method_std, key=key + ".in_proj_qkvz", **common)
        self.in_proj_ba = PL.ColumnParallelLinear(cfg.hidden_size, self.hk * 2 * self.ratio, bias=False,
                                                  init_std=cfg.init_method_std, key=key + ".in_proj_ba", **common)
        # The FULL parameters are drawn from a seed that depends only on the key, then sliced to this rank's heads, so
        # that every tensor-parallel layout starts from the same model. Conv channels are laid out type-major
        # [q heads | k heads | v heads]; a rank keeps its head range of each type.
        g = torch.Generator().manual_seed(zlib.crc32((key + ".conv1d").encode()) & 0x7FFFFFFF)
        full_conv = (torch.rand(self.hk * (2 * self.dk + self.ratio * self.dv), self.K, generator=g) * 2 - 1) * self.K ** -0.5
        qf, kf, vf = full_conv.split([self.hk * self.dk, self.hk * self.dk, self.hv * self.dv], dim=0)
        r0 = st.tp_rank
        local = torch.cat([qf.view(self.hk, self.dk, -1)[r0 * self.hk_l:(r0 + 1) * self.hk_l].reshape(-1, self.K),
                           kf.view(self.hk, self.dk, -1)[r0 * self.hk_l:(r0 + 1) * self.hk_l].reshape(-1, self.K),
                           vf.view(self.hv, self.dv, -1)[r0 * self.hv_l:(r0 + 1) * self.hv_l].reshape(-1, self.K)], 0)
        self.conv_weight = nn.Parameter(local.to(device=device, dtype=cfg.params_dtype))
        self.dt_bias = nn.Parameter(torch.ones(self.hv_l, device=device))
        A = torch.empty(self.hv).uniform_(1e-3, 16.0, generator=g)[r0 * self.hv_l:(r0 + 1) * self.hv_l]
        self.A_log = nn.Parameter(torch.log(A).to(device=device))
        for p in (self.conv_weight, self.dt_bias, self.A_log):
            PL.mark_tp(p, 0 if tp > 1 else None)
        self.out_norm = GatedRMSNorm(self.dv, cfg.layernorm_epsilon, device=device)
        PL.mark_tp(self.out_norm.weight, None)
        if tp > 1:
            PL.mark_tp_partial_grad(self.out_norm)
        self.out_proj = PL.RowParallelLinear(self.hv * self.dv, cfg.hidden_size, bias=False,
                                             init_std=cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers),
                                             key=key + ".out_proj", **common)

    def forward(self, x, rotary=None, packed: Optional[PackedSeqParams] = None, residual=None):
        hk, r, dk, dv = self.hk_l, self.ratio, self.dk, self.dv
        qkvz = self.in_proj_qkvz(x)
        T = qkvz.shape[0]
        qkvz = qkvz.view(T, hk, 2 * dk + 2 * r * dv)
        ba = self.in_proj_ba(x).view(T, hk, 2 * r)
        q, k, v, z = qkvz.split([dk, dk, r * dv, r * dv], dim=-1)
        b, a = ba.split([r, r], dim=-1)
        cu = packed.cu_seqlens if packed is not None else None
        # conv over [q | k | v] channels, laid out type-major like the conv weight
        mixed = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], dim=-1)
        own = None
        if self.cp > 1:
            # The convolution window and the recurrent state cross the chunk boundaries of context parallelism: run
            # both on the gathered sequence (token-wise projections stay local) and keep this rank's outputs.
            from ..parallel.context_parallel import gather_full_sequence
            (mixed, b, a), own = gather_full_sequence([mixed, b.reshape(T, -1), a.reshape(T, -1)],
                                                      packed.row_length if packed is not None else None)
            T_loc, T = T, mixed.shape[0]
        mixed = LA.causal_conv1d(mixed, self.conv_weight, cu_seqlens=cu, activation="silu")
        q, k, v = mixed.split([hk * dk, hk * dk, hk * r * dv], dim=-1)
        q = q.view(T, hk, dk).repeat_interleave(r, dim=1)
        k = k.view(T, hk, dk).repeat_interleave(r, dim=1)
        v = v.view(T, hk * r, dv)
        beta = torch.sigmoid(b.reshape(T, hk * r).float())
        g = -self.A_log.float().exp() * F.softplus(a.reshape(T, hk * r).float() + self.dt_bias.float())
        o = LA.gated_delta_rule(q, k, v, g, beta, cu_seqlens=cu, qk_l2norm=True)
        if own is not None:
            o, T = o.index_select(0, own), T_loc
        o = self.out_norm(o, z.reshape(T, hk * r, dv))
        return self.out_proj(o.reshape(T, hk * r * dv), residual)
