"""Decoder building blocks on a packed-token layout.

Activations are ``[T, hidden]`` (T = all tokens of the micro-batch, sequence boundaries in
``cu_seqlens``); under sequence parallelism the tensors between blocks are ``[T/tp, hidden]``.
Module and parameter names reproduce Megatron's so that ``state_dict`` keys equal the
reference's checkpoint keys (configs/models/llama3/ckpt_convert/llama3_convert.yaml:43-70):
``self_attention.linear_qkv.{layer_norm_weight,weight,bias}``, ``self_attention.linear_proj``,
``mlp.linear_fc1.{layer_norm_weight,weight}``, ``mlp.linear_fc2``, ``pre_mlp_layernorm``,
``input_layernorm``, ``self_attention.{q,k}_layernorm``.

The packed QKV weight uses Megatron's per-group row order ``[q_0..q_{r-1}, k, v]``
(tools/convert_checkpoint/huggingface/util/hf_attn_converter.py:62-78) and FC1 is
``[gate; up]`` (tools/convert_checkpoint/huggingface/huggingface_base.py:495-524).
"""
from __future__ import annotations

import dataclasses
import math
from typing import Optional

import torch
import torch.nn as nn
import torch.utils.checkpoint

from ..ops import functional as OF
from ..parallel import layers as PL
from ..parallel import state as ps
from .config import TransformerConfig


@dataclasses.dataclass
class PackedSeqParams:
    """Sequence boundaries of a packed ("thd") micro-batch."""
    cu_seqlens: Optional[torch.Tensor] = None  # int32 [num_seqs + 1]
    max_seqlen: Optional[int] = None
    # Context parallelism cuts every ROW of the micro-batch into 2*cp chunks; with several rows per micro-batch this is
    # the full (unsliced) row length, and `cu_seqlens` are offsets in the concatenation of the full rows. None = one row.
    row_length: Optional[int] = None


@dataclasses.dataclass
class RotaryInputs:
    freqs: torch.Tensor  # fp32 [P, rot_dim/2] angle table, or per-token angles [T, rot_dim/2]
    pos_ids: Optional[torch.Tensor] = None  # int32 [T] rows of `freqs`; None = row t
    mscale: float = 1.0


class Norm(nn.Module):
    def __init__(self, hidden: int, cfg: TransformerConfig, device=None, sequence_parallel: bool = False):
        super().__init__()
        self.kind = cfg.normalization
        self.eps = cfg.layernorm_epsilon
        self.offset = 1.0 if cfg.layernorm_zero_centered_gamma else 0.0
        init = 0.0 if cfg.layernorm_zero_centered_gamma else 1.0
        self.weight = nn.Parameter(torch.full((hidden,), init, dtype=cfg.params_dtype, device=device))
        PL.mark_tp(self.weight, None, sequence_parallel=sequence_parallel)
        if self.kind == "LayerNorm":
            self.bias = nn.Parameter(torch.zeros(hidden, dtype=cfg.params_dtype, device=device))
            PL.mark_tp(self.bias, None, sequence_parallel=sequence_parallel)
        else:
            self.register_parameter("bias", None)

    def forward(self, x):
        return apply_norm(x, self.weight, self.bias, self.kind, self.eps, self.offset)


class TPRMSNorm(nn.Module):
    """RMSNorm over a feature dimension that is SHARDED across tensor-parallel ranks: each rank holds its
    slice of the features and of the weight; the sum of squares is all-reduced over the TP group
    (MiniMax full-width QK norm, loongforge/models/foundation/minimax/attention.py:143,170,230-239;
    InternViT's TP-aware norm, loongforge/models/encoder/internvl_vision_models/intern_vision_attention.py:116)."""

    def __init__(self, full_dim: int, cfg: TransformerConfig, key: str, device=None, parallel_state=None):
        super().__init__()
        st = ps.get_state(parallel_state)
        self.state_name, self.full_dim, self.eps = parallel_state, full_dim, cfg.layernorm_epsilon
        self.weight = nn.Parameter(torch.ones(full_dim // st.dims.tp, device=device, dtype=cfg.params_dtype))
        PL.mark_tp(self.weight, 0 if st.dims.tp > 1 else None)

    def forward(self, x):
        st = ps.get_state(self.state_name)
        ss = x.float().pow(2).sum(-1, keepdim=True)
        if st.dims.tp > 1:
            from ..parallel import mappings as M
            # every rank normalises its own feature slice with the SHARED statistic: gradients flow back from all ranks
            ss = M.all_reduce_forward_and_backward(ss, st.group("tp"))
        return (x.float() * torch.rsqrt(ss / self.full_dim + self.eps) * self.weight.float()).to(x.dtype)


def apply_norm(x, weight, bias, kind, eps, offset=0.0):
    if kind == "RMSNorm":
        return OF.rmsnorm(x, weight, eps, offset)
    w = weight + offset if offset else weight
    return torch.nn.functional.layer_norm(x, (x.shape[-1],), w.to(x.dtype), bias.to(x.dtype) if bias is not None else None, eps)


class LayerNormColumnParallelLinear(PL.ColumnParallelLinear):
    """Norm fused in front of a column-parallel linear (norm runs on the sequence shard,
    before the all-gather). Parameter names: ``layer_norm_weight`` / ``layer_norm_bias``."""

    def __init__(self, in_features, out_features, cfg: TransformerConfig, **kw):
        super().__init__(in_features, out_features, **kw)
        dev = self.weight.device
        init = 0.0 if cfg.layernorm_zero_centered_gamma else 1.0
        self.layer_norm_weight = nn.Parameter(torch.full((in_features,), init, dtype=cfg.params_dtype, device=dev))
        PL.mark_tp(self.layer_norm_weight, None, sequence_parallel=self.sequence_parallel)
        if cfg.normalization == "LayerNorm":
            self.layer_norm_bias = nn.Parameter(torch.zeros(in_features, dtype=cfg.params_dtype, device=dev))
            PL.mark_tp(self.layer_norm_bias, None, sequence_parallel=self.sequence_parallel)
        else:
            self.register_parameter("layer_norm_bias", None)
        self._norm = (cfg.normalization, cfg.layernorm_epsilon, 1.0 if cfg.layernorm_zero_centered_gamma else 0.0)

    def forward(self, x):
        kind, eps, off = self._norm
        if (self.tp == 1 and kind == "RMSNorm" and not self.gather_output
                and OF.norm_linear_supported(x, self.layer_norm_weight, self.weight)):
            # single-GPU tensor layout: fused block that does not store the normalised activations
            return OF.norm_linear(x, self.layer_norm_weight, self.weight, self.bias, eps, off)
        return super().forward(apply_norm(x, self.layer_norm_weight, self.layer_norm_bias, kind, eps, off))


def _act(name: str):
    import torch.nn.functional as F
    return {"gelu": F.gelu, "relu": F.relu, "silu": F.silu,
            "quick_gelu": lambda x: x * torch.sigmoid(1.702 * x),
            "gelu_tanh": lambda x: F.gelu(x, approximate="tanh")}[name]


def clamped_swiglu(h: torch.Tensor, limit: float) -> torch.Tensor:
    """SwiGLU with bounded pre-activations (DeepSeek-V4 ``swiglu_limit``): gate clamped from above, the linear branch
    to [-limit, limit], so that a few huge activations cannot dominate the product."""
    g, u = h.chunk(2, dim=-1)
    return torch.nn.functional.silu(g.clamp(max=limit)) * u.clamp(min=-limit, max=limit)


class MLP(nn.Module):
    def __init__(self, cfg: TransformerConfig, key: str, *, ffn_hidden: Optional[int] = None, fused_norm: bool = True,
                 device=None, parallel_state=None, is_expert: bool = False, sequence_parallel: Optional[bool] = None):
        super().__init__()
        f = ffn_hidden or cfg.ffn_hidden_size
        sp = cfg.sequence_parallel if sequence_parallel is None else sequence_parallel
        glu = cfg.gated_linear_unit
        common = dict(init_std=cfg.init_method_std, sequence_parallel=sp, params_dtype=cfg.params_dtype,
                      device=device, parallel_state=parallel_state, tp_comm_overlap=cfg.tp_comm_overlap,
                      is_expert=is_expert)
        fc1_kw = dict(bias=cfg.add_bias_linear, key=key + ".linear_fc1", stride=2 if glu else 1, **common)
        if fused_norm:
            self.linear_fc1 = LayerNormColumnParallelLinear(cfg.hidden_size, f * (2 if glu else 1), cfg, **fc1_kw)
        else:
            self.linear_fc1 = PL.ColumnParallelLinear(cfg.hidden_size, f * (2 if glu else 1), **fc1_kw)
        out_std = cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers)
        common["init_std"] = out_std
        self.linear_fc2 = PL.RowParallelLinear(f, cfg.hidden_size, bias=cfg.add_bias_linear, key=key + ".linear_fc2",
                                               **common)
        self.glu = glu
        self.act_name = cfg.activation
        self.swiglu_limit = cfg.swiglu_limit

    def forward(self, x, residual=None):
        h = self.linear_fc1(x)
        if self.glu and self.act_name == "swiglu" and self.swiglu_limit:
            return self.linear_fc2(clamped_swiglu(h, self.swiglu_limit), residual)
        if (self.glu and self.act_name == "swiglu" and self.linear_fc2.tp == 1 and self.linear_fc2.bias is None
                and OF.swiglu_linear_supported(h, self.linear_fc2.weight)):
            return OF.swiglu_linear(h, self.linear_fc2.weight, residual)
        if self.glu and self.act_name == "swiglu":
            h = OF.swiglu(h)
        elif self.glu:
            g, u = h.chunk(2, dim=-1)
            h = _act("gelu" if self.act_name == "geglu" else self.act_name)(g) * u
        else:
            h = _act(self.act_name)(h)
        return self.linear_fc2(h, residual)


class SelfAttention(nn.Module):
    """GQA self attention with a packed QKV projection, optional per-head QK RMSNorm (Qwen3),
    RoPE / M-RoPE applied in place on the packed buffer, and packed-sequence attention."""

    def __init__(self, cfg: TransformerConfig, key: str, *, fused_norm: bool = True, device=None, parallel_state=None):
        super().__init__()
        st = ps.get_state(parallel_state)
        tp = st.dims.tp
        self.cfg = cfg
        self.d = cfg.kv_channels
        self.nq, self.ng = cfg.num_attention_heads, cfg.num_query_groups
        assert self.ng % tp == 0 and self.nq % self.ng == 0, "kv groups must divide by TP"
        self.r = self.nq // self.ng
        self.ng_local = self.ng // tp
        self.nq_local = self.nq // tp
        qkv_out = (self.nq + 2 * self.ng) * self.d
        common = dict(sequence_parallel=cfg.sequence_parallel, params_dtype=cfg.params_dtype, device=device,
                      parallel_state=parallel_state, tp_comm_overlap=cfg.tp_comm_overlap)
        kw = dict(bias=cfg.add_bias_linear or cfg.add_qkv_bias, init_std=cfg.init_method_std,
                  key=key + ".linear_qkv", **common)
        if fused_norm:
            self.linear_qkv = LayerNormColumnParallelLinear(cfg.hidden_size, qkv_out, cfg, **kw)
        else:
            self.linear_qkv = PL.ColumnParallelLinear(cfg.hidden_size, qkv_out, **kw)
        if cfg.qk_layernorm_full:
            # MiniMax: one RMSNorm over ALL heads of q (and of k); under TP the statistic is all-reduced
            self.q_layernorm = TPRMSNorm(self.nq * self.d, cfg, key + ".q_layernorm", device=device,
                                         parallel_state=parallel_state)
            self.k_layernorm = TPRMSNorm(self.ng * self.d, cfg, key + ".k_layernorm", device=device,
                                         parallel_state=parallel_state)
        elif cfg.qk_layernorm:
            self.q_layernorm = Norm(self.d, cfg, device=device)
            self.k_layernorm = Norm(self.d, cfg, device=device)
            if tp > 1:
                PL.mark_tp_partial_grad(self.q_layernorm)
                PL.mark_tp_partial_grad(self.k_layernorm)
        else:
            self.q_layernorm = self.k_layernorm = None
        self.linear_proj = PL.RowParallelLinear(self.nq * self.d, cfg.hidden_size, bias=cfg.add_bias_linear,
                                                init_std=cfg.init_method_std / math.sqrt(2.0 * cfg.num_layers),
                                                key=key + ".linear_proj", **common)
        self.scale = cfg.attention_softmax_scale or 1.0 / math.sqrt(self.d)
        self.rot_dim = int(self.d * cfg.rotary_percent)

    def forward(self, x, rotary: Optional[RotaryInputs], packed: Optional[PackedSeqParams], residual=None):
        cfg = self.cfg
        qkv = self.linear_qkv(x)  # [T, ng_local * (r + 2) * d]
        T = qkv.shape[0]
        g, r, d = self.ng_local, self.r, self.d
        cu = packed.cu_seqlens if packed is not None else None
        if self.q_layernorm is None:
            if rotary is not None:
                qkv = self._rope_packed(qkv, rotary)
            if (ps.get_state().dims.cp == 1 and not CHUNK_PREFIX["active"] and OF.attention_packed_supported(qkv, d)
                    and not (self.training and cfg.attention_dropout > 0)):
                # tcgen05 attention reads q/k/v straight out of the packed GEMM output
                o = OF.attention_packed(qkv, g, r, causal=cfg.causal, scale=self.scale, cu_seqlens=cu)
                return self.linear_proj(o.view(T, g * r * d), residual)
            pk4 = qkv.view(T, g, r + 2, d)
            q = pk4[:, :, :r].reshape(T, g * r, d)
            k = pk4[:, :, r]
            v = pk4[:, :, r + 1]
        else:
            pk4 = qkv.view(T, g, r + 2, d)
            if cfg.qk_layernorm_full:
                q = self.q_layernorm(pk4[:, :, :r].reshape(T, g * r * d)).view(T, g * r, d)
                k = self.k_layernorm(pk4[:, :, r].reshape(T, g * d)).view(T, g, d)
            else:
                q = self.q_layernorm(pk4[:, :, :r].reshape(T, g * r, d))
                k = self.k_layernorm(pk4[:, :, r].contiguous())
            v = pk4[:, :, r + 1]
            if rotary is not None:
                q = self._rope(q, rotary)
                k = self._rope(k, rotary)
        o = core_attention(q, k, v, causal=cfg.causal, scale=self.scale, cu_seqlens=cu, cfg=cfg,
                           row_length=packed.row_length if packed is not None else None, training=self.training)
        return self.linear_proj(o.reshape(T, g * r * d), residual)

    def _rope_kw(self, rotary):
        cfg = self.cfg
        return dict(pos_ids=rotary.pos_ids, rot_dim=self.rot_dim, interleaved=cfg.rotary_interleaved,
                    mscale=rotary.mscale)

    def _rope(self, t, rotary):
        if rotary.freqs.dim() == 3:  # M-RoPE: per-token angles already mixed from the t/h/w streams
            return OF.rope(t, rotary.freqs[:, 0], rot_dim=self.rot_dim, interleaved=False, mscale=rotary.mscale)
        return OF.rope(t, rotary.freqs, **self._rope_kw(rotary))

    def _rope_packed(self, pk, rotary):
        f = rotary.freqs[:, 0] if rotary.freqs.dim() == 3 else rotary.freqs
        kw = self._rope_kw(rotary)
        if rotary.freqs.dim() == 3:
            kw.update(pos_ids=None, interleaved=False)
        return OF.rope(pk, f, group=self.r + 2, rope_in_group=self.r + 1, inplace=True, head_dim=self.d, **kw)


# Sequence-chunk pipelining (runtime/chunkpipe.py): while "active", every attention call sees the keys / values of
# the sequence's earlier chunks as a prefix ("past") and publishes its own keys / values ("out").
CHUNK_PREFIX = {"active": False, "past": None, "out": None}


def core_attention(q, k, v, *, causal, scale, cu_seqlens, cfg: Optional[TransformerConfig] = None,
                   row_length: Optional[int] = None, training: bool = False):
    """Attention over packed tokens; context parallelism is applied here when enabled."""
    st = ps.get_state()
    if CHUNK_PREFIX["active"]:
        assert cu_seqlens is None and st.dims.cp == 1, "chunk pipelining runs one unpacked sequence per micro-batch"
        past = CHUNK_PREFIX["past"]
        CHUNK_PREFIX["out"] = (k, v)
        kk, vv = (torch.cat([past[0], k]), torch.cat([past[1], v])) if past is not None else (k, v)
        # fewer queries than keys: the causal mask is aligned to the bottom right, i.e. the chunk follows its prefix
        return OF.attention(q, kk, vv, causal=causal, scale=scale)
    p_drop = cfg.attention_dropout if (cfg is not None and training) else 0.0
    if p_drop > 0:
        return _attention_with_dropout(q, k, v, causal, scale, cu_seqlens, p_drop, st)
    if st.dims.cp > 1:
        from ..parallel import context_parallel as CP
        return CP.ring_attention(q, k, v, causal=causal, scale=scale, cu_seqlens=cu_seqlens, row_length=row_length)
    return OF.attention(q, k, v, causal=causal, scale=scale, cu_seqlens=cu_seqlens)


def _attention_with_dropout(q, k, v, causal, scale, cu_seqlens, p_drop, st):
    """Attention-probability dropout (``--attention-dropout`` > 0). The flash kernels carry no dropout, so this path
    computes the probabilities in PyTorch; heads are sharded over the TP group, hence the masks come from the
    tracker's model-parallel stream. Context parallelism and this path exclude each other."""
    if st.dims.cp > 1:
        raise ValueError("attention dropout is not available together with context parallelism")
    from ..parallel import random as PR
    import contextlib

    Tq, Hq, _ = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    s = torch.einsum("qhd,khd->hqk", q.float(), k.float().repeat_interleave(rep, 1)) * scale
    seg, pos, _ = OF._seq_ids(Tq, cu_seqlens, q.device)
    mask = seg[:, None] == seg[None, :]
    if causal:
        mask &= pos[None, :] <= pos[:, None]
    pr = torch.softmax(s.masked_fill(~mask, float("-inf")), dim=-1)
    ctx = PR.get_rng_tracker().fork() if st.dims.tp > 1 else contextlib.nullcontext()
    with ctx:
        pr = torch.nn.functional.dropout(pr, p_drop, training=True)
    return torch.einsum("hqk,khd->qhd", pr, v.float().repeat_interleave(rep, 1)).to(q.dtype)


def hidden_dropout(t: torch.Tensor, p: float, cfg: TransformerConfig) -> torch.Tensor:
    """Dropout on a sub-layer output. With sequence parallelism every tensor-parallel rank holds different tokens, so
    the masks come from the tracker's model-parallel stream (different per TP rank); otherwise the activations are
    replicated over the TP group and the default stream, seeded alike on its ranks, keeps the masks identical
    (reference: loongforge/models/foundation/language_transformer_block.py:199-202, Megatron's bias-dropout-add)."""
    from ..parallel import random as PR

    if cfg.sequence_parallel and ps.get_state().dims.tp > 1:
        with PR.get_rng_tracker().fork():
            return torch.nn.functional.dropout(t, p, training=True)
    return torch.nn.functional.dropout(t, p, training=True)


class TransformerLayer(nn.Module):
    """Pre-norm decoder layer: x + Attn(LN(x)), then x + MLP(LN(x)). The residual adds are
    folded into the output-projection / FC2 epilogues."""

    def __init__(self, cfg: TransformerConfig, layer_number: int, *, device=None, parallel_state=None):
        super().__init__()
        self.cfg = cfg
        self.layer_number = layer_number  # 0-based global index
        key = f"decoder.layers.{layer_number}"
        self.is_moe = cfg.is_moe_layer(layer_number)
        if cfg.csa_compress_ratios is not None:
            from .csa import CompressedSparseAttention
            self.input_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.self_attention = CompressedSparseAttention(cfg, key + ".self_attention", layer_number, device=device,
                                                            parallel_state=parallel_state)
        elif cfg.multi_latent_attention:
            from .mla import MLASelfAttention
            self.input_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.self_attention = MLASelfAttention(cfg, key + ".self_attention", layer_number, device=device,
                                                   parallel_state=parallel_state)
        elif cfg.layer_type(layer_number) == "linear_attention":
            from .hybrid import GatedDeltaNet
            self.input_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.self_attention = GatedDeltaNet(cfg, key + ".self_attention", device=device,
                                                parallel_state=parallel_state)
        elif cfg.attention_output_gate:
            from .hybrid import GatedAttention
            self.input_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.self_attention = GatedAttention(cfg, key + ".self_attention", device=device,
                                                 parallel_state=parallel_state)
        else:
            self.input_layernorm = None
            self.self_attention = SelfAttention(cfg, key + ".self_attention", device=device,
                                                parallel_state=parallel_state)
        if self.is_moe:
            from .moe import MoELayer
            if cfg.moe_multi_type:
                from .ernie import MultiTypeMoELayer as MoELayer  # noqa: N811
            self.pre_mlp_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.mlp = MoELayer(cfg, key + ".mlp", layer_number, device=device, parallel_state=parallel_state)
        elif cfg.multi_latent_attention or cfg.csa_compress_ratios is not None:
            self.pre_mlp_layernorm = Norm(cfg.hidden_size, cfg, device=device, sequence_parallel=cfg.sequence_parallel)
            self.mlp = MLP(cfg, key + ".mlp", fused_norm=False, device=device, parallel_state=parallel_state)
        else:
            self.pre_mlp_layernorm = None
            self.mlp = MLP(cfg, key + ".mlp", device=device, parallel_state=parallel_state)
        if cfg.enable_hyper_connections:
            from .hyper_connections import HyperConnection
            assert self.input_layernorm is not None and self.pre_mlp_layernorm is not None, \
                "hyper-connections need the un-fused norm layout"
            hc = dict(n=cfg.num_residual_streams, sinkhorn_iters=cfg.mhc_sinkhorn_iterations,
                      gate_init=cfg.mhc_init_gating_factor, eps=cfg.layernorm_epsilon, device=device,
                      sequence_parallel=cfg.sequence_parallel)
            self.hc_attention = HyperConnection(cfg.hidden_size, key=key + ".hc_attention", **hc)
            self.hc_mlp = HyperConnection(cfg.hidden_size, key=key + ".hc_mlp", **hc)

    def _forward_hyper(self, xs, rotary, packed):
        """xs [T, n, C]: both sub-layers read one mixed vector and write back into all streams."""
        h, maps = self.hc_attention.read(xs)
        xs = self.hc_attention.write(xs, self.self_attention(self.input_layernorm(h), rotary, packed), maps)
        h, maps = self.hc_mlp.read(xs)
        return self.hc_mlp.write(xs, self.mlp(self.pre_mlp_layernorm(h)), maps)

    def forward(self, x, rotary=None, packed=None):
        if self.cfg.enable_hyper_connections:
            return self._forward_hyper(x, rotary, packed)
        drop = self.cfg.hidden_dropout if self.training else 0.0
        h = self.input_layernorm(x) if self.input_layernorm is not None else x
        if drop > 0:
            # dropout sits between the sub-layer and the residual add, so the add leaves the GEMM epilogue
            x = x + hidden_dropout(self.self_attention(h, rotary, packed, residual=None), drop, self.cfg)
        else:
            x = self.self_attention(h, rotary, packed, residual=x)
        h = self.pre_mlp_layernorm(x) if self.pre_mlp_layernorm is not None else x
        if drop > 0:
            return x + hidden_dropout(self.mlp(h), drop, self.cfg)
        if self.is_moe:
            return x + self.mlp(h)
        return self.mlp(h, residual=x)


class TransformerBlock(nn.Module):
    """The layers owned by this pipeline stage (+ final norm on the last stage), with
    full / uniform / block activation recomputation
    (loongforge/models/foundation/language_transformer_block.py:230-245,449-503)."""

    def __init__(self, cfg: TransformerConfig, layer_numbers, *, post_process: bool = True, device=None,
                 parallel_state=None):
        super().__init__()
        self.cfg = cfg
        self.layers = nn.ModuleList([TransformerLayer(cfg, n, device=device, parallel_state=parallel_state)
                                     for n in layer_numbers])
        self.layer_numbers = list(layer_numbers)
        if (cfg.use_dsa and cfg.dsa_indexer_topk_freq > 1 and self.layer_numbers
                and not cfg.dsa_computes_topk(self.layer_numbers[0])):
            raise ValueError(f"layer {self.layer_numbers[0]} reuses another layer's top-k indices (IndexShare): every "
                             "pipeline stage must start on a layer that computes them")
        self.final_layernorm = Norm(cfg.hidden_size, cfg, device=device,
                                    sequence_parallel=cfg.sequence_parallel) if post_process else None
        self.deepstack_hook = None  # callable(layer_idx, hidden) -> hidden, used by Qwen3-VL
        self.pre_process = True  # set False by pipeline stages that receive hidden states
        if cfg.enable_hyper_connections and post_process:
            from .hyper_connections import HyperHead
            self.head_hyper_connection = HyperHead(cfg.hidden_size, cfg.num_residual_streams,
                                                   cfg.mhc_init_gating_factor, cfg.layernorm_epsilon,
                                                   "decoder.head_hyper_connection", device=device,
                                                   sequence_parallel=cfg.sequence_parallel)

    def _run(self, layer, x, rotary, packed, shared_idx=None):
        if shared_idx is not None and hasattr(layer.self_attention, "shared_topk_indices"):
            layer.self_attention.shared_topk_indices = shared_idx  # IndexShare: top-k indices of the source layer
        return layer(x, rotary, packed)

    def forward(self, x, rotary=None, packed=None):
        cfg = self.cfg
        n = len(self.layers)
        rec = cfg.recompute_granularity == "full" and torch.is_grad_enabled()
        rec_n = cfg.recompute_num_layers if cfg.recompute_num_layers is not None else n
        method = cfg.recompute_method or "block"
        hyper = cfg.enable_hyper_connections
        if hyper:
            # streams travel between pipeline stages flattened as [T, n * C]; the first stage replicates the embedding
            ns = cfg.num_residual_streams
            x = x.unsqueeze(1).expand(-1, ns, -1).contiguous() if x.shape[-1] == cfg.hidden_size else \
                x.view(x.shape[0], ns, cfg.hidden_size)
        share = cfg.use_dsa and cfg.dsa_indexer_topk_freq > 1
        shared_idx = None
        for i, layer in enumerate(self.layers):
            do_rec = rec and ((method == "block" and i < rec_n) or method == "uniform")
            if do_rec and self.training and (cfg.hidden_dropout > 0 or cfg.attention_dropout > 0):
                # dropout inside: the recomputation must replay the default AND the tracked random streams
                from ..parallel import random as PR
                x = PR.checkpoint(lambda t, _l=layer, _s=shared_idx: self._run(_l, t, rotary, packed, _s), x)
            elif do_rec:
                # the shared top-k indices are an explicit input, so a recomputed layer sees those of ITS forward
                x = torch.utils.checkpoint.checkpoint(self._run, layer, x, rotary, packed, shared_idx, use_reentrant=False)
            else:
                x = self._run(layer, x, rotary, packed, shared_idx)
            if share:
                shared_idx = getattr(layer.self_attention, "last_topk_indices", shared_idx)
            if self.deepstack_hook is not None:
                x = self.deepstack_hook(self.layer_numbers[i], x)
        if hyper:
            x = self.head_hyper_connection(x) if self.final_layernorm is not None else x.reshape(x.shape[0], -1)
        if self.final_layernorm is not None:
            x = self.final_layernorm(x)
        return x
