"""Hugging Face <-> Megatron-core parameter mapping for decoder-only language models.

The reference drives its converter with per-family YAML name maps
(configs/models/*/ckpt_convert/*.yaml; e.g. llama3_convert.yaml:17-70) and a two-step pipeline
HF -> "common" -> mcore (tools/convert_checkpoint/module_convertor/model.py:250-383). Here the common
form is simply the UNSHARDED Megatron state dict; one table describes a family:

  * plain renames (embedding, norms, proj, fc2, router, lm head),
  * packed QKV: per KV group rows ``[q_0 .. q_{r-1}, k, v]`` (hf_attn_converter.py:62-78),
  * SwiGLU FC1 = ``cat([gate, up])`` (huggingface_base.py:495-524),
  * MoE experts as ``experts.linear_fc{1,2}.weight{e}`` (mcore_moe.py:60-74).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional

import torch


@dataclasses.dataclass
class FamilyMap:
    name: str
    qkv_bias: bool = False
    qk_norm: bool = False
    moe: bool = False
    hf_prefix: str = "model."
    hf_layers: str = "model.layers.{i}."
    expert_tpl: str = "mlp.experts.{e}."
    router: str = "mlp.gate.weight"
    shared_expert: Optional[str] = None  # e.g. "mlp.shared_experts."
    mla: bool = False  # DeepSeek-style multi-latent attention (+ optional DSA indexer, router bias, MTP layers)
    # families whose Hugging Face files spell the same tensors differently: (theirs, canonical) substring pairs applied
    # to the part of a key after the layer prefix, and (theirs, canonical) prefixes for the keys outside the layers
    layer_alias: tuple = ()
    top_alias: tuple = ()
    hybrid: bool = False  # Qwen3-Next / Qwen3.5: GatedDeltaNet layers + gated full attention, gated shared expert
    packed_qkv: Optional[str] = None  # HF key suffix of an already packed per-group [q.., k, v] projection
    # multi-token-prediction layers of the non-MLA families: HF prefix and the names of the four extra tensors
    mtp_layers: Optional[str] = None  # e.g. "model.mtp_layers.{i}."
    mtp_names: tuple = (("enorm.weight", "enorm.weight"), ("hnorm.weight", "hnorm.weight"),
                        ("eh_proj.weight", "eh_proj.weight"), ("final_layernorm.weight", "shared_head.norm.weight"))


FAMILIES: Dict[str, FamilyMap] = {
    "llama": FamilyMap("llama"),
    "llama2": FamilyMap("llama2"),
    "llama3": FamilyMap("llama3"),
    "qwen2": FamilyMap("qwen2", qkv_bias=True),
    "qwen2.5": FamilyMap("qwen2.5", qkv_bias=True),
    "qwen3": FamilyMap("qwen3", qk_norm=True),
    "qwen3_moe": FamilyMap("qwen3_moe", qk_norm=True, moe=True),
    # DeepSeek-V2 / V3 / V3.2 and GLM-5.x share one layout: MLA projections, optional lightning indexer, dense-then-MoE
    # layers with a shared expert and a router bias, multi-token-prediction layers appended after the last layer
    "deepseek": FamilyMap("deepseek", moe=True, mla=True, shared_expert="mlp.shared_experts."),
    "glm": FamilyMap("glm", moe=True, mla=True, shared_expert="mlp.shared_experts."),
    # (configs/models/qwen3_next/ckpt_convert/qwen3_next_moe_convert.yaml:17-100)
    "qwen3_next": FamilyMap("qwen3_next", qk_norm=True, moe=True, hybrid=True, shared_expert="mlp.shared_expert."),
    "qwen3_5": FamilyMap("qwen3_5", qk_norm=True, moe=True, hybrid=True, shared_expert="mlp.shared_expert."),
    "kimi_k2": FamilyMap("kimi_k2", moe=True, mla=True, shared_expert="mlp.shared_experts."),
    # InternLM2 / 2.5: packed wqkv, w1/w3/w2 feed-forward (configs/models/internlm2.5/ckpt_convert/internlm2_5_convert.yaml)
    "internlm2": FamilyMap("internlm2", packed_qkv="self_attn.wqkv.weight",
                           layer_alias=(("attention.wqkv.", "self_attn.wqkv."), ("attention.wo.", "self_attn.o_proj."),
                                        ("feed_forward.w1.", "mlp.gate_proj."), ("feed_forward.w3.", "mlp.up_proj."),
                                        ("feed_forward.w2.", "mlp.down_proj."), ("attention_norm.", "input_layernorm."),
                                        ("ffn_norm.", "post_attention_layernorm.")),
                           top_alias=(("model.tok_embeddings.", "model.embed_tokens."), ("output.", "lm_head."))),
    # MiniMax-M2: block_sparse_moe with w1/w3/w2 experts, router bias, q/k norms
    # (configs/models/minimax/ckpt_convert/minimax_convert.yaml)
    "minimax": FamilyMap("minimax", qk_norm=True, moe=True,
                         layer_alias=(("block_sparse_moe.experts.", "mlp.experts."), (".w1.", ".gate_proj."),
                                      (".w3.", ".up_proj."), (".w2.", ".down_proj."),
                                      ("block_sparse_moe.gate.", "mlp.gate."),
                                      ("block_sparse_moe.e_score_correction_bias", "mlp.gate.e_score_correction_bias"))),
    # MiMo: Qwen2-style layers plus multi-token-prediction layers under model.mtp_layers
    # (configs/models/mimo/ckpt_convert/mimo_convert.yaml)
    "mimo": FamilyMap("mimo", qkv_bias=True, mtp_layers="model.mtp_layers.{i}.",
                      mtp_names=(("enorm.weight", "token_layernorm.weight"), ("hnorm.weight", "hidden_layernorm.weight"),
                                 ("eh_proj.weight", "input_proj.weight"),
                                 ("final_layernorm.weight", "final_layernorm.weight"))),
}


# vision-language compositions: name -> family of their language model
# the InternLM presets of this package use family "internlm"; MiniMax / Kimi checkpoints share their families' maps
FAMILIES["internlm"] = FAMILIES["internlm2.5"] = FAMILIES["internlm2"]
FAMILIES["kimi"] = FAMILIES["kimi_k2"]

VLM_FAMILIES: Dict[str, str] = {"qwen2_vl": "qwen2", "qwen2_5_vl": "qwen2.5", "qwen2.5_vl": "qwen2.5"}


def pack_qkv(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, num_groups: int) -> torch.Tensor:
    """[nq*d, ...], [ng*d, ...], [ng*d, ...] -> Megatron packed [(nq + 2 ng) * d, ...] per-group order."""
    tail = q.shape[1:]
    d = k.shape[0] // num_groups
    r = q.shape[0] // k.shape[0]
    qg = q.reshape(num_groups, r * d, *tail)
    kg = k.reshape(num_groups, d, *tail)
    vg = v.reshape(num_groups, d, *tail)
    return torch.cat([qg, kg, vg], dim=1).reshape(-1, *tail)


def unpack_qkv(w: torch.Tensor, num_heads: int, num_groups: int):
    tail = w.shape[1:]
    d = w.shape[0] // (num_heads + 2 * num_groups)
    r = num_heads // num_groups
    g = w.reshape(num_groups, (r + 2) * d, *tail)
    q = g[:, : r * d].reshape(-1, *tail)
    k = g[:, r * d:(r + 1) * d].reshape(-1, *tail)
    v = g[:, (r + 1) * d:].reshape(-1, *tail)
    return q.contiguous(), k.contiguous(), v.contiguous()


def pad_vocab(w: torch.Tensor, padded: int) -> torch.Tensor:
    """Pad the vocabulary dimension by repeating the last row (tools/convert_checkpoint/utils/utils.py:71-98)."""
    if w.shape[0] >= padded:
        return w
    return torch.cat([w, w[-1:].expand(padded - w.shape[0], -1)], 0).contiguous()


# (Megatron suffix, Hugging Face suffix) inside one MLA layer; entries absent from a checkpoint are skipped
_MLA_LAYER = [
    ("input_layernorm.weight", "input_layernorm.weight"),
    ("self_attention.linear_q_proj.weight", "self_attn.q_proj.weight"),
    ("self_attention.linear_q_down_proj.weight", "self_attn.q_a_proj.weight"),
    ("self_attention.q_layernorm.weight", "self_attn.q_a_layernorm.weight"),
    ("self_attention.linear_q_up_proj.weight", "self_attn.q_b_proj.weight"),
    ("self_attention.linear_kv_down_proj.weight", "self_attn.kv_a_proj_with_mqa.weight"),
    ("self_attention.kv_layernorm.weight", "self_attn.kv_a_layernorm.weight"),
    ("self_attention.linear_kv_up_proj.weight", "self_attn.kv_b_proj.weight"),
    ("self_attention.linear_proj.weight", "self_attn.o_proj.weight"),
    ("self_attention.core_attention.indexer.linear_wq_b.weight", "self_attn.indexer.wq_b.weight"),
    ("self_attention.core_attention.indexer.linear_wk.weight", "self_attn.indexer.wk.weight"),
    ("self_attention.core_attention.indexer.k_norm.weight", "self_attn.indexer.k_norm.weight"),
    ("self_attention.core_attention.indexer.k_norm.bias", "self_attn.indexer.k_norm.bias"),
    ("self_attention.core_attention.indexer.linear_weights_proj.weight", "self_attn.indexer.weights_proj.weight"),
    ("pre_mlp_layernorm.weight", "post_attention_layernorm.weight"),
    ("mlp.router.weight", "mlp.gate.weight"),
    ("mlp.router.expert_bias", "mlp.gate.e_score_correction_bias"),
]
_MTP_EXTRA = [("enorm.weight", "enorm.weight"), ("hnorm.weight", "hnorm.weight"), ("eh_proj.weight", "eh_proj.weight"),
              ("final_layernorm.weight", "shared_head.norm.weight")]


def _mla_layer_to_mcore(hf, h: str, m: str, out, fam: FamilyMap, num_experts) -> None:
    for mk, hk in _MLA_LAYER:
        if h + hk in hf:
            out[m + mk] = hf[h + hk]
    glu = lambda p: torch.cat([hf[p + "gate_proj.weight"], hf[p + "up_proj.weight"]], 0)  # noqa: E731
    if h + "mlp.gate.weight" in hf:
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            out[m + f"mlp.experts.linear_fc1.weight{e}"] = glu(p)
            out[m + f"mlp.experts.linear_fc2.weight{e}"] = hf[p + "down_proj.weight"]
        if fam.shared_expert and h + fam.shared_expert + "gate_proj.weight" in hf:
            out[m + "mlp.shared_experts.linear_fc1.weight"] = glu(h + fam.shared_expert)
            out[m + "mlp.shared_experts.linear_fc2.weight"] = hf[h + fam.shared_expert + "down_proj.weight"]
    else:
        out[m + "mlp.linear_fc1.weight"] = glu(h + "mlp.")
        out[m + "mlp.linear_fc2.weight"] = hf[h + "mlp.down_proj.weight"]


def _mla_layer_to_hf(mc, m: str, h: str, out, fam: FamilyMap, num_experts) -> None:
    for mk, hk in _MLA_LAYER:
        if m + mk in mc:
            out[h + hk] = mc[m + mk]

    def unglu(w, p):
        g, u = w.chunk(2, 0)
        out[p + "gate_proj.weight"], out[p + "up_proj.weight"] = g.contiguous(), u.contiguous()

    if m + "mlp.router.weight" in mc:
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            unglu(mc[m + f"mlp.experts.linear_fc1.weight{e}"], p)
            out[p + "down_proj.weight"] = mc[m + f"mlp.experts.linear_fc2.weight{e}"]
        if m + "mlp.shared_experts.linear_fc1.weight" in mc:
            unglu(mc[m + "mlp.shared_experts.linear_fc1.weight"], h + fam.shared_expert)
            out[h + fam.shared_expert + "down_proj.weight"] = mc[m + "mlp.shared_experts.linear_fc2.weight"]
    else:
        unglu(mc[m + "mlp.linear_fc1.weight"], h + "mlp.")
        out[h + "mlp.down_proj.weight"] = mc[m + "mlp.linear_fc2.weight"]


def _mla_to_mcore(hf, fam, num_layers, padded_vocab, num_experts, tie_embeddings):
    """Multi-token-prediction layers follow the decoder in the Hugging Face file as layers L, L+1, ... (with their own
    copies of the embedding and the head, which the Megatron side shares with the main model)."""
    out: Dict[str, torch.Tensor] = {}
    emb = hf[fam.hf_prefix + "embed_tokens.weight"]
    out["embedding.word_embeddings.weight"] = pad_vocab(emb, padded_vocab or emb.shape[0])
    for i in range(num_layers):
        _mla_layer_to_mcore(hf, fam.hf_layers.format(i=i), f"decoder.layers.{i}.", out, fam, num_experts)
    k = 0
    while fam.hf_layers.format(i=num_layers + k) + "eh_proj.weight" in hf:
        h, m = fam.hf_layers.format(i=num_layers + k), f"mtp.layers.{k}."
        for mk, hk in _MTP_EXTRA:
            out[m + mk] = hf[h + hk]
        _mla_layer_to_mcore(hf, h, m + "transformer_layer.", out, fam, num_experts)
        k += 1
    out["decoder.final_layernorm.weight"] = hf[fam.hf_prefix + "norm.weight"]
    if not tie_embeddings:
        head = hf.get("lm_head.weight", emb)
        out["output_layer.weight"] = pad_vocab(head, padded_vocab or head.shape[0])
    return out


def _mla_to_hf(mc, fam, num_layers, vocab_size, num_experts, tie_embeddings):
    out: Dict[str, torch.Tensor] = {}
    strip = lambda w: w[:vocab_size].contiguous() if vocab_size else w  # noqa: E731
    emb = strip(mc["embedding.word_embeddings.weight"])
    out[fam.hf_prefix + "embed_tokens.weight"] = emb
    for i in range(num_layers):
        _mla_layer_to_hf(mc, f"decoder.layers.{i}.", fam.hf_layers.format(i=i), out, fam, num_experts)
    head = strip(mc["output_layer.weight"]) if (not tie_embeddings and "output_layer.weight" in mc) else emb
    k = 0
    while f"mtp.layers.{k}.eh_proj.weight" in mc:
        m, h = f"mtp.layers.{k}.", fam.hf_layers.format(i=num_layers + k)
        for mk, hk in _MTP_EXTRA:
            out[h + hk] = mc[m + mk]
        _mla_layer_to_hf(mc, m + "transformer_layer.", h, out, fam, num_experts)
        # separate copies: the Hugging Face file stores the MTP layer's embedding and head as tensors of their own
        out[h + "embed_tokens.weight"], out[h + "shared_head.head.weight"] = emb.clone(), head.clone()
        k += 1
    out[fam.hf_prefix + "norm.weight"] = mc["decoder.final_layernorm.weight"]
    if not tie_embeddings and "output_layer.weight" in mc:
        out["lm_head.weight"] = head
    return out


def _layer_keys(fam: FamilyMap, num_layers: int, mtp: int = 8):
    """Layer prefixes of a family (decoder layers, then whatever MTP prefixes it uses)."""
    pre = [fam.hf_layers.format(i=i) for i in range(num_layers + (mtp if fam.mla else 0))]
    if fam.mtp_layers:
        pre += [fam.mtp_layers.format(i=i) for i in range(mtp)]
    return pre


def _rename(keys_in: Dict[str, torch.Tensor], fam: FamilyMap, num_layers: int, to_canonical: bool):
    """Family spelling <-> canonical (Llama-style) spelling of the Hugging Face keys."""
    if not fam.layer_alias and not fam.top_alias:
        return keys_in
    layer = [(a, b) if to_canonical else (b, a) for a, b in fam.layer_alias]
    top = [(a, b) if to_canonical else (b, a) for a, b in fam.top_alias]
    if not to_canonical:
        layer.reverse()
    prefixes = _layer_keys(fam, num_layers)
    out = {}
    for k, v in keys_in.items():
        pre = next((p for p in prefixes if k.startswith(p)), None)
        if pre is not None:
            tail = k[len(pre):]
            for a, b in layer:
                tail = tail.replace(a, b)
            out[pre + tail] = v
            continue
        for a, b in top:
            if k.startswith(a):
                k = b + k[len(a):]
                break
        out[k] = v
    return out


def _std_layer_to_mcore(hf, h: str, m: str, out, fam: FamilyMap, num_groups: int, num_experts) -> None:
    out[m + "self_attention.linear_qkv.layer_norm_weight"] = hf[h + "input_layernorm.weight"]
    if fam.packed_qkv:
        out[m + "self_attention.linear_qkv.weight"] = hf[h + fam.packed_qkv]  # already [q.., k, v] per group
    else:
        out[m + "self_attention.linear_qkv.weight"] = pack_qkv(hf[h + "self_attn.q_proj.weight"],
                                                               hf[h + "self_attn.k_proj.weight"],
                                                               hf[h + "self_attn.v_proj.weight"], num_groups)
    if fam.qkv_bias:
        out[m + "self_attention.linear_qkv.bias"] = pack_qkv(hf[h + "self_attn.q_proj.bias"],
                                                             hf[h + "self_attn.k_proj.bias"],
                                                             hf[h + "self_attn.v_proj.bias"], num_groups)
    if fam.qk_norm:
        out[m + "self_attention.q_layernorm.weight"] = hf[h + "self_attn.q_norm.weight"]
        out[m + "self_attention.k_layernorm.weight"] = hf[h + "self_attn.k_norm.weight"]
    out[m + "self_attention.linear_proj.weight"] = hf[h + "self_attn.o_proj.weight"]
    post = hf[h + "post_attention_layernorm.weight"]
    if fam.moe and (h + fam.router) in hf:
        out[m + "pre_mlp_layernorm.weight"] = post
        out[m + "mlp.router.weight"] = hf[h + fam.router]
        if h + "mlp.gate.e_score_correction_bias" in hf:
            out[m + "mlp.router.expert_bias"] = hf[h + "mlp.gate.e_score_correction_bias"]
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            out[m + f"mlp.experts.linear_fc1.weight{e}"] = torch.cat([hf[p + "gate_proj.weight"],
                                                                      hf[p + "up_proj.weight"]], 0)
            out[m + f"mlp.experts.linear_fc2.weight{e}"] = hf[p + "down_proj.weight"]
    else:
        out[m + "mlp.linear_fc1.layer_norm_weight"] = post
        out[m + "mlp.linear_fc1.weight"] = torch.cat([hf[h + "mlp.gate_proj.weight"], hf[h + "mlp.up_proj.weight"]], 0)
        out[m + "mlp.linear_fc2.weight"] = hf[h + "mlp.down_proj.weight"]


def _std_layer_to_hf(mc, m: str, h: str, out, fam: FamilyMap, num_heads: int, num_groups: int, num_experts) -> None:
    out[h + "input_layernorm.weight"] = mc[m + "self_attention.linear_qkv.layer_norm_weight"]
    if fam.packed_qkv:
        out[h + fam.packed_qkv] = mc[m + "self_attention.linear_qkv.weight"]
    else:
        q, k, v = unpack_qkv(mc[m + "self_attention.linear_qkv.weight"], num_heads, num_groups)
        out[h + "self_attn.q_proj.weight"], out[h + "self_attn.k_proj.weight"], out[h + "self_attn.v_proj.weight"] = q, k, v
    if fam.qkv_bias:
        qb, kb, vb = unpack_qkv(mc[m + "self_attention.linear_qkv.bias"], num_heads, num_groups)
        out[h + "self_attn.q_proj.bias"], out[h + "self_attn.k_proj.bias"], out[h + "self_attn.v_proj.bias"] = qb, kb, vb
    if fam.qk_norm:
        out[h + "self_attn.q_norm.weight"] = mc[m + "self_attention.q_layernorm.weight"]
        out[h + "self_attn.k_norm.weight"] = mc[m + "self_attention.k_layernorm.weight"]
    out[h + "self_attn.o_proj.weight"] = mc[m + "self_attention.linear_proj.weight"]
    if (m + "mlp.router.weight") in mc:
        out[h + "post_attention_layernorm.weight"] = mc[m + "pre_mlp_layernorm.weight"]
        out[h + fam.router] = mc[m + "mlp.router.weight"]
        if m + "mlp.router.expert_bias" in mc:
            out[h + "mlp.gate.e_score_correction_bias"] = mc[m + "mlp.router.expert_bias"]
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            g, u = mc[m + f"mlp.experts.linear_fc1.weight{e}"].chunk(2, 0)
            out[p + "gate_proj.weight"], out[p + "up_proj.weight"] = g.contiguous(), u.contiguous()
            out[p + "down_proj.weight"] = mc[m + f"mlp.experts.linear_fc2.weight{e}"]
    else:
        out[h + "post_attention_layernorm.weight"] = mc[m + "mlp.linear_fc1.layer_norm_weight"]
        g, u = mc[m + "mlp.linear_fc1.weight"].chunk(2, 0)
        out[h + "mlp.gate_proj.weight"], out[h + "mlp.up_proj.weight"] = g.contiguous(), u.contiguous()
        out[h + "mlp.down_proj.weight"] = mc[m + "mlp.linear_fc2.weight"]


# ---- Qwen3-Next / Qwen3.5 hybrid layers ----------------------------------------------------------
_GDN = [("self_attention.in_proj_qkvz.weight", "linear_attn.in_proj_qkvz.weight"),
        ("self_attention.in_proj_ba.weight", "linear_attn.in_proj_ba.weight"),
        ("self_attention.dt_bias", "linear_attn.dt_bias"), ("self_attention.A_log", "linear_attn.A_log"),
        ("self_attention.out_norm.weight", "linear_attn.norm.weight"),
        ("self_attention.out_proj.weight", "linear_attn.out_proj.weight")]


def _pack_qgkv(qg, k, v, num_heads: int, num_groups: int):
    """HF ``q_proj`` rows are per head ``[q_h; gate_h]``; the packed projection holds per KV group
    ``[q heads | gate heads | k | v]`` so that a tensor-parallel shard keeps whole groups."""
    d = k.shape[0] // num_groups
    r = num_heads // num_groups
    tail = qg.shape[1:]
    qg = qg.reshape(num_groups, r, 2, d, *tail)
    q, g = qg[:, :, 0].reshape(num_groups, r * d, *tail), qg[:, :, 1].reshape(num_groups, r * d, *tail)
    return torch.cat([q, g, k.reshape(num_groups, d, *tail), v.reshape(num_groups, d, *tail)], 1).reshape(-1, *tail)


def _unpack_qgkv(w, num_heads: int, num_groups: int):
    r = num_heads // num_groups
    d = w.shape[0] // (num_groups * (2 * r + 2))
    tail = w.shape[1:]
    y = w.reshape(num_groups, 2 * r + 2, d, *tail)
    q, g = y[:, :r], y[:, r:2 * r]
    qg = torch.stack([q, g], 2).reshape(num_heads * 2 * d, *tail)
    return qg.contiguous(), y[:, 2 * r].reshape(-1, *tail).contiguous(), y[:, 2 * r + 1].reshape(-1, *tail).contiguous()


def _hybrid_mlp_to_mcore(hf, h, m, out, fam, num_experts):
    glu = lambda p: torch.cat([hf[p + "gate_proj.weight"], hf[p + "up_proj.weight"]], 0)  # noqa: E731
    out[m + "pre_mlp_layernorm.weight"] = hf[h + "post_attention_layernorm.weight"]
    if h + fam.router in hf:
        out[m + "mlp.router.weight"] = hf[h + fam.router]
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            out[m + f"mlp.experts.linear_fc1.weight{e}"] = glu(p)
            out[m + f"mlp.experts.linear_fc2.weight{e}"] = hf[p + "down_proj.weight"]
        if h + fam.shared_expert + "gate_proj.weight" in hf:
            out[m + "mlp.shared_experts.linear_fc1.weight"] = glu(h + fam.shared_expert)
            out[m + "mlp.shared_experts.linear_fc2.weight"] = hf[h + fam.shared_expert + "down_proj.weight"]
        if h + "mlp.shared_expert_gate.weight" in hf:
            out[m + "mlp.shared_experts.gate_weight"] = hf[h + "mlp.shared_expert_gate.weight"]
    else:
        out[m + "mlp.linear_fc1.weight"] = glu(h + "mlp.")
        out[m + "mlp.linear_fc2.weight"] = hf[h + "mlp.down_proj.weight"]


def _hybrid_mlp_to_hf(mc, m, h, out, fam, num_experts):
    def unglu(w, p):
        g, u = w.chunk(2, 0)
        out[p + "gate_proj.weight"], out[p + "up_proj.weight"] = g.contiguous(), u.contiguous()

    out[h + "post_attention_layernorm.weight"] = mc[m + "pre_mlp_layernorm.weight"]
    if m + "mlp.router.weight" in mc:
        out[h + fam.router] = mc[m + "mlp.router.weight"]
        for e in range(num_experts):
            p = h + fam.expert_tpl.format(e=e)
            unglu(mc[m + f"mlp.experts.linear_fc1.weight{e}"], p)
            out[p + "down_proj.weight"] = mc[m + f"mlp.experts.linear_fc2.weight{e}"]
        if m + "mlp.shared_experts.linear_fc1.weight" in mc:
            unglu(mc[m + "mlp.shared_experts.linear_fc1.weight"], h + fam.shared_expert)
            out[h + fam.shared_expert + "down_proj.weight"] = mc[m + "mlp.shared_experts.linear_fc2.weight"]
        if m + "mlp.shared_experts.gate_weight" in mc:
            out[h + "mlp.shared_expert_gate.weight"] = mc[m + "mlp.shared_experts.gate_weight"]
    else:
        unglu(mc[m + "mlp.linear_fc1.weight"], h + "mlp.")
        out[h + "mlp.down_proj.weight"] = mc[m + "mlp.linear_fc2.weight"]


# Qwen3-Next keeps its multi-token-prediction block under ``mtp.``: four tensors without a layer index, then the layers
# (qwen3_next_moe_convert.yaml:73-88)
_HYBRID_MTP = [("enorm.weight", "mtp.pre_fc_norm_embedding.weight"), ("hnorm.weight", "mtp.pre_fc_norm_hidden.weight"),
               ("eh_proj.weight", "mtp.fc.weight"), ("final_layernorm.weight", "mtp.norm.weight")]


def _hybrid_layer_to_mcore(hf, h, m, out, fam, num_heads, num_groups, num_experts):
    out[m + "input_layernorm.weight"] = hf[h + "input_layernorm.weight"]
    if h + "linear_attn.A_log" in hf:
        for mk, hk in _GDN:
            out[m + mk] = hf[h + hk]
        out[m + "self_attention.conv_weight"] = hf[h + "linear_attn.conv1d.weight"].squeeze(1)  # [C, 1, K] -> [C, K]
    else:
        out[m + "self_attention.linear_qgkv.weight"] = _pack_qgkv(
            hf[h + "self_attn.q_proj.weight"], hf[h + "self_attn.k_proj.weight"], hf[h + "self_attn.v_proj.weight"],
            num_heads, num_groups)
        out[m + "self_attention.q_layernorm.weight"] = hf[h + "self_attn.q_norm.weight"]
        out[m + "self_attention.k_layernorm.weight"] = hf[h + "self_attn.k_norm.weight"]
        out[m + "self_attention.linear_proj.weight"] = hf[h + "self_attn.o_proj.weight"]
    _hybrid_mlp_to_mcore(hf, h, m, out, fam, num_experts)


def _hybrid_layer_to_hf(mc, m, h, out, fam, num_heads, num_groups, num_experts):
    out[h + "input_layernorm.weight"] = mc[m + "input_layernorm.weight"]
    if m + "self_attention.A_log" in mc:
        for mk, hk in _GDN:
            out[h + hk] = mc[m + mk]
        out[h + "linear_attn.conv1d.weight"] = mc[m + "self_attention.conv_weight"].unsqueeze(1)
    else:
        qg, k, v = _unpack_qgkv(mc[m + "self_attention.linear_qgkv.weight"], num_heads, num_groups)
        out[h + "self_attn.q_proj.weight"], out[h + "self_attn.k_proj.weight"], out[h + "self_attn.v_proj.weight"] = qg, k, v
        out[h + "self_attn.q_norm.weight"] = mc[m + "self_attention.q_layernorm.weight"]
        out[h + "self_attn.k_norm.weight"] = mc[m + "self_attention.k_layernorm.weight"]
        out[h + "self_attn.o_proj.weight"] = mc[m + "self_attention.linear_proj.weight"]
    _hybrid_mlp_to_hf(mc, m, h, out, fam, num_experts)


def _hybrid_to_mcore(hf, fam, num_layers, num_heads, num_groups, padded_vocab, num_experts, tie_embeddings):
    out: Dict[str, torch.Tensor] = {}
    emb = hf[fam.hf_prefix + "embed_tokens.weight"]
    out["embedding.word_embeddings.weight"] = pad_vocab(emb, padded_vocab or emb.shape[0])
    args = (fam, num_heads, num_groups, num_experts)
    for i in range(num_layers):
        _hybrid_layer_to_mcore(hf, fam.hf_layers.format(i=i), f"decoder.layers.{i}.", out, *args)
    if "mtp.fc.weight" in hf:  # one set of the four extra tensors; the layers follow under mtp.layers.{k}.
        for mk, hk in _HYBRID_MTP:
            out["mtp.layers.0." + mk] = hf[hk]
        k = 0
        while f"mtp.layers.{k}.input_layernorm.weight" in hf:
            _hybrid_layer_to_mcore(hf, f"mtp.layers.{k}.", f"mtp.layers.{k}.transformer_layer.", out, *args)
            k += 1
    out["decoder.final_layernorm.weight"] = hf[fam.hf_prefix + "norm.weight"]
    if not tie_embeddings:
        head = hf.get("lm_head.weight", emb)
        out["output_layer.weight"] = pad_vocab(head, padded_vocab or head.shape[0])
    return out


def _hybrid_to_hf(mc, fam, num_layers, num_heads, num_groups, vocab_size, num_experts, tie_embeddings):
    out: Dict[str, torch.Tensor] = {}
    strip = lambda w: w[:vocab_size].contiguous() if vocab_size else w  # noqa: E731
    out[fam.hf_prefix + "embed_tokens.weight"] = strip(mc["embedding.word_embeddings.weight"])
    args = (fam, num_heads, num_groups, num_experts)
    for i in range(num_layers):
        _hybrid_layer_to_hf(mc, f"decoder.layers.{i}.", fam.hf_layers.format(i=i), out, *args)
    if "mtp.layers.0.eh_proj.weight" in mc:
        if "mtp.layers.1.eh_proj.weight" in mc:
            raise NotImplementedError("the Hugging Face layout of this family holds one multi-token-prediction block")
        for mk, hk in _HYBRID_MTP:
            out[hk] = mc["mtp.layers.0." + mk]
        _hybrid_layer_to_hf(mc, "mtp.layers.0.transformer_layer.", "mtp.layers.0.", out, *args)
    out[fam.hf_prefix + "norm.weight"] = mc["decoder.final_layernorm.weight"]
    if not tie_embeddings and "output_layer.weight" in mc:
        out["lm_head.weight"] = strip(mc["output_layer.weight"])
    return out


def hf_to_mcore(hf: Dict[str, torch.Tensor], fam: FamilyMap, *, num_layers: int, num_heads: int, num_groups: int,
                padded_vocab: Optional[int] = None, num_experts: Optional[int] = None,
                tie_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    hf = _rename(hf, fam, num_layers, True)
    if fam.hybrid:
        return _hybrid_to_mcore(hf, fam, num_layers, num_heads, num_groups, padded_vocab, num_experts, tie_embeddings)
    if fam.mla:
        return _mla_to_mcore(hf, fam, num_layers, padded_vocab, num_experts, tie_embeddings)
    out: Dict[str, torch.Tensor] = {}
    emb = hf[fam.hf_prefix + "embed_tokens.weight"]
    out["embedding.word_embeddings.weight"] = pad_vocab(emb, padded_vocab or emb.shape[0])
    for i in range(num_layers):
        _std_layer_to_mcore(hf, fam.hf_layers.format(i=i), f"decoder.layers.{i}.", out, fam, num_groups, num_experts)
    k = 0
    while fam.mtp_layers and fam.mtp_layers.format(i=k) + fam.mtp_names[2][1] in hf:
        h, m = fam.mtp_layers.format(i=k), f"mtp.layers.{k}."
        for mk, hk in fam.mtp_names:
            out[m + mk] = hf[h + hk]
        _std_layer_to_mcore(hf, h, m + "transformer_layer.", out, fam, num_groups, num_experts)
        k += 1
    out["decoder.final_layernorm.weight"] = hf[fam.hf_prefix + "norm.weight"]
    if not tie_embeddings:
        head = hf.get("lm_head.weight", emb)
        out["output_layer.weight"] = pad_vocab(head, padded_vocab or head.shape[0])
    return out


def mcore_to_hf(mc: Dict[str, torch.Tensor], fam: FamilyMap, *, num_layers: int, num_heads: int, num_groups: int,
                vocab_size: Optional[int] = None, num_experts: Optional[int] = None,
                tie_embeddings: bool = False) -> Dict[str, torch.Tensor]:
    if fam.hybrid:
        return _hybrid_to_hf(mc, fam, num_layers, num_heads, num_groups, vocab_size, num_experts, tie_embeddings)
    if fam.mla:
        return _rename(_mla_to_hf(mc, fam, num_layers, vocab_size, num_experts, tie_embeddings), fam, num_layers, False)
    out: Dict[str, torch.Tensor] = {}

    def strip(w):
        return w[:vocab_size].contiguous() if vocab_size else w

    out[fam.hf_prefix + "embed_tokens.weight"] = strip(mc["embedding.word_embeddings.weight"])
    for i in range(num_layers):
        _std_layer_to_hf(mc, f"decoder.layers.{i}.", fam.hf_layers.format(i=i), out, fam, num_heads, num_groups,
                         num_experts)
    k = 0
    while fam.mtp_layers and f"mtp.layers.{k}.eh_proj.weight" in mc:
        m, h = f"mtp.layers.{k}.", fam.mtp_layers.format(i=k)
        for mk, hk in fam.mtp_names:
            out[h + hk] = mc[m + mk]
        _std_layer_to_hf(mc, m + "transformer_layer.", h, out, fam, num_heads, num_groups, num_experts)
        k += 1
    out[fam.hf_prefix + "norm.weight"] = mc["decoder.final_layernorm.weight"]
    if not tie_embeddings and "output_layer.weight" in mc:
        out["lm_head.weight"] = strip(mc["output_layer.weight"])
    return _rename(out, fam, num_layers, False)


# ---- tensor / pipeline / expert sharding of the unsharded Megatron dict -----------------------
def tp_rule(key: str):
    """(partition_dim, stride) of a Megatron key, or None when replicated."""
    if key.endswith(("linear_qkv.weight", "linear_qkv.bias", "embedding.word_embeddings.weight", "output_layer.weight",
                     "self_attention.linear_q_proj.weight", "self_attention.linear_q_up_proj.weight",
                     "self_attention.linear_kv_up_proj.weight", "eh_proj.weight")):
        return 0, 1
    if key.endswith(("linear_fc1.weight", "linear_fc1.bias")) and ".experts." not in key:
        return 0, (1 if "image_projector." in key else 2)  # the projector's first linear is not gated
    if key.endswith(("linear_proj.weight", "linear_fc2.weight", "self_attention.out_proj.weight")) and ".experts." not in key:
        return 1, 1
    # gated full attention packs whole KV groups, GatedDeltaNet projections whole key heads; per-value-head vectors
    if key.endswith(("linear_qgkv.weight", "in_proj_qkvz.weight", "in_proj_ba.weight", "self_attention.dt_bias",
                     "self_attention.A_log")):
        return 0, 1
    if _QK_NORM_FULL["on"] and key.endswith(("self_attention.q_layernorm.weight", "self_attention.k_layernorm.weight")):
        return 0, 1  # MiniMax: one norm over all heads, the weight is split with the heads
    if key.endswith("self_attention.conv_weight"):
        # channels are type-major [q heads | k heads | v heads]: three blocks of different sizes, each split by head
        if _GDN_GEOMETRY["blocks"] is None:
            raise ValueError("tensor-parallel conversion of GatedDeltaNet layers needs set_linear_attention_geometry()")
        return 0, list(_GDN_GEOMETRY["blocks"])
    return None


_GDN_GEOMETRY = {"blocks": None}
_QK_NORM_FULL = {"on": False}


def set_qk_norm_over_all_heads(flag: bool) -> None:
    """MiniMax normalises q (and k) over ALL heads at once; its norm weights are then sharded over TP ranks."""
    _QK_NORM_FULL["on"] = bool(flag)


def set_linear_attention_geometry(num_key_heads: int, key_dim: int, num_value_heads: int, value_dim: int) -> None:
    """Sizes of the q / k / v channel blocks of the GatedDeltaNet convolution (needed to split it over TP ranks)."""
    _GDN_GEOMETRY["blocks"] = (num_key_heads * key_dim, num_key_heads * key_dim, num_value_heads * value_dim)


def shard_tp(key: str, w: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    rule = tp_rule(key)
    if rule is None or tp == 1:
        return w
    dim, stride = rule
    if isinstance(stride, list):
        return torch.cat([b.chunk(tp, dim)[rank] for b in w.split(stride, dim)], dim).contiguous()
    if stride == 1:
        return w.chunk(tp, dim)[rank].contiguous()
    return torch.cat([b.chunk(tp, dim)[rank] for b in w.chunk(stride, dim)], dim).contiguous()


def merge_tp(key: str, shards: List[torch.Tensor]) -> torch.Tensor:
    rule = tp_rule(key)
    if rule is None or len(shards) == 1:
        return shards[0]
    dim, stride = rule
    if isinstance(stride, list):
        tp = len(shards)
        blocks = [s.split([n // tp for n in stride], dim) for s in shards]
        return torch.cat([torch.cat([b[j] for b in blocks], dim) for j in range(len(stride))], dim)
    if stride == 1:
        return torch.cat(shards, dim)
    blocks = [s.chunk(stride, dim) for s in shards]
    return torch.cat([torch.cat([b[j] for b in blocks], dim) for j in range(stride)], dim)


# ---- vision-language models: Qwen2-VL / Qwen2.5-VL vision tower + merger ---------------------------------------------
def _vit_pack_qkv(w: torch.Tensor, num_heads: int) -> torch.Tensor:
    """HF fused ``[q_all; k_all; v_all]`` rows -> Megatron per-head ``[q_h, k_h, v_h]`` rows."""
    tail = w.shape[1:]
    d = w.shape[0] // (3 * num_heads)
    return w.reshape(3, num_heads, d, *tail).transpose(0, 1).reshape(-1, *tail).contiguous()


def _vit_unpack_qkv(w: torch.Tensor, num_heads: int) -> torch.Tensor:
    tail = w.shape[1:]
    d = w.shape[0] // (3 * num_heads)
    return w.reshape(num_heads, 3, d, *tail).transpose(0, 1).reshape(-1, *tail).contiguous()


_VIT_LAYER = [  # (Megatron suffix, HF suffix) inside one vision block
    ("self_attention.linear_qkv.layer_norm_weight", "norm1.weight"),
    ("self_attention.linear_proj.weight", "attn.proj.weight"), ("self_attention.linear_proj.bias", "attn.proj.bias"),
    ("mlp.linear_fc1.layer_norm_weight", "norm2.weight"),
    ("mlp.linear_fc2.weight", "mlp.down_proj.weight"), ("mlp.linear_fc2.bias", "mlp.down_proj.bias"),
]
_VIT_TOP = [("image_encoder.patch_embed.proj.weight", "patch_embed.proj.weight"),
            ("image_projector.layernorm.weight", "merger.ln_q.weight"),
            ("image_projector.linear_fc1.weight", "merger.mlp.0.weight"), ("image_projector.linear_fc1.bias", "merger.mlp.0.bias"),
            ("image_projector.linear_fc2.weight", "merger.mlp.2.weight"), ("image_projector.linear_fc2.bias", "merger.mlp.2.bias")]


def qwen_vision_to_mcore(hf: Dict[str, torch.Tensor], prefix: str, num_layers: int, num_heads: int) -> Dict[str, torch.Tensor]:
    """``visual.*`` tensors -> ``image_encoder.* / image_projector.*`` (SwiGLU FC1 = [gate; up], packed QKV per head)."""
    out = {mk: hf[prefix + hk] for mk, hk in _VIT_TOP}
    for i in range(num_layers):
        h, m = f"{prefix}blocks.{i}.", f"image_encoder.decoder.layers.{i}."
        for mk, hk in _VIT_LAYER:
            out[m + mk] = hf[h + hk]
        out[m + "self_attention.linear_qkv.weight"] = _vit_pack_qkv(hf[h + "attn.qkv.weight"], num_heads)
        out[m + "self_attention.linear_qkv.bias"] = _vit_pack_qkv(hf[h + "attn.qkv.bias"], num_heads)
        out[m + "mlp.linear_fc1.weight"] = torch.cat([hf[h + "mlp.gate_proj.weight"], hf[h + "mlp.up_proj.weight"]], 0)
        out[m + "mlp.linear_fc1.bias"] = torch.cat([hf[h + "mlp.gate_proj.bias"], hf[h + "mlp.up_proj.bias"]], 0)
    return out


def qwen_vision_to_hf(mc: Dict[str, torch.Tensor], prefix: str, num_layers: int, num_heads: int) -> Dict[str, torch.Tensor]:
    out = {prefix + hk: mc[mk] for mk, hk in _VIT_TOP}
    for i in range(num_layers):
        h, m = f"{prefix}blocks.{i}.", f"image_encoder.decoder.layers.{i}."
        for mk, hk in _VIT_LAYER:
            out[h + hk] = mc[m + mk]
        out[h + "attn.qkv.weight"] = _vit_unpack_qkv(mc[m + "self_attention.linear_qkv.weight"], num_heads)
        out[h + "attn.qkv.bias"] = _vit_unpack_qkv(mc[m + "self_attention.linear_qkv.bias"], num_heads)
        for name in ("weight", "bias"):
            g, u = mc[m + f"mlp.linear_fc1.{name}"].chunk(2, 0)
            out[h + f"mlp.gate_proj.{name}"], out[h + f"mlp.up_proj.{name}"] = g.contiguous(), u.contiguous()
    return out


def _vlm_prefixes(hf: Dict[str, torch.Tensor]):
    """(language prefix, vision prefix) of the two Hugging Face layouts in circulation."""
    if any(k.startswith("model.language_model.") for k in hf):
        return "model.language_model.", "model.visual."
    return "model.", "visual."


def vlm_hf_to_mcore(hf: Dict[str, torch.Tensor], fam: FamilyMap, *, vit_layers: int, vit_heads: int,
                    **lm_kw) -> Dict[str, torch.Tensor]:
    """Whole vision-language checkpoint -> ``foundation_model.* / encoder_model.image_encoder.* /
    encoder_model.image_projector.*`` (the composition of models/omni.py)."""
    lp, vp = _vlm_prefixes(hf)
    lm_fam = dataclasses.replace(fam, hf_prefix=lp, hf_layers=lp + "layers.{i}.")
    lm = hf_to_mcore({k: v for k, v in hf.items() if not k.startswith(vp)}, lm_fam, **lm_kw)
    vis = qwen_vision_to_mcore(hf, vp, vit_layers, vit_heads)
    out = {"foundation_model." + k: v for k, v in lm.items()}
    out.update({"encoder_model." + k: v for k, v in vis.items()})
    return out


def vlm_mcore_to_hf(mc: Dict[str, torch.Tensor], fam: FamilyMap, *, vit_layers: int, vit_heads: int,
                    nested: bool = False, **lm_kw) -> Dict[str, torch.Tensor]:
    lp, vp = ("model.language_model.", "model.visual.") if nested else ("model.", "visual.")
    lm_fam = dataclasses.replace(fam, hf_prefix=lp, hf_layers=lp + "layers.{i}.")
    out = mcore_to_hf({k[len("foundation_model."):]: v for k, v in mc.items() if k.startswith("foundation_model.")},
                      lm_fam, **lm_kw)
    out.update(qwen_vision_to_hf({k[len("encoder_model."):]: v for k, v in mc.items() if k.startswith("encoder_model.")},
                                 vp, vit_layers, vit_heads))
    return out


# ---- Qwen3-VL vision tower with DeepStack taps --------------------------------------------------------
# (configs/models/image_encoder/ckpt_convert/qwen3_vit_convert.yaml:31-90)
_Q3VIT_LAYER = [("self_attention.linear_qkv.layer_norm_weight", "norm1.weight"),
                ("self_attention.linear_qkv.layer_norm_bias", "norm1.bias"),
                ("self_attention.linear_proj.weight", "attn.proj.weight"), ("self_attention.linear_proj.bias", "attn.proj.bias"),
                ("mlp.linear_fc1.layer_norm_weight", "norm2.weight"), ("mlp.linear_fc1.layer_norm_bias", "norm2.bias"),
                ("mlp.linear_fc1.weight", "mlp.linear_fc1.weight"), ("mlp.linear_fc1.bias", "mlp.linear_fc1.bias"),
                ("mlp.linear_fc2.weight", "mlp.linear_fc2.weight"), ("mlp.linear_fc2.bias", "mlp.linear_fc2.bias")]
_Q3VIT_TOP = [("pos_embed", "pos_embed.weight"), ("patch_embed.proj.weight", "patch_embed.proj.weight"),
              ("patch_embed.proj.bias", "patch_embed.proj.bias")]
_Q3VIT_TAP = [("norms.{k}.weight", "deepstack_merger_list.{k}.norm.weight"),
              ("norms.{k}.bias", "deepstack_merger_list.{k}.norm.bias"),
              ("fc1.{k}.weight", "deepstack_merger_list.{k}.linear_fc1.weight"),
              ("fc1.{k}.bias", "deepstack_merger_list.{k}.linear_fc1.bias"),
              ("fc2.{k}.weight", "deepstack_merger_list.{k}.linear_fc2.weight"),
              ("fc2.{k}.bias", "deepstack_merger_list.{k}.linear_fc2.bias")]


def qwen3_vision_to_hf(vit: Dict[str, torch.Tensor], taps: Dict[str, torch.Tensor], *, num_layers: int, num_heads: int,
                       prefix: str = "model.visual.") -> Dict[str, torch.Tensor]:
    """State dicts of the vision tower and of its DeepStack mergers -> ``model.visual.*`` tensors. Entries that a
    model does not have (norm biases, patch-embedding bias) are skipped."""
    out: Dict[str, torch.Tensor] = {}
    for mk, hk in _Q3VIT_TOP:
        if mk in vit:
            out[prefix + hk] = vit[mk]
    for i in range(num_layers):
        m, h = f"decoder.layers.{i}.", f"{prefix}blocks.{i}."
        for mk, hk in _Q3VIT_LAYER:
            if m + mk in vit:
                out[h + hk] = vit[m + mk]
        for suffix in ("weight", "bias"):
            if m + f"self_attention.linear_qkv.{suffix}" in vit:
                out[h + f"attn.qkv.{suffix}"] = _vit_unpack_qkv(vit[m + f"self_attention.linear_qkv.{suffix}"], num_heads)
    k = 0
    while f"fc1.{k}.weight" in taps:
        for mk, hk in _Q3VIT_TAP:
            if mk.format(k=k) in taps:
                out[prefix + hk.format(k=k)] = taps[mk.format(k=k)]
        k += 1
    return out


def qwen3_vision_to_mcore(hf: Dict[str, torch.Tensor], *, num_layers: int, num_heads: int,
                          prefix: str = "model.visual."):
    """Inverse of :func:`qwen3_vision_to_hf`: (vision tower state dict, DeepStack merger state dict)."""
    vit: Dict[str, torch.Tensor] = {}
    taps: Dict[str, torch.Tensor] = {}
    for mk, hk in _Q3VIT_TOP:
        if prefix + hk in hf:
            vit[mk] = hf[prefix + hk]
    for i in range(num_layers):
        m, h = f"decoder.layers.{i}.", f"{prefix}blocks.{i}."
        for mk, hk in _Q3VIT_LAYER:
            if h + hk in hf:
                vit[m + mk] = hf[h + hk]
        for suffix in ("weight", "bias"):
            if h + f"attn.qkv.{suffix}" in hf:
                vit[m + f"self_attention.linear_qkv.{suffix}"] = _vit_pack_qkv(hf[h + f"attn.qkv.{suffix}"], num_heads)
    k = 0
    while f"{prefix}deepstack_merger_list.{k}.linear_fc1.weight" in hf:
        for mk, hk in _Q3VIT_TAP:
            if prefix + hk.format(k=k) in hf:
                taps[mk.format(k=k)] = hf[prefix + hk.format(k=k)]
        k += 1
    return vit, taps


# ---- InternViT (InternVL2.5 / 3.5) and MoonViT (Kimi-VL / K2.5 / K2.6) towers with their projectors --------------------
# (configs/models/image_encoder/ckpt_convert/{internvl_vit_*,moon_vit_3d}_convert.yaml,
#  configs/models/image_projector/ckpt_convert/{intern_mlp_adapter,patch_merger_adapter}_convert.yaml)
_GENERIC_VIT = {
    "intern_vit": dict(
        prefix="vision_model.", proj_prefix="mlp1.",
        top=[("patch_embed.proj.weight", "embeddings.patch_embedding.weight"), ("patch_embed.proj.bias", "embeddings.patch_embedding.bias"),
             ("pos_embed", "embeddings.position_embedding"), ("cls_token", "embeddings.class_embedding")],
        layer_prefix="encoder.layers.",
        layer=[("self_attention.linear_qkv.layer_norm_weight", "norm1.weight"), ("self_attention.linear_qkv.layer_norm_bias", "norm1.bias"),
               ("self_attention.linear_qkv.weight", "attn.qkv.weight"), ("self_attention.linear_qkv.bias", "attn.qkv.bias"),
               ("self_attention.q_layernorm.weight", "attn.q_norm.weight"), ("self_attention.k_layernorm.weight", "attn.k_norm.weight"),
               ("self_attention.linear_proj.weight", "attn.proj.weight"), ("self_attention.linear_proj.bias", "attn.proj.bias"),
               ("ls1", "ls1"), ("ls2", "ls2"),
               ("mlp.linear_fc1.layer_norm_weight", "norm2.weight"), ("mlp.linear_fc1.layer_norm_bias", "norm2.bias"),
               ("mlp.linear_fc1.weight", "mlp.fc1.weight"), ("mlp.linear_fc1.bias", "mlp.fc1.bias"),
               ("mlp.linear_fc2.weight", "mlp.fc2.weight"), ("mlp.linear_fc2.bias", "mlp.fc2.bias")],
        projector=[("norm.weight", "0.weight"), ("norm.bias", "0.bias"), ("fc1.weight", "1.weight"), ("fc1.bias", "1.bias"),
                   ("fc2.weight", "3.weight"), ("fc2.bias", "3.bias")]),
    "moon_vit": dict(
        prefix="vision_tower.", proj_prefix="multi_modal_projector.",
        top=[("patch_embed.proj.weight", "patch_embed.proj.weight"), ("patch_embed.proj.bias", "patch_embed.proj.bias"),
             ("pos_embed", "patch_embed.pos_emb.weight"), ("post_layernorm.weight", "encoder.final_layernorm.weight"),
             ("post_layernorm.bias", "encoder.final_layernorm.bias")],
        layer_prefix="encoder.blocks.",
        layer=[("self_attention.linear_qkv.layer_norm_weight", "norm0.weight"), ("self_attention.linear_qkv.layer_norm_bias", "norm0.bias"),
               ("self_attention.linear_qkv.weight", "wqkv.weight"), ("self_attention.linear_qkv.bias", "wqkv.bias"),
               ("self_attention.linear_proj.weight", "wo.weight"), ("self_attention.linear_proj.bias", "wo.bias"),
               ("mlp.linear_fc1.layer_norm_weight", "norm1.weight"), ("mlp.linear_fc1.layer_norm_bias", "norm1.bias"),
               ("mlp.linear_fc1.weight", "mlp.fc0.weight"), ("mlp.linear_fc1.bias", "mlp.fc0.bias"),
               ("mlp.linear_fc2.weight", "mlp.fc1.weight"), ("mlp.linear_fc2.bias", "mlp.fc1.bias")],
        projector=[("pre_norm.weight", "pre_norm.weight"), ("pre_norm.bias", "pre_norm.bias"), ("fc1.weight", "linear_1.weight"),
                   ("fc1.bias", "linear_1.bias"), ("fc2.weight", "linear_2.weight"), ("fc2.bias", "linear_2.bias")]),
}


def _vit_shape_to_mcore(family: str, key: str, t: torch.Tensor, num_heads: int) -> torch.Tensor:
    if key.endswith("linear_qkv.weight") or key.endswith("linear_qkv.bias"):
        return _vit_pack_qkv(t, num_heads)
    if key == "patch_embed.proj.weight" and t.dim() == 4:
        return t.unsqueeze(2)                                       # Conv2d -> the Conv3d shape with one frame per patch
    if key == "pos_embed":
        return t.reshape(-1, t.shape[-1])                           # [1, 1 + N, C] (InternViT) or [H, W, C] (MoonViT) -> rows
    if key == "cls_token":
        return t.reshape(1, -1)
    return t


def _vit_shape_to_hf(family: str, key: str, t: torch.Tensor, num_heads: int) -> torch.Tensor:
    if key.endswith("linear_qkv.weight") or key.endswith("linear_qkv.bias"):
        return _vit_unpack_qkv(t, num_heads)
    if key == "patch_embed.proj.weight" and t.dim() == 5:
        return t.squeeze(2)
    if key == "pos_embed":
        if family == "intern_vit":
            return t.unsqueeze(0)
        side = int(round(t.shape[0] ** 0.5))
        return t.reshape(side, side, t.shape[-1])
    if key == "cls_token":
        return t.reshape(1, 1, -1)
    return t


def generic_vision_to_mcore(hf: Dict[str, torch.Tensor], family: str, num_layers: int, num_heads: int) -> Dict[str, torch.Tensor]:
    """Vision tower and projector tensors of an InternVL / Kimi-VL checkpoint -> ``image_encoder.* / image_projector.*``
    (entries the checkpoint does not have, like q / k norms of the small InternViT, are skipped)."""
    spec = _GENERIC_VIT[family]
    out: Dict[str, torch.Tensor] = {}
    for mk, hk in spec["top"]:
        if spec["prefix"] + hk in hf:
            out["image_encoder." + mk] = _vit_shape_to_mcore(family, mk, hf[spec["prefix"] + hk], num_heads)
    for i in range(num_layers):
        for mk, hk in spec["layer"]:
            src = f"{spec['prefix']}{spec['layer_prefix']}{i}.{hk}"
            if src in hf:
                out[f"image_encoder.decoder.layers.{i}.{mk}"] = _vit_shape_to_mcore(family, mk, hf[src], num_heads)
    for mk, hk in spec["projector"]:
        if spec["proj_prefix"] + hk in hf:
            out["image_projector." + mk] = hf[spec["proj_prefix"] + hk]
    return out


def generic_vision_to_hf(mc: Dict[str, torch.Tensor], family: str, num_layers: int, num_heads: int) -> Dict[str, torch.Tensor]:
    spec = _GENERIC_VIT[family]
    out: Dict[str, torch.Tensor] = {}
    for mk, hk in spec["top"]:
        if "image_encoder." + mk in mc:
            out[spec["prefix"] + hk] = _vit_shape_to_hf(family, mk, mc["image_encoder." + mk], num_heads)
    for i in range(num_layers):
        for mk, hk in spec["layer"]:
            src = f"image_encoder.decoder.layers.{i}.{mk}"
            if src in mc:
                out[f"{spec['prefix']}{spec['layer_prefix']}{i}.{hk}"] = _vit_shape_to_hf(family, mk, mc[src], num_heads)
    for mk, hk in spec["projector"]:
        if "image_projector." + mk in mc:
            out[spec["proj_prefix"] + hk] = mc["image_projector." + mk]
    return out


# vision-language checkpoints that keep the language model under ``language_model.`` next to a tower of its own:
# composition name -> vision family of ``_GENERIC_VIT``
COMPOSITE_VLM = {"internvl": "intern_vit", "internvl2.5": "intern_vit", "internvl3.5": "intern_vit",
                 "kimi_vl": "moon_vit", "kimi_k2.5": "moon_vit", "kimi_k2.6": "moon_vit"}


def composite_vlm_hf_to_mcore(hf: Dict[str, torch.Tensor], lm_fam: FamilyMap, vision_family: str, *, vit_layers: int,
                              vit_heads: int, **lm_kw) -> Dict[str, torch.Tensor]:
    """InternVL / Kimi-VL checkpoint -> ``foundation_model.* / encoder_model.image_encoder.* / image_projector.*``."""
    lang = {k[len("language_model."):]: v for k, v in hf.items() if k.startswith("language_model.")}
    out = {"foundation_model." + k: v for k, v in hf_to_mcore(lang, lm_fam, **lm_kw).items()}
    out.update({"encoder_model." + k: v for k, v in generic_vision_to_mcore(hf, vision_family, vit_layers, vit_heads).items()})
    return out


def composite_vlm_mcore_to_hf(mc: Dict[str, torch.Tensor], lm_fam: FamilyMap, vision_family: str, *, vit_layers: int,
                              vit_heads: int, **lm_kw) -> Dict[str, torch.Tensor]:
    lang = mcore_to_hf({k[len("foundation_model."):]: v for k, v in mc.items() if k.startswith("foundation_model.")}, lm_fam, **lm_kw)
    out = {"language_model." + k: v for k, v in lang.items()}
    out.update(generic_vision_to_hf({k[len("encoder_model."):]: v for k, v in mc.items() if k.startswith("encoder_model.")},
                                    vision_family, vit_layers, vit_heads))
    return out
