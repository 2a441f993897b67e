"""Online Hugging Face bridge: load HF weights straight into the running (sharded) model at start-up
and export HF safetensors from it at the end, without an offline conversion step
(tools/dist_checkpoint/checkpoint/hf_checkpoint_loader.py:97-284, hf_checkpoint_saver.py:115-412,
core/tp_gather.py:35-380). Each rank converts the full HF dict to Megatron names, keeps the slice for
its (tp, pp, ep) coordinates and loads it strictly; export gathers the TP shards inside the TP group
and lets the first data-parallel rank of every pipeline stage contribute its layers."""
from __future__ import annotations

import os
import re
from typing import Dict, Optional

import torch
import torch.distributed as dist

from ..parallel import state as ps

_LAYER = re.compile(r"^decoder\.layers\.(\d+)\.(.*)$")
_EXPERT = re.compile(r"\.experts\.linear_fc[12]\.weight(\d+)$")


def _nm():
    from tools.convert_checkpoint import name_maps
    return name_maps


def load_hf_checkpoint_online(trainer, hf_dir: str, family: str = "llama3", upcycle: bool = False) -> int:
    """Returns the number of tensors loaded into this rank's model chunks. ``upcycle``: the directory holds the DENSE
    model that this mixture-of-experts model grows from; every expert starts as (a slice of) the dense feed-forward
    block and the routers are drawn from one seed on all ranks (``--moe-use-upcycling``)."""
    from tools.convert_checkpoint.convert import load_hf

    nm = _nm()
    cfg = trainer.mcfg
    st = trainer.st
    _set_geometry(cfg)
    hf = load_hf(hf_dir)
    lm_kw = dict(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, num_groups=cfg.num_query_groups,
                 padded_vocab=cfg.padded_vocab_size, num_experts=cfg.num_moe_experts,
                 tie_embeddings=not cfg.untie_embeddings_and_output_weights)
    enc_mc: Dict[str, torch.Tensor] = {}
    if family in nm.VLM_FAMILIES:
        # vision tower + merger + language model in one Hugging Face checkpoint
        vit = trainer.vit_cfg
        both = nm.vlm_hf_to_mcore(hf, nm.FAMILIES[nm.VLM_FAMILIES[family]], vit_layers=vit.num_layers,
                                  vit_heads=vit.num_attention_heads, **lm_kw)
        mc = {k[len("foundation_model."):]: v for k, v in both.items() if k.startswith("foundation_model.")}
        enc_mc = {k[len("encoder_model."):]: v for k, v in both.items() if k.startswith("encoder_model.")}
    elif upcycle and cfg.num_moe_experts:
        import dataclasses

        from ..runtime.upcycling import upcycle_state_dict
        dense_family = dataclasses.replace(nm.FAMILIES[family], moe=False)
        mc = nm.hf_to_mcore(hf, dense_family, **{**lm_kw, "num_experts": None})
        dense_ffn = mc["decoder.layers.0.mlp.linear_fc2.weight"].shape[1]
        moe_ffn = cfg.moe_ffn_hidden_size or cfg.ffn_hidden_size
        if dense_ffn % moe_ffn:
            raise ValueError(f"dense FFN width {dense_ffn} must divide by the expert width {moe_ffn}")
        mc = upcycle_state_dict(mc, cfg.num_moe_experts, granularity=dense_ffn // moe_ffn, glu=cfg.gated_linear_unit,
                                router_std=cfg.init_method_std,
                                moe_layers={i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)})
    else:
        mc = nm.hf_to_mcore(hf, nm.FAMILIES[family], **lm_kw)
    e_local = (cfg.num_moe_experts // st.dims.ep) if cfg.num_moe_experts else 0
    n = 0
    for chunk in trainer.models:
        mod = chunk.module
        lm = getattr(mod, "foundation_model", mod)
        numbers = lm.decoder.layer_numbers
        local_of = {g: l for l, g in enumerate(numbers)}
        sd = {}
        for k, w in mc.items():
            m = _LAYER.match(k)
            if m:
                g = int(m.group(1))
                if g not in local_of:
                    continue
                key = f"decoder.layers.{local_of[g]}.{m.group(2)}"
            else:
                key = k
            em = _EXPERT.search(key)
            if em:
                e = int(em.group(1))
                if not (st.ep_rank * e_local <= e < (st.ep_rank + 1) * e_local):
                    continue
                key = key[: em.start(1)] + str(e - st.ep_rank * e_local)
            sd[key] = nm.shard_tp(k, w, st.tp_rank, st.dims.tp)
        own = dict(lm.state_dict())
        load = {k: v.to(own[k].dtype) for k, v in sd.items() if k in own}
        missing = [k for k in own if k not in load and not k.endswith("_extra_state") and "expert_bias" not in k
                   and "local_tokens_per_expert" not in k]
        if missing:
            raise KeyError(f"HF checkpoint does not provide: {missing[:5]} ...")
        with torch.no_grad():
            for k, v in load.items():
                own[k].copy_(v)
        n += len(load)
        enc = getattr(mod, "encoder_model", None)
        if enc is not None and enc_mc:
            e_rank, e_tp = _encoder_tp(trainer)
            params = dict(enc.named_parameters())
            with torch.no_grad():
                for k, t in enc.state_dict().items():
                    if k not in enc_mc:
                        raise KeyError(f"HF checkpoint does not provide the vision parameter {k}")
                    t.copy_(_shard_like(params.get(k), enc_mc[k], e_rank, e_tp).to(t.dtype))
                    n += 1
    trainer.optimizer.reload_model_params()
    return n


def _set_geometry(cfg) -> None:
    """Two of the converter's TP rules depend on the model: the GatedDeltaNet convolution needs the sizes of its
    q / k / v channel blocks, and MiniMax's q / k norms over all heads are split with the heads."""
    _nm().set_qk_norm_over_all_heads(getattr(cfg, "qk_layernorm_full", False))
    if getattr(cfg, "linear_num_key_heads", None):
        _nm().set_linear_attention_geometry(cfg.linear_num_key_heads, cfg.linear_key_head_dim,
                                            cfg.linear_num_value_heads, cfg.linear_value_head_dim)



_HF_ARCH = {"llama": ("llama", "LlamaForCausalLM"), "llama2": ("llama", "LlamaForCausalLM"),
            "llama3": ("llama", "LlamaForCausalLM"), "internlm": ("internlm2", "InternLM2ForCausalLM"),
            "qwen2": ("qwen2", "Qwen2ForCausalLM"), "qwen2.5": ("qwen2", "Qwen2ForCausalLM"),
            "qwen3": ("qwen3", "Qwen3ForCausalLM"), "qwen3_moe": ("qwen3_moe", "Qwen3MoeForCausalLM"),
            "deepseek": ("deepseek_v3", "DeepseekV3ForCausalLM"), "glm": ("glm_moe_dsa", "GlmMoeDsaForCausalLM"),
            "internlm2": ("internlm2", "InternLM2ForCausalLM"), "kimi_k2": ("kimi_k2", "DeepseekV3ForCausalLM"),
            "minimax": ("minimax_m2", "MiniMaxM2ForCausalLM"), "mimo": ("mimo", "MiMoForCausalLM"),
            "qwen3_next": ("qwen3_next", "Qwen3NextForCausalLM"), "qwen3_5": ("qwen3_5_moe", "Qwen3_5MoeForCausalLM")}


def hf_config_from_model(cfg, family: str) -> dict:
    """``config.json`` contents for the exported weights, derived from the training configuration."""
    model_type, arch = _HF_ARCH.get(family, ("llama", "LlamaForCausalLM"))
    out = {
        "architectures": [arch], "model_type": model_type, "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.ffn_hidden_size, "num_hidden_layers": cfg.num_layers,
        "num_attention_heads": cfg.num_attention_heads, "num_key_value_heads": cfg.num_query_groups,
        "head_dim": cfg.kv_channels, "vocab_size": cfg.vocab_size, "rms_norm_eps": cfg.layernorm_epsilon,
        "rope_theta": cfg.rotary_base, "max_position_embeddings": cfg.max_position_embeddings,
        "tie_word_embeddings": not cfg.untie_embeddings_and_output_weights, "hidden_act": "silu",
        "attention_bias": bool(cfg.add_qkv_bias), "torch_dtype": str(cfg.params_dtype).replace("torch.", ""),
    }
    if cfg.multi_latent_attention:
        out.update(q_lora_rank=cfg.q_lora_rank, kv_lora_rank=cfg.kv_lora_rank, qk_nope_head_dim=cfg.qk_head_dim,
                   qk_rope_head_dim=cfg.qk_pos_emb_head_dim, v_head_dim=cfg.v_head_dim,
                   num_nextn_predict_layers=cfg.mtp_num_layers, n_routed_experts=cfg.num_moe_experts,
                   n_shared_experts=1 if cfg.moe_shared_expert_intermediate_size else 0)
        if cfg.use_dsa:
            out.update(index_n_heads=cfg.dsa_indexer_n_heads, index_head_dim=cfg.dsa_indexer_head_dim,
                       index_topk=cfg.dsa_indexer_topk)
    if cfg.num_moe_experts:
        out.update(num_experts=cfg.num_moe_experts, num_experts_per_tok=cfg.moe_router_topk,
                   moe_intermediate_size=cfg.moe_ffn_hidden_size, norm_topk_prob=True)
    return out


def _shard_like(p, full: torch.Tensor, rank: int, tp: int) -> torch.Tensor:
    """This rank's piece of `full` according to the sharding the parameter itself declares (partition dim and
    stride set by the tensor-parallel layers); replicated parameters take the whole tensor."""
    dim = getattr(p, "partition_dim", -1) if p is not None else -1
    if tp == 1 or dim < 0 or not getattr(p, "tensor_model_parallel", False) or getattr(p, "tp_shards", tp) == 1:
        return full
    stride = getattr(p, "partition_stride", 1)
    if stride == 1:
        return full.chunk(tp, dim)[rank].contiguous()
    return torch.cat([b.chunk(tp, dim)[rank] for b in full.chunk(stride, dim)], dim).contiguous()


def _encoder_tp(trainer):
    """(rank, size) of the vision encoder's own tensor-parallel group."""
    from ..models.omni import ENCODER_STATE
    from ..parallel import state as ps

    if ENCODER_STATE in ps._STATES:
        est = ps.get_state(ENCODER_STATE)
        return est.tp_rank, est.dims.tp
    return trainer.st.tp_rank, trainer.st.dims.tp


def save_hf_checkpoint(trainer, out_dir: str, family: str = "llama3", hf_config: Optional[dict] = None) -> None:
    """Gather the model to rank 0 (TP shards merged, pipeline stages concatenated) and write safetensors."""
    from tools.convert_checkpoint.convert import save_hf

    nm = _nm()
    cfg, st = trainer.mcfg, trainer.st
    _set_geometry(cfg)
    e_local = (cfg.num_moe_experts // st.dims.ep) if cfg.num_moe_experts else 0
    local: Dict[str, torch.Tensor] = {}
    enc_meta: Dict[str, tuple] = {}  # encoder tensors sharded over TP: key -> (dim, stride), from the parameters
    for chunk in trainer.models:
        lm = getattr(chunk.module, "foundation_model", chunk.module)
        numbers = lm.decoder.layer_numbers
        for k, v in lm.state_dict().items():
            m = _LAYER.match(k)
            key = f"decoder.layers.{numbers[int(m.group(1))]}.{m.group(2)}" if m else k
            em = _EXPERT.search(key)
            if em:
                key = key[: em.start(1)] + str(int(em.group(1)) + st.ep_rank * e_local)
            local[key] = v.detach().cpu()
        enc = getattr(chunk.module, "encoder_model", None)
        if enc is not None and family in nm.VLM_FAMILIES and getattr(chunk.module, "pre_process", True):
            e_rank, e_tp = _encoder_tp(trainer)
            if e_tp not in (1, st.dims.tp):
                raise NotImplementedError("the encoder's TP degree must be 1 or the decoder's for the HF export")
            params = dict(enc.named_parameters())
            for k, v in enc.state_dict().items():
                p_ = params.get(k)
                sharded = (e_tp > 1 and p_ is not None and getattr(p_, "tensor_model_parallel", False)
                           and getattr(p_, "partition_dim", -1) >= 0 and getattr(p_, "tp_shards", e_tp) > 1)
                if sharded:
                    enc_meta["encoder_model." + k] = (p_.partition_dim, getattr(p_, "partition_stride", 1))
                if sharded or st.tp_rank == 0:  # replicated tensors: one copy is enough
                    local["encoder_model." + k] = v.detach().cpu()
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world > 1:
        payload = (st.tp_rank, st.rank_in("dp_cp"), st.ep_rank, local) if st.rank_in("dp") == 0 or st.dims.ep > 1 else None
        gathered = [None] * world
        dist.gather_object(payload, gathered if dist.get_rank() == 0 else None, dst=0)
        if dist.get_rank() != 0:
            dist.barrier()
            return
        pieces: Dict[str, Dict[int, torch.Tensor]] = {}
        for item in gathered:
            if item is None:
                continue
            t_rank, _, _, sd = item
            for k, v in sd.items():
                pieces.setdefault(k, {}).setdefault(t_rank, v)
        def merge(k, shards):
            if not k.startswith("encoder_model."):
                return nm.merge_tp(k, shards)
            if k not in enc_meta or len(shards) == 1:
                return shards[0]
            dim, stride = enc_meta[k]
            if stride == 1:
                return torch.cat(shards, dim)
            blocks = [s_.chunk(stride, dim) for s_ in shards]
            return torch.cat([torch.cat([b[j] for b in blocks], dim) for j in range(stride)], dim)

        full = {k: merge(k, [v[t] for t in sorted(v)]) for k, v in pieces.items()}
    else:
        full = local
    out_kw = dict(num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads, num_groups=cfg.num_query_groups,
                  vocab_size=cfg.vocab_size, num_experts=cfg.num_moe_experts,
                  tie_embeddings=not cfg.untie_embeddings_and_output_weights)
    if family in nm.VLM_FAMILIES:
        vit = trainer.vit_cfg
        lm_family = nm.VLM_FAMILIES[family]
        both = {("foundation_model." + k if not k.startswith("encoder_model.") else k): v for k, v in full.items()}
        hf = nm.vlm_mcore_to_hf(both, nm.FAMILIES[lm_family], vit_layers=vit.num_layers,
                                vit_heads=vit.num_attention_heads, **out_kw)
        if hf_config is None:
            hf_config = {"model_type": family, "architectures": ["Qwen2_5_VLForConditionalGeneration"],
                         "text_config": hf_config_from_model(cfg, lm_family),
                         "vision_config": {"depth": vit.num_layers, "num_heads": vit.num_attention_heads,
                                           "hidden_size": vit.hidden_size, "patch_size": vit.patch_size,
                                           "spatial_merge_size": vit.spatial_merge_size,
                                           "temporal_patch_size": vit.temporal_patch_size}}
    else:
        hf = nm.mcore_to_hf(full, nm.FAMILIES[family], **out_kw)
    save_hf(hf, out_dir, hf_config or hf_config_from_model(cfg, family))
    if world > 1:
        dist.barrier()
