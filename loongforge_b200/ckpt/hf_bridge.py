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


def load_hf_checkpoint_online(trainer, hf_dir: str, family: str = "llama3") -> int:
    """Returns the number of tensors loaded into this rank's model chunks."""
    from tools.convert_checkpoint.convert import load_hf

    nm = _nm()
    cfg = trainer.mcfg
    st = trainer.st
    hf = load_hf(hf_dir)
    mc = nm.hf_to_mcore(hf, nm.FAMILIES[family], num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads,
                        num_groups=cfg.num_query_groups, padded_vocab=cfg.padded_vocab_size,
                        num_experts=cfg.num_moe_experts,
                        tie_embeddings=not cfg.untie_embeddings_and_output_weights)
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
    trainer.optimizer.reload_model_params()
    return n


_HF_ARCH = {"llama": ("llama", "LlamaForCausalLM"), "llama2": ("llama", "LlamaForCausalLM"),
            "llama3": ("llama", "LlamaForCausalLM"), "internlm": ("internlm2", "InternLM2ForCausalLM"),
            "qwen2": ("qwen2", "Qwen2ForCausalLM"), "qwen2.5": ("qwen2", "Qwen2ForCausalLM"),
            "qwen3": ("qwen3", "Qwen3ForCausalLM"), "qwen3_moe": ("qwen3_moe", "Qwen3MoeForCausalLM"),
            "deepseek": ("deepseek_v3", "DeepseekV3ForCausalLM"), "glm": ("glm_moe_dsa", "GlmMoeDsaForCausalLM")}


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


def save_hf_checkpoint(trainer, out_dir: str, family: str = "llama3", hf_config: Optional[dict] = None) -> None:
    """Gather the model to rank 0 (TP shards merged, pipeline stages concatenated) and write safetensors."""
    from tools.convert_checkpoint.convert import save_hf

    nm = _nm()
    cfg, st = trainer.mcfg, trainer.st
    e_local = (cfg.num_moe_experts // st.dims.ep) if cfg.num_moe_experts else 0
    local: Dict[str, torch.Tensor] = {}
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
        full = {k: nm.merge_tp(k, [v[t] for t in sorted(v)]) for k, v in pieces.items()}
    else:
        full = local
    hf = nm.mcore_to_hf(full, nm.FAMILIES[family], num_layers=cfg.num_layers, num_heads=cfg.num_attention_heads,
                        num_groups=cfg.num_query_groups, vocab_size=cfg.vocab_size, num_experts=cfg.num_moe_experts,
                        tie_embeddings=not cfg.untie_embeddings_and_output_weights)
    save_hf(hf, out_dir, hf_config or hf_config_from_model(cfg, family))
    if world > 1:
        dist.barrier()
