"""Turn (CLI args, model YAML) into the three config objects the runtime uses, with validation.

Mirrors the reference's flow: model name -> YAML (loongforge/utils/config_map.py:439-460), YAML keys
copied onto the args / config dataclass (loongforge/train/validators.py:79-122), Megatron-style
consistency checks (validators.py:140-620). YAML keys use the reference's spelling; the table
below maps the ones whose name differs from ``TransformerConfig``.
"""
from __future__ import annotations

import dataclasses
import os
from typing import Any, Dict, List, Optional, Tuple

import torch

from ..models.config import TransformerConfig
from ..models.registry import get_model_config, list_models
from ..parallel.state import ParallelDims
from ..runtime.trainer import TrainConfig
from . import yaml_compose

REPO_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
CONFIG_DIR = os.path.join(REPO_ROOT, "configs", "models")

# model name -> yaml path relative to configs/models (names follow the reference's --model-name values)
def _scan_model_yaml() -> Dict[str, str]:
    """Every ``configs/models/<dir>/<file>.yaml`` whose first line is ``# <model-name> (...)`` registers that name."""
    out: Dict[str, str] = {}
    if not os.path.isdir(CONFIG_DIR):
        return out
    for d in sorted(os.listdir(CONFIG_DIR)):
        sub = os.path.join(CONFIG_DIR, d)
        if not os.path.isdir(sub):
            continue
        for f in sorted(os.listdir(sub)):
            if f.endswith(".yaml"):
                with open(os.path.join(sub, f)) as fh:
                    first = fh.readline()
                if first.startswith("# ") and "(" in first:
                    out[first[2:first.index("(")].strip().lower()] = f"{d}/{f}"
    return out


MODEL_YAML = {
    "llama3-8b": "llama3/llama3_8b.yaml",
    "qwen2.5-7b": "qwen2.5/qwen2_5_7b.yaml",
    "qwen3-30b-a3b": "qwen3/qwen3_30b_a3b.yaml",
    "deepseek-v3.2": "deepseek3/deepseek_v3_2.yaml",
    "qwen2.5-vl-7b": "qwen2.5vl/qwen2_5_vl_7b.yaml",
    **_scan_model_yaml(),
}

_YAML_ALIASES = {"norm_epsilon": "layernorm_epsilon", "num_experts": "num_moe_experts",
                 "rotary_emb_base": "rotary_base", "activation_func": "activation"}
_FIELDS = {f.name for f in dataclasses.fields(TransformerConfig)}


def family_of(model_type: Optional[str]) -> str:
    mt = (model_type or "llama").lower()
    for fam in ("deepseek", "qwen3", "qwen2", "llama", "glm", "internlm", "minimax", "mimo", "ernie"):
        if mt.startswith(fam) or fam in mt:
            return fam
    return mt


def transformer_config_from_yaml(node: Dict[str, Any], base: Optional[TransformerConfig] = None) -> TransformerConfig:
    """One model section of a YAML file -> TransformerConfig (unknown keys are kept in ``.extra``)."""
    kw: Dict[str, Any] = dataclasses.asdict(base) if base is not None else {}
    extra: Dict[str, Any] = {}
    for k, v in node.items():
        k2 = _YAML_ALIASES.get(k, k)
        if k2 == "swiglu":
            if v:
                kw["activation"], kw["gated_linear_unit"] = "swiglu", True
        elif k2 == "group_query_attention":
            extra[k] = v
        elif k2 == "model_type":
            kw["model_family"] = family_of(v)
            extra[k] = v
        elif k2 == "moe_layer_freq" and isinstance(v, str):
            kw[k2] = yaml_compose._moe_freq(v)
        elif k2 in _FIELDS:
            kw[k2] = v
        else:
            extra[k] = v
    if extra.get("group_query_attention") is False:
        kw["num_query_groups"] = None
    if isinstance(kw.get("params_dtype"), str):
        kw["params_dtype"] = getattr(torch, kw["params_dtype"].replace("torch.", ""))
    cfg = TransformerConfig(**kw)
    cfg.extra = extra
    return cfg


def load_model_yaml(args, overrides: List[str]) -> Optional[dict]:
    path = args.config_file
    if path is None and args.model_name:
        rel = MODEL_YAML.get(args.model_name.lower().replace("_", "-"))
        if rel and os.path.isfile(os.path.join(CONFIG_DIR, rel)):
            path = os.path.join(CONFIG_DIR, rel)
    if path is None:
        return None
    os.environ.setdefault("LOONGFORGE_PATH", REPO_ROOT)
    return yaml_compose.compose(path, overrides)


_ARG_TO_CFG = {
    "num_layers": "num_layers", "hidden_size": "hidden_size", "ffn_hidden_size": "ffn_hidden_size",
    "num_attention_heads": "num_attention_heads", "num_query_groups": "num_query_groups",
    "kv_channels": "kv_channels", "max_position_embeddings": "max_position_embeddings",
    "position_embedding_type": "position_embedding_type", "rotary_base": "rotary_base",
    "rotary_percent": "rotary_percent", "rotary_scaling_factor": "rotary_scaling_factor",
    "normalization": "normalization", "norm_epsilon": "layernorm_epsilon", "init_method_std": "init_method_std",
    "vocab_size": "vocab_size", "num_experts": "num_moe_experts", "moe_router_topk": "moe_router_topk",
    "moe_ffn_hidden_size": "moe_ffn_hidden_size",
    "moe_shared_expert_intermediate_size": "moe_shared_expert_intermediate_size",
    "moe_shared_expert_gate": "moe_shared_expert_gate",
    "moe_router_score_function": "moe_router_score_function",
    "moe_router_bias_update_rate": "moe_router_bias_update_rate", "moe_router_num_groups": "moe_router_num_groups",
    "moe_router_group_topk": "moe_router_group_topk",
    "moe_router_topk_scaling_factor": "moe_router_topk_scaling_factor",
    "moe_router_load_balancing_type": "moe_router_load_balancing_type", "moe_aux_loss_coeff": "moe_aux_loss_coeff",
    "moe_z_loss_coeff": "moe_z_loss_coeff", "mtp_num_layers": "mtp_num_layers",
    "mtp_loss_scaling_factor": "mtp_loss_scaling_factor", "moe_token_dispatcher_type": "moe_token_dispatcher_type",
    "recompute_granularity": "recompute_granularity",
    "recompute_method": "recompute_method", "recompute_num_layers": "recompute_num_layers",
    "attention_dropout": "attention_dropout", "hidden_dropout": "hidden_dropout",
}
_FLAG_TO_CFG = {"swiglu": ("activation", "swiglu"), "add_qkv_bias": ("add_qkv_bias", True),
                "qk_layernorm": ("qk_layernorm", True), "disable_bias_linear": ("add_bias_linear", False),
                "untie_embeddings_and_output_weights": ("untie_embeddings_and_output_weights", True),
                "moe_router_pre_softmax": ("moe_router_pre_softmax", True),
                "moe_router_enable_expert_bias": ("moe_router_enable_expert_bias", True),
                "multi_latent_attention": ("multi_latent_attention", True), "use_dsa_fused": ("use_dsa", True),
                "use_dsa_sp_first": ("dsa_sp_first", True),
                "sequence_parallel": ("sequence_parallel", True), "tp_comm_overlap": ("tp_comm_overlap", True),
                "no_gradient_accumulation_fusion": ("gradient_accumulation_fusion", False),
                "moe_grouped_gemm": ("moe_grouped_gemm", True),
                "cross_entropy_loss_fusion": ("cross_entropy_loss_fusion", True)}


def build_configs(args, overrides: Optional[List[str]] = None) -> Tuple[TransformerConfig, TrainConfig, ParallelDims, dict]:
    """(model config, train config, parallel dims, raw yaml). Raises ValueError on inconsistent input."""
    overrides = overrides or []
    raw = load_model_yaml(args, overrides) or {}
    node = raw.get("model", raw) if isinstance(raw, dict) else {}
    lm_node = node.get("foundation", node) if isinstance(node, dict) else {}
    base = None
    if args.model_name and args.model_name.lower().replace("_", "-") in list_models():
        base = get_model_config(args.model_name)
    if lm_node:
        cfg = transformer_config_from_yaml({k: v for k, v in lm_node.items() if not isinstance(v, dict)}, base)
    elif base is not None:
        cfg = base
    else:
        cfg = TransformerConfig()
    for a, c in _ARG_TO_CFG.items():
        v = getattr(args, a, None)
        if v is not None:
            setattr(cfg, c, v)
    for a, (c, val) in _FLAG_TO_CFG.items():
        if getattr(args, a, False):
            setattr(cfg, c, val)
    if isinstance(getattr(args, "moe_layer_freq", None), str):
        cfg.moe_layer_freq = yaml_compose._moe_freq(args.moe_layer_freq)
    if cfg.fp8 is None and args.fp8_format:
        cfg.fp8 = "blockwise" if (args.fp8_recipe or "blockwise") == "blockwise" else args.fp8_recipe
    cfg.__post_init__()
    vpp = args.num_virtual_stages_per_pipeline_rank
    per_virtual = getattr(args, "num_layers_per_virtual_pipeline_stage", None)
    if not vpp and per_virtual:
        pp_ = args.pipeline_model_parallel_size
        if cfg.num_layers % (pp_ * per_virtual):
            raise ValueError("num_layers must divide by pipeline size x layers per virtual stage")
        vpp = cfg.num_layers // (pp_ * per_virtual)
    dims = ParallelDims(tp=args.tensor_model_parallel_size, pp=args.pipeline_model_parallel_size,
                        cp=args.context_parallel_size, ep=args.expert_model_parallel_size,
                        etp=args.expert_tensor_parallel_size, vpp=vpp)
    dt = {"fp32": torch.float32, "bf16": torch.bfloat16}
    from ..parallel.pipeline_layout import resolve_stage_layers
    _ints = lambda v: [int(x) for x in v.split(",") if x.strip()] if v else None  # noqa: E731
    custom_layers = resolve_stage_layers(
        cfg.num_layers, dims.pp, dims.vpp or 1, layout=getattr(args, "pipeline_model_parallel_layout", None),
        custom_pipeline_layers=_ints(args.custom_pipeline_layers),
        custom_virtual_pipeline_layers=_ints(getattr(args, "custom_virtual_pipeline_layers", None)),
        mtp_num_layers=cfg.mtp_num_layers)
    recompute_layers = _ints(getattr(args, "custom_pipeline_recompute_layers", None))
    if recompute_layers is not None and len(recompute_layers) != dims.pp:
        raise ValueError("--custom-pipeline-recompute-layers needs one count per pipeline stage")
    gbs = args.global_batch_size or args.micro_batch_size
    train_iters = args.train_iters or 0
    if not train_iters and getattr(args, "train_samples", None):
        train_iters = int(args.train_samples) // gbs  # sample-based length (constant batch size)
    decay_iters = args.lr_decay_iters
    warmup_iters = args.lr_warmup_iters
    if getattr(args, "lr_warmup_fraction", None) is not None:
        warmup_iters = int(float(args.lr_warmup_fraction) * (decay_iters or train_iters))
    tc = TrainConfig(
        micro_batch_size=args.micro_batch_size, global_batch_size=gbs,
        seq_length=args.seq_length or cfg.max_position_embeddings, train_iters=train_iters, lr=args.lr,
        min_lr=args.min_lr, lr_decay_style=args.lr_decay_style, lr_warmup_iters=warmup_iters,
        lr_decay_iters=decay_iters, rampup_batch_size=getattr(args, "rampup_batch_size", None),
        grad_reduce_in_fp32=(True if getattr(args, "accumulate_allreduce_grads_in_fp32", False) or args.bf16 else False), weight_decay=args.weight_decay, adam_beta1=args.adam_beta1,
        adam_beta2=args.adam_beta2, adam_eps=args.adam_eps, clip_grad=args.clip_grad, bf16=args.bf16, seed=args.seed,
        log_interval=args.log_interval, save=args.save, load=args.load, save_interval=args.save_interval,
        ckpt_format="torch_dist" if args.ckpt_format in ("torch_dist", "torch_dcp") else args.ckpt_format,
        async_save=bool(getattr(args, "async_save", False)),
        fp8_policy_file=getattr(args, "fp8_dynamic_policy_path", None),
        chunkpipe_chunks=(max(1, args.seq_length // int(args.chunksize))
                          if getattr(args, "enable_chunkpipe", False) and getattr(args, "chunksize", None) else 0),
        overlap_moe_expert_parallel_comm=bool(getattr(args, "overlap_moe_expert_parallel_comm", False)),
        rerun_mode=getattr(args, "rerun_mode", "disabled") or "disabled",
        error_injection_rate=int(getattr(args, "error_injection_rate", 0) or 0),
        error_injection_type=getattr(args, "error_injection_type", "transient_error"),
        iterations_to_skip=list(getattr(args, "iterations_to_skip", []) or []),
        check_weight_hash_interval=int(getattr(args, "check_weight_hash_across_dp_replicas_interval", 0) or 0),
        eval_interval=int(getattr(args, "eval_interval", 0) or 0), eval_iters=int(getattr(args, "eval_iters", 0) or 0),
        no_save_optim=bool(getattr(args, "no_save_optim", False)), no_save_rng=bool(getattr(args, "no_save_rng", False)),
        log_memory_stats=bool(getattr(args, "log_memory_stats", False)),
        dp_balance=bool(getattr(args, "use_vlm_dp_balance", False)),
        optimizer_cpu_offload=bool(getattr(args, "optimizer_cpu_offload", False)),
        timing_log_level=int(getattr(args, "timing_log_level", 0) or 0),
        log_timers_to_tensorboard=bool(getattr(args, "log_timers_to_tensorboard", False)),
        optimizer_offload_fraction=float(getattr(args, "optimizer_offload_fraction", 1.0) or 0.0),
        optimizer=(getattr(args, "optimizer", None) or "adam").lower(), sgd_momentum=getattr(args, "sgd_momentum", 0.9),
        use_fsdp=bool(getattr(args, "use_torch_fsdp2", False) or getattr(args, "use_megatron_fsdp", False)),
        fsdp_sharding_strategy=getattr(args, "data_parallel_sharding_strategy", None) or "optim_grads_params",
        use_distributed_optimizer=args.use_distributed_optimizer, overlap_grad_reduce=args.overlap_grad_reduce,
        overlap_param_gather=args.overlap_param_gather, exp_avg_dtype=dt[args.exp_avg_dtype],
        exp_avg_sq_dtype=dt[args.exp_avg_sq_dtype], calculate_per_token_loss=args.calculate_per_token_loss,
        custom_pipeline_layers=custom_layers, custom_pipeline_recompute_layers=recompute_layers, training_phase=args.training_phase,
        freeze_parameters=list(getattr(args, "freeze_parameters", None) or []),
        freeze_parameters_regex=getattr(args, "freeze_parameters_regex", None),
        trainable_modules=list(getattr(args, "trainable_modules", None) or []),
        check_for_nan_in_loss=not bool(getattr(args, "no_check_for_nan_in_loss_and_grad", False)),
        log_throughput=True)  # --log-throughput: the TFLOP/s field is always part of the log line
    from .validators import validate
    validate(args, cfg, tc, dims)
    return cfg, tc, dims, raw
