"""Training entry point: ``torchrun ... -m loongforge_b200.train <flags> [yaml overrides]``
(same role and flag spelling as the reference's loongforge/train.py:17-27)."""
from __future__ import annotations

import os
import sys
from typing import List, Optional


def main(argv: Optional[List[str]] = None) -> int:
    import torch.distributed as dist

    from .config.arguments import parse_args
    from .config.build import build_configs
    from .data.synthetic import synthetic_batch_iterator
    from .runtime.trainer import init_distributed
    from .runtime.trainer_builder import build_model_trainer

    args, overrides = parse_args(argv)
    from .config.validators import apply_aliases, unwired_flag_notes
    apply_aliases(args)
    device = init_distributed(backend=args.distributed_backend if args.distributed_backend == "gloo" else None,
                              timeout_s=args.distributed_timeout_minutes * 60)
    model_cfg, train_cfg, dims, raw = build_configs(args, overrides)
    # process-wide handles: library code far from the trainer (tokenizer / template helpers, position-id functions,
    # user hooks) reads the parsed arguments, the composed YAML and the model configuration from here
    from .config import global_vars
    global_vars.set_args(args)
    global_vars.set_yaml_config(raw)
    global_vars.set_model_config(model_cfg)
    rank = dist.get_rank() if dist.is_initialized() else 0
    if rank == 0:
        print("------------------------ arguments ------------------------", flush=True)
        for k, v in sorted(vars(args).items()):
            print(f"  {k} {'.' * max(1, 48 - len(k))} {v}", flush=True)
        print("-------------------- end of arguments ---------------------", flush=True)
        for note in unwired_flag_notes(args):
            print(f"WARNING: {note}", flush=True)
    if args.cp_comm_type not in ("auto", None):
        from .parallel.context_parallel import set_cp_comm_type
        kinds = ("p2p", "allgather", "a2a", "a2a+p2p")
        set_cp_comm_type(args.cp_comm_type if args.cp_comm_type in kinds else "auto",
                         getattr(args, "context_parallel_ulysses_degree", None))
    if args.attention_backend in ("native", "sdpa"):
        from .ops.functional import set_attention_impl
        set_attention_impl(args.attention_backend)
    node = raw.get("model", raw) if isinstance(raw, dict) else {}
    family = (node.get("model_type") if isinstance(node, dict) and "foundation" in node else None) or model_cfg.model_family
    extra = {}
    enc = node.get("image_encoder") if isinstance(node, dict) else None
    if isinstance(enc, dict):
        # VLM YAML: the encoder section becomes its own config; its model_type selects the encoder family
        from .config.build import transformer_config_from_yaml
        from .models.vision_zoo import VISION_FAMILIES
        vt = str(enc.get("model_type", "qwen2_5_vit"))
        extra["vit_cfg"] = transformer_config_from_yaml({k: v for k, v in enc.items() if not isinstance(v, dict)
                                                          and k not in ("freeze", "vision_options")})
        extra["vision_family"] = vt if vt in VISION_FAMILIES else "qwen2_vit"
        extra["vision_options"] = enc.get("vision_options")
        extra["freeze_encoder"] = bool(enc.get("freeze", False))
        extra["encoder_tp"] = int(getattr(args, "encoder_tensor_model_parallel_size", None) or 1)
        extra["encoder_hetero_dp"] = bool(getattr(args, "enable_encoder_hetero_dp", False))
        extra["full_hetero_dp"] = bool(getattr(args, "enable_full_hetero_dp", False))
        extra["full_hetero_cpu_offload"] = bool(getattr(args, "full_hetero_dp_cpu_offload", False))
        if getattr(args, "image_resolution", None):
            extra["image_size"] = int(args.image_resolution)
    peft = node.get("peft_config") if isinstance(node, dict) else None
    if isinstance(peft, dict) and train_cfg.training_phase == "sft":
        # adapters described in the model YAML (configs/models/lora/*.yaml composed as `model.peft_config`)
        extra["lora"] = dict(rank=int(peft.get("dim", peft.get("rank", 16))), alpha=float(peft.get("alpha", 32)),
                             dropout=float(peft.get("dropout", 0.0)),
                             targets=tuple(peft.get("target_modules") or ("linear_qkv", "linear_proj", "linear_fc1", "linear_fc2")),
                             canonical=bool(peft.get("canonical", False)))
        if isinstance(enc, dict):
            extra["lora"].update(apply_to_foundation=bool(peft.get("apply_to_foundation", True)),
                                 apply_to_image_encoder=bool(peft.get("apply_to_image_encoder", False)),
                                 apply_to_image_projector=bool(peft.get("apply_to_image_projector", False)))
    if getattr(args, "peft_type", None) and train_cfg.training_phase == "sft" and "lora" not in extra:
        extra["lora"] = dict(rank=args.lora_rank, alpha=args.lora_alpha, dropout=args.lora_dropout,
                             targets=tuple(args.lora_target_modules), canonical=args.peft_type == "canonical_lora")
        if isinstance(enc, dict):  # vision-language model: which components get adapters
            extra["lora"].update(apply_to_foundation=not getattr(args, "lora_skip_foundation", False),
                                 apply_to_image_encoder=bool(getattr(args, "lora_apply_to_image_encoder", False)),
                                 apply_to_image_projector=bool(getattr(args, "lora_apply_to_image_projector", False)))
    from .runtime.diffusion_trainer import build_diffusion_trainer, is_diffusion_model
    if is_diffusion_model(args.model_name):
        # diffusion transformers (WAN, Qwen-Image): their own model configuration, the common loop around it
        over = {k: v for k, v in (("num_layers", args.num_layers), ("hidden_size", args.hidden_size),
                                  ("ffn_hidden_size", args.ffn_hidden_size), ("num_heads", args.num_attention_heads))
                if v is not None}
        trainer = build_diffusion_trainer(args.model_name, train_cfg, dims, device=device, dit_overrides=over,
                                          recompute=args.recompute_granularity == "full")
        family = trainer.kind
    else:
        trainer = build_model_trainer(family, train_cfg.training_phase, model_cfg=model_cfg, train_cfg=train_cfg,
                                      dims=dims, device=device, **extra)
    _load_initial_state(trainer, args, train_cfg, family)
    data_iter = trainer.build_data_iterator(args) if hasattr(trainer, "build_data_iterator") else None
    prefetch = None
    collective_in_data_path = bool(getattr(args, "use_vlm_dp_balance", False) or getattr(args, "enable_full_hetero_dp", False))
    if data_iter is not None and int(getattr(args, "num_workers", 0) or 0) > 0 and not collective_in_data_path:
        # (data paths that exchange samples between ranks stay in the training thread: their collectives must keep
        # their order relative to the step's)
        from .data.samplers import PrefetchIterator
        data_iter = prefetch = PrefetchIterator(data_iter, depth=2 * int(args.num_workers))   # host work overlaps the step
    if data_iter is None:
        st = trainer.st
        data_iter = synthetic_batch_iterator(model_cfg.vocab_size, train_cfg.seq_length, train_cfg.micro_batch_size,
                                             dp_rank=st.dp_rank, dp_size=st.dp_size, seed=train_cfg.seed,
                                             start_sample=trainer.consumed_samples)
    from .runtime.hooks import build_hooks
    trainer.hooks = build_hooks(args, trainer)
    trainer.train(data_iter)
    if prefetch is not None:
        prefetch.close()
    if train_cfg.save:
        trainer.save_checkpoint(train_cfg.save)
    if _truthy(getattr(args, "save_hf", False)) and trainer.iteration >= train_cfg.train_iters:
        # Hugging Face weights of the final model (reference: loongforge/train/training_utils.py:622-632)
        from .ckpt.hf_bridge import save_hf_checkpoint
        out = args.save_hf_path or (os.path.join(train_cfg.save, "release_hf_weights") if train_cfg.save else None)
        if out is None:
            raise ValueError("--save-hf needs --save-hf-path or --save")
        save_hf_checkpoint(trainer, out, family=_hf_family(family, model_cfg))
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    return 0


def _truthy(v) -> bool:
    return v is True or str(v).lower() in ("1", "true", "yes")


def _hf_family(family: str, cfg) -> str:
    """Key of the Hugging Face name map (tools/convert_checkpoint/name_maps.py) for a model family."""
    from tools.convert_checkpoint.name_maps import FAMILIES, VLM_FAMILIES
    if family in VLM_FAMILIES:
        return family
    if family == "qwen3" and cfg.num_moe_experts:
        return "qwen3_moe"
    if family in FAMILIES:
        return family
    return {"llama": "llama3", "qwen": "qwen2"}.get(family, "llama3")


def is_hf_checkpoint(path: Optional[str]) -> bool:
    return bool(path) and os.path.isfile(os.path.join(path, "config.json")) and any(
        f.endswith((".safetensors", ".bin")) for f in os.listdir(path))


def _load_initial_state(trainer, args, train_cfg, family: str) -> str:
    """Where training starts from, in the reference's order of precedence (loongforge/train/training_utils.py:1184-1204,
    loongforge/train/checkpointing.py:1721-1730): a checkpoint of THIS run under ``--load`` (resume: weights, optimizer,
    RNG, iteration; ``--ckpt-step`` picks the iteration); else Hugging Face weights (``--load`` pointing at an HF
    directory, or ``--load-hf --hf-checkpoint-path``); else ``--pretrained-checkpoint`` (weights only, iteration 0).
    ``--finetune`` keeps the weights of whatever was loaded and starts the schedule from iteration 0."""
    from .ckpt.checkpointing import read_tracker

    hf_dir = args.hf_checkpoint_path if getattr(args, "load_hf", False) else None
    if hf_dir is None and is_hf_checkpoint(train_cfg.load):
        hf_dir = train_cfg.load
    resume_dir = train_cfg.load if (train_cfg.load and hf_dir != train_cfg.load) else None
    has_own = bool(resume_dir) and os.path.isdir(resume_dir) and (
        read_tracker(resume_dir)[0] is not None or getattr(args, "ckpt_step", None) is not None)
    how = "scratch"
    if has_own:
        finetune = bool(args.finetune)
        trainer.load_checkpoint(resume_dir, load_optim=not args.no_load_optim and not finetune,
                                load_rng=not args.no_load_rng and not finetune,
                                **({"iteration": args.ckpt_step} if getattr(args, "ckpt_step", None) is not None else {}))
        how = "resume"
        if finetune:
            trainer.iteration, trainer.consumed_samples, trainer.num_flops_so_far = 0, 0, 0.0
            how = "finetune"
    elif hf_dir:
        from .ckpt.hf_bridge import load_hf_checkpoint_online
        load_hf_checkpoint_online(trainer, hf_dir, family=_hf_family(family, trainer.mcfg),
                                  upcycle=bool(getattr(args, "moe_use_upcycling", False)))
        trainer.optimizer.reload_model_params()
        how = "hf"
    elif getattr(args, "pretrained_checkpoint", None):
        trainer.load_checkpoint(args.pretrained_checkpoint, load_optim=False, load_rng=False)
        trainer.iteration, trainer.consumed_samples, trainer.num_flops_so_far = 0, 0, 0.0
        how = "pretrained"
    return how


if __name__ == "__main__":
    sys.exit(main())
