"""Three-layer configuration of the embodied stack: CLI overrides > YAML file > dataclass defaults, with a
model-name -> YAML map and validators (reference: loongforge/embodied/train/parser.py, training_args.py,
config_map.py, validators.py)."""
from __future__ import annotations

import argparse
import dataclasses
import os
from typing import Any, Dict, List, Optional

import yaml


@dataclasses.dataclass
class EmbodiedArgs:
    # ---- model / data
    model_name: str = "pi05"
    model_overrides: Dict[str, Any] = dataclasses.field(default_factory=dict)
    dataset_type: str = "synthetic"  # synthetic | npz_episodes | lerobot | hdf5
    dataset_path: Optional[str] = None
    action_horizon: int = 16
    action_dim: int = 7
    state_dim: int = 8
    image_size: int = 56
    num_cameras: int = 1
    max_text_len: int = 16
    use_transforms: bool = False       # per-policy sample pipeline of embodied/transforms.py (resize, augment, normalise, prompt / ids)
    stats_path: Optional[str] = None   # stats.json (or a data-set directory with meta/stats.json); else computed and stored in output_dir
    stats_samples: int = 2048          # samples read when the statistics are computed here
    normalization_mode: Optional[str] = None  # mean_std | min_max | q99 | scale | identity; default by policy
    image_augmentation: bool = False
    image_resize_mode: str = "pad"     # pad | crop | stretch
    relative_action_mask: List[bool] = dataclasses.field(default_factory=list)  # channels trained as offsets from the state
    embodiment_tags: Dict[str, int] = dataclasses.field(default_factory=dict)   # tag / domain name -> id
    robot_description: Optional[str] = None
    dataset_mixture: List[Dict[str, Any]] = dataclasses.field(default_factory=list)  # [{type, path, weight}]: several data sets in fixed proportions
    mixture_epoch_length: Optional[int] = None
    precomputed_cache: Optional[str] = None  # features written by tools/data_preprocess/embodied_precompute.py
    video_frames: int = 0  # world-model policies: future frames per sample (1 + 4k; 0 = none), camera 0, one per `video_frame_stride` steps
    video_frame_stride: int = 1
    # ---- optimisation
    train_steps: int = 100
    per_device_batch_size: int = 4
    gradient_accumulation_steps: int = 1
    lr: float = 1e-4
    min_lr: float = 0.0
    weight_decay: float = 0.01
    warmup_steps: int = 0
    lr_scheduler: str = "cosine"  # constant | linear | cosine | cosine_restarts | polynomial | wsd
    lr_decay_steps: Optional[int] = None   # where the decay ends (default: train_steps)
    lr_num_cycles: int = 1
    lr_power: float = 1.0
    lr_mults: Dict[str, float] = dataclasses.field(default_factory=dict)  # parameter-name prefix -> lr multiplier
    optimizer: str = "adamw"      # adamw | adam | sgd | lion
    adam_eps: float = 1e-8
    adam_beta1: float = 0.9
    adam_beta2: float = 0.95
    max_grad_norm: float = 1.0
    nan_clean: bool = True
    bf16: bool = False
    seed: int = 1234
    deterministic_mode: bool = False   # deterministic algorithms + no cuDNN autotuning
    disable_tf32: bool = False
    check_for_nan_in_loss: bool = True  # stop with an error when the loss is not finite
    pretrained_checkpoint: Optional[str] = None  # .pt / .safetensors file or a directory of them: weights loaded before training
    pretrained_strict: bool = False
    freeze_modules: List[str] = dataclasses.field(default_factory=list)  # dot paths or globs of sub-modules kept frozen
    num_workers: int = 0
    video_backend: str = "opencv"  # opencv | pyav | decord | torchcodec (the last three when installed)
    sampler: str = "distributed"  # distributed (samples dealt to ranks) | block_shard (whole batches dealt to ranks)
    save_training_state: bool = True   # False: checkpoints hold the weights only
    async_save: bool = False           # pt format: the file is written by a background thread from a CPU copy
    profile_step_start: int = -1       # torch profiler over [start, end) on rank 0, trace in output_dir/profile
    profile_step_end: int = -1
    fsdp_param_dtype: Optional[str] = None    # FSDP mixed precision: dtype of the gathered parameters (bf16)
    fsdp_reduce_dtype: Optional[str] = None   # ... and of the gradient reduce-scatter (fp32)
    ddp_find_unused_parameters: bool = False
    ddp_broadcast_buffers: bool = True
    # ---- distribution
    strategy: str = "ddp"  # ddp | zero1 | fsdp | hsdp
    fsdp_wrap_patterns: List[str] = dataclasses.field(default_factory=lambda: ["blocks.*", "layers.*"])
    fsdp_prefetch: int = 1
    fsdp_min_num_params: int = 1_000_000            # automatic plan ([auto]): smallest group of repeated layers
    fsdp_leftover_min_num_params: int = 10_000_000  # ... and smallest single leaf that gets a unit of its own
    fsdp_no_wrap_modules: List[str] = dataclasses.field(default_factory=list)  # class names never taken as one unit
    fsdp_reshard_default: Any = True                # reshard_after_forward of the units (bool or int)
    fsdp_reshard_root: Any = False
    fsdp_reshard_module_overrides: Dict[str, Any] = dataclasses.field(default_factory=dict)  # glob -> bool | int
    hsdp_shard_size: Optional[int] = None
    ddp_bucket_mb: int = 25
    ddp_comm_hook: Optional[str] = None  # None | bf16_compress
    ddp_static_graph: bool = True
    activation_checkpoint_patterns: List[str] = dataclasses.field(default_factory=list)
    fp32_master_weights: bool = False
    # ---- LoRA
    lora_rank: int = 0
    lora_alpha: float = 16.0
    lora_targets: List[str] = dataclasses.field(default_factory=lambda: ["q", "k", "v", "o"])  # names, globs, all-linear; [] = the policy's own
    lora_dropout: float = 0.0
    lora_use_rslora: bool = False
    lora_init: str = "kaiming"  # kaiming | gaussian
    lora_exclude: List[str] = dataclasses.field(default_factory=list)
    lora_modules_to_save: List[str] = dataclasses.field(default_factory=list)
    lora_adapter_path: Optional[str] = None  # start from a stored adapter (directory with adapter_model.pt + adapter_config.json)
    # ---- CUDA graphs
    per_microbatch_cuda_graph: bool = False
    cuda_graph_warmup_steps: int = 3       # eager micro-batches per input signature before capture
    cuda_graph_pad_length: int = 1         # token fields are padded to a multiple of this (fewer distinct signatures)
    cuda_graph_max_graphs: int = 4
    # ---- checkpoint / logging
    output_dir: str = "./outputs"
    save_interval: int = 0
    checkpoint_format: str = "pt"  # pt | dcp
    resume: bool = False
    log_interval: int = 1
    log_stage_times: bool = False      # data / forward-backward / optimizer time per step, slowest rank
    tensorboard: bool = False
    wandb_project: Optional[str] = None  # written offline unless WANDB_MODE says otherwise
    run_name: Optional[str] = None
    manual_gc_interval: int = 0


MODEL_CONFIG_MAP = {name: f"configs/embodied/{name}.yaml" for name in
                    ("pi05", "groot_n1_6", "groot_n1_7", "xvla", "lingbot_va", "fastwam", "dreamzero", "cosmos3")}


def validate(a: EmbodiedArgs) -> EmbodiedArgs:
    if a.strategy not in ("ddp", "zero1", "fsdp", "hsdp"):
        raise ValueError(f"unknown strategy {a.strategy}")
    if a.strategy == "hsdp" and not a.hsdp_shard_size:
        raise ValueError("hsdp needs hsdp_shard_size")
    if a.gradient_accumulation_steps < 1 or a.per_device_batch_size < 1:
        raise ValueError("batch sizes must be positive")
    if a.checkpoint_format not in ("pt", "dcp"):
        raise ValueError(f"unknown checkpoint format {a.checkpoint_format}")
    if a.per_microbatch_cuda_graph and a.strategy in ("fsdp", "hsdp"):
        raise ValueError("per-microbatch CUDA graphs need parameters resident on the device (ddp / zero1)")
    if a.lr_scheduler not in ("constant", "linear", "cosine", "cosine_restarts", "polynomial", "wsd"):
        raise ValueError(f"unknown lr_scheduler {a.lr_scheduler}")
    if a.optimizer not in ("adamw", "adam", "sgd", "lion"):
        raise ValueError(f"unknown optimizer {a.optimizer}")
    if a.async_save and a.checkpoint_format != "pt":
        raise ValueError("async_save writes the single-file format (checkpoint_format: pt)")
    if a.ddp_find_unused_parameters and a.ddp_static_graph:
        a.ddp_static_graph = False  # a static graph cannot have parameters that come and go
    if a.lora_rank < 0:
        raise ValueError("lora_rank must be >= 0")
    return a


def _coerce(value: str, current: Any) -> Any:
    if isinstance(current, bool):
        return value.lower() in ("1", "true", "yes")
    if isinstance(current, (list, dict)) or current is None:
        return yaml.safe_load(value)
    return type(current)(value)


def parse_args(argv: Optional[List[str]] = None, repo_root: Optional[str] = None) -> EmbodiedArgs:
    """``--config file.yaml`` or ``--model-name NAME`` (looked up in MODEL_CONFIG_MAP) plus ``key=value`` overrides."""
    ap = argparse.ArgumentParser("loongforge_b200.embodied.train")
    ap.add_argument("--config", default=None)
    ap.add_argument("--model-name", default=None)
    ap.add_argument("overrides", nargs="*")
    ns = ap.parse_args(argv)
    args = EmbodiedArgs()
    path = ns.config
    if path is None and ns.model_name:
        cand = os.path.join(repo_root or os.getcwd(), MODEL_CONFIG_MAP.get(ns.model_name, ""))
        path = cand if os.path.isfile(cand) else None
        args.model_name = ns.model_name
    if path:
        with open(path) as f:
            for k, v in (yaml.safe_load(f) or {}).items():
                if not hasattr(args, k):
                    raise KeyError(f"unknown config key {k!r} in {path}")
                setattr(args, k, v)
    for ov in ns.overrides:
        k, _, v = ov.partition("=")
        k = k.lstrip("-").replace("-", "_")
        if not hasattr(args, k):
            raise KeyError(f"unknown override {k!r}")
        setattr(args, k, _coerce(v, getattr(args, k)))
    return validate(args)


_GLOBAL: Dict[str, Any] = {}


def set_global_args(a: EmbodiedArgs) -> None:
    _GLOBAL["args"] = a


def get_global_args() -> EmbodiedArgs:
    return _GLOBAL["args"]
