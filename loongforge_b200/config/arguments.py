"""Command-line interface: Megatron-style training flags plus the framework's own groups.

The reference parses Megatron's argparse flags first and its own groups second, with
``parse_known_args`` so that left-over tokens become YAML overrides
(loongforge/train/parser.py:80-108, loongforge/train/arguments.py:23-53,95-1439). Flag spellings
are kept so that the reference's launch scripts (examples/**/*.sh) drive this framework unchanged;
flags that select a code path this framework does not have are accepted and validated in
``validators.py``.
"""
from __future__ import annotations

import argparse
from typing import List, Optional, Tuple


def _add_model_args(p: argparse.ArgumentParser):
    g = p.add_argument_group("model")
    g.add_argument("--model-name", type=str, default=None, help="registered model name (see models/registry.py)")
    g.add_argument("--config-file", type=str, default=None, help="model YAML (same schema as configs/models/**)")
    g.add_argument("--num-layers", type=int, default=None)
    g.add_argument("--hidden-size", type=int, default=None)
    g.add_argument("--ffn-hidden-size", type=int, default=None)
    g.add_argument("--num-attention-heads", type=int, default=None)
    g.add_argument("--num-query-groups", type=int, default=None)
    g.add_argument("--group-query-attention", action="store_true")
    g.add_argument("--kv-channels", type=int, default=None)
    g.add_argument("--max-position-embeddings", type=int, default=None)
    g.add_argument("--position-embedding-type", type=str, default=None)
    g.add_argument("--rotary-base", type=float, default=None)
    g.add_argument("--rotary-percent", type=float, default=None)
    g.add_argument("--rotary-scaling-factor", type=float, default=None)
    g.add_argument("--normalization", type=str, default=None)
    g.add_argument("--norm-epsilon", type=float, default=None)
    g.add_argument("--swiglu", action="store_true")
    g.add_argument("--disable-bias-linear", action="store_true")
    g.add_argument("--add-qkv-bias", action="store_true")
    g.add_argument("--qk-layernorm", action="store_true")
    g.add_argument("--untie-embeddings-and-output-weights", action="store_true")
    g.add_argument("--init-method-std", type=float, default=None)
    g.add_argument("--attention-dropout", type=float, default=None)
    g.add_argument("--hidden-dropout", type=float, default=None)
    g.add_argument("--vocab-size", type=int, default=None)
    g.add_argument("--make-vocab-size-divisible-by", type=int, default=128)
    g.add_argument("--attention-backend", type=str, default="auto", choices=["auto", "native", "flash", "fused", "sdpa"])
    g.add_argument("--use-dsa-fused", action="store_true")
    g.add_argument("--use-dsa-sp-first", action="store_true")
    g.add_argument("--absorb-backend", type=str, default="einsum")
    g.add_argument("--multi-latent-attention", action="store_true")
    g.add_argument("--mtp-num-layers", type=int, default=None)
    g.add_argument("--mtp-loss-scaling-factor", type=float, default=None)


def _add_moe_args(p):
    g = p.add_argument_group("moe")
    g.add_argument("--num-experts", type=int, default=None)
    g.add_argument("--moe-router-topk", type=int, default=None)
    g.add_argument("--moe-ffn-hidden-size", type=int, default=None)
    g.add_argument("--moe-shared-expert-intermediate-size", type=int, default=None)
    g.add_argument("--moe-shared-expert-gate", action="store_true", default=None,
                   help="sigmoid gate on the shared expert's output (Qwen3-Next, Qwen3.5)")
    g.add_argument("--moe-layer-freq", type=str, default=None)
    g.add_argument("--moe-router-score-function", type=str, default=None, choices=[None, "softmax", "sigmoid"])
    g.add_argument("--moe-router-pre-softmax", action="store_true")
    g.add_argument("--moe-router-enable-expert-bias", action="store_true")
    g.add_argument("--moe-router-bias-update-rate", type=float, default=None)
    g.add_argument("--moe-router-num-groups", type=int, default=None)
    g.add_argument("--moe-router-group-topk", type=int, default=None)
    g.add_argument("--moe-router-topk-scaling-factor", type=float, default=None)
    g.add_argument("--moe-router-load-balancing-type", type=str, default=None)
    g.add_argument("--moe-aux-loss-coeff", type=float, default=None)
    g.add_argument("--moe-z-loss-coeff", type=float, default=None)
    g.add_argument("--moe-grouped-gemm", action="store_true")
    g.add_argument("--moe-permute-fusion", action="store_true")
    g.add_argument("--moe-token-dispatcher-type", type=str, default="alltoall",
                   choices=["alltoall", "allgather", "flex", "peer"],
                   help="peer: dispatch / combine kernels over NVLink peer memory (CUDA only)")
    g.add_argument("--moe-enable-deepep", action="store_true")
    g.add_argument("--overlap-moe-expert-parallel-comm", action="store_true")
    g.add_argument("--delay-wgrad-compute", action="store_true")
    g.add_argument("--moe-use-upcycling", action="store_true")


def _add_parallel_args(p):
    g = p.add_argument_group("parallel")
    g.add_argument("--tensor-model-parallel-size", type=int, default=1)
    g.add_argument("--pipeline-model-parallel-size", type=int, default=1)
    g.add_argument("--num-virtual-stages-per-pipeline-rank", type=int, default=None)
    g.add_argument("--num-layers-per-virtual-pipeline-stage", type=int, default=None)
    g.add_argument("--pipeline-model-parallel-layout", type=str, default=None)
    g.add_argument("--custom-pipeline-layers", type=str, default=None)
    g.add_argument("--custom-pipeline-recompute-layers", type=str, default=None)
    g.add_argument("--custom-virtual-pipeline-layers", type=str, default=None,
                   help="layers per virtual stage: every pipeline rank's chunk 0, then every rank's chunk 1, ...")
    g.add_argument("--context-parallel-size", type=int, default=1)
    g.add_argument("--cp-comm-type", type=str, default="auto")
    g.add_argument("--context-parallel-ulysses-degree", type=int, default=None)
    g.add_argument("--expert-model-parallel-size", type=int, default=1)
    g.add_argument("--expert-tensor-parallel-size", type=int, default=1)
    g.add_argument("--sequence-parallel", action="store_true")
    g.add_argument("--tp-comm-overlap", action="store_true")
    g.add_argument("--use-distributed-optimizer", action="store_true")
    g.add_argument("--overlap-grad-reduce", action="store_true")
    g.add_argument("--overlap-param-gather", action="store_true")
    g.add_argument("--use-torch-fsdp2", action="store_true")
    g.add_argument("--use-megatron-fsdp", action="store_true")
    g.add_argument("--data-parallel-sharding-strategy", type=str, default="optim")
    g.add_argument("--distributed-backend", type=str, default="nccl", choices=["nccl", "gloo"])
    g.add_argument("--distributed-timeout-minutes", type=int, default=30)
    g.add_argument("--encoder-tensor-model-parallel-size", type=int, default=None)
    g.add_argument("--enable-encoder-hetero-dp", action="store_true")
    g.add_argument("--enable-full-hetero-dp", action="store_true")
    g.add_argument("--full-hetero-dp-cpu-offload", action="store_true")
    g.add_argument("--use-vlm-dp-balance", action="store_true")
    g.add_argument("--enable-chunkpipe", action="store_true")
    g.add_argument("--chunksize", type=int, default=None)


def _add_training_args(p):
    g = p.add_argument_group("training")
    g.add_argument("--training-phase", type=str, default="pretrain", choices=["pretrain", "sft"])
    g.add_argument("--micro-batch-size", type=int, default=1)
    g.add_argument("--global-batch-size", type=int, default=None)
    g.add_argument("--rampup-batch-size", nargs=3, type=int, default=None)
    g.add_argument("--seq-length", type=int, default=None)
    g.add_argument("--train-iters", type=int, default=None)
    g.add_argument("--train-samples", type=int, default=None)
    g.add_argument("--exit-interval", type=int, default=None)
    g.add_argument("--exit-duration-in-mins", type=int, default=None)
    g.add_argument("--lr", type=float, default=1e-4)
    g.add_argument("--min-lr", type=float, default=0.0)
    g.add_argument("--lr-decay-style", type=str, default="cosine")
    g.add_argument("--lr-decay-iters", type=int, default=None)
    g.add_argument("--lr-warmup-iters", type=int, default=0)
    g.add_argument("--lr-warmup-fraction", type=float, default=None)
    g.add_argument("--weight-decay", type=float, default=0.01)
    g.add_argument("--adam-beta1", type=float, default=0.9)
    g.add_argument("--adam-beta2", type=float, default=0.999)
    g.add_argument("--adam-eps", type=float, default=1e-8)
    g.add_argument("--clip-grad", type=float, default=1.0)
    g.add_argument("--optimizer", type=str, default="adam", choices=["adam", "sgd"])
    g.add_argument("--sgd-momentum", type=float, default=0.9)
    g.add_argument("--optimizer-offload-fraction", type=float, default=1.0,
                   help="with --optimizer-cpu-offload: part of the optimizer state kept on the host")
    g.add_argument("--use-precision-aware-optimizer", action="store_true")
    g.add_argument("--exp-avg-dtype", type=str, default="fp32", choices=["fp32", "bf16"])
    g.add_argument("--exp-avg-sq-dtype", type=str, default="fp32", choices=["fp32", "bf16"])
    g.add_argument("--optimizer-cpu-offload", action="store_true")
    g.add_argument("--bf16", action="store_true")
    g.add_argument("--fp16", action="store_true")
    g.add_argument("--fp8-format", type=str, default=None)
    g.add_argument("--fp8-recipe", type=str, default=None)
    g.add_argument("--fp8-dynamic-policy-path", type=str, default=None,
                   help="JSON rules that pick FP8 or BF16 per linear-layer kind, token count and TP size")
    g.add_argument("--fp8-param-gather", action="store_true")
    g.add_argument("--accumulate-allreduce-grads-in-fp32", action="store_true")
    g.add_argument("--seed", type=int, default=1234)
    g.add_argument("--recompute-granularity", type=str, default=None, choices=[None, "full", "selective"])
    g.add_argument("--recompute-method", type=str, default=None, choices=[None, "uniform", "block"])
    g.add_argument("--recompute-num-layers", type=int, default=None)
    g.add_argument("--cross-entropy-loss-fusion", action="store_true")
    g.add_argument("--cross-entropy-fusion-impl", type=str, default="linear")
    g.add_argument("--calculate-per-token-loss", action="store_true")
    g.add_argument("--use-flash-attn", action="store_true")
    g.add_argument("--no-gradient-accumulation-fusion", action="store_true")
    g.add_argument("--enable-cuda-graph", action="store_true")
    g.add_argument("--cuda-graph-scope", type=str, default=None)
    g.add_argument("--iterations-to-skip", type=int, nargs="*", default=[])
    g.add_argument("--error-injection-rate", type=int, default=0)
    g.add_argument("--error-injection-type", type=str, default="transient_error")
    g.add_argument("--rerun-mode", type=str, default="disabled",
                   choices=["disabled", "validate_results", "report_stats"])
    g.add_argument("--check-weight-hash-across-dp-replicas-interval", type=int, default=None)
    g.add_argument("--manual-gc", action="store_true")
    g.add_argument("--manual-gc-interval", type=int, default=0)
    g.add_argument("--ema-decay", type=float, default=None)


def _add_data_args(p):
    g = p.add_argument_group("data")
    g.add_argument("--data-path", nargs="*", default=None)
    g.add_argument("--split", type=str, default="949,50,1")
    g.add_argument("--mock-data", action="store_true")
    g.add_argument("--num-workers", type=int, default=2)
    g.add_argument("--tokenizer-type", type=str, default="HFTokenizer")
    g.add_argument("--hf-tokenizer-path", type=str, default=None)
    g.add_argument("--tokenizer-model", type=str, default=None)
    g.add_argument("--use-fast-tokenizer", action="store_true")
    g.add_argument("--chat-template", type=str, default=None)
    g.add_argument("--sft-dataset", nargs="*", default=None)
    g.add_argument("--sft-dataset-config", type=str, default=None)
    g.add_argument("--sft-data-streaming", action="store_true")
    g.add_argument("--packing-sft-data", action="store_true")
    g.add_argument("--packing-batch-size", type=int, default=None)
    g.add_argument("--train-on-prompt", action="store_true")
    g.add_argument("--eod-mask-loss", action="store_true")
    g.add_argument("--dataloader-type", type=str, default="single")
    g.add_argument("--image-resolution", type=int, default=None)
    g.add_argument("--min-pixels", type=int, default=None)
    g.add_argument("--max-pixels", type=int, default=None)
    g.add_argument("--frame-num", type=int, default=None)
    g.add_argument("--fps", type=float, default=None)
    g.add_argument("--variable-seq-lengths", action="store_true")


def _add_ckpt_logging_args(p):
    g = p.add_argument_group("checkpointing and logging")
    g.add_argument("--save", type=str, default=None)
    g.add_argument("--load", type=str, default=None)
    g.add_argument("--pretrained-checkpoint", type=str, default=None)
    g.add_argument("--save-interval", type=int, default=None)
    g.add_argument("--ckpt-format", type=str, default="torch_dist", choices=["torch", "torch_dist", "torch_dcp", "zarr", "fsdp_dtensor"])
    g.add_argument("--ckpt-step", type=int, default=None)
    g.add_argument("--no-load-optim", action="store_true")
    g.add_argument("--no-load-rng", action="store_true")
    g.add_argument("--no-save-optim", action="store_true")
    g.add_argument("--no-save-rng", action="store_true")
    g.add_argument("--finetune", action="store_true")
    g.add_argument("--async-save", action="store_true")
    g.add_argument("--save-hf", nargs="?", const="true", default="false", choices=["true", "false"],
                   help="write Hugging Face weights of the final model (to --save-hf-path or <save>/release_hf_weights)")
    g.add_argument("--save-hf-path", type=str, default=None)
    g.add_argument("--load-hf", action="store_true")
    g.add_argument("--hf-checkpoint-path", type=str, default=None)
    g.add_argument("--dist-ckpt-strictness", type=str, default="assume_ok_unexpected")
    g.add_argument("--log-interval", type=int, default=1)
    g.add_argument("--log-throughput", action="store_true")
    g.add_argument("--log-memory-stats", action="store_true")
    g.add_argument("--log-timers-to-tensorboard", action="store_true")
    g.add_argument("--timing-log-level", type=int, default=0)
    g.add_argument("--detail-log-interval", type=int, default=None)
    g.add_argument("--tensorboard-dir", type=str, default=None)
    g.add_argument("--wandb-project", type=str, default=None)
    g.add_argument("--wandb-exp-name", type=str, default=None)
    g.add_argument("--eval-interval", type=int, default=None)
    g.add_argument("--eval-iters", type=int, default=0)
    g.add_argument("--profile", action="store_true")
    g.add_argument("--profile-step-start", type=int, default=10)
    g.add_argument("--profile-step-end", type=int, default=12)
    g.add_argument("--profile-ranks", type=int, nargs="*", default=[0])
    g.add_argument("--use-pytorch-profiler", action="store_true")
    g.add_argument("--record-memory-history", action="store_true")
    g.add_argument("--enable-log-tensor", action="store_true")
    g.add_argument("--log-tensor-name-pattern", type=str, default=None)
    g.add_argument("--log-straggler", action="store_true")
    g.add_argument("--heartbeat-timeout-s", type=float, default=None,
                   help="report ranks whose per-step heartbeat in the job store stopped for this long; checkpoint and exit")


def _add_peft_args(p):
    g = p.add_argument_group("peft")
    g.add_argument("--peft-type", type=str, default=None, choices=[None, "lora", "canonical_lora"])
    g.add_argument("--lora-rank", type=int, default=16)
    g.add_argument("--lora-alpha", type=int, default=32)
    g.add_argument("--lora-dropout", type=float, default=0.0)
    g.add_argument("--lora-target-modules", nargs="*", default=["linear_qkv", "linear_proj", "linear_fc1", "linear_fc2"])


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("loongforge_b200 training", allow_abbrev=False)
    for add in (_add_model_args, _add_moe_args, _add_parallel_args, _add_training_args, _add_data_args,
                _add_ckpt_logging_args, _add_peft_args):
        add(p)
    return p


def parse_args(argv: Optional[List[str]] = None) -> Tuple[argparse.Namespace, List[str]]:
    """Returns (args, yaml_overrides). Unknown tokens of the form ``key=value`` / ``+key=value`` /
    ``~key`` are YAML overrides; anything else unknown is an error."""
    from .yaml_compose import is_override_token

    args, unknown = build_parser().parse_known_args(argv)
    bad = [u for u in unknown if not is_override_token(u)]
    if bad:
        raise SystemExit(f"unrecognised arguments: {' '.join(bad)}")
    return args, unknown
