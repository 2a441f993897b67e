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
    g.add_argument("--train-data-path", nargs="*", default=None, help="separate training data (then --split is not used)")
    g.add_argument("--valid-data-path", nargs="*", default=None)
    g.add_argument("--test-data-path", nargs="*", default=None)
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
    g.add_argument("--lora-apply-to-image-encoder", action="store_true",
                   help="vision-language models: adapters on the vision tower's linears as well")
    g.add_argument("--lora-apply-to-image-projector", action="store_true")
    g.add_argument("--lora-skip-foundation", action="store_true",
                   help="vision-language models: no adapters on the language model (it keeps training or stays frozen)")


# (flag, kind, default) with kind: "flag" store_true, "noflag" store_false, int / float / str, "list" nargs="*".
# The reference's own flags (loongforge/train/arguments.py:95-1439) that no group above defines, plus the Megatron
# flags its example launchers pass. They are accepted so that those launchers run unchanged; `COMPAT_WIRED` lists the
# ones the trainers act on, the rest describe code paths this framework covers differently (noted by the validators).
_COMPAT_FLAGS = [
    # tensor inspection / debugging
    ("--log-tensor-stage", str, "forward"), ("--log-tensor-iter-pattern", str, None),
    ("--log-tensor-mbs-pattern", str, None), ("--log-tensor-layer-pattern", str, None), ("--log-tensor-rank", str, "0"),
    ("--save-tensor", "flag", False), ("--save-tensor-dir", str, ""), ("--random-fallback-cpu", "flag", False),
    ("--no-detail-log", "noflag", True),
    # low precision
    ("--fp8-force-no-requant", "flag", False), ("--force-pow-2-scales", "flag", False), ("--amax-epsilon", float, 0.0),
    ("--hf-dequantize-int4", "flag", False), ("--hf-dequantize-mxfp4", "flag", False),
    ("--hf-dequantize-dtype", str, "bfloat16"), ("--hf-quant-config-file", str, None), ("--quant-method", str, "te"),
    ("--pretrain-as-fp8", "flag", False), ("--enable-fp8-comm", "flag", False),
    # model / attention
    ("--enable-fa-within-mla", "flag", False), ("--language-model-type", str, None),
    ("--should-get-embedding-weights-for-mtp", "flag", False), ("--cuda-graph-pad-length", int, None),
    ("--rotary-seq-len-interpolation-factor", float, None), ("--no-position-embedding", "flag", False),
    ("--attention-softmax-in-fp32", "flag", False), ("--no-masked-softmax-fusion", "flag", False),
    ("--no-bias-gelu-fusion", "flag", False), ("--no-bias-dropout-fusion", "flag", False), ("--no-rope-fusion", "flag", False),
    ("--mscale", float, None), ("--mscale-all-dim", float, None), ("--original-max-position-embeddings", int, None),
    ("--moe-router-dtype", str, None), ("--moe-shared-expert-overlap", "flag", False),
    # freezing / adapters
    ("--freeze-parameters", "list", []), ("--freeze-parameters-regex", str, None), ("--trainable-modules", "list", ["all"]),
    ("--allow-missing-adapter-checkpoint", "flag", False), ("--lora-dim", int, None),
    # tokenizer
    ("--hf-processor-path", str, None), ("--split-special-tokens", "flag", False), ("--padding-side", str, "right"),
    ("--additional-special-tokens", str, None), ("--vocab-size-in-config-file", int, None), ("--padded-vocab-size", int, None),
    # SFT data
    ("--task-encoder", str, None), ("--chat-template-kwargs", str, None), ("--sft-train-dataset", "list", None),
    ("--sft-valid-dataset", "list", None), ("--sft-test-dataset", "list", None), ("--sft-sort-batch", "flag", False),
    ("--streaming-buffer-size", int, 16384), ("--sft-data-mix-strategy", str, "concat"),
    ("--sft-num-preprocess-workers", int, None), ("--history-mask-loss", "flag", False), ("--is-tokenized-data", "flag", False),
    ("--enable-discard-sample", "flag", False), ("--packing-buffer-size", int, 10000), ("--use-fixed-seq-lengths", "flag", False),
    ("--sample-type", str, None), ("--packing-pretrain-data", "flag", False), ("--add-question-in-pretrain", "flag", False),
    ("--data-shuffle-buffer-size", int, 0), ("--data-max-samples-per-sequence", int, 0), ("--dataloader-save", str, None),
    ("--save-dataset-state", "flag", False), ("--dataloader-prefetch-factor", int, 2), ("--data-cache-path", str, None),
    ("--no-create-attention-mask-in-dataloader", "flag", False),
    # loss
    ("--loss-reduction", str, "square"), ("--loss-reduction-all-gather", "flag", False),
    ("--legacy-reporting-loss-reduction", "flag", False), ("--force-all-weight-decay", "flag", False),
    # video / latent (diffusion) data
    ("--latent-in-channels", int, None), ("--latent-out-channels", int, None), ("--caption-channels", int, None),
    ("--latent-patch-size", str, None), ("--latent-space-scale", float, 1.0), ("--latent-time-scale", float, 1.0),
    ("--num-latent-frames", int, None), ("--max-latent-height", int, None), ("--max-latent-width", int, None),
    ("--max-text-length", int, None), ("--max-video-length", int, 32760), ("--max-image-length", int, None),
    ("--max-timestep-boundary", float, 1.0), ("--min-timestep-boundary", float, 0.0), ("--dataset-metadata-path", str, None),
    # multimodal (InternVL / Qwen-VL / RICE) data
    ("--training-rice-vl-max-answer-length", int, 4096), ("--conv-style", str, "internvl2_5"), ("--force-image-size", int, 448),
    ("--num-images-expected", int, 48), ("--pad2square", "flag", False), ("--down-sample-ratio", float, 0.5),
    ("--max-buffer-size", int, 20), ("--max-packed-tokens", int, 8192), ("--strict-mode", "flag", False),
    ("--replacement", "flag", False), ("--patch-size", int, 14), ("--group-by-length", "flag", False),
    ("--min-num-frame", int, 8), ("--max-num-frame", int, 32), ("--dynamic-image-size", "flag", False),
    ("--min-dynamic-patch", int, 1), ("--max-dynamic-patch", int, 12), ("--use_thumbnail", "flag", False),
    ("--normalize_type", str, "imagenet"), ("--use-packed-ds", "flag", False), ("--frame-min-pixels", int, 128 * 28 * 28),
    ("--frame-max-pixels", int, 768 * 28 * 28), ("--video-max-pixels", int, 65536 * 28 * 28), ("--fps-min-frames", int, 4),
    ("--fps-max-frames", int, 768), ("--energon-pack-algo", str, "balanced"),
    # data-parallel balancing of VLM batches
    ("--use-vit-dp-balance", "flag", False), ("--vlm-dp-balance-warmup-iters", "list", [2, 5]),
    ("--dp-balance-verbose", "flag", False), ("--dp-balance-max-len-ratio-vlm", float, 1.2),
    ("--dp-balance-max-len-ratio-vit", float, None), ("--dp-balance-trigger-threshold-vlm", float, 0.2),
    ("--dp-balance-trigger-threshold-vit", float, 0.2),
    # EMA
    ("--enable-ema", "flag", False), ("--save-ema", str, None), ("--load-ema", str, None),
    # Megatron flags of the example launchers
    ("--initial-loss-scale", float, 65536.0), ("--no-check-for-nan-in-loss-and-grad", "flag", False),
    ("--empty-unused-memory-level", int, 0), ("--log-memory-to-tensorboard", "flag", False),
    ("--log-validation-ppl-to-tensorboard", "flag", False), ("--tp-comm-overlap-bootstrap-backend", str, "nccl"),
    ("--use-fp32-dtype-for-param-pattern", "list", None), ("--use-cpu-initialization", "flag", False),
    ("--no-initialization", "flag", False), ("--reduce-variable-seq-shape-p2p-comm", "flag", False),
    ("--offload-optimizer", str, None), ("--offload-optimizer-percent", float, None),
    ("--overlap-cpu-optimizer-d2h-h2d", "flag", False), ("--ckpt-fully-parallel-load", "flag", False),
    ("--no-strict-fsdp-dtensor-load", "flag", False), ("--suggested-communication-unit-size", int, None),
    ("--timing-log-option", str, "minmax"), ("--disable-turn-off-bucketing", "flag", False),
    ("--enable-experimental", "flag", False), ("--rope-scaling-factor", float, None),
    ("--disable-rotate-activation", "flag", False),
]

# compat flags that change what the trainers do (the others are accepted and recorded in the argument dump)
COMPAT_WIRED = {"--freeze-parameters", "--freeze-parameters-regex", "--trainable-modules", "--force-pow-2-scales",
                "--amax-epsilon", "--enable-ema", "--no-check-for-nan-in-loss-and-grad", "--padded-vocab-size",
                "--offload-optimizer", "--offload-optimizer-percent", "--no-position-embedding", "--group-by-length",
                "--sft-sort-batch", "--vlm-dp-balance-warmup-iters", "--sft-train-dataset",
                "--streaming-buffer-size", "--sft-data-mix-strategy", "--sft-valid-dataset"}


def _add_compat_args(p):
    g = p.add_argument_group("reference compatibility")
    have = {o for a in p._actions for o in a.option_strings}
    for name, kind, default in _COMPAT_FLAGS:
        if name in have:
            continue
        if kind == "flag":
            # some launchers spell these with underscores
            names = [name] + ([name.replace("-", "_").replace("__", "--", 1)] if name in (
                "--fp8-force-no-requant", "--force-pow-2-scales") else [])
            g.add_argument(*names, action="store_true", default=default)
        elif kind == "noflag":
            g.add_argument(name, action="store_false", default=default)
        elif kind == "list":
            g.add_argument(name, nargs="*", default=default)
        else:
            g.add_argument(name, type=kind, default=default)


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser("loongforge_b200 training", allow_abbrev=False)
    for add in (_add_model_args, _add_moe_args, _add_parallel_args, _add_training_args, _add_data_args,
                _add_ckpt_logging_args, _add_peft_args, _add_compat_args):
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
