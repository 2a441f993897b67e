#!/bin/bash
# Hugging Face kimi-k2 checkpoint -> training layout sharded for TP4 + SP, PP2, EP64.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/kimi_k2_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom kimi_k2 --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 4 --pipeline_model_parallel_size 2 --expert_parallel_size 64 --safetensors --torch_dtype bfloat16
