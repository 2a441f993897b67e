#!/bin/bash
# Hugging Face qwen3.5-4b checkpoint -> training layout sharded for DP8.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/qwen3_5_4b_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom qwen3_5 --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 1 --pipeline_model_parallel_size 1 --safetensors --torch_dtype bfloat16
