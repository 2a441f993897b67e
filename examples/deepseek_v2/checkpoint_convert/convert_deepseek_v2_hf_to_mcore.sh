#!/bin/bash
# Hugging Face deepseek-v2 checkpoint -> training layout sharded for TP8 + SP, PP4, EP8.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/deepseek_v2_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom deepseek --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 8 --pipeline_model_parallel_size 4 --expert_parallel_size 8 --safetensors --torch_dtype bfloat16
