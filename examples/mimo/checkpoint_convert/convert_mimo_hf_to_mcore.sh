#!/bin/bash
# Hugging Face mimo checkpoint -> training layout sharded for DP8.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/mimo_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom mimo --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 1 --pipeline_model_parallel_size 1 --safetensors --torch_dtype bfloat16
