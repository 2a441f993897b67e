#!/bin/bash
# Hugging Face llama3-70b checkpoint -> training layout sharded for TP8 + SP.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/llama3_70b_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom llama3 --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 8 --pipeline_model_parallel_size 1 --safetensors --torch_dtype bfloat16
