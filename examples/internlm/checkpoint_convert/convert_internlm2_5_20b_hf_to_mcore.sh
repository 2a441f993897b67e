#!/bin/bash
# Hugging Face internlm2.5-20b checkpoint -> training layout sharded for TP2 + SP.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/internlm2_5_20b_mcore}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom internlm2.5 --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 2 --pipeline_model_parallel_size 1 --safetensors --torch_dtype bfloat16
