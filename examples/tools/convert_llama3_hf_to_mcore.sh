#!/bin/bash
# Hugging Face Llama-3 checkpoint -> Megatron layout sharded for TP2 x PP1, and back.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
HF=${1:?path to the Hugging Face checkpoint directory}
OUT=${2:-$REPO/outputs/llama3_8b_mcore_tp2}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --model_type_custom llama3 --load_ckpt_path "$HF" --save_ckpt_path "$OUT" \
  --tensor_model_parallel_size 2 --pipeline_model_parallel_size 1 --safetensors --torch_dtype bfloat16
python -m tools.convert_checkpoint.convert --load_platform mcore --save_platform huggingface \
  --model_type_custom llama3 --load_ckpt_path "$OUT" --save_ckpt_path "$OUT"_hf --safetensors
