#!/bin/bash
# Training checkpoint of qwen3.5-4b -> Hugging Face safetensors (shards of any TP / PP / EP layout are merged).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
IN=${1:?path to the training checkpoint}
OUT=${2:-$REPO/outputs/qwen3_5_4b_hf}
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform mcore --save_platform huggingface \
  --model_type_custom qwen3_5 --load_ckpt_path "$IN" --save_ckpt_path "$OUT" --safetensors --torch_dtype bfloat16
