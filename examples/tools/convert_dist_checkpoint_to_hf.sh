#!/bin/bash
# torch_dist checkpoint (any parallel layout) -> Hugging Face safetensors, offline, and back into a weights-only
# checkpoint that loads under any layout.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
cd "$REPO"
python -m tools.dist_checkpoint.convert_dist_checkpoint --to hf --load "${CKPT:?checkpoint directory}" \
  --save "${HF_OUT:?output directory}" --family "${FAMILY:-llama3}"
# python -m tools.dist_checkpoint.convert_dist_checkpoint --to dist --load "$HF_OUT" --save "$CKPT2" \
#   --family llama3 --model-name llama3-8b
