#!/bin/bash
# Qwen-Image (double-stream MMDiT), flow matching on 2 x 2 packed image latents: data parallel with the
# distributed optimizer.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
CKPT=${CKPT:-$REPO/outputs/qwen_image_edit_2511}
DATA_PATH=${DATA_PATH:-}      # directory of *.pt samples: {"latents", "text", }
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH")

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen-image-edit-2511 \
  --use-distributed-optimizer --overlap-grad-reduce --recompute-granularity full \
  --micro-batch-size 1 --global-batch-size 16 --seq-length 4096 \
  --bf16 --lr 1e-5 --lr-decay-style constant --weight-decay 0.01 --clip-grad 1.0 \
  --train-iters 1000 --log-interval 10 \
  --save "$CKPT" --save-interval 200 \
  "${DATA_ARGS[@]}"
