#!/bin/bash
# Qwen2.5-72B pretraining, TP4 + SP, PP2
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
CKPT=${CKPT:-$REPO/outputs/qwen2_5_72b}
DATA_PATH=${DATA_PATH:-}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --split 99,1,0)

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen2.5-72b \
  --tensor-model-parallel-size 4 --sequence-parallel \
  --pipeline-model-parallel-size 2 \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 8192 \
  --bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --recompute-granularity full --recompute-method uniform \
  --train-iters 5000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}"
