#!/bin/bash
# deepseek-v4-flash-lite-6l (40.1 B parameters) pretraining, sequence length 4096
# Layout for 1 node(s) of 8 B200 (EP8, DP8); estimated 97 GB of 180 GB per GPU. Written by
# tools/generate_launchers.py; run it on every node with NODE_RANK set (one node: no variables needed).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${GPUS:-8}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
CKPT=${CKPT:-$REPO/outputs/deepseek_v4_flash_lite_6l}
DATA_PATH=${DATA_PATH:-}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --split 99,1,0)

cd "$REPO"
python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
  -m loongforge_b200.train \
  --model-name deepseek-v4-flash-lite-6l \
  --expert-model-parallel-size 8 --moe-token-dispatcher-type alltoall --moe-grouped-gemm \
  --use-distributed-optimizer --overlap-grad-reduce --overlap-param-gather \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 4096 \
  --bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --train-iters 5000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}"
