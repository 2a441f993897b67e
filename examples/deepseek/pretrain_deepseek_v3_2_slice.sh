#!/bin/bash
# DeepSeek-V3.2 (reduced-layer slice): multi-latent attention with the sparse-attention indexer, sigmoid router with
# selection bias and group-limited top-k, multi-token prediction, expert parallel 8.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name deepseek-v3.2-slice --use-dsa-fused \
  --expert-model-parallel-size "$GPUS" \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 8192 \
  --bf16 --lr 2e-4 --lr-decay-style cosine --lr-warmup-iters 100 --clip-grad 1.0 \
  --recompute-granularity full --recompute-method uniform --recompute-num-layers 1 \
  --train-iters 1000 --log-interval 5 --mock-data
