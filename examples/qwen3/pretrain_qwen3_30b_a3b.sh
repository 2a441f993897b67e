#!/bin/bash
# Qwen3-30B-A3B (128 experts, top-8) pretraining: expert parallel over the 8 GPUs of a node, grouped tcgen05 GEMMs
# for the experts. MOE_DISPATCHER=peer selects the NVLink peer-memory dispatch / combine kernels (validated on 2 GPUs).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
MOE_DISPATCHER=${MOE_DISPATCHER:-alltoall}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen3-30b-a3b \
  --expert-model-parallel-size "$GPUS" --moe-token-dispatcher-type "$MOE_DISPATCHER" --moe-grouped-gemm \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 4096 \
  --bf16 --lr 2e-4 --lr-decay-style cosine --lr-warmup-iters 100 --weight-decay 0.1 --clip-grad 1.0 \
  --train-iters 2000 --log-interval 10 --mock-data \
  --save "${CKPT:-$REPO/outputs/qwen3_30b_a3b}" --save-interval 500
