#!/bin/bash
# Llama-3-8B pretraining on one node of 8 B200s: TP2 + sequence parallel with the fused all-gather->GEMM /
# GEMM->reduce-scatter kernels, DP4 with the distributed optimizer, no activation recompute.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
DATA_PATH=${DATA_PATH:-}            # prefix of a .bin/.idx pair from tools/data_preprocess/preprocess_pretrain_data.py
CKPT=${CKPT:-$REPO/outputs/llama3_8b}
GPUS=${GPUS:-8}

export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --split 99,1,0)

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name llama3-8b \
  --tensor-model-parallel-size 2 --sequence-parallel --tp-comm-overlap \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 8192 \
  --bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-iters 200 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --train-iters 5000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist --async-save \
  "${DATA_ARGS[@]}"
