#!/bin/bash
# DeepSeek-V3.2 slice (MLA + sparse attention with the lightning indexer), blockwise FP8 linears
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
CKPT=${CKPT:-$REPO/outputs/deepseek_v3_2}
DATA_PATH=${DATA_PATH:-}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --split 99,1,0)

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name deepseek-v3.2 \
  --tensor-model-parallel-size 2 --sequence-parallel \
  --expert-model-parallel-size 4 --moe-grouped-gemm \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 64 --seq-length 4096 \
  --bf16 --lr 3e-4 --min-lr 3e-5 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --num-layers 4 --moe-layer-freq "[0]+[1]*3" --fp8-format e4m3 --fp8-recipe blockwise \
  --train-iters 5000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}"
