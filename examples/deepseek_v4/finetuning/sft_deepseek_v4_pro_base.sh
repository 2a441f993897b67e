#!/bin/bash
# deepseek-v4-pro-base chat fine-tuning, packed sequences of 8192 tokens
# Layout for 32 node(s) of 8 B200 (PP16, EP16, DP16, selective recompute); estimated 122 GB of 180 GB per GPU. Written by
# tools/generate_launchers.py; run it on every node with NODE_RANK set (one node: no variables needed).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${GPUS:-8}
NNODES=${NNODES:-32}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
CKPT=${CKPT:-$REPO/outputs/sft_deepseek_v4_pro_base}
DATA_PATH=${DATA_PATH:-}
TOKENIZER=${TOKENIZER:-}   # Hugging Face tokenizer directory
LOAD=${LOAD:-}             # converted base checkpoint
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--sft-dataset "$DATA_PATH" --tokenizer-type HFTokenizer --hf-tokenizer-path "$TOKENIZER")
[ -n "$LOAD" ] && DATA_ARGS+=(--load "$LOAD" --finetune)

cd "$REPO"
python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
  -m loongforge_b200.train \
  --model-name deepseek-v4-pro-base \
  --pipeline-model-parallel-size 16 --custom-pipeline-layers 4,4,4,4,4,4,4,4,4,4,4,4,4,3,3,3 \
  --expert-model-parallel-size 16 --moe-token-dispatcher-type alltoall --moe-grouped-gemm \
  --use-distributed-optimizer --overlap-grad-reduce --overlap-param-gather \
  --recompute-granularity selective \
  --micro-batch-size 1 --global-batch-size 128 --seq-length 8192 \
  --bf16 --lr 1e-5 --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --training-phase sft --packing-sft-data --chat-template deepseek \
  --train-iters 1000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}"
