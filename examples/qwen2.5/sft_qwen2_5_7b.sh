#!/bin/bash
# Qwen2.5-7B chat SFT with sequence packing
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
CKPT=${CKPT:-$REPO/outputs/sft_qwen2_5_7b}
DATA_PATH=${DATA_PATH:-}
TOKENIZER=${TOKENIZER:-}   # Hugging Face tokenizer directory
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--sft-dataset "$DATA_PATH" --tokenizer-type HFTokenizer --hf-tokenizer-path "$TOKENIZER")

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen2.5-7b \
  --tensor-model-parallel-size 2 --sequence-parallel \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 64 --seq-length 8192 \
  --bf16 --lr 1e-5 --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.01 --weight-decay 0.1 \
  --adam-beta1 0.9 --adam-beta2 0.95 --clip-grad 1.0 \
  --training-phase sft --packing-sft-data --chat-template chatml \
  --train-iters 1000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}"
