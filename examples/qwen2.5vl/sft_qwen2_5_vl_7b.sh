#!/bin/bash
# Qwen2.5-VL-7B supervised fine-tuning: language model TP4, vision encoder TP1 (heterogeneous tensor parallelism),
# encoder heterogeneous DP inside the TP group, packed variable-length samples. Tokens after the flags that start
# with '+' override keys of the composed YAML (here: freeze the vision encoder).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen2.5-vl-7b --training-phase sft \
  --tensor-model-parallel-size 4 --encoder-tensor-model-parallel-size 1 --sequence-parallel --enable-encoder-hetero-dp \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 32 --seq-length 4096 --packing-sft-data --variable-seq-lengths \
  --bf16 --lr 1e-5 --lr-decay-style cosine --lr-warmup-fraction 0.03 --clip-grad 1.0 \
  --train-iters 1000 --log-interval 5 --mock-data \
  --save "${CKPT:-$REPO/outputs/qwen2_5_vl_7b_sft}" --save-interval 250 \
  +model.image_encoder.freeze=True
