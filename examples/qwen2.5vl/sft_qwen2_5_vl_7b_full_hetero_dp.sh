#!/bin/bash
# Qwen2.5-VL-7B supervised fine-tuning with FULL heterogeneous data parallelism: the language model runs TP2 + SP x PP2,
# the vision encoder (TP1, recomputed) runs data parallel over all four ranks of each model-parallel group: every
# encoder round happens before the pipeline starts, the embeddings are broadcast to the ranks that need them and
# their gradients return to the encoding rank after the pipeline's backward.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
CKPT=${CKPT:-$REPO/outputs/qwen2_5_vl_7b_full_hetero}
DATA_PATH=${DATA_PATH:-}      # directory of WebDataset shards from tools/data_preprocess/vlm_to_webdataset.py
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH")

cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.train \
  --model-name qwen2.5-vl-7b --training-phase sft \
  --tensor-model-parallel-size 2 --sequence-parallel --pipeline-model-parallel-size 2 \
  --encoder-tensor-model-parallel-size 1 --enable-full-hetero-dp \
  --use-distributed-optimizer --overlap-grad-reduce \
  --micro-batch-size 1 --global-batch-size 64 --seq-length 8192 \
  --bf16 --lr 1e-5 --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.03 --weight-decay 0.1 --clip-grad 1.0 \
  --train-iters 1000 --log-interval 10 --log-throughput \
  --save "$CKPT" --save-interval 500 \
  "${DATA_ARGS[@]}"
