#!/bin/bash
# qwen2.5-vl-3b-lora supervised fine-tuning on image-text conversations (language model: qwen2.5-3b); the vision encoder keeps
# tensor-parallel size 1 and is spread over the TP ranks by encoder heterogeneous DP
# Layout for 1 node(s) of 8 B200 (DP8); estimated 35 GB of 180 GB per GPU. Written by
# tools/generate_launchers.py; run it on every node with NODE_RANK set (one node: no variables needed).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${GPUS:-8}
NNODES=${NNODES:-1}
NODE_RANK=${NODE_RANK:-0}
MASTER_ADDR=${MASTER_ADDR:-127.0.0.1}
MASTER_PORT=${MASTER_PORT:-29500}
CKPT=${CKPT:-$REPO/outputs/sft_qwen2_5_vl_3b_lora}
DATA_PATH=${DATA_PATH:-}        # WebDataset shards written by tools/data_preprocess/vlm_to_webdataset.py
TOKENIZER=${TOKENIZER:-}
export PYTORCH_CUDA_ALLOC_CONF=expandable_segments:True
DATA_ARGS=(--mock-data)
[ -n "$DATA_PATH" ] && DATA_ARGS=(--data-path "$DATA_PATH" --tokenizer-type HFTokenizer --hf-tokenizer-path "$TOKENIZER")

cd "$REPO"
python -m torch.distributed.run --nnodes "$NNODES" --node-rank "$NODE_RANK" --nproc-per-node "$GPUS" \
  --master-addr "$MASTER_ADDR" --master-port "$MASTER_PORT" \
  -m loongforge_b200.train \
  --model-name qwen2.5-vl-3b-lora --training-phase sft \
  --use-distributed-optimizer --overlap-grad-reduce --overlap-param-gather \
  --micro-batch-size 1 --global-batch-size 32 --seq-length 4096 --packing-sft-data --variable-seq-lengths \
  --bf16 --lr 1e-5 --min-lr 1e-6 --lr-decay-style cosine --lr-warmup-fraction 0.03 --weight-decay 0.1 --clip-grad 1.0 \
  --train-iters 1000 --log-interval 5 --log-throughput \
  --save "$CKPT" --save-interval 250 --ckpt-format torch_dist \
  "${DATA_ARGS[@]}" \
  +model.image_encoder.freeze=True
