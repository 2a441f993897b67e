#!/bin/bash
# LoRA fine-tuning of lingbot_va: adapters on the policy's default projections, base weights from PRETRAINED.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${GPUS:-8}
OUT=${OUT:-$REPO/outputs/lingbot_va_lora}
DATA=${DATA:-}            # LeRobot v2 data set directory (empty: synthetic episodes)
DATA_ARGS=(dataset_type=synthetic)
[ -n "$DATA" ] && DATA_ARGS=(dataset_type=lerobot dataset_path="$DATA" use_transforms=true stats_path="$DATA")
cd "$REPO"
PRETRAINED=${PRETRAINED:-}
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.embodied.train --config configs/embodied/lingbot_va.yaml \
  strategy=ddp lora_rank=16 lora_alpha=32 'lora_targets=[]' per_device_batch_size=4 lr=2e-4 train_steps=2000 save_interval=500 \
  output_dir="$OUT" "${DATA_ARGS[@]}" ${PRETRAINED:+pretrained_checkpoint="$PRETRAINED"} "$@"
