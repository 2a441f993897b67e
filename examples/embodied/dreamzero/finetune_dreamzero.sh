#!/bin/bash
# Fine-tune the dreamzero policy (fsdp); key=value tokens after the script name override the recipe.
# CACHE=<dir> trains from features written by precompute_dreamzero.sh.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
GPUS=${GPUS:-8}
OUT=${OUT:-$REPO/outputs/dreamzero}
DATA=${DATA:-}            # LeRobot v2 data set directory (empty: synthetic episodes)
DATA_ARGS=(dataset_type=synthetic)
[ -n "$DATA" ] && DATA_ARGS=(dataset_type=lerobot dataset_path="$DATA" use_transforms=true stats_path="$DATA")
cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.embodied.train --config configs/embodied/dreamzero.yaml \
  strategy=fsdp 'fsdp_wrap_patterns=[auto]' fsdp_reduce_dtype=fp32 per_device_batch_size=1 train_steps=2000 save_interval=500 log_stage_times=true \
  output_dir="$OUT" "${DATA_ARGS[@]}" ${CACHE:+precomputed_cache="$CACHE"} "$@"
