#!/bin/bash
# Fine-tune the pi05 flow-matching policy with DDP; key=value tokens override the YAML recipe.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
GPUS=${GPUS:-8}
cd "$REPO"
python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 --master-port 29500 \
  -m loongforge_b200.embodied.train --model-name pi05 \
  strategy=ddp ddp_comm_hook=bf16_compress per_device_batch_size=16 train_steps=2000 \
  output_dir="${OUT:-$REPO/outputs/pi05}" save_interval=500 "$@"
