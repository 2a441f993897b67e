#!/bin/bash
# Cache the codec latents / text embeddings of a data set for dreamzero (train afterwards with CACHE=<dir>).
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
DATA=${1:?LeRobot v2 data set directory}
CACHE=${2:?output directory}
cd "$REPO"
python -m tools.data_preprocess.embodied_precompute build --output "$CACHE" --config configs/embodied/dreamzero.yaml \
  dataset_type=lerobot dataset_path="$DATA" ${PRETRAINED:+pretrained_checkpoint="$PRETRAINED"}
python -m tools.data_preprocess.embodied_precompute validate --cache "$CACHE" --deep
