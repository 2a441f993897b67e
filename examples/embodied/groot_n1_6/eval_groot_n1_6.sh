#!/bin/bash
# Serve the newest checkpoint of a groot_n1_6 run and roll out evaluation episodes against it.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../../.." && pwd)
RUN=${1:?run directory (output_dir of the training)}
PORT=${PORT:-18600}
cd "$REPO"
python -m loongforge_b200.embodied.eval serve --checkpoint "$RUN" --port "$PORT" model_name=groot_n1_6 output_dir="$RUN" &
SERVER=$!
trap 'kill "$SERVER"' EXIT
sleep 20
python -m loongforge_b200.embodied.eval run --port "$PORT" --episodes "${EPISODES:-20}" --output-dir "$RUN/eval"
