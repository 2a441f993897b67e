#!/bin/bash
# DeepSeek-V3 / V3.2 / GLM-5 layout (MLA, indexer, shared expert, router bias, MTP layers) -> Megatron per-rank files.
set -euo pipefail
REPO=$(cd "$(dirname "$0")/../.." && pwd)
cd "$REPO"
python -m tools.convert_checkpoint.convert --load_platform huggingface --save_platform mcore \
  --load_ckpt_path "${HF:?Hugging Face directory}" --save_ckpt_path "${OUT:?output directory}" \
  --model_type_custom deepseek --tensor_model_parallel_size "${TP:-2}" --pipeline_model_parallel_size "${PP:-2}" \
  --expert_parallel_size "${EP:-4}" --torch_dtype bfloat16
