#!/usr/bin/env bash
# HF base model (Qwen3-0.6B, SmolLM2-360M, any Llama-family checkpoint) -> step-0 DCP of a target config
# (reference: scripts/convert_*_to_*.sh).
#
#   HF_MODEL=/models/Qwen3-0.6B MODEL=ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k FAMILY=ipttcd ./scripts/convert_to_dcp.sh
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL=${MODEL:-ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k}
FAMILY=${FAMILY:-ipttcd}
CONFIG_PATH=${CONFIG_PATH:-configs/${FAMILY}/${MODEL}.json}
OUTPUT_DCP=${OUTPUT_DCP:-exp/${MODEL}/checkpoint/step-0}
python -m flame.utils.convert_qwen_to_ipttcd_dcp --model "${HF_MODEL:?set HF_MODEL}" --config "${CONFIG_PATH}" \
  --tokenizer "${TOKENIZER:-tokenizers/Qwen3-0.6B-Base}" --checkpoint "${OUTPUT_DCP}"
echo "wrote ${OUTPUT_DCP}"
