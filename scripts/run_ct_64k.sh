#!/usr/bin/env bash
# Continued-training recipe at 64K context (the recipe of the reference's scripts/run_*_ct_64k*.sh:44-79),
# one script for every model family:
#
#   MODEL=ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k FAMILY=ipttcd DATASET=/data/books_65k ./scripts/run_ct_64k.sh
#   MODEL=ipttt_qwen3_0.6B_64k_swa8k_ct       FAMILY=ipttt  ...
#   MODEL=transformer_qwen3_0.6B_swa8k         FAMILY=transformer ...
#
# Environment: NGPU (default 8), DATASET (HF dataset dir, `mds:/path?...` or `synthetic`), TOKENIZER, EXP_DIR,
# LR, LR_FINAL, WARMUP_STEPS, TOTAL_STEPS, BATCH_SIZE, GRAD_ACCUM, AC (none|full|ttt), CP, TP, MUON=1.
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL=${MODEL:-ipttcdv9_qwen3_0.6B_ct_64k_v2_swa8k}
FAMILY=${FAMILY:-ipttcd}
NGPU=${NGPU:-8}
SEQ_LEN=${SEQ_LEN:-65536}
CONTEXT_LEN=${CONTEXT_LEN:-${SEQ_LEN}}
CONFIG_PATH=${CONFIG_PATH:-configs/${FAMILY}/${MODEL}.json}
TOKENIZER=${TOKENIZER:-tokenizers/Qwen3-0.6B-Base}
EXP_DIR=${EXP_DIR:-exp/${MODEL}}
DATASET=${DATASET:-synthetic}
DCP_INIT=${DCP_INIT:-${EXP_DIR}/checkpoint/step-0}
mkdir -p "${EXP_DIR}"
EXTRA=()
[ -d "${DCP_INIT}" ] && EXTRA+=(--checkpoint.initial_load_path "${DCP_INIT}" --checkpoint.initial_load_model_weights_only)
[ "${MUON:-0}" = "1" ] && EXTRA+=(--optimizer.enable_muon)
[ "${CP:-1}" != "1" ] && EXTRA+=(--experimental.context_parallel_degree "${CP}")
[ "${TP:-1}" != "1" ] && EXTRA+=(--training.tensor_parallel_degree "${TP}")

python -m torch.distributed.run --nproc-per-node "${NGPU}" --master-addr 127.0.0.1 --master-port "${MASTER_PORT:-29500}" \
  -m flame.train \
  --job.config_file flame/models/fla.toml \
  --job.dump_folder "${EXP_DIR}" \
  --model.config "${CONFIG_PATH}" \
  --model.tokenizer_path "${TOKENIZER}" \
  --optimizer.name AdamW --optimizer.eps 1e-15 --optimizer.lr "${LR:-1e-5}" \
  --lr_scheduler.warmup_steps "${WARMUP_STEPS:-100}" --lr_scheduler.lr_min_absolute "${LR_FINAL:-1e-6}" \
  --lr_scheduler.decay_type cosine \
  --training.batch_size "${BATCH_SIZE:-1}" --training.seq_len "${SEQ_LEN}" --training.context_len "${CONTEXT_LEN}" \
  --training.gradient_accumulation_steps "${GRAD_ACCUM:-1}" --training.steps "${TOTAL_STEPS:-10000}" \
  --training.max_norm 1.0 --training.skip_nan_inf \
  --training.dataset "${DATASET}" --training.dataset_split train --training.num_workers 4 --training.prefetch_factor 2 \
  --training.seed 42 \
  --checkpoint.enable_checkpoint --checkpoint.interval 2000 --checkpoint.load_step -1 --checkpoint.keep_latest_k 2 \
  --metrics.log_freq 10 \
  --activation_checkpoint.mode "${AC:-none}" \
  --comm.train_timeout_seconds 600 \
  "${EXTRA[@]}" "$@"
