#!/usr/bin/env bash
# Supervised fine-tuning. data.train_files: parquet / jsonl with a `messages` column (multi-turn) or prompt/response keys.
set -euo pipefail
# CONTROLLER=1: one driver process with a worker group of training workers behind it (verl_b200.trainer.sft_trainer_ray)
# instead of one SPMD process per GPU.
NGPU=${NGPU:-1}
LAUNCH="python"
MODULE=verl_b200.trainer.sft_trainer
EXTRA=""
if [ "${CONTROLLER:-0}" = "1" ]; then
  MODULE=verl_b200.trainer.sft_trainer_ray
  EXTRA="trainer.n_gpus_per_node=$NGPU"
elif [ "$NGPU" -gt 1 ]; then
  LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
fi
$LAUNCH -m $MODULE $EXTRA \
  model.path=${MODEL:-preset:qwen2.5-0.5b} \
  data.train_files=${TRAIN:-synthetic:4096:64:512:2000:0} data.val_files=${VAL:-synthetic:256:64:512:2000:1} \
  data.multiturn=false data.train_batch_size=$((64 * NGPU)) data.max_length=1024 data.max_token_len_per_gpu=16384 \
  optim.lr=1e-5 trainer.total_epochs=1 trainer.logger='[console]' trainer.save_freq=-1 "$@"
