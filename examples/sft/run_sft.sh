#!/usr/bin/env bash
# Supervised fine-tuning. data.train_files: parquet / jsonl with a `messages` column (multi-turn) or prompt/response keys.
set -euo pipefail
NGPU=${NGPU:-1}
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
$LAUNCH -m verl_b200.trainer.sft_trainer \
  model.path=${MODEL:-preset:qwen2.5-0.5b} \
  data.train_files=${TRAIN:-synthetic:4096:64:512:2000:0} data.val_files=${VAL:-synthetic:256:64:512:2000:1} \
  data.multiturn=false data.train_batch_size=$((64 * NGPU)) data.max_length=1024 data.max_token_len_per_gpu=16384 \
  optim.lr=1e-5 trainer.total_epochs=1 trainer.logger='[console]' trainer.save_freq=-1 "$@"
