#!/usr/bin/env bash
# GRPO, Qwen2.5-7B architecture, one process per GPU. NGPU=1 runs in a single process.
set -euo pipefail
NGPU=${NGPU:-8}
MODEL=${MODEL:-preset:qwen2.5-7b}            # or a HF checkpoint directory
TRAIN=${TRAIN:-synthetic:4096:256:512:100:151000:0:synthetic/contains_token:4242}
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
$LAUNCH -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo \
  actor_rollout_ref.model.path="$MODEL" \
  data.train_files="$TRAIN" data.val_files=null \
  data.train_batch_size=$((16 * NGPU)) data.max_prompt_length=512 data.max_response_length=1024 \
  actor_rollout_ref.rollout.n=8 actor_rollout_ref.rollout.temperature=1.0 \
  actor_rollout_ref.rollout.gpu_memory_utilization=0.12 actor_rollout_ref.rollout.max_num_seqs=128 \
  actor_rollout_ref.actor.ppo_mini_batch_size=$((16 * NGPU)) actor_rollout_ref.actor.use_dynamic_bsz=true \
  actor_rollout_ref.actor.ppo_max_token_len_per_gpu=16384 \
  actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=true actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu=32768 \
  actor_rollout_ref.ref.log_prob_use_dynamic_bsz=true actor_rollout_ref.ref.log_prob_max_token_len_per_gpu=32768 \
  actor_rollout_ref.actor.use_kl_loss=true actor_rollout_ref.actor.kl_loss_coef=0.001 actor_rollout_ref.actor.optim.lr=1e-6 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=${ROLLOUT_TP:-1} \
  trainer.n_gpus_per_node="$NGPU" trainer.nnodes=1 trainer.logger='[console]' trainer.val_before_train=false \
  trainer.total_epochs=1 trainer.save_freq=-1 trainer.test_freq=-1 "$@"
