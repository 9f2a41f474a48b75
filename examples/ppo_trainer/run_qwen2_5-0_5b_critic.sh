#!/usr/bin/env bash
# PPO with a critic (GAE), Qwen2.5-0.5B architecture.
set -euo pipefail
NGPU=${NGPU:-1}
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
$LAUNCH -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=gae algorithm.gamma=1.0 algorithm.lam=1.0 \
  actor_rollout_ref.model.path=${MODEL:-preset:qwen2.5-0.5b} critic.model.path=${MODEL:-preset:qwen2.5-0.5b} \
  data.train_files=${TRAIN:-synthetic:2048:64:256:100:151000:0} data.val_files=null \
  data.train_batch_size=$((64 * NGPU)) data.max_prompt_length=256 data.max_response_length=512 \
  actor_rollout_ref.rollout.n=1 actor_rollout_ref.actor.ppo_mini_batch_size=$((64 * NGPU)) \
  actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=16 actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=32 \
  actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=32 critic.ppo_micro_batch_size_per_gpu=16 \
  actor_rollout_ref.actor.use_kl_loss=false critic.optim.lr=1e-5 actor_rollout_ref.actor.optim.lr=1e-6 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=${ROLLOUT_TP:-1} \
  trainer.n_gpus_per_node="$NGPU" trainer.nnodes=1 trainer.logger='[console]' trainer.val_before_train=false \
  trainer.total_epochs=1 trainer.save_freq=-1 trainer.test_freq=-1 "$@"
