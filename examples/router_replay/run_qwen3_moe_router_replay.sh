#!/usr/bin/env bash
# GRPO on a Qwen3-MoE architecture with router replay. MODE=R2: the experts chosen in compute_log_prob are replayed in
# the update; MODE=R3: the rollout engine records the experts of every token and both passes replay them (the prefix
# cache of the rollout engine is off while it records).
set -euo pipefail
NGPU=${NGPU:-1}
MODE=${MODE:-R2}
MODEL=${MODEL:-preset:tiny-qwen3-moe}        # preset:qwen3-30b-a3b or a HF checkpoint directory for the real size
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
R3=false; [ "$MODE" = "R3" ] && R3=true
$LAUNCH -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo actor_rollout_ref.model.path="$MODEL" \
  data.train_files="${TRAIN:-synthetic:256:32:64:16:2000:0}" data.val_files=null \
  data.train_batch_size=$((8 * NGPU)) data.max_prompt_length=128 data.max_response_length=128 \
  actor_rollout_ref.rollout.n=4 actor_rollout_ref.actor.ppo_mini_batch_size=$((4 * NGPU)) \
  actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4 actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=8 \
  actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=8 \
  actor_rollout_ref.actor.router_replay.mode="$MODE" actor_rollout_ref.rollout.enable_rollout_routing_replay=$R3 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=${ROLLOUT_TP:-1} \
  trainer.n_gpus_per_node="$NGPU" trainer.nnodes=1 trainer.logger='[console]' trainer.val_before_train=false \
  trainer.total_epochs=1 trainer.save_freq=-1 trainer.test_freq=-1 "$@"
