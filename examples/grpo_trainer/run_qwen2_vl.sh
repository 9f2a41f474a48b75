#!/usr/bin/env bash
# GRPO on a Qwen2-VL / Qwen2.5-VL / Qwen3-VL architecture: images travel as multi_modal_inputs, the vision tower runs at admission in the
# rollout engine and trains with the embedding unit. Synthetic image prompts; a random-init preset by default.
set -euo pipefail
NGPU=${NGPU:-1}
MODEL=${MODEL:-preset:tiny-qwen2-vl}         # preset:tiny-qwen2.5-vl, preset:tiny-qwen3-vl; preset:qwen2-vl-7b,
                                             # qwen2.5-vl-7b, qwen3-vl-8b or a HF checkpoint directory for the real size
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
$LAUNCH -m verl_b200.trainer.main_ppo \
  algorithm.adv_estimator=grpo actor_rollout_ref.model.path="$MODEL" \
  data.train_files="${TRAIN:-synthetic:256:16:32:16:2000:0}" data.val_files=null data.synthetic_image_size=${IMAGE_SIZE:-16} \
  data.train_batch_size=$((4 * NGPU)) data.max_prompt_length=128 data.max_response_length=64 \
  actor_rollout_ref.rollout.n=4 actor_rollout_ref.actor.ppo_mini_batch_size=$((4 * NGPU)) \
  actor_rollout_ref.actor.ppo_micro_batch_size_per_gpu=4 actor_rollout_ref.rollout.log_prob_micro_batch_size_per_gpu=4 \
  actor_rollout_ref.ref.log_prob_micro_batch_size_per_gpu=4 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=${ROLLOUT_TP:-1} \
  trainer.n_gpus_per_node="$NGPU" trainer.nnodes=1 trainer.logger='[console]' trainer.val_before_train=false \
  trainer.total_epochs=1 trainer.save_freq=-1 trainer.test_freq=-1 "$@"
