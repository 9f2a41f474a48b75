#!/usr/bin/env bash
# One launcher for the advantage estimators and policy losses beside GRPO / PPO:
#   ALGO=rloo | remax | reinforce_plus_plus | reinforce_plus_plus_baseline | opo | gpg | grpo_passk | otb |
#        gspo | sapo | gmpo | cispo | clip_cov | kl_cov
# DRY_RUN=1 prints the algorithm's overrides (one per line) and exits.
set -euo pipefail
ALGO=${ALGO:-rloo}
NGPU=${NGPU:-1}
MODEL=${MODEL:-preset:qwen2.5-0.5b}
A=actor_rollout_ref.actor
case "$ALGO" in
  rloo|remax|reinforce_plus_plus|reinforce_plus_plus_baseline|opo|grpo_passk)
    # critic-free estimators with the KL penalty inside the reward
    OV="algorithm.adv_estimator=$ALGO $A.use_kl_loss=false algorithm.use_kl_in_reward=true algorithm.kl_penalty=kl algorithm.kl_ctrl.kl_coef=0.001" ;;
  gpg)
    OV="algorithm.adv_estimator=gpg $A.policy_loss.loss_mode=gpg $A.use_kl_loss=false $A.entropy_coeff=0 algorithm.use_kl_in_reward=false" ;;
  otb)
    # optimal token baseline: compute_log_prob also returns the sum of squared token probabilities
    OV="algorithm.adv_estimator=optimal_token_baseline $A.calculate_sum_pi_squared=true $A.use_kl_loss=false $A.entropy_coeff=0" ;;
  gspo)
    OV="algorithm.adv_estimator=grpo $A.policy_loss.loss_mode=gspo $A.clip_ratio_low=3e-4 $A.clip_ratio_high=4e-4 $A.loss_agg_mode=seq-mean-token-mean $A.use_kl_loss=false" ;;
  sapo)
    OV="algorithm.adv_estimator=grpo $A.policy_loss.loss_mode=sapo $A.tau_pos=1.0 $A.tau_neg=1.05 $A.use_kl_loss=false" ;;
  gmpo)
    OV="algorithm.adv_estimator=grpo $A.policy_loss.loss_mode=geo_mean $A.clip_ratio_low=0.4 $A.clip_ratio_high=0.4 $A.use_kl_loss=false $A.entropy_coeff=0" ;;
  cispo)
    OV="algorithm.adv_estimator=grpo $A.policy_loss.loss_mode=cispo $A.clip_ratio_low=10 $A.clip_ratio_high=0.2 $A.use_kl_loss=true $A.kl_loss_coef=0.001 $A.kl_loss_type=low_var_kl" ;;
  clip_cov|kl_cov)
    OV="algorithm.adv_estimator=grpo $A.policy_loss.loss_mode=$ALGO $A.use_kl_loss=false" ;;
  *) echo "unknown ALGO=$ALGO" >&2; exit 2 ;;
esac
if [ "${DRY_RUN:-0}" = "1" ]; then printf '%s\n' $OV; exit 0; fi
LAUNCH="python"
[ "$NGPU" -gt 1 ] && LAUNCH="python -m torch.distributed.run --nnodes=1 --nproc-per-node $NGPU --master-addr 127.0.0.1 --master-port ${PORT:-29500}"
$LAUNCH -m verl_b200.trainer.main_ppo $OV \
  actor_rollout_ref.model.path="$MODEL" \
  data.train_files="${TRAIN:-synthetic:1024:128:256:100:151000:0:synthetic/contains_token:4242}" data.val_files=null \
  data.train_batch_size=$((16 * NGPU)) data.max_prompt_length=256 data.max_response_length=512 \
  actor_rollout_ref.rollout.n=${N:-4} $A.ppo_mini_batch_size=$((16 * NGPU)) $A.use_dynamic_bsz=true \
  $A.ppo_max_token_len_per_gpu=16384 actor_rollout_ref.rollout.log_prob_use_dynamic_bsz=true \
  actor_rollout_ref.rollout.log_prob_max_token_len_per_gpu=32768 actor_rollout_ref.ref.log_prob_use_dynamic_bsz=true \
  actor_rollout_ref.ref.log_prob_max_token_len_per_gpu=32768 $A.optim.lr=1e-6 \
  actor_rollout_ref.rollout.tensor_model_parallel_size=${ROLLOUT_TP:-1} \
  trainer.n_gpus_per_node="$NGPU" trainer.nnodes=1 trainer.logger='[console]' trainer.val_before_train=false \
  trainer.total_epochs=1 trainer.save_freq=-1 trainer.test_freq=-1 "$@"
