#!/usr/bin/env bash
# GRPO with rollout correction: the rollout engine's log-probs of the sampled tokens correct the off-policy gap between
# the rollout and the training numerics. MODE=token_is (truncated importance weights per token, the default here) |
# seq_is (per sequence) | token_rs (rejection: tokens whose ratio leaves the band are masked out) | bypass (the rollout
# log-probs stand in for old_log_probs: no compute_log_prob pass).
set -euo pipefail
MODE=${MODE:-token_is}
C=algorithm.rollout_correction
case "$MODE" in
  token_is) OV="$C.rollout_is=token $C.rollout_is_threshold=2.0" ;;
  seq_is)   OV="$C.rollout_is=sequence $C.rollout_is_threshold=2.0" ;;
  token_rs) OV="$C.rollout_rs=token_k1 $C.rollout_rs_threshold=0.5_2.0" ;;
  bypass)   OV="$C.bypass_mode=true $C.rollout_is=token $C.rollout_is_threshold=2.0" ;;
  *) echo "unknown MODE=$MODE" >&2; exit 2 ;;
esac
if [ "${DRY_RUN:-0}" = "1" ]; then printf '%s\n' $OV; exit 0; fi
exec "$(dirname "$0")/../grpo_trainer/run_qwen2_5-7b.sh" actor_rollout_ref.rollout.calculate_log_probs=true $OV "$@"
