#!/usr/bin/env bash
# GRPO with shared-prefix evaluation: in the forward-only passes (old log-probs, reference log-probs) every distinct
# prompt of a micro-batch is evaluated once and its n responses attend to its keys.
set -euo pipefail
exec "$(dirname "$0")/../grpo_trainer/run_qwen2_5-7b.sh" \
  actor_rollout_ref.actor.use_prefix_grouper=true "$@"
