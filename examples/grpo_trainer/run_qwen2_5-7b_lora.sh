#!/usr/bin/env bash
# GRPO with LoRA: frozen base (no optimizer state), adapters trained, merged weights pushed to the rollout copy.
set -euo pipefail
exec "$(dirname "$0")/run_qwen2_5-7b.sh" \
  actor_rollout_ref.model.lora_rank=32 actor_rollout_ref.model.lora_alpha=32 \
  actor_rollout_ref.model.target_modules=all-linear actor_rollout_ref.actor.optim.lr=3e-5 "$@"
