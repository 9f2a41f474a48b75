#!/usr/bin/env bash
# GRPO on a Qwen3-MoE architecture; the rollout engine quantises the linear layers to block-scaled fp8
# (128 x 128 weight blocks, 1 x 128 activation blocks) after every weight sync.
set -euo pipefail
MODEL=${MODEL:-preset:tiny-qwen3-moe} exec "$(dirname "$0")/run_qwen2_5-7b.sh" \
  actor_rollout_ref.rollout.quantization=fp8 "$@"
