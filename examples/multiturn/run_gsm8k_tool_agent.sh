#!/usr/bin/env bash
# Multi-turn GRPO: rollouts go through the tool agent loop (Hermes-style <tool_call> parsing) and the token-in /
# token-out server; tool tokens are masked out of the loss. Needs a chat model and GSM8K parquet files whose
# extra_info carries tools_kwargs (ground truth) to be meaningful.
set -euo pipefail
HERE=$(cd "$(dirname "$0")" && pwd)
exec "$HERE/../grpo_trainer/run_qwen2_5-7b.sh" \
  actor_rollout_ref.rollout.multi_turn.enable=true \
  actor_rollout_ref.rollout.multi_turn.tool_config_path="$HERE/gsm8k_tool_config.yaml" \
  actor_rollout_ref.rollout.multi_turn.max_assistant_turns=5 \
  actor_rollout_ref.rollout.agent.default_agent_loop=tool_agent data.return_raw_chat=true "$@"
