#!/usr/bin/env bash
# GRPO on the Qwen2.5-7B architecture with a model-parallel layout of the training engine and / or the rollout.
#   LAYOUT=tp2        tensor-parallel training (2 ranks per model copy, ZeRO over the copies) + TP = 2 rollout replicas
#   LAYOUT=pp2        two pipeline stages
#   LAYOUT=cp2        context parallelism: 2 ranks share a micro-batch, zig-zag chunks of every sequence
#   LAYOUT=sp2        Ulysses sequence parallelism
#   LAYOUT=hsdp4      hybrid sharding: ZeRO inside groups of 4, gradient all-reduce between the groups
# The reference policy follows the actor's layout unless its own keys are set.
set -euo pipefail
NGPU=${NGPU:-8}
LAYOUT=${LAYOUT:-tp2}
EXTRA=()
case "$LAYOUT" in
  tp2)   EXTRA+=(actor_rollout_ref.actor.fsdp_config.tensor_model_parallel_size=2 actor_rollout_ref.rollout.tensor_model_parallel_size=2) ;;
  pp2)   EXTRA+=(actor_rollout_ref.actor.fsdp_config.pipeline_model_parallel_size=2) ;;
  cp2)   EXTRA+=(actor_rollout_ref.actor.fsdp_config.context_parallel_size=2) ;;
  sp2)   EXTRA+=(actor_rollout_ref.actor.ulysses_sequence_parallel_size=2) ;;
  hsdp4) EXTRA+=(actor_rollout_ref.actor.fsdp_config.fsdp_size=4) ;;
  *) echo "unknown LAYOUT=$LAYOUT" >&2; exit 2 ;;
esac
exec "$(dirname "$0")/run_qwen2_5-7b.sh" "${EXTRA[@]}" "$@"
