#!/usr/bin/env bash
# Offline generation (n samples per prompt with the native rollout engine) and rule-based evaluation of the result.
# PROMPTS: parquet / jsonl with a `prompt` column (chat messages or text) as examples/data_preprocess/rl_data.py writes.
set -euo pipefail
MODEL=${MODEL:-preset:tiny-qwen2}            # or a HF checkpoint directory
PROMPTS=${PROMPTS:?set PROMPTS to a parquet / jsonl file of prompts}
OUT=${OUT:-generation.jsonl}
python -m verl_b200.trainer.main_generation model.path="$MODEL" data.path="$PROMPTS" data.output_path="$OUT" \
  rollout.n=${N:-4} rollout.temperature=${TEMPERATURE:-1.0} rollout.prompt_length=1024 rollout.response_length=${RESPONSE_LENGTH:-512} "$@"
python -m verl_b200.trainer.main_eval data.path="$OUT" data.response_key=responses
