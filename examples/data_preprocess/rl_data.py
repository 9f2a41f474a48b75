#!/usr/bin/env python
"""Raw question / answer files -> the parquet schema the RL and SFT datasets read.

    python examples/data_preprocess/rl_data.py --task gsm8k --input train.jsonl --output ~/data/gsm8k/train.parquet
    python examples/data_preprocess/rl_data.py --task math  --input math_train.jsonl --output ~/data/math/train.parquet
    python examples/data_preprocess/rl_data.py --task gsm8k --input train.jsonl --output train_tool.parquet --with-tool
    python examples/data_preprocess/rl_data.py --task gsm8k --input train.jsonl --output sft.parquet --sft

Role of the reference's examples/data_preprocess/{gsm8k,math_dataset,gsm8k_multiturn_w_tool,gsm8k_multiturn_sft}.py, which
pull the datasets from the hub; this script takes LOCAL copies (``.jsonl`` / ``.json`` / ``.parquet``; GSM8K rows with
``question`` / ``answer``, MATH rows with ``problem`` / ``solution``) because the machines this framework targets often have
no network. Every output row has ``data_source``, ``prompt`` (a chat message list), ``ability``,
``reward_model = {style: rule, ground_truth}`` and ``extra_info = {split, index, question, answer, ...}``:
the fields ``RLHFDataset``, the reward managers and ``utils/reward_score`` dispatch on.
"""

from __future__ import annotations

import argparse
import json
import os
import re

GSM8K_SUFFIX = 'Let\'s think step by step and output the final answer after "####".'
MATH_SUFFIX = "Let's think step by step and output the final answer within \\boxed{}."


def read_rows(path: str) -> list[dict]:
    path = os.path.expanduser(path)
    if path.endswith(".parquet"):
        import pandas as pd

        return pd.read_parquet(path).to_dict("records")
    if path.endswith(".jsonl"):
        return [json.loads(line) for line in open(path) if line.strip()]
    data = json.load(open(path))
    return data if isinstance(data, list) else data.get("data", data.get("rows"))


def gsm8k_answer(solution: str) -> str:
    """The number after the last ``####`` of a GSM8K solution, without thousands separators."""
    m = re.findall(r"#### *(-?[0-9.,]+)", solution)
    if not m:
        raise ValueError(f"no '#### <number>' in {solution[-80:]!r}")
    return m[-1].replace(",", "").rstrip(".")


def last_boxed(text: str) -> str:
    """Contents of the last ``\\boxed{...}`` (balanced braces) of a MATH solution."""
    i = text.rfind("\\boxed{")
    if i < 0:
        raise ValueError(f"no \\boxed{{}} in {text[-80:]!r}")
    depth, j = 0, i + len("\\boxed{") - 1
    for k in range(j, len(text)):
        depth += text[k] == "{"
        depth -= text[k] == "}"
        if depth == 0:
            return text[j + 1 : k]
    raise ValueError("unbalanced \\boxed{")


def make_row(task: str, raw: dict, split: str, index: int, with_tool: bool = False, sft: bool = False) -> dict:
    if task == "gsm8k":
        question, solution = raw["question"], raw["answer"]
        truth, source, suffix = gsm8k_answer(solution), "openai/gsm8k", GSM8K_SUFFIX
    elif task == "math":
        question, solution = raw["problem"], raw["solution"]
        truth, source, suffix = last_boxed(solution), "DigitalLearningGmbH/MATH-lighteval", MATH_SUFFIX
    else:
        raise ValueError(f"unknown task {task!r}")
    user = {"role": "user", "content": f"{question} {suffix}"}
    if sft:  # multi-turn SFT rows: the dataset masks everything but the assistant turns
        return {"messages": [user, {"role": "assistant", "content": solution}], "data_source": source}
    row = {"data_source": source, "prompt": [user], "ability": "math", "reward_model": {"style": "rule", "ground_truth": truth},
           "extra_info": {"split": split, "index": index, "question": question, "answer": solution}}
    if with_tool:
        # the tool agent loop creates one answer-checking tool instance per sample with these arguments
        row["prompt"] = [{"role": "system", "content": "You are a math expert. Check your answer with the `calc_gsm8k_reward` "
                                                       "tool once before you give the final answer."}, user]
        row["agent_name"] = "tool_agent"
        row["extra_info"]["need_tools_kwargs"] = True
        row["extra_info"]["tools_kwargs"] = {"calc_gsm8k_reward": {"create_kwargs": {"ground_truth": truth}}}
    return row


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--task", choices=["gsm8k", "math"], required=True)
    ap.add_argument("--input", required=True, help="local .jsonl / .json / .parquet file with the raw rows")
    ap.add_argument("--output", required=True, help="parquet file to write")
    ap.add_argument("--split", default="train")
    ap.add_argument("--with-tool", action="store_true", help="rows for the multi-turn tool agent loop")
    ap.add_argument("--sft", action="store_true", help="rows with a `messages` column for the SFT trainers")
    ap.add_argument("--max-rows", type=int, default=-1)
    a = ap.parse_args(argv)
    import pandas as pd

    raws = read_rows(a.input)
    if a.max_rows > 0:
        raws = raws[: a.max_rows]
    rows = [make_row(a.task, r, a.split, i, a.with_tool, a.sft) for i, r in enumerate(raws)]
    out = os.path.expanduser(a.output)
    os.makedirs(os.path.dirname(out) or ".", exist_ok=True)
    pd.DataFrame(rows).to_parquet(out)
    print(json.dumps({"rows": len(rows), "output": out}))


if __name__ == "__main__":
    main()
