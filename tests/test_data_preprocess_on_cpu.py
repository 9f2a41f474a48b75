"""examples/data_preprocess/rl_data.py: local raw files -> parquet rows that the datasets and the reward functions accept."""
import importlib.util
import json
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _mod():
    spec = importlib.util.spec_from_file_location("rl_data", os.path.join(ROOT, "examples", "data_preprocess", "rl_data.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_gsm8k_rows_load_and_score(tmp_path):
    import zlib

    from verl_b200.utils.dataset.rl_dataset import RLHFDataset
    from verl_b200.utils.reward_score import default_compute_score
    from verl_b200.utils.tokenizer import IntTokenizer

    class WordTokenizer(IntTokenizer):  # words -> ids by a stable hash: enough to tokenize real text in a test
        def encode(self, text, add_special_tokens=False):
            return [3 + zlib.crc32(w.encode()) % (self.vocab_size - 3) for w in text.split()]

    m = _mod()
    raw = tmp_path / "raw.jsonl"
    raw.write_text("\n".join(json.dumps(r) for r in [
        {"question": "1 2 3", "answer": "3 plus 4 is 7\n#### 7"},
        {"question": "4 5", "answer": "a lot\n#### 1,234."}]))
    out = tmp_path / "o" / "train.parquet"
    m.main(["--task", "gsm8k", "--input", str(raw), "--output", str(out)])
    ds = RLHFDataset(str(out), WordTokenizer(512), {"max_prompt_length": 64, "prompt_key": "prompt"})
    assert len(ds) == 2
    it = ds[1]
    assert it["data_source"] == "openai/gsm8k" and it["reward_model"]["ground_truth"] == "1234"
    assert it["extra_info"]["index"] == 1 and it["extra_info"]["split"] == "train"
    assert default_compute_score("openai/gsm8k", "so the answer is #### 1234", "1234") == 1.0
    assert default_compute_score("openai/gsm8k", "#### 12", "1234") == 0.0
    # rows for the tool agent loop and for SFT
    tool = m.make_row("gsm8k", {"question": "q", "answer": "#### 5"}, "train", 0, with_tool=True)
    assert tool["agent_name"] == "tool_agent" and tool["extra_info"]["tools_kwargs"]["calc_gsm8k_reward"]["create_kwargs"] == {"ground_truth": "5"}
    sft = m.make_row("gsm8k", {"question": "q", "answer": "w\n#### 5"}, "train", 0, sft=True)
    assert [t["role"] for t in sft["messages"]] == ["user", "assistant"]
    with pytest.raises(ValueError):
        m.gsm8k_answer("no marker")


def test_math_rows_extract_the_last_balanced_box():
    m = _mod()
    row = m.make_row("math", {"problem": "p", "solution": "first \\boxed{1} then \\boxed{\\frac{a}{b^{2}}}."}, "test", 3)
    assert row["reward_model"]["ground_truth"] == "\\frac{a}{b^{2}}" and row["data_source"].endswith("MATH-lighteval")
    assert row["prompt"][0]["content"].endswith("\\boxed{}.")
    from verl_b200.utils.reward_score import default_compute_score

    assert default_compute_score(row["data_source"], "thus \\boxed{\\frac{a}{b^{2}}}", row["reward_model"]["ground_truth"]) == 1.0
