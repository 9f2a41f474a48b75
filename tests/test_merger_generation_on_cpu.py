"""Model merger CLI, offline generation and offline evaluation on CPU."""

import json

import torch


def test_merge_checkpoint_roundtrip(tmp_path):
    from verl_b200.model_merger import merge_checkpoint, test_merged
    from verl_b200.model_merger.merger import main as merger_main
    from verl_b200.models import preset
    from verl_b200.models.hf_io import load_hf_checkpoint
    from verl_b200.workers.engine.native import NativeEngine

    cfg = preset("tiny-qwen2")
    eng = NativeEngine(cfg, None, {"lr": 1e-3}, device="cpu", seed=5).initialize()
    ref = {k: v.detach().clone() for k, v in eng.model.named_parameters()}
    eng.save_checkpoint(str(tmp_path / "actor"), global_step=1)
    merge_checkpoint(str(tmp_path / "actor"), str(tmp_path / "hf"), dtype=torch.float32)
    cfg2, sd = load_hf_checkpoint(tmp_path / "hf")
    assert cfg2.hidden_size == cfg.hidden_size
    for k, v in ref.items():
        torch.testing.assert_close(sd[k].float(), v.float())
    test_merged(str(tmp_path / "actor"), str(tmp_path / "hf"))
    merger_main(["merge", "--backend", "fsdp", "--local_dir", str(tmp_path / "actor"), "--target_dir", str(tmp_path / "hf2")])
    merger_main(["test", "--backend", "fsdp", "--local_dir", str(tmp_path / "actor"), "--test_hf_dir", str(tmp_path / "hf2")])


def test_generation_and_eval(tmp_path):
    from verl_b200.trainer.main_eval import main as eval_main
    from verl_b200.trainer.main_generation import main as gen_main

    rows = [{"prompt": "1 2 3", "data_source": "openai/gsm8k", "reward_model": {"ground_truth": "7"}} for _ in range(3)]
    (tmp_path / "p.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    gen_main(["model.path=preset:tiny-qwen2", f"data.path={tmp_path}/p.jsonl", f"data.output_path={tmp_path}/o.jsonl",
              "rollout.n=2", "rollout.response_length=8", "rollout.prompt_length=32", "trainer.device=cpu",
              "rollout.max_num_seqs=8", "rollout.max_num_batched_tokens=256"])
    out = [json.loads(line) for line in (tmp_path / "o.jsonl").read_text().splitlines()]
    assert len(out) == 3 and all(len(r["responses"]) == 2 for r in out)
    eval_main([f"data.path={tmp_path}/o.jsonl"])


def test_generation_through_standalone_servers(tmp_path):
    """Two standalone replicas behind HTTP; greedy decoding gives the same text for identical prompts whichever
    replica served them."""
    from verl_b200.trainer.main_generation_server import main as gen_main

    rows = [{"prompt": "1 2 3", "id": i} for i in range(4)]
    (tmp_path / "p.jsonl").write_text("\n".join(json.dumps(r) for r in rows))
    out = gen_main(["model.path=preset:tiny-qwen2", f"data.path={tmp_path}/p.jsonl", f"data.output_path={tmp_path}/o.jsonl",
                    "rollout.n=2", "rollout.response_length=6", "rollout.prompt_length=32", "trainer.device=cpu",
                    "rollout.max_num_seqs=8", "rollout.max_num_batched_tokens=256", "rollout.num_replicas=2",
                    "rollout.do_sample=false"])
    saved = [json.loads(line) for line in (tmp_path / "o.jsonl").read_text().splitlines()]
    assert len(out) == len(saved) == 4 and all(len(r["responses"]) == 2 for r in saved)
    texts = {t for r in saved for t in r["responses"]}
    assert len(texts) == 1 and len(next(iter(texts)).split()) > 0


def test_init_random_model_and_print_cfg(tmp_path, capsys):
    from verl_b200.models.init_random_model import main as init_main
    from verl_b200.trainer.print_cfg import main as print_main
    from verl_b200.workers.engine_workers import resolve_model_config

    out = init_main(["--preset", "tiny-qwen2", "--out", str(tmp_path / "m"), "--seed", "3", "--dtype", "float32",
                     "--override", "num_hidden_layers=1"])
    assert (tmp_path / "m" / "config.json").exists()
    cfg, state = resolve_model_config({"path": out})
    assert cfg.num_hidden_layers == 1 and state is not None and any(k.startswith("layers.0.") for k in state)
    text = print_main(["ppo_trainer", "data.train_batch_size=7"])
    assert "train_batch_size: 7" in text and "actor_rollout_ref" in text
