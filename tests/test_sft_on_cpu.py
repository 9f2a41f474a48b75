"""SFT trainer on CPU: loss goes down on a tiny model, checkpoints resume, datasets build the right loss masks."""

import json
import os

import torch

from verl_b200.utils.config import compose
from verl_b200.utils.tokenizer import IntTokenizer


def _config(tmp_path, **over):
    ov = [
        "model.path=preset:tiny-qwen2", "data.train_files=synthetic:64:24:48:250:1", "data.val_files=synthetic:8:24:48:250:2",
        "data.train_batch_size=8", "data.micro_batch_size_per_gpu=4", "data.max_token_len_per_gpu=128", "data.max_length=48",
        "data.multiturn=false", "data.pad_mode=right", "optim.lr=3e-3", "trainer.total_epochs=1", "trainer.total_training_steps=6",
        "trainer.device=cpu", f"trainer.default_local_dir={tmp_path}/ckpt", "trainer.save_freq=3", "trainer.test_freq=3",
        "trainer.logger=[console]",
    ] + [f"{k}={v}" for k, v in over.items()]
    return compose("sft_trainer", ov)


def test_sft_loss_decreases_and_resumes(tmp_path):
    from verl_b200.trainer.sft_trainer import SFTTrainer

    cfg = _config(tmp_path)
    tr = SFTTrainer(cfg, tokenizer=IntTokenizer(256))
    losses = []
    for step, (_, idx) in enumerate(tr._batches(0)):
        from verl_b200.utils.dataset.sft_dataset import sft_collate_fn

        m = tr.train_step(sft_collate_fn([tr.train_dataset[i] for i in idx]))
        losses.append(m["train/loss"])
        tr.global_step += 1
        if step == 2:
            tr.save_checkpoint()
            v = tr.validate()
            assert v["val/loss"] > 0
    assert losses[-1] < losses[0]
    # a new trainer picks up the step-3 checkpoint and reproduces the weights saved there
    tr2 = SFTTrainer(cfg, tokenizer=IntTokenizer(256))
    assert tr2.global_step == 3
    out = tr2.fit()
    assert tr2.global_step == 6 and "train/loss" in out


def test_sft_dataset_masks(tmp_path):
    from verl_b200.utils.dataset.sft_dataset import MultiTurnSFTDataset, SFTDataset

    tok = IntTokenizer(512)
    rows = [{"prompt": "1 2 3", "response": "4 5", "messages": [{"role": "user", "content": "1 2 3"},
                                                                 {"role": "assistant", "content": "4 5"},
                                                                 {"role": "user", "content": "6"},
                                                                 {"role": "assistant", "content": "7 8 9"}]}]
    f = tmp_path / "d.jsonl"
    f.write_text("\n".join(json.dumps(r) for r in rows))
    ds = SFTDataset(str(f), tok, {"max_length": 64, "pad_mode": "right", "truncation": "right"})
    it = ds[0]
    n = int(it["attention_mask"].sum())
    assert it["input_ids"].shape == (64,) and it["loss_mask"][n - 1] == 0
    # the last prompt position predicts the first response token
    first = int(torch.nonzero(it["loss_mask"])[0])
    assert it["loss_mask"][first:n - 1].all() and not it["loss_mask"][:first].any()
    mt = MultiTurnSFTDataset(str(f), tok, {"max_length": 128, "pad_mode": "no_padding"})
    it = mt[0]
    assert it["input_ids"].numel() == it["loss_mask"].numel() < 128
    assert 0 < int(it["loss_mask"].sum()) < it["loss_mask"].numel()


def test_controller_driven_sft_trains_validates_and_resumes(tmp_path):
    """The single-controller SFT trainer: two TrainingWorker processes (gloo) behind a worker group, one no-padding
    TensorDict per step, checkpoints through the CheckpointHandler; a second trainer resumes at the saved step with the
    sampler's position and ends with the same loss as an uninterrupted run."""
    from verl_b200.trainer.sft_trainer_ray import SFTTrainer, StatefulBatchSampler

    s = StatefulBatchSampler(20, 4, 2, shuffle=True, seed=1)
    first = [b for _, b in zip(range(3), s)]
    s2 = StatefulBatchSampler(20, 4, 2, shuffle=True, seed=1)
    s2.load_state_dict(s.state_dict())
    rest, full = list(s2), list(StatefulBatchSampler(20, 4, 2, shuffle=True, seed=1))
    assert first + rest == full and len(full) == 10 and sorted(sum(full[:5], [])) == list(range(20))

    def run(sub, **over):
        cfg = _config(tmp_path / sub, **{"trainer.n_gpus_per_node": 2, "data.pad_mode": "no_padding", **over})
        tr = SFTTrainer(cfg, tokenizer=IntTokenizer(256))
        try:
            return tr, tr.fit()
        finally:
            tr.shutdown()

    ref, out_ref = run("a", **{"trainer.total_training_steps": 6, "trainer.save_freq": -1})
    assert ref.global_step == 6 and out_ref["val/loss"] > 0 and out_ref["train/grad_norm"] > 0
    tr1, out1 = run("b", **{"trainer.total_training_steps": 3})
    assert tr1.global_step == 3 and os.path.isdir(tmp_path / "b" / "ckpt" / "global_step_3")
    assert os.path.exists(tmp_path / "b" / "ckpt" / "global_step_3" / "data_0.pt")
    tr2, out2 = run("b", **{"trainer.total_training_steps": 6})
    assert tr2.resume_global_step == 3 and tr2.global_step == 6
    assert abs(out2["train/loss"] - out_ref["train/loss"]) < 2e-3, (out2["train/loss"], out_ref["train/loss"])
    assert out2["train/loss"] < out1["train/loss"] + 0.5


def test_sft_with_the_megatron_engine_and_optimizer_choices(tmp_path):
    """``engine=megatron optim=megatron`` (the reference's group choices) compose and train on the native engine."""
    from verl_b200.trainer.sft_trainer import SFTTrainer

    cfg = _config(tmp_path, **{"engine": "megatron", "optim": "megatron", "optim.lr_decay_style": "cosine", "optim.lr": "3e-3",
                               "trainer.total_training_steps": 3, "trainer.save_freq": -1, "trainer.test_freq": -1})
    assert cfg.engine.strategy == "megatron" and cfg.optim.lr_scheduler_type == "cosine"
    out = SFTTrainer(cfg, tokenizer=IntTokenizer(256)).fit()
    assert out["train/loss"] > 0 and out["train/grad_norm"] > 0
