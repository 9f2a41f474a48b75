"""TrainingWorker (train_mini_batch / train_batch / infer_batch on TensorDict batches in the no-padding layout)."""

from functools import partial

import torch

from verl_b200.utils import tensordict_utils as tu


class C(dict):
    __getattr__ = dict.get


def _worker(lr=5e-3, **eng):
    from verl_b200.models import preset
    from verl_b200.workers.training_worker import TrainingWorker

    cfg = C(model_type="language_model", model_config=preset("tiny-qwen2"),
            engine_config=C(strategy="fsdp", micro_batch_size_per_gpu=2, infer_micro_batch_size_per_gpu=4, seed=1, **eng),
            optimizer_config=C(lr=lr, weight_decay=0.0, clip_grad=1.0))
    w = TrainingWorker(cfg, device_name="cpu")
    w.reset()
    return w


def _sft_batch(n=8, seed=0):
    g = torch.Generator().manual_seed(seed)
    seqs = [torch.randint(3, 200, (int(L),), generator=g) for L in torch.randint(6, 20, (n,), generator=g)]
    masks = [torch.cat([torch.zeros(3, dtype=torch.long), torch.ones(len(s) - 3, dtype=torch.long)]) for s in seqs]
    nt = lambda xs: torch.nested.as_nested_tensor(xs, layout=torch.jagged)  # noqa: E731
    return tu.get_tensordict({"input_ids": nt(seqs), "loss_mask": nt(masks)}, {"temperature": 1.0})


def test_sft_training_lowers_the_loss_and_infer_returns_log_probs():
    from verl_b200.workers.utils.losses import sft_loss_on_batch

    w = _worker()
    w.set_loss_fn(partial(sft_loss_on_batch, None))
    batch = _sft_batch()
    first = tu.get(w.infer_batch(_sft_batch()), "metrics")["loss"]
    out = w.train_mini_batch(tu.get_tensordict({k: batch[k] for k in ("input_ids", "loss_mask")},
                                               {"temperature": 1.0, "mini_batch_size": 4, "epochs": 6, "seed": 3}))
    m = tu.get(out, "metrics")
    assert len(m["loss"]) == 12 and len(m["grad_norm"]) == 12 and "lr" in m and "mfu" in m
    res = w.infer_batch(_sft_batch())
    last = tu.get(res, "metrics")["loss"]
    assert last < first - 0.3, (first, last)
    lp = res["log_probs"]
    assert lp.is_nested and torch.equal(lp.offsets(), _sft_batch()["input_ids"].offsets()) and bool((lp.values() <= 0).all())


def test_ppo_loss_through_the_batch_interface_matches_the_dp_actor():
    """One optimizer step with ``ppo_loss_on_batch`` on a no-padding batch = ``DataParallelPPOActor.update_policy`` on
    the padded batch of the same samples."""
    from verl_b200 import DataProto
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.utils.losses import ppo_loss_on_batch

    g = torch.Generator().manual_seed(5)
    B, P, R = 4, 6, 8
    ids = torch.randint(3, 2000, (B, P + R), generator=g)
    mask = torch.ones(B, P + R, dtype=torch.long)
    mask[0, :2] = 0       # left padding of a prompt
    mask[1, -3:] = 0      # right padding of a response
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    adv = torch.randn(B, R, generator=g)
    nested = torch.nested.as_nested_tensor([ids[i][mask[i].bool()] for i in range(B)], layout=torch.jagged)
    # behaviour log-probs: the current policy's, slightly perturbed so that ratios differ from 1 without clipping
    from verl_b200.workers.utils.losses import slice_response_from_unpad_output

    probe = _worker(lr=1e-3)
    lp_now = probe.infer_batch(tu.get_tensordict({"input_ids": nested}, {"temperature": 1.0, "compute_loss": False}))["log_probs"]
    old = slice_response_from_unpad_output(lp_now, {"prompts": ids[:, :P], "responses": ids[:, P:], "attention_mask": mask})
    old = (old + 0.05 * torch.randn(B, R, generator=g)) * mask[:, P:]
    acfg = FSDPActorConfig(ppo_mini_batch_size=B, ppo_micro_batch_size_per_gpu=2, use_kl_loss=False, clip_ratio=0.2,
                           ppo_epochs=2)  # two epochs: the actor then uses the given old log-probs, not its own
    w1 = _worker(lr=1e-3)
    actor = DataParallelPPOActor(acfg, w1.engine)
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, P:],
                                "response_mask": mask[:, P:], "old_log_probs": old, "advantages": adv},
                               meta_info={"temperature": 1.0})
    with w1.engine.train_mode():
        m1 = actor.update_policy(data)
    w2 = _worker(lr=1e-3)
    w2.set_loss_fn(partial(ppo_loss_on_batch, FSDPActorConfig(ppo_mini_batch_size=B, use_kl_loss=False, clip_ratio=0.2)))
    td = tu.get_tensordict({"input_ids": nested, "prompts": ids[:, :P], "responses": ids[:, P:], "attention_mask": mask,
                            "response_mask": mask[:, P:], "old_log_probs": old, "advantages": adv}, {"temperature": 1.0})
    m2 = tu.get(w2.train_batch(td), "metrics")
    assert abs(m2["grad_norm"] - m1["actor/grad_norm"][0]) < 1e-4 * max(1.0, m2["grad_norm"]), (m1, m2)
    assert m2["grad_norm"] > 1e-2
