"""Shared-prefix evaluation (``use_prefix_grouper``): every distinct prompt of a micro-batch is evaluated once and its
n responses attend to its keys; log-probs and entropies equal those of the plain layout that repeats the prompt."""

import torch


def _batch(n_prompts=3, n=4, P=12, R=9, vocab=1500, seed=0):
    g = torch.Generator().manual_seed(seed)
    B = n_prompts * n
    ids = torch.zeros(B, P + R, dtype=torch.long)
    mask = torch.zeros(B, P + R, dtype=torch.long)
    for p in range(n_prompts):
        plen = int(torch.randint(3, P + 1, (1,), generator=g))
        prompt = torch.randint(5, vocab, (plen,), generator=g)
        for s in range(n):
            i = p * n + s
            rlen = int(torch.randint(1, R + 1, (1,), generator=g))
            ids[i, P - plen : P] = prompt
            mask[i, P - plen : P] = 1
            ids[i, P : P + rlen] = torch.randint(5, vocab, (rlen,), generator=g)
            mask[i, P : P + rlen] = 1
    pos = (mask.cumsum(-1) - 1).clamp(min=0)
    return ids, mask, pos, R


def test_shared_prefix_layout():
    from verl_b200.trainer.ppo.prefix_grouper_utils import shared_prefix_batch

    ids, mask, pos, R = _batch()
    packed, rows, labels, bj, saving = shared_prefix_batch(ids, mask, R)
    ps = packed.prefix_share
    P = ids.shape[1] - R
    n_prompt = sum(int(mask[i, :P].sum()) for i in range(0, 12, 4))
    assert ps["n_prompt_tokens"] == n_prompt and packed.input_ids.numel() == n_prompt + int(mask[:, P:].sum())
    assert 0.3 < saving < 0.8 and rows.numel() == labels.numel() == bj.shape[0] == int(mask[:, P:].sum())
    # the row that predicts a response's first token is the last token of its prompt (stored once per group)
    first = rows[bj[:, 1] == 0]
    assert first.numel() == 12 and len(set(first.tolist())) == 3 and int(first.max()) < n_prompt
    # keys of a response = its prompt's positions, then its own
    lens_k = (ps["cu_k"][1:] - ps["cu_k"][:-1]).tolist()
    assert lens_k == [int(mask[i].sum()) for i in range(12)]
    assert torch.equal(packed.input_ids[rows[bj[:, 1] > 0] + 1], labels[bj[:, 1] > 0])


def test_actor_log_probs_with_shared_prefix_equal_the_plain_layout():
    from verl_b200 import DataProto
    from verl_b200.models import preset
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    for name in ("tiny-qwen2", "tiny-qwen3-moe"):
        eng = NativeEngine(preset(name), C(), C(lr=1e-3, clip_grad=1.0), device="cpu", seed=3).initialize()
        ids, mask, pos, R = _batch(seed=4)
        data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, -R:],
                                    "response_mask": mask[:, -R:]}, meta_info={"temperature": 0.8, "micro_batch_size": 8})
        res = {}
        for flag in (False, True):
            actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=12, ppo_micro_batch_size_per_gpu=8,
                                                         use_prefix_grouper=flag), eng)
            res[flag] = actor.compute_log_prob(data, calculate_entropy=True)
            if flag:  # micro-batches of 8 and 4 samples: two whole groups, then one
                assert 0.2 < actor.last_prefix_saving < 0.8
        m = mask[:, -R:].bool()
        torch.testing.assert_close(res[True][0][m], res[False][0][m], atol=2e-5, rtol=1e-4)
        torch.testing.assert_close(res[True][1][m], res[False][1][m], atol=2e-5, rtol=1e-4)
        assert float(res[True][0][~m].abs().sum()) == 0.0


import pytest  # noqa: E402


@pytest.mark.gpu
def test_shared_prefix_on_the_kernels():
    """Same comparison on a GPU: the response part runs the key-stream form of the tcgen05 forward kernel."""
    from verl_b200 import DataProto
    from verl_b200.models import preset
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    cfg = preset("qwen2.5-0.5b", num_hidden_layers=3, vocab_size=32768, num_attention_heads=4, num_key_value_heads=2,
                 head_dim=128, hidden_size=512, intermediate_size=1024)
    eng = NativeEngine(cfg, C(), C(lr=1e-5), device="cuda:0", seed=3).initialize()
    ids, mask, pos, R = _batch(n_prompts=4, n=8, P=200, R=150, vocab=30000, seed=7)
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, -R:],
                                "response_mask": mask[:, -R:]}, meta_info={"temperature": 1.0, "micro_batch_size": 16})
    res = {}
    for flag in (False, True):
        actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=32, ppo_micro_batch_size_per_gpu=16,
                                                     use_prefix_grouper=flag), eng)
        res[flag] = actor.compute_log_prob(data, calculate_entropy=True)
    m = mask[:, -R:].bool()
    d = (res[True][0].cpu()[m] - res[False][0].cpu()[m]).abs()
    assert float(d.max()) < 0.08 and float(d.mean()) < 0.01, (float(d.max()), float(d.mean()))


def test_token_budget_micro_batches_keep_groups_together():
    from verl_b200 import DataProto
    from verl_b200.models import preset
    from verl_b200.workers.actor.dp_actor import DataParallelPPOActor
    from verl_b200.workers.config import FSDPActorConfig
    from verl_b200.workers.engine.native import NativeEngine

    class C(dict):
        __getattr__ = dict.get

    eng = NativeEngine(preset("tiny-qwen2"), C(), C(lr=1e-3), device="cpu", seed=3).initialize()
    ids, mask, pos, R = _batch(n_prompts=5, n=4, seed=9)
    perm = torch.randperm(20, generator=torch.Generator().manual_seed(1))  # the samples of a prompt arrive scattered
    ids, mask, pos = ids[perm], mask[perm], pos[perm]
    data = DataProto.from_dict({"input_ids": ids, "attention_mask": mask, "position_ids": pos, "responses": ids[:, -R:],
                                "response_mask": mask[:, -R:]},
                               meta_info={"temperature": 1.0, "use_dynamic_bsz": True, "max_token_len": 90})
    res = {}
    for flag in (False, True):
        actor = DataParallelPPOActor(FSDPActorConfig(ppo_mini_batch_size=20, use_dynamic_bsz=True, use_prefix_grouper=flag), eng)
        res[flag] = actor.compute_log_prob(data, calculate_entropy=False)[0]
        if flag:
            with torch.no_grad():
                micros, bins = actor._micro_batches(data, 90, None, True)
            P = ids.shape[1] - R
            for mb in micros:  # whole groups only: 4 samples per distinct prompt
                keys = [mb.batch["input_ids"][i, :P][mb.batch["attention_mask"][i, :P].bool()].numpy().tobytes() for i in range(len(mb))]
                assert all(keys.count(k) == 4 for k in set(keys))
            assert sorted(i for b in bins for i in b) == list(range(20)) and len(micros) >= 2
            assert actor.last_prefix_saving > 0.2
    m = mask[:, -R:].bool()
    torch.testing.assert_close(res[True][m], res[False][m], atol=2e-5, rtol=1e-4)
