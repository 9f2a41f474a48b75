"""Transfer-queue data plane and the embodied env loop with the synthetic environment."""

import threading
import time

import numpy as np
import pytest
import torch

from verl_b200.protocol import DataProto


def test_transfer_queue_bridge_moves_only_needed_columns():
    from verl_b200.experimental.transfer_queue import BatchMeta, TransferQueue, set_transfer_queue, tqbridge

    q = TransferQueue()
    set_transfer_queue(q)
    ids = q.allocate(4)
    cols = q.put(ids, DataProto.from_dict(tensors={"input_ids": torch.arange(8).view(4, 2), "big": torch.zeros(4, 1000)},
                                          non_tensors={"uid": np.array(list("abcd"), dtype=object)}))
    meta = BatchMeta(ids, cols, {"step": 3})

    class Worker:
        @tqbridge(reads=["input_ids", "uid"])
        def compute(self, data: DataProto) -> DataProto:
            assert set(data.batch.keys()) == {"input_ids"}
            if "uid" in data.non_tensor_batch:  # came through the queue
                assert data.meta_info["step"] == 3
            return DataProto.from_dict(tensors={"out": data.batch["input_ids"].sum(-1)}, meta_info={"ok": 1})

    before = q.bytes_get
    out = Worker().compute(meta)
    assert isinstance(out, BatchMeta) and out.columns == ["out"] and out.meta_info == {"ok": 1}
    assert q.bytes_get - before == 4 * 2 * 8  # the 'big' column never moved
    merged = meta.union(out)
    got = q.get(merged.global_indexes, ["out", "uid"])
    assert got.batch["out"].tolist() == [1, 5, 9, 13] and got.non_tensor_batch["uid"].tolist() == list("abcd")
    # a plain DataProto call bypasses the queue
    d = Worker().compute(DataProto.from_dict(tensors={"input_ids": torch.ones(2, 2, dtype=torch.long)}))
    assert isinstance(d, DataProto)
    halves = meta.chunk(2)
    assert BatchMeta.concat(halves).global_indexes == ids
    # consumers wait for producers
    ids2 = q.allocate(1)
    t = threading.Thread(target=lambda: (time.sleep(0.05), q.put(ids2, DataProto.from_dict(tensors={"x": torch.ones(1)}))))
    t.start()
    assert q.get(ids2, ["x"], timeout=2.0).batch["x"].item() == 1.0
    t.join()
    with pytest.raises(TimeoutError):
        q.get(q.allocate(1), ["x"], timeout=0.05)
    set_transfer_queue(None)


def test_env_loop_pipeline_and_trajectory_layout():
    from verl_b200.experimental.vla import EnvLoop, SyntheticReachEnv
    from verl_b200.experimental.vla.env_loop import ActionTokenizer

    tok = ActionTokenizer(256)
    x = np.array([[-1.0, 0.0, 0.999]])
    assert np.abs(tok.decode(tok.encode(x)) - x).max() < 1 / 128

    def expert(obs):
        a = SyntheticReachEnv.expert_action(obs["state"])
        return tok.encode(a), np.zeros(a.shape, np.float32)

    loop = EnvLoop([lambda s=s: SyntheticReachEnv(6, seed=s) for s in range(2)], expert, tok, max_steps=12)
    trajs = loop.run()
    loop.close()
    data = loop.to_dataproto(trajs)
    assert len(data) == 12 and data.batch["responses"].shape == (12, 24)
    score = data.batch["token_level_scores"].sum(-1)
    assert score.mean() > 0.9  # the expert reaches the goal
    mask = data.batch["response_mask"]
    last = mask.sum(-1) - 1
    assert (data.batch["token_level_scores"][torch.arange(12), last] == score).all()
    assert (mask.sum(-1) < 24).any()  # finished episodes stop contributing tokens


def test_token_policy_drives_the_env_loop():
    from verl_b200.experimental.vla import EnvLoop, NaiveRolloutRob, SyntheticReachEnv
    from verl_b200.models import preset
    from verl_b200.models.transformer import CausalLM

    cfg = preset("tiny-qwen2")
    m = CausalLM(cfg, dtype=torch.float32, device="cpu")
    m.init_weights(0)
    loop = EnvLoop([lambda: SyntheticReachEnv(4, seed=1)], NaiveRolloutRob(m, action_dim=2), max_steps=3)
    data = loop.to_dataproto(loop.run())
    loop.close()
    assert data.batch["responses"].shape == (4, 6) and torch.isfinite(data.batch["rollout_log_probs"]).all()
    assert (data.batch["rollout_log_probs"][data.batch["response_mask"].bool()] < 0).all()
