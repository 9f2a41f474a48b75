"""DataProto semantics (role of the reference's tests/test_protocol_on_cpu.py)."""

import pickle

import numpy as np
import pytest
import torch

from verl_b200.protocol import DataProto, DataProtoConfig, pad_dataproto_to_divisor, unpad_dataproto


def _dp(n=6):
    obs = torch.arange(n * 3, dtype=torch.float32).view(n, 3)
    labels = np.array([f"s{i}" for i in range(n)], dtype=object)
    return DataProto.from_dict(tensors={"obs": obs, "act": torch.arange(n)}, non_tensors={"labels": labels},
                               meta_info={"name": "abc"})


def test_len_getitem_and_slices():
    d = _dp()
    assert len(d) == 6
    item = d[2]
    assert torch.equal(item.batch["obs"], torch.tensor([6.0, 7.0, 8.0])) and item.non_tensor_batch["labels"] == "s2"
    s = d[1:4]
    assert len(s) == 3 and s.non_tensor_batch["labels"].tolist() == ["s1", "s2", "s3"]
    idx = d[torch.tensor([5, 0])]
    assert idx.batch["act"].tolist() == [5, 0]
    mask = d[torch.tensor([True, False, True, False, False, False])]
    assert mask.non_tensor_batch["labels"].tolist() == ["s0", "s2"]
    assert d.slice(0, 6, 2).batch["act"].tolist() == [0, 2, 4]


def test_inconsistent_batch_raises():
    with pytest.raises(Exception):
        DataProto.from_dict(tensors={"a": torch.zeros(3), "b": torch.zeros(4)})
    with pytest.raises(Exception):
        DataProto.from_dict(tensors={"a": torch.zeros(3)}, non_tensors={"x": np.array(["a", "b"], dtype=object)})


def test_select_pop_rename_union():
    d = _dp()
    sel = d.select(batch_keys=["obs"], non_tensor_batch_keys=[])
    assert list(sel.batch.keys()) == ["obs"] and not sel.non_tensor_batch
    popped = d.pop(batch_keys=["act"], non_tensor_batch_keys=["labels"])
    assert "act" not in d.batch.keys() and "labels" not in d.non_tensor_batch and "act" in popped.batch.keys()
    d.rename("obs", "state")
    assert "state" in d.batch.keys()
    u = d.union(popped)
    assert set(u.batch.keys()) == {"state", "act"}
    clash = DataProto.from_dict(tensors={"state": torch.zeros(6, 3)})
    with pytest.raises(AssertionError):
        d.union(clash)
    same = DataProto.from_dict(tensors={"state": d.batch["state"].clone()})
    d.union(same)  # equal values are fine


def test_chunk_split_concat_roundtrip_and_metrics_merge():
    d = _dp(6)
    parts = d.chunk(3)
    assert [len(p) for p in parts] == [2, 2, 2]
    for i, p in enumerate(parts):
        p.meta_info = {"name": "abc", "metrics": [{"loss": float(i)}]}  # chunks share the parent's meta_info dict
    back = DataProto.concat(parts)
    assert torch.equal(back.batch["obs"], d.batch["obs"]) and back.non_tensor_batch["labels"].tolist() == d.non_tensor_batch["labels"].tolist()
    assert back.meta_info["metrics"] == {"loss": [0.0, 1.0, 2.0]}
    assert [len(p) for p in d.split(4)] == [4, 2]
    with pytest.raises(AssertionError):
        d.chunk(4)


def test_auto_padding_chunk():
    d = _dp(5)
    DataProtoConfig.auto_padding = True
    try:
        d2 = DataProto.from_dict(tensors={"a": torch.arange(5)}, auto_padding=True)
        parts = d2.chunk(2)
        assert [len(p) for p in parts] == [3, 2]  # uneven chunks are allowed once padding is enabled (the dispatcher pads)
    finally:
        DataProtoConfig.auto_padding = False
    padded, pad = pad_dataproto_to_divisor(d, 4)
    assert len(padded) == 8 and pad == 3 and padded.batch["act"][5:].tolist() == [0, 1, 2]
    assert len(unpad_dataproto(padded, pad)) == 5


def test_repeat_and_reorder():
    d = _dp(3)
    r = d.repeat(2, interleave=True)
    assert r.batch["act"].tolist() == [0, 0, 1, 1, 2, 2] and r.non_tensor_batch["labels"].tolist() == ["s0", "s0", "s1", "s1", "s2", "s2"]
    r2 = d.repeat(2, interleave=False)
    assert r2.batch["act"].tolist() == [0, 1, 2, 0, 1, 2]
    s = d.sample_level_repeat([1, 0, 2])
    assert s.batch["act"].tolist() == [0, 2, 2]
    d.reorder(torch.tensor([2, 0, 1]))
    assert d.batch["act"].tolist() == [2, 0, 1] and d.non_tensor_batch["labels"].tolist() == ["s2", "s0", "s1"]


def test_pickle_and_disk_roundtrip(tmp_path):
    d = _dp()
    d2 = pickle.loads(pickle.dumps(d))
    assert torch.equal(d2.batch["obs"], d.batch["obs"]) and d2.meta_info == d.meta_info
    d.save_to_disk(str(tmp_path / "d.pt"))
    d3 = DataProto.load_from_disk(str(tmp_path / "d.pt"))
    assert d3.non_tensor_batch["labels"].tolist() == d.non_tensor_batch["labels"].tolist()


def test_make_iterator_epochs_and_seed():
    d = _dp(8)
    it = d.make_iterator(mini_batch_size=4, epochs=2, seed=1)
    batches = list(it)
    assert len(batches) == 4 and all(len(b) == 4 for b in batches)
    first_epoch = torch.cat([b.batch["act"] for b in batches[:2]]).sort().values
    assert first_epoch.tolist() == list(range(8))
    again = list(d.make_iterator(mini_batch_size=4, epochs=2, seed=1))
    assert all(torch.equal(a.batch["act"], b.batch["act"]) for a, b in zip(batches, again))


def test_from_single_dict_and_tensordict_roundtrip():
    d = DataProto.from_single_dict({"x": torch.ones(2, 2), "names": np.array(["a", "b"], dtype=object)})
    assert "x" in d.batch.keys() and "names" in d.non_tensor_batch
    td = d.to_tensordict()
    back = DataProto.from_tensordict(td)
    assert torch.equal(back.batch["x"], d.batch["x"]) and back.non_tensor_batch["names"].tolist() == ["a", "b"]


def test_dataproto_future_chunk_and_get():
    import concurrent.futures as cf

    from verl_b200.protocol import DataProtoFuture

    d = _dp(4)
    with cf.ThreadPoolExecutor(2) as ex:
        futs = [ex.submit(lambda p=p: p, p) for p in d.chunk(2)]
        fut = DataProtoFuture(collect_fn=DataProto.concat, futures=futs)
        halves = fut.chunk(2)
        got = [h.get() for h in halves]
    assert [len(g) for g in got] == [2, 2] and torch.equal(torch.cat([g.batch["act"] for g in got]), d.batch["act"])
