"""Single-controller runtime on CPU processes: dispatch modes, futures, colocated workers, failures."""
import pytest
import torch

from verl_b200 import DataProto
from verl_b200.single_controller.base import ClassWithInitArgs
from verl_b200.single_controller.ray import (RayClassWithInitArgs, RayResourcePool, RayWorkerGroup,
                                             create_colocated_worker_cls, split_resource_pool)
from verl_b200.single_controller.mp import RemoteError

from _sc_workers import EchoWorker, MeshWorker, OtherWorker


@pytest.fixture(scope="module")
def wg():
    pool = RayResourcePool([4], use_gpu=False)
    g = RayWorkerGroup(pool, RayClassWithInitArgs(MeshWorker, scale=1.0), device_name="cpu")
    yield g
    g.shutdown()


def test_one_to_all_and_env(wg):
    out = wg.whoami()
    assert [o[0] for o in out] == [0, 1, 2, 3] and all(o[1] == 4 for o in out)
    assert len({o[2] for o in out}) == 1


def test_dp_compute_proto_and_metrics(wg):
    data = DataProto.from_dict({"x": torch.arange(8.0)})
    out = wg.double(data)
    assert torch.equal(out.batch["y"], torch.arange(8.0) * 2)
    assert out.meta_info["metrics"]["rank"] == [0, 1, 2, 3]


def test_auto_padding_chunk(wg):
    data = DataProto.from_dict({"x": torch.arange(6.0)}, auto_padding=True)
    out = wg.double(data)
    assert torch.equal(out.batch["y"], torch.arange(6.0) * 2)


def test_non_blocking_future(wg):
    fut = wg.double_async(DataProto.from_dict({"x": torch.arange(4.0)}))
    assert torch.equal(fut.get().batch["y"], torch.arange(4.0) * 2)


def test_rank_zero_and_dp_compute(wg):
    assert wg.only_zero(5) == (0, 5)
    assert wg.per_rank([10, 20, 30, 40]) == [10, 21, 32, 43]


def test_mesh_dispatch_collect(wg):
    # 4 workers, dp groups {0,1} and {2,3}; only even ranks are collected
    out = wg.mesh_double(DataProto.from_dict({"x": torch.arange(4.0)}))
    assert torch.equal(out.batch["y"], torch.arange(4.0) * 2)
    assert out.batch["r"].tolist() == [0, 0, 2, 2]


def test_remote_exception_has_traceback(wg):
    with pytest.raises(RemoteError, match="intended failure"):
        wg.boom()
    assert wg.whoami()[0][0] == 0  # workers survive an exception


def test_torch_distributed_rendezvous(wg):
    assert wg.allreduce() == [10.0] * 4


def test_colocated_workers_and_spawn():
    pool = RayResourcePool([2], use_gpu=False)
    fused = create_colocated_worker_cls({"a": ClassWithInitArgs(EchoWorker, scale=2.0), "b": ClassWithInitArgs(OtherWorker)})
    g = RayWorkerGroup(pool, fused, device_name="cpu")
    try:
        views = g.spawn({"a", "b"})
        out = views["a"].double(DataProto.from_dict({"x": torch.ones(2)}))
        assert torch.equal(out.batch["y"], torch.full((2,), 4.0))
        assert views["b"].hello() == ["other0", "other1"]
    finally:
        g.shutdown()


def test_split_pool_and_worker_death_detection():
    pools = split_resource_pool(RayResourcePool([4], use_gpu=False), 2)
    assert [p.world_size for p in pools] == [2, 2]
    g = RayWorkerGroup(pools[0], RayClassWithInitArgs(EchoWorker), device_name="cpu")
    try:
        assert all(g._is_worker_alive(w) for w in g.workers)
        with pytest.raises(RemoteError):
            g.die()
        g.workers[0].proc.join(5)
        assert not g._is_worker_alive(g.workers[0])
    finally:
        g.shutdown()
