"""Worker classes used by the single-controller tests (importable by spawned processes)."""
import os

import torch

from verl_b200 import DataProto
from verl_b200.single_controller.base import Dispatch, Execute, Worker, register


class EchoWorker(Worker):
    def __init__(self, scale=1.0):
        super().__init__()
        self.scale = scale
        self._register_dispatch_collect_info("pair", dp_rank=self.rank // 2, is_collect=self.rank % 2 == 0)

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def whoami(self):
        return (self.rank, self.world_size, os.environ.get("MASTER_PORT"))

    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO)
    def double(self, data: DataProto):
        out = DataProto.from_dict({"y": data.batch["x"] * 2 * self.scale})
        out.meta_info["metrics"] = {"rank": self.rank}
        return out

    @register(dispatch_mode=Dispatch.DP_COMPUTE_PROTO, blocking=False)
    def double_async(self, data: DataProto):
        return DataProto.from_dict({"y": data.batch["x"] * 2 * self.scale})

    @register(dispatch_mode=Dispatch.ALL_TO_ALL, execute_mode=Execute.RANK_ZERO)
    def only_zero(self, v):
        return (self.rank, v)

    @register(dispatch_mode=Dispatch.DP_COMPUTE)
    def per_rank(self, v):
        return v + self.rank

    @register(dispatch_mode={"dispatch_fn": None, "collect_fn": None} if False else Dispatch.ONE_TO_ALL)
    def boom(self):
        raise ValueError("intended failure")

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def allreduce(self):
        import torch.distributed as dist

        if not dist.is_initialized():
            dist.init_process_group("gloo")
        t = torch.tensor([float(self.rank + 1)])
        dist.all_reduce(t)
        return t.item()

    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def die(self):
        os._exit(3)


from verl_b200.single_controller.base.decorator import make_nd_compute_dataproto_dispatch_fn  # noqa: E402


class MeshWorker(EchoWorker):
    @register(dispatch_mode=make_nd_compute_dataproto_dispatch_fn("pair"))
    def mesh_double(self, data: DataProto):
        return DataProto.from_dict({"y": data.batch["x"] * 2, "r": torch.full((len(data),), self.rank)})


class OtherWorker(Worker):
    @register(dispatch_mode=Dispatch.ONE_TO_ALL)
    def hello(self):
        return f"other{self.rank}"
