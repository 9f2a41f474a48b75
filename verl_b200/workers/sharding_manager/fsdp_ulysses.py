"""Data re-sharding for Ulysses sequence parallelism (verl/workers/sharding_manager/fsdp_ulysses.py:26-76).

Batches are dispatched over all data-parallel ranks, but the ranks of one sequence-parallel group must work on the
same samples: ``preprocess_data`` all-gathers the group's shares, ``postprocess_data`` hands every rank its share of
the result back. Inside the ``with`` block the group is the process-wide Ulysses group. (The engine workers here get
the same effect from their dispatch registration; this class serves code written against the manager interface.)

``sp_group``: the sequence-parallel process group, or a ``DeviceMesh`` with an ``"sp"`` dimension, or None.
"""

from __future__ import annotations

import torch.distributed as dist

from ...protocol import DataProto, all_gather_data_proto
from ...utils.ulysses import get_ulysses_sequence_parallel_group, set_ulysses_sequence_parallel_group
from .base import BaseShardingManager


class FSDPUlyssesShardingManager(BaseShardingManager):
    def __init__(self, device_mesh=None):
        super().__init__()
        self.device_mesh = device_mesh
        self.seed_offset = 12345
        self.prev_sp_group = None

    def _group(self):
        m = self.device_mesh
        if m is None:
            return None
        if hasattr(m, "mesh_dim_names") or hasattr(m, "get_group"):
            try:
                return m["sp"].get_group()
            except Exception:
                return m.get_group()
        return m  # already a process group

    def __enter__(self):
        g = self._group()
        if g is not None:
            self.prev_sp_group = get_ulysses_sequence_parallel_group()
            set_ulysses_sequence_parallel_group(g)
        return self

    def __exit__(self, exc_type, exc_value, traceback):
        if self._group() is not None:
            set_ulysses_sequence_parallel_group(self.prev_sp_group)
        return False

    def preprocess_data(self, data: DataProto) -> DataProto:
        g = self._group()
        if g is not None:
            all_gather_data_proto(data=data, process_group=g)
        return data

    def postprocess_data(self, data: DataProto) -> DataProto:
        g = self._group()
        if g is not None:
            data = data.chunk(chunks=dist.get_world_size(g))[dist.get_rank(g)]
        return data
