"""Engine abstraction shared by all training backends (verl/workers/engine/base.py:1-336)."""

from __future__ import annotations

from typing import Any, Callable, Generator, Optional

import torch


class BaseEngine:
    """A training/inference engine for one model replica spread over a process group."""

    def initialize(self):
        raise NotImplementedError

    def train_mode(self, **kwargs):
        raise NotImplementedError

    def eval_mode(self, **kwargs):
        raise NotImplementedError

    def optimizer_zero_grad(self):
        raise NotImplementedError

    def optimizer_step(self):
        raise NotImplementedError

    def lr_scheduler_step(self):
        raise NotImplementedError

    def forward_backward_batch(self, data, loss_function: Callable, forward_only: bool = False) -> Any:
        raise NotImplementedError

    def train_batch(self, data, loss_function: Callable) -> Any:
        self.optimizer_zero_grad()
        out = self.forward_backward_batch(data, loss_function, forward_only=False)
        grad_norm = self.optimizer_step()
        if self.is_mp_src_rank_with_outputs():
            out.setdefault("metrics", {})["grad_norm"] = grad_norm
        return out

    def infer_batch(self, data, loss_function: Optional[Callable] = None) -> Any:
        with torch.no_grad():
            return self.forward_backward_batch(data, loss_function, forward_only=True)

    def get_per_tensor_param(self) -> Generator:
        raise NotImplementedError

    def get_data_parallel_size(self) -> int:
        raise NotImplementedError

    def get_data_parallel_rank(self) -> int:
        raise NotImplementedError

    def get_data_parallel_group(self):
        raise NotImplementedError

    def to(self, device: str, model: bool = True, optimizer: bool = True, grad: bool = True):
        raise NotImplementedError

    def save_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, global_step: int = 0,
                        max_ckpt_to_keep: Optional[int] = None, **kwargs) -> None:
        raise NotImplementedError

    def load_checkpoint(self, local_path: str, hdfs_path: Optional[str] = None, del_local_after_load: bool = True,
                        **kwargs) -> None:
        raise NotImplementedError

    def is_mp_src_rank_with_outputs(self) -> bool:
        return True


class BaseEngineCtx:
    """Loads offloaded state to the device on enter and offloads again on exit."""

    def __init__(self, engine: BaseEngine, mode: str, **kwargs):
        self.engine, self.mode, self.kwargs = engine, mode, kwargs

    def __enter__(self):
        self.engine._enter_mode(self.mode, **self.kwargs)
        return self.engine

    def __exit__(self, *exc):
        self.engine._exit_mode(self.mode)
        return False


class EngineRegistry:
    """``(model_type, backend, device) -> engine class`` (verl/workers/engine/base.py EngineRegistry)."""

    _engines: dict = {}

    @classmethod
    def register(cls, model_type: str, backend: list[str] | str, device: list[str] | str = "cuda"):
        backends = backend if isinstance(backend, list) else [backend]
        devices = device if isinstance(device, list) else [device]

        def deco(engine_cls):
            for b in backends:
                for d in devices:
                    cls._engines.setdefault(model_type, {}).setdefault(b, {})[d] = engine_cls
            return engine_cls

        return deco

    @classmethod
    def get_engine_cls(cls, model_type: str, backend: str, device: Optional[str] = None):
        assert model_type in cls._engines, f"Unknown model_type: {model_type}"
        by_backend = cls._engines[model_type]
        assert backend in by_backend, f"Unknown backend: {backend}"
        if device is None:
            device = "cuda" if torch.cuda.is_available() else "cpu"
        by_dev = by_backend[backend]
        assert device in by_dev, f"Unknown device: {device}"
        return by_dev[device]

    @classmethod
    def new(cls, model_type: str, backend: str, *args, **kwargs):
        return cls.get_engine_cls(model_type, backend, kwargs.pop("device_name", None))(*args, **kwargs)
