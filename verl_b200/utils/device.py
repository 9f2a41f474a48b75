"""Device helpers (role of verl/utils/device.py:1-180; the NPU switch of the reference has no counterpart: this
framework targets sm_100a only, with a CPU path for tests)."""

from __future__ import annotations

import os

import torch


def is_cuda_available() -> bool:
    return torch.cuda.is_available()


is_npu_available = False


def get_device_name() -> str:
    return "cuda" if torch.cuda.is_available() else "cpu"


def get_torch_device():
    return torch.cuda if torch.cuda.is_available() else torch.cpu


def get_device_id() -> int:
    return torch.cuda.current_device() if torch.cuda.is_available() else 0


def get_nccl_backend() -> str:
    return "nccl" if torch.cuda.is_available() else "gloo"


def get_visible_devices_keyword() -> str:
    return "CUDA_VISIBLE_DEVICES"


def set_expandable_segments(enable: bool) -> None:
    if torch.cuda.is_available():
        torch.cuda.memory._set_allocator_settings(f"expandable_segments:{enable}")


def get_device_capability(device_id: int = 0):
    return torch.cuda.get_device_capability(device_id) if torch.cuda.is_available() else (None, None)


def is_blackwell(device_id: int = 0) -> bool:
    major, _ = get_device_capability(device_id)
    return major == 10


def auto_set_device(config) -> None:
    """``trainer.device`` falls back to cpu when no GPU is visible."""
    if config.trainer.get("device", "cuda") == "cuda" and not torch.cuda.is_available():
        config.trainer.device = "cpu"


def local_rank() -> int:
    return int(os.environ.get("LOCAL_RANK", "0"))


def is_torch_npu_available() -> bool:
    """This framework targets NVIDIA B200 only."""
    return False


def get_resource_name() -> str:
    """Name of the accelerator resource a scheduler hands out per worker."""
    return "GPU" if is_cuda_available() else "CPU"
