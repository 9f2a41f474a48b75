"""SFT collation modes (verl/utils/dataset/dataset_utils.py:22-80)."""

from __future__ import annotations

from enum import Enum

import torch


class DatasetPadMode(str, Enum):
    RIGHT = "right"
    LEFT_RIGHT = "left_right"
    NO_PADDING = "no_padding"


class SFTTensorCollator:
    """``NO_PADDING``: per-sample 1-D tensors of different lengths become one jagged nested tensor per key; the other
    modes stack equally long tensors."""

    def __init__(self, pad_mode: DatasetPadMode = DatasetPadMode.LEFT_RIGHT):
        self.pad_mode = DatasetPadMode(pad_mode)

    def __call__(self, batch: list[dict]) -> dict:
        if self.pad_mode == DatasetPadMode.NO_PADDING:
            return self.collate_variable_batch(batch)
        return {k: torch.stack([b[k] for b in batch]) if isinstance(batch[0][k], torch.Tensor) else [b[k] for b in batch]
                for k in batch[0]}

    def collate_variable_batch(self, batch: list[dict]) -> dict:
        out = {}
        for k in batch[0]:
            vals = [b[k] for b in batch]
            if isinstance(vals[0], torch.Tensor):
                out[k] = torch.nested.as_nested_tensor(vals, layout=torch.jagged)
            else:
                out[k] = vals
        return out
