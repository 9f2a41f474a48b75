"""Left-padded-prompt / right-padded-response batches <-> packed (no-padding) streams
(verl/workers/utils/padding.py:1-106). The native engine consumes ``PackedBatch``."""

from __future__ import annotations

import torch

from ...models.transformer import PackedBatch


def left_right_2_no_padding(input_ids: torch.Tensor, attention_mask: torch.Tensor, position_ids: torch.Tensor | None = None):
    """[B, S] padded tensors -> (PackedBatch, flat indices of the kept tokens in the [B*S] layout)."""
    return PackedBatch.from_padded(input_ids, attention_mask, position_ids)


def no_padding_2_padding(values: torch.Tensor, flat_indices: torch.Tensor, batch_size: int, seq_len: int,
                         pad_value: float = 0.0) -> torch.Tensor:
    """Scatter per-token values of the packed stream back to [B, S] (pad positions get ``pad_value``)."""
    out = torch.full((batch_size * seq_len,) + tuple(values.shape[1:]), pad_value, dtype=values.dtype, device=values.device)
    out[flat_indices] = values
    return out.view(batch_size, seq_len, *values.shape[1:])


def response_from_padded(x: torch.Tensor, response_length: int) -> torch.Tensor:
    """Values predicted for the response tokens: positions [S - R - 1, S - 1) of a [B, S] tensor."""
    return x[:, -response_length - 1 : -1]
