"""Metric reduction helpers (verl/utils/metric/utils.py:25-149)."""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum
from typing import Any, Union

import numpy as np
import torch


def reduce_metrics(metrics: dict[str, Union["Metric", list[Any]]]) -> dict[str, Any]:
    out = {}
    for key, val in metrics.items():
        if isinstance(val, Metric):
            out[key] = val.aggregate()
        elif "max" in key:
            out[key] = float(np.max(val))
        elif "min" in key:
            out[key] = float(np.min(val))
        else:
            out[key] = float(np.mean(val))
    return out


class AggregationType(Enum):
    MEAN = "mean"
    SUM = "sum"
    MIN = "min"
    MAX = "max"


Numeric = Union[int, float, torch.Tensor, np.ndarray]


class Metric:
    """A typed metric that knows how to aggregate its values (also across DP ranks' lists)."""

    def __init__(self, aggregation: str | AggregationType, value: Numeric | list | None = None) -> None:
        self.aggregation = AggregationType(aggregation) if isinstance(aggregation, str) else aggregation
        self.values: list = []
        if value is not None:
            self.extend(value) if isinstance(value, list) else self.append(value)

    def append(self, value: "Metric | Numeric") -> None:
        if isinstance(value, Metric):
            self.extend(value)
            return
        if isinstance(value, torch.Tensor):
            value = value.detach().item()
        if isinstance(value, np.ndarray):
            value = value.item()
        self.values.append(value)

    def extend(self, values: "Metric | list") -> None:
        if isinstance(values, Metric):
            if values.aggregation != self.aggregation:
                raise ValueError(f"Aggregation type mismatch: {self.aggregation} != {values.aggregation}")
            values = values.values
        for v in values:
            self.append(v)

    def aggregate(self) -> float:
        fn = {AggregationType.MEAN: np.mean, AggregationType.SUM: np.sum, AggregationType.MIN: np.min,
              AggregationType.MAX: np.max}[self.aggregation]
        return float(fn(self.values))

    @classmethod
    def chain(cls, metric_lists: list["Metric"]) -> "Metric":
        """One metric holding the values of all (same aggregation); an empty list gives an empty mean metric."""
        out = cls(metric_lists[0].aggregation if metric_lists else AggregationType.MEAN)
        for m in metric_lists:
            out.extend(m)
        return out

    @classmethod
    def aggregate_dp(cls, metric_lists: list["Metric"]) -> float:
        vals = [v for m in metric_lists for v in m.values]
        return cls(metric_lists[0].aggregation, vals).aggregate()

    @classmethod
    def from_dict(cls, data: dict[str, Numeric], aggregation) -> dict[str, "Metric"]:
        return {k: cls(aggregation, v) for k, v in data.items()}

    def init_list(self) -> "Metric":
        return Metric(self.aggregation)
