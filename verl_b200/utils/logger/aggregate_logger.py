"""Console logger and rank-aware print helpers (verl/utils/logger/aggregate_logger.py:26-140)."""

from __future__ import annotations

import datetime
import logging
import numbers

import torch


def concat_dict_to_str(d: dict, step) -> str:
    parts = [f"step:{step}"] + [f"{k}:{v:.3f}" for k, v in d.items() if isinstance(v, numbers.Number)]
    return " - ".join(parts)


class LocalLogger:
    def __init__(self, print_to_console: bool = True):
        self.print_to_console = print_to_console

    def flush(self):
        pass

    def log(self, data, step):
        if self.print_to_console:
            print(concat_dict_to_str(data, step=step), flush=True)


def _rank() -> int:
    return torch.distributed.get_rank() if torch.distributed.is_initialized() else 0


class DecoratorLoggerBase:
    """Base of decorators that log around a call: prints or logs ``[role] message`` on rank 0 (or every rank)."""

    def __init__(self, role: str, logger: logging.Logger | None = None, level=logging.DEBUG, rank: int | None = None,
                 log_only_rank_0: bool = True):
        self.role, self.logger, self.level = role, logger, level
        self.rank = _rank() if rank is None else rank
        self.log_only_rank_0 = log_only_rank_0
        self.logging_function = self.log_by_print if logger is None else self.log_by_logging

    def log_by_print(self, log_str):
        if not self.log_only_rank_0 or self.rank == 0:
            print(f"{self.role} {log_str}", flush=True)

    def log_by_logging(self, log_str):
        if not self.log_only_rank_0 or self.rank == 0:
            self.logger.log(self.level, f"{self.role} {log_str}")


def print_rank_0(message):
    if _rank() == 0:
        print(message, flush=True)


def print_with_rank(message: str, rank: int = 0, log_only_rank_0: bool = False):
    if not log_only_rank_0 or rank == 0:
        print(f"[Rank {rank}] {message}", flush=True)


def print_with_rank_and_timer(message: str, rank: int = 0, log_only_rank_0: bool = False):
    if not log_only_rank_0 or rank == 0:
        print(f"[{datetime.datetime.now():%Y-%m-%d %H:%M:%S}] [Rank {rank}] {message}", flush=True)


def log_with_rank(message: str, rank, logger: logging.Logger, level=logging.INFO, log_only_rank_0: bool = False):
    if not log_only_rank_0 or rank == 0:
        logger.log(level, f"[Rank {rank}] {message}")
