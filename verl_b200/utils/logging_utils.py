"""Logging helpers (verl/utils/logging_utils.py:21-32)."""

import logging
import os

import torch


def set_basic_config(level) -> None:
    logging.basicConfig(format="%(levelname)s:%(asctime)s:%(message)s", level=level)


def log_to_file(string) -> None:
    print(string)
    if os.path.isdir("logs"):
        rank = torch.distributed.get_rank() if torch.distributed.is_initialized() else 0
        with open(f"logs/log_{rank}", "a+") as f:
            f.write(str(string) + "\n")
