"""Helpers shared by engines and workers (verl/workers/engine/utils.py:30-154): reproducibility switches, micro-batch
preparation for the TensorDict batch interface, and re-assembly of per-micro-batch outputs."""

from __future__ import annotations

import os
import random
from typing import Optional

import numpy as np
import torch

from ...utils import tensordict_utils as tu
from ...utils.py_functional import append_to_dict
from ...utils.seqlen_balancing import rearrange_micro_batches, restore_dynamic_batch


def enable_full_determinism(seed: int) -> None:
    """Seeds every generator and asks the libraries for deterministic algorithms. The kernels of this package are
    deterministic by construction (fixed summation orders, no atomics in GEMM / attention backward); the switches
    below cover what torch and the libraries add around them."""
    os.environ["PYTHONHASHSEED"] = str(seed)
    os.environ.setdefault("CUBLAS_WORKSPACE_CONFIG", ":16:8")
    os.environ["NCCL_DETERMINISTIC"] = "1"
    os.environ["FLASH_ATTENTION_DETERMINISTIC"] = "1"
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
    torch.use_deterministic_algorithms(True, warn_only=True)
    torch.backends.cudnn.deterministic = True
    torch.backends.cudnn.benchmark = False


def prepare_micro_batches(data, dp_group=None, num_batches_divided_by: Optional[int] = None, same_micro_num_in_dp: bool = True,
                          min_num_micro_batch: Optional[int] = None, use_dynamic_bsz_balance: bool = True):
    """TensorDict -> (micro-batches, row indices of each micro-batch or None). ``use_dynamic_bsz`` (default on) packs by
    the token budget ``max_token_len_per_gpu`` (times ``sp_size``: the ranks of a sequence-parallel group share their
    samples); otherwise equal chunks of ``micro_batch_size_per_gpu`` rows."""
    if tu.get_non_tensor_data(data, "use_dynamic_bsz", True):
        budget = tu.get_non_tensor_data(data, "max_token_len_per_gpu", None)
        assert budget is not None, "max_token_len_per_gpu must be set when use_dynamic_bsz is True"
        sp = int(tu.get_non_tensor_data(data, "sp_size", 1) or 1)
        return rearrange_micro_batches(data, int(budget) * sp, dp_group, num_batches_divided_by, same_micro_num_in_dp,
                                       min_num_micro_batch, use_dynamic_bsz_balance)
    mbs = int(tu.get_non_tensor_data(data, "micro_batch_size_per_gpu", len(data)))
    return tu.chunk_tensordict(data, max(len(data) // max(mbs, 1), 1)), None


def postprocess_batch_func(output_lst: list, indices, data) -> dict:
    """Per-micro-batch ``{"model_output", "loss", "metrics"}`` dicts -> one dict: jagged model outputs concatenated in
    the ORIGINAL row order (the permutation of the dynamic batching undone), the list of losses, metrics appended."""
    dyn = bool(tu.get_non_tensor_data(data, "use_dynamic_bsz", True))
    merged: dict = {}
    for o in output_lst:
        for k, v in (o.get("model_output") or {}).items():
            merged.setdefault(k, []).append(v)
    out_model = {}
    for k, parts in merged.items():
        rows = [t for nt in parts for t in (nt.unbind() if nt.is_nested else nt)]
        cat = torch.nested.as_nested_tensor(rows, layout=torch.jagged)
        out_model[k] = restore_dynamic_batch(cat, indices) if dyn and indices is not None else cat
    metrics: dict = {}
    for o in output_lst:
        if o.get("metrics"):
            append_to_dict(metrics, o["metrics"])
    return {"model_output": out_model, "loss": [o["loss"] for o in output_lst if "loss" in o], "metrics": metrics}
