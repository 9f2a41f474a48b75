"""Precision names <-> torch dtypes (the helper class of verl/utils/torch_dtypes.py, table-driven here)."""

import torch

# every spelling a config may use -> (dtype, canonical short name)
_TABLE = {}
for _dtype, _short, _names in ((torch.float16, "fp16", (16, "16", "fp16", "float16", "half")),
                               (torch.float32, "fp32", (32, "32", "fp32", "float32", "float")),
                               (torch.bfloat16, "bf16", ("bf16", "bfloat16")),
                               (torch.float64, "fp64", (64, "64", "fp64", "float64", "double"))):
    for _n in (*_names, _dtype):
        _TABLE[_n] = (_dtype, _short)


def _lookup(precision):
    try:
        return _TABLE[precision]
    except (KeyError, TypeError):
        raise RuntimeError(f"unexpected precision: {precision}") from None


class PrecisionType:
    HALF, FLOAT, FULL, BFLOAT, MIXED = "16", "32", "64", "bf16", "mixed"

    @staticmethod
    def supported_types() -> list[str]:
        return [PrecisionType.HALF, PrecisionType.FLOAT, PrecisionType.FULL, PrecisionType.BFLOAT, PrecisionType.MIXED]

    @staticmethod
    def supported_type(precision) -> bool:
        return precision in PrecisionType.supported_types()

    @staticmethod
    def is_fp16(precision) -> bool:
        return _TABLE.get(precision, (None,))[0] is torch.float16

    @staticmethod
    def is_fp32(precision) -> bool:
        return _TABLE.get(precision, (None,))[0] is torch.float32

    @staticmethod
    def is_bf16(precision) -> bool:
        return _TABLE.get(precision, (None,))[0] is torch.bfloat16

    @staticmethod
    def to_dtype(precision) -> torch.dtype:
        return _lookup(precision)[0]

    @staticmethod
    def to_str(precision) -> str:
        return _lookup(precision)[1]
