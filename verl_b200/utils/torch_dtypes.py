"""Precision names <-> torch dtypes (verl/utils/torch_dtypes.py:25-82)."""

import torch

HALF_LIST = [16, "16", "fp16", "float16", torch.float16]
FLOAT_LIST = [32, "32", "fp32", "float32", torch.float32]
BFLOAT_LIST = ["bf16", "bfloat16", torch.bfloat16]


class PrecisionType:
    HALF, FLOAT, FULL, BFLOAT, MIXED = "16", "32", "64", "bf16", "mixed"

    @staticmethod
    def supported_type(precision) -> bool:
        return any(x == precision for x in PrecisionType.supported_types())

    @staticmethod
    def supported_types() -> list[str]:
        return [PrecisionType.HALF, PrecisionType.FLOAT, PrecisionType.FULL, PrecisionType.BFLOAT, PrecisionType.MIXED]

    @staticmethod
    def is_fp16(precision) -> bool:
        return precision in HALF_LIST

    @staticmethod
    def is_fp32(precision) -> bool:
        return precision in FLOAT_LIST

    @staticmethod
    def is_bf16(precision) -> bool:
        return precision in BFLOAT_LIST

    @staticmethod
    def to_dtype(precision) -> torch.dtype:
        if precision in HALF_LIST:
            return torch.float16
        if precision in FLOAT_LIST:
            return torch.float32
        if precision in BFLOAT_LIST:
            return torch.bfloat16
        raise RuntimeError(f"unexpected precision: {precision}")

    @staticmethod
    def to_str(precision) -> str:
        if precision == torch.float16:
            return "fp16"
        if precision == torch.float32:
            return "fp32"
        if precision == torch.bfloat16:
            return "bf16"
        raise RuntimeError(f"unexpected precision: {precision}")
