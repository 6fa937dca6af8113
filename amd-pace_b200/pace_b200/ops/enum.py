"""Operator / backend / dtype names of the operator plug-in API (reference: pace/ops/enum.py:21-80)."""
from enum import StrEnum, auto
from typing import List

import torch


class OperatorType(StrEnum):
    MHA = auto()


class BackendType(StrEnum):
    # the reference's names are kept so an operator config written for it still parses;
    # for MHA every one of them resolves to the single sm_100a implementation
    NATIVE = auto()
    JIT = auto()
    TPP = auto()
    IMBPS = auto()
    B200 = auto()


class DataType(StrEnum):
    FLOAT32 = auto()
    BFLOAT16 = auto()

    @classmethod
    def from_torch(cls, dtype):
        if dtype == torch.float32:
            return DataType.FLOAT32
        if dtype == torch.bfloat16:
            return DataType.BFLOAT16
        raise ValueError(f"Unsupported dtype: {dtype}")

    def to_torch_dtype(self):
        return torch.float32 if self == DataType.FLOAT32 else torch.bfloat16


FALLBACK_BACKEND: List[BackendType] = [BackendType.B200]
