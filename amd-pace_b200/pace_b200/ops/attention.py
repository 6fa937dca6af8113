"""MultiHeadAttention operator front end (reference: pace/ops/attention.py:15-41)."""
from typing import Optional

import torch

from pace_b200.ops.base import OperatorBase
from pace_b200.ops.enum import BackendType, DataType, OperatorType


class MultiHeadAttention(OperatorBase):
    """``forward(query, key, value, attention_mask=None)`` -> ``[B, Hq, S, D]``.

    ``key`` / ``value`` are what the KV cache's ``update_cache`` returned (paged
    handles) or dense ``[B, Hkv, L, D]`` CUDA tensors.  Extra keyword arguments
    (``kv_start``, ``q_lens``) are forwarded to the backend; callers written for
    the reference never pass them.
    """

    @property
    def operator_type(self):
        return OperatorType.MHA

    def __init__(self, dtype: Optional[DataType] = None, backend_impl: BackendType = BackendType.NATIVE):
        if dtype is None:
            dtype = DataType.BFLOAT16   # the caches are bf16
        super().__init__(backend_impl=backend_impl, dtype=dtype)

    def forward(self, query: torch.Tensor, key, value, attention_mask: Optional[torch.Tensor] = None,
                **kwargs) -> torch.Tensor:
        return self.backend.execute(query=query, key=key, value=value, attention_mask=attention_mask, **kwargs)

    def extra_repr(self):
        return f"dtype={self.dtype}, backend={self.backend}"
