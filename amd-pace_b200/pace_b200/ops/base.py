"""Operator / backend base classes (reference: pace/ops/base.py:17-113)."""
from abc import ABC, abstractmethod
from typing import Optional, Type

from torch import get_default_dtype, nn

from pace_b200.ops.enum import BackendType, DataType, OperatorType
from pace_b200.ops.registry import backend_registry


class BackendBase(ABC):
    def create_extra_params(self, layer: nn.Module):
        pass

    def preprocess(self, layer: nn.Module):
        pass

    @abstractmethod
    def execute(self, *args, **kwargs):
        ...

    def __repr__(self):
        return f"{self.__class__.__name__}"


class OperatorBase(nn.Module, ABC):
    """Picks its backend class from the registry at construction (base.py:25-47)."""

    def __init__(self, backend_impl: Optional[BackendType] = None, dtype: Optional[DataType] = None):
        super().__init__()
        dtype = dtype if dtype is not None else get_default_dtype()
        dtype = dtype if isinstance(dtype, DataType) else DataType.from_torch(dtype)
        self.dtype = dtype
        self.backend_impl = backend_impl
        self.backend_cls: Type[BackendBase] = backend_registry.get(self.operator_type, backend_impl, dtype)
        if self.backend_cls is not None:
            self.backend: BackendBase = self.backend_cls()
            self.backend.create_extra_params(self)
        else:
            self.backend = None

    @property
    @abstractmethod
    def operator_type(cls) -> OperatorType:
        ...

    def load_weights(self, *args, **kwargs):
        pass

    @abstractmethod
    def forward(self, *args, **kwargs):
        ...

    @abstractmethod
    def extra_repr(self) -> str:
        ...
