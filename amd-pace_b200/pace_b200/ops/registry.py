"""Backend registry keyed by (operator, backend, dtype) (reference: pace/ops/registry.py:20-106).

Same surface - ``register`` as a class decorator, ``get``, ``get_available_backends`` -
but no multi-backend dispatch is rebuilt: an unknown (backend, dtype) pair resolves
to the one sm_100a implementation registered for the operator.
"""
from collections import defaultdict
from typing import Dict, List, Tuple, Type

from pace_b200.ops.enum import BackendType, DataType, OperatorType, FALLBACK_BACKEND


class BackendRegistry:
    def __init__(self):
        self._registry: Dict[OperatorType, Dict[Tuple[BackendType, DataType], Type]] = defaultdict(dict)

    def register(self, operator: OperatorType, backend: BackendType, dtype: List[DataType]):
        for dt in dtype:
            if (backend, dt) in self._registry.get(operator, {}):
                raise AssertionError(f"Duplicate registration of {operator} with backend {backend} and dtype {dt}")

        def decorator(cls):
            for dt in dtype:
                self._registry[operator][(backend, dt)] = cls
            return cls

        return decorator

    def get_available_backends(self, operator: OperatorType) -> List[Tuple[BackendType, DataType]]:
        return list(self._registry.get(operator, {}).keys())

    def get(self, operator: OperatorType, backend: BackendType, dtype: DataType):
        if operator not in self._registry:
            return None
        table = self._registry[operator]
        if (backend, dtype) in table:
            return table[(backend, dtype)]
        for fb in FALLBACK_BACKEND:
            if (fb, dtype) in table:
                return table[(fb, dtype)]
        raise AssertionError(f"No backend found for {operator} with {backend}, {dtype}")

    def __repr__(self):
        return str(dict(self._registry))


backend_registry = BackendRegistry()
