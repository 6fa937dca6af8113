from pace_b200.ops.enum import OperatorType, BackendType, DataType  # noqa: F401
from pace_b200.ops.registry import backend_registry  # noqa: F401
from pace_b200.ops.base import OperatorBase, BackendBase  # noqa: F401
from pace_b200.ops.backends import b200  # noqa: F401  (registers the CUDA backend)
from pace_b200.ops.attention import MultiHeadAttention  # noqa: F401
from pace_b200.ops.rotary_embedding import RotaryEmbedding  # noqa: F401
from pace_b200.ops import custom_op  # noqa: F401  (torch.ops.pace.attention on CUDA)
