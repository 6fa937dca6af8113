"""``torch.ops.pace.attention`` for CUDA tensors.

The reference registers ``pace::attention(Tensor input_Q, Tensor input_K, Tensor input_V,
Tensor? input_mask, Scalar? use_KQ) -> Tensor`` from its C++ extension
(csrc/ops/attention.cpp:104-108) with a CPU implementation.  Importing this module defines the same
schema (when no extension has defined it already) and gives it a CUDA implementation on the
hand-written kernels.  ``use_KQ`` only selected among equivalent CPU evaluation orders
(attention_kernels.cpp:192-214); it is validated and otherwise has no effect here.
"""
import torch

from pace_b200.ops.backends.b200 import dense_attention

_SCHEMA = "attention(Tensor input_Q, Tensor input_K, Tensor input_V, Tensor? input_mask, Scalar? use_KQ) -> Tensor"

_lib = torch.library.Library("pace", "FRAGMENT")
try:
    _lib.define(_SCHEMA)
except RuntimeError:
    pass  # the reference's own extension is loaded and has defined the op


def _attention_cuda(input_Q, input_K, input_V, input_mask=None, use_KQ=None):
    if input_mask is None:
        # the reference dereferences the mask unconditionally (attention.cpp:26-28)
        raise RuntimeError("pace::SDPA attention requires 4D inputs, but recieved no attention mask")
    kq = 0 if use_KQ is None else int(use_KQ)
    if kq not in (0, 1):
        raise RuntimeError(f"pace::SDPA attention requires use_KQ to be 0 or 1 but recieved:  use_KQ - {kq}")
    return dense_attention(input_Q, input_K, input_V, input_mask)


_lib.impl("attention", _attention_cuda, "CUDA")
