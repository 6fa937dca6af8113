"""Linear layers of a decode step.

The reference's ``Linear`` operator picks a GEMM back end per layer (pace/ops/linear.py, back ends
pace/ops/backends/tpp.py:19-63, imbps.py:19-92).  On the GPU the projections, the MLP and the LM head of
a decode step see at most a few dozen tokens: they are bound by reading the weights once, which is what
``pace_linear_skinny`` is built for (csrc/linear_skinny.cu).  Measured on the four layer shapes of a
Llama-3.1-8B-shaped step (``bench.py --workload linear``, chains of launches in one CUDA graph) the kernel
streams at the copy rate but pays 4-6 us after its last chunk to settle the row tiles that several CTAs
share; it is ahead of the library GEMM only at K = 14336 and, between the model's other kernels (which
do not overlap with it the way its own launches do), not even there.  ``linear()`` - what the model calls -
is therefore the library GEMM; ``linear_skinny()`` runs the kernel, for the side measurement, the tests and
callers that chain several such layers.
"""
from typing import Dict, Optional, Tuple

import torch
import torch.nn.functional as F

from pace_b200 import _C

MAX_TOKENS = 32
_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def _workspace(device: torch.device, n: int) -> torch.Tensor:
    """Zeroed scratch of the kernel, one per device and stream (launches on one stream are ordered; the
    kernel leaves the scratch zeroed for the next one)."""
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    nbytes = _C.lib.pace_linear_workspace_bytes(n)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def fits(x: torch.Tensor, weight: torch.Tensor) -> bool:
    if not x.is_cuda or x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or weight.dim() != 2:
        return False
    n, k = weight.shape
    if x.shape[-1] != k or n % 128 or k % 128 or weight.stride(1) != 1 or weight.stride(0) % 8:
        return False
    return 0 < x.numel() // k <= MAX_TOKENS


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.linear(x, weight, bias)`` on the library GEMM (see the module text for why)."""
    return F.linear(x, weight, bias)


def linear_skinny(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x W^T on the weight-streaming kernel; raises where the shape does not fit it."""
    if not fits(x, weight):
        raise RuntimeError("linear_skinny: needs bf16 CUDA operands, at most 32 token rows, N and K multiples of 128")
    k = weight.shape[1]
    x2 = x.reshape(-1, k)
    if x2.stride(1) != 1 or x2.stride(0) % 8 or x2.data_ptr() % 16:
        x2 = x2.contiguous()
    out = torch.empty(x2.shape[0], weight.shape[0], dtype=torch.bfloat16, device=x.device)
    torch.ops.pace_b200.linear_skinny(x2, weight, out, _workspace(x.device, weight.shape[0]))
    return out.view(*x.shape[:-1], weight.shape[0])
