"""The sm_100a attention backend behind ``MultiHeadAttention``.

Takes the place of the reference's NATIVE and JIT attention backends
(pace/ops/backends/native.py:32-47, pace/ops/backends/jit.py:31-47): same
``execute(query, key, value, attention_mask)`` contract, but the computation is
the hand-written CUDA kernels of libpace_b200.so.  There is no fallback: a
tensor that is not on a CUDA device is an error.
"""
import ctypes as C
import math
from typing import Dict, Optional, Tuple

import torch

from pace_b200 import _C
from pace_b200.llm.cache import PagedKV
from pace_b200.ops.base import BackendBase
from pace_b200.ops.enum import BackendType, DataType, OperatorType
from pace_b200.ops.registry import backend_registry

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}
_OPS = torch.ops.pace_b200   # defined by pace_b200.torch_ops (imported with the cache module)


def workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch shared by every attention call on a device.

    Calls on one stream are ordered, so one buffer serves them all; a call on
    another stream gets its own (keyed by stream) because overlapping kernels
    would race on it.
    """
    key = (device.index if device.index is not None else torch.cuda.current_device(),
           torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def kv_start_from_mask(mask: torch.Tensor) -> Optional[torch.Tensor]:
    """Left padding expressed by an additive ``[B,1,S,L]`` mask -> first visible key per row.

    The reference encodes padding as finfo.min columns (llama.py:294-310); the
    kernels take the count of leading masked keys of the last query row instead.
    """
    if mask is None or mask.dim() != 4:
        return None
    row = mask[:, 0, -1, :]
    hidden = (row < -1e30).to(torch.int32)
    return torch.cumprod(hidden, dim=-1).sum(dim=-1).to(torch.int32)


_sm_counts: Dict[int, int] = {}


def even_lengths(lens, n_kv_heads: int, head_dim: int, page_tokens: int, device: Optional[torch.device],
                 sms: Optional[int] = None) -> bool:
    """True when giving every thread block whole (sequence, KV head) units loads the busiest block
    at most 1.3x an even share - the test the decode kernel makes on the device, made here on the
    host mirror of the lengths (the reference keeps one ``seq_len`` per layer on the host as well,
    cache.py:184).  Such a launch may be told never to cut a unit (``PACE_ATTN_WHOLE_UNITS``): it
    then touches no workspace, and the append behind it need not wait for it."""
    if not lens:
        return False
    if sms is None:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        sms = _sm_counts.get(idx)
        if sms is None:
            sms = _sm_counts[idx] = torch.cuda.get_device_properties(idx).multi_processor_count
    grid = 2 * sms                                      # decode: two thread blocks per SM
    if page_tokens <= 64:
        chunk = min(64 // page_tokens, 16 // max(head_dim // 64, 1)) * page_tokens
    else:
        chunk = 64
    chunks = [(n + chunk - 1) // chunk for n in lens]
    units = len(lens) * n_kv_heads
    per_block = (units + grid - 1) // grid
    return per_block * max(chunks) * grid * 10 <= sum(chunks) * n_kv_heads * 13


def paged_attention(query: torch.Tensor, key: PagedKV, kv_start: Optional[torch.Tensor] = None,
                    q_lens: Optional[torch.Tensor] = None, scale: Optional[float] = None,
                    out: Optional[torch.Tensor] = None, max_ctas: int = 0, decode_kernel: Optional[str] = None,
                    whole_units: Optional[bool] = None, one_cta_per_sm: bool = False,
                    no_early_kv: bool = False) -> torch.Tensor:
    """Attention of ``query`` [B, Hq, S, D] over one layer of the paged pool.

    The last five arguments choose among schedules that give the same result (tests walk through
    them; callers normally leave them alone): ``max_ctas`` limits the thread blocks,
    ``decode_kernel`` forces ``"cuda"`` (CUDA-core kernel) or ``"mma"`` (tensor-core kernel) for
    S == 1, ``whole_units`` overrides the host's own test for ``PACE_ATTN_WHOLE_UNITS``,
    ``one_cta_per_sm`` keeps decode on eight-warp thread blocks, ``no_early_kv`` makes a decode
    launch wait for the kernel in front of it before it fetches anything."""
    cache = key.cache
    pool, mgr = cache.pool, cache.manager
    if query.device != pool.device:
        raise RuntimeError("query must live on the KV pool's CUDA device")
    if query.dtype != torch.bfloat16:
        raise TypeError("pace_b200 attention computes on bf16 queries")
    if query.dim() != 4:
        raise RuntimeError("pace_b200 attention requires 4D inputs")
    B, Hq, S, D = query.shape
    if B != len(mgr.slots) or D != pool.head_dim or Hq % pool.n_kv_heads:
        raise ValueError(f"query {tuple(query.shape)} does not fit the cache "
                         f"(B={len(mgr.slots)}, Hkv={pool.n_kv_heads}, D={pool.head_dim})")
    if query.stride(3) != 1 or any(s % 8 for s in query.stride()[:3]) or query.data_ptr() % 16:
        query = query.contiguous()
    # a staged row (deferred append) rides along as the newest key of a one-token decode launch on the
    # tensor-core kernel; anything else needs it in the pool first
    pending = cache.pending
    if pending and (S != 1 or Hq // pool.n_kv_heads >= 33 or decode_kernel == "cuda"):
        mgr.commit()
        pending = False
    # [B, S, Hq, D] storage so the caller's transpose(1, 2).reshape(B, S, Hq*D) is a view
    if out is None:
        out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=query.device).transpose(1, 2)
    elif out.shape != query.shape or out.dtype != torch.bfloat16 or out.stride(3) != 1 or out.device != query.device:
        raise ValueError("out must be a bf16 [B, Hq, S, D] tensor (any strides, last dim contiguous) on the same device")
    nbytes = _C.lib.pace_attn_workspace_bytes(B, Hq, pool.n_kv_heads, D, S)
    ws = workspace(query.device, nbytes)
    flags = 0
    if whole_units is None:
        whole_units = S == 1 and even_lengths(cache._lens, pool.n_kv_heads, D, pool.page_tokens, query.device)
    if S == 1 and whole_units:
        flags |= _C.ATTN_WHOLE_UNITS
    if one_cta_per_sm:
        flags |= _C.ATTN_ONE_CTA_PER_SM
    if no_early_kv:
        flags |= _C.ATTN_NO_EARLY_KV
    k_pend = v_pend = None
    if pending:
        k_pend, v_pend = mgr.staging(cache.layer)
        flags |= _C.ATTN_PENDING_ROW
        mgr._row_stored.add(cache.layer)    # the launch below puts the staged row in its slot of the pool
    if S == 1 and decode_kernel == "cuda":
        op = _OPS.attn_decode_cuda_cores
    elif S == 1 and decode_kernel != "mma":
        op = _OPS.attn_decode
    elif S <= 64:
        op = _OPS.attn_verify
    else:
        op = _OPS.attn_prefill
    # a manager that owns its pool uses slots 0..B-1: no seq_ids tells the kernels so and saves them a dependent load
    op(pool.handle, pool.pages, cache.layer, query, out, None if mgr.identity_slots else mgr.slots_dev, kv_start, q_lens,
       ws, float(scale) if scale is not None else 1.0 / math.sqrt(D), flags, k_pend, v_pend, int(max_ctas))
    return out


def dense_attention(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor,
                    mask: Optional[torch.Tensor]) -> torch.Tensor:
    """The reference custom op's operands (csrc/ops/attention.cpp:18-97) on CUDA tensors."""
    if query.dim() != 4 or key.dim() != 4 or value.dim() != 4 or (mask is not None and mask.dim() != 4):
        raise RuntimeError("pace::SDPA attention requires 4D inputs")
    if key.shape != value.shape:
        raise RuntimeError("pace::SDPA attention requires Key and Value sizes to be of same shape")
    for t, name in ((query, "Query"), (key, "Key"), (value, "Value")):
        if t.dtype not in (torch.float32, torch.bfloat16):
            raise RuntimeError(f"pace::SDPA attention only support the dtypes Float and BF16 types for input {name}")
    if mask is not None and mask.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError("pace::SDPA attention only support the dtypes Float and BF16 types for input Attention mask")
    if query.device.type != "cuda":
        raise RuntimeError("pace_b200 attention takes CUDA tensors (there is no CPU path)")
    out_dtype = query.dtype
    q, k, v = (t.to(torch.bfloat16).contiguous() for t in (query, key, value))
    B, N, S, H = q.shape
    Nkv, L = k.shape[1], k.shape[2]
    if k.shape[0] != B or k.shape[3] != H or N % Nkv:
        raise RuntimeError("pace::SDPA attention: key/value shape does not match the query")
    m_ptr, m_fp32, m_rows = None, 0, 1
    if mask is not None:
        if mask.shape[0] != B or mask.shape[1] != 1 or mask.shape[3] != L or mask.shape[2] not in (1, S):
            raise RuntimeError("pace::SDPA attention: mask must be [B, 1, 1|S, L]")
        mask = mask.contiguous()
        m_ptr, m_fp32, m_rows = mask.data_ptr(), int(mask.dtype == torch.float32), mask.shape[2]
    out = torch.empty_like(q)
    nbytes = _C.lib.pace_attn_workspace_bytes(B, N, Nkv, H, S)
    ws = workspace(q.device, nbytes)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    with torch.cuda.device(q.device):
        _C.check(_C.lib.pace_attention_dense(q.data_ptr(), k.data_ptr(), v.data_ptr(), m_ptr, m_fp32, m_rows,
                                             out.data_ptr(), B, N, Nkv, S, L, H, ws.data_ptr(), ws.numel(), stream),
                 "pace_attention_dense")
    return out.to(out_dtype)


class B200Attention(BackendBase):
    def execute(self, query: torch.Tensor, key, value, attention_mask: Optional[torch.Tensor] = None,
                kv_start: Optional[torch.Tensor] = None, q_lens: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None, **schedule) -> torch.Tensor:
        if isinstance(key, PagedKV):
            if not isinstance(value, PagedKV) or value.cache is not key.cache:
                raise ValueError("key and value must come from the same update_cache call")
            if kv_start is None and attention_mask is not None:
                kv_start = kv_start_from_mask(attention_mask)
            return paged_attention(query, key, kv_start=kv_start, q_lens=q_lens, out=out, **schedule)
        return dense_attention(query, key, value, attention_mask)


for _bt in (BackendType.B200, BackendType.NATIVE, BackendType.JIT):
    backend_registry.register(OperatorType.MHA, _bt, [DataType.BFLOAT16, DataType.FLOAT32])(B200Attention)
