"""CPU restatement of the reference attention arithmetic.  TEST INFRASTRUCTURE ONLY.

Two flavours, matching the reference's two shipped attention backends:

* ``sdpa_native``  - pace/ops/backends/native.py:32-47: torch's CPU
  scaled_dot_product_attention with an additive mask, scale 1/sqrt(D), no
  causal flag, no dropout.
* ``sdpa_jit_restated`` - csrc/ops/kernels/attention_kernels.cpp:188,218-257
  (the live "Method 1" sequence): scores = (Q K^T) * 1/sqrt(D) stored in the
  INPUT dtype, += mask in place, softmax over the last axis in place, then
  P V, every step accumulating in fp32 and rounding to the input dtype when it
  stores.  The arithmetic itself lives in oneDNN v3.8 (fetched at build time by
  cmake/BuildJITBackend.cmake:18-44, not vendored in the reference tree), so
  this restates the published semantics of matmul / binary_add /
  softmax_accurate; the reference's own test keeps the same restatement in
  torch ops (tests/ops/test_sdpa.py:44-60).

Plus the pieces either side that decide WHAT is attended over:
``repeat_kv`` (pace/llm/models/llama.py:50-61), the 2-D -> 4-D additive mask
(transformers' AttentionMaskConverter.to_4d as called at llama.py:294-299) and
the BMC mask padding (cache.py:195-222).
"""
import math
from typing import Optional

import torch
import torch.nn.functional as F


def repeat_kv(x: torch.Tensor, n_rep: int) -> torch.Tensor:
    """[B, Hkv, T, D] -> [B, Hkv*n_rep, T, D]; head h*n_rep+r is a copy of head h."""
    if n_rep == 1:
        return x
    b, h, t, d = x.shape
    return x.unsqueeze(2).expand(b, h, n_rep, t, d).reshape(b, h * n_rep, t, d)


def additive_mask_4d(mask2d: torch.Tensor, q_len: int, kv_len: int, dtype) -> torch.Tensor:
    """[B, kv_len] 0/1 mask -> [B, 1, q_len, kv_len] additive mask.

    Entry (i, j) is 0 when key j is visible to query i, i.e. j <= past + i with
    past = kv_len - q_len and mask2d[b, j] == 1; otherwise finfo(dtype).min.
    """
    lo = torch.finfo(dtype).min
    past = kv_len - q_len
    i = torch.arange(q_len).unsqueeze(1)
    j = torch.arange(kv_len).unsqueeze(0)
    causal_ok = j <= (past + i)                                  # [q, kv]
    keep = causal_ok.unsqueeze(0) & (mask2d[:, None, :kv_len] != 0)  # [B, q, kv]
    out = torch.zeros(keep.shape, dtype=dtype)
    out.masked_fill_(~keep, lo)
    return out.unsqueeze(1)


def sdpa_native(q, k, v, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.scaled_dot_product_attention(q, k, v, attn_mask=mask)


def sdpa_jit_restated(q, k, v, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    dt = q.dtype
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = (torch.matmul(q.float(), k.float().transpose(2, 3)) * scale).to(dt)
    if mask is not None:
        s = (s.float() + mask.float()).to(dt)
    p = torch.softmax(s.float(), dim=-1).to(dt)
    return torch.matmul(p.float(), v.float()).to(dt)


def sdpa_exact(q, k, v, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 everywhere; the yardstick the two flavours above are measured against."""
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.matmul(q.float(), k.float().transpose(2, 3)) * scale
    if mask is not None:
        s = s + mask.float()
    return torch.matmul(torch.softmax(s, dim=-1), v.float())


def attend_over_cache(q, k_cache, v_cache, seq_len: int, left_pad: int = 0,
                      flavour: str = "native") -> torch.Tensor:
    """What one reference layer does after update_cache returned its buffers.

    q        [1, Hq, S, D]      the S newest tokens' queries
    k_cache  [1, Hkv, cap, D]   the whole (padded) buffer, GQA heads NOT expanded
    seq_len  valid tokens in the buffer (the S new ones included)
    left_pad leading cached positions that are padding (masked)

    The reference expands K/V to Hq heads before caching (llama.py:152-158),
    builds the causal+padding mask for the real columns (llama.py:294-299) and
    pads it with finfo.min up to the buffer's capacity (cache.py:195-222).
    """
    hq, hkv = q.shape[1], k_cache.shape[1]
    s = q.shape[2]
    cap = k_cache.shape[2]
    k = repeat_kv(k_cache, hq // hkv)
    v = repeat_kv(v_cache, hq // hkv)
    m2 = torch.ones(1, seq_len, dtype=torch.long)
    m2[:, :left_pad] = 0
    m4 = additive_mask_4d(m2, s, seq_len, q.dtype)
    if cap > seq_len:
        pad = torch.full((1, 1, s, cap - seq_len), torch.finfo(q.dtype).min, dtype=q.dtype)
        m4 = torch.cat([m4, pad], dim=-1)
    fn = {"native": sdpa_native, "jit": sdpa_jit_restated, "exact": sdpa_exact}[flavour]
    return fn(q, k, v, m4)
