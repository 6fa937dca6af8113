"""CPU restatement of the reference KV-cache bookkeeping.  TEST INFRASTRUCTURE ONLY.

Follows pace/llm/cache.py of the reference:
  * split arithmetic          cache.py:175-181
  * BMC append + growth rule  cache.py:242-326  (growth test is ``>=``, :300)
  * BMC rollback              cache.py:224-240  (length only, buffer untouched)
  * BMC mask padding          cache.py:195-222
  * dynamic append / rollback cache.py:352-400
  * beam gather               cache.py:161-167
  * manager fan-out           cache.py:48-123

The classes here keep dense ``[B, H, cap, D]`` tensors exactly as the reference
does, so cache *contents* (including zero padding and stale rolled-back rows)
can be compared with what the paged CUDA cache holds.
"""
import math
import os
from typing import List, Optional, Tuple

import torch

OVER_REMOVE_MSG = "Cannot remove more tokens than available in cache."


def bmc_tokens_per_split(max_seq_length: int) -> int:
    """Segment size of the BMC policy (cache.py:177-181)."""
    n_splits = int(os.getenv("PACE_BMC_NUM_SPLITS", int(math.sqrt(max_seq_length))))
    return max_seq_length // n_splits


def bmc_capacity_after(capacity: int, seq_len: int, n_new: int, tps: int) -> int:
    """Capacity (tokens) after appending n_new tokens (cache.py:292-313).

    A fresh buffer is made when none exists or when the new length reaches the
    current capacity; its size is the new length rounded up to whole segments.
    """
    upd = seq_len + n_new
    if capacity == 0 or upd >= capacity:
        return ((upd - 1) // tps + 1) * tps
    return capacity


class SegmentedCacheRef:
    """One layer's cache under the BMC policy."""

    policy = "bmc"

    def __init__(self, max_seq_length: int):
        self.tps = bmc_tokens_per_split(max_seq_length)
        self.k: Optional[torch.Tensor] = None
        self.v: Optional[torch.Tensor] = None
        self.seq_len = 0
        self.axis: Optional[int] = None
        self.capacity_trace: List[int] = []

    # -- append ---------------------------------------------------------
    def append(self, k_new: torch.Tensor, v_new: torch.Tensor, axis: int):
        if self.axis is None:
            self.axis = axis
        assert self.axis == axis, "concat_dim should be the same for all updates"
        n = k_new.size(axis)
        upd = self.seq_len + n
        cap = 0 if self.k is None else self.k.size(axis)
        new_cap = bmc_capacity_after(cap, self.seq_len, n, self.tps)
        if self.k is None or upd >= cap:
            shape = list(k_new.shape)
            shape[axis] = new_cap
            fresh_k = torch.zeros(shape, dtype=k_new.dtype)
            fresh_v = torch.zeros(shape, dtype=v_new.dtype)
            if self.k is not None:
                fresh_k.narrow(axis, 0, cap).copy_(self.k)
                fresh_v.narrow(axis, 0, cap).copy_(self.v)
            self.k, self.v = fresh_k, fresh_v
        self.k.narrow(axis, self.seq_len, n).copy_(k_new)
        self.v.narrow(axis, self.seq_len, n).copy_(v_new)
        self.seq_len = upd
        self.capacity_trace.append(self.k.size(axis))
        return self.k, self.v

    # -- rollback -------------------------------------------------------
    def remove(self, n: int) -> None:
        if self.k is None:
            return  # silent no-op on an empty cache (cache.py:235)
        if n > self.seq_len:
            raise ValueError(OVER_REMOVE_MSG)
        self.seq_len -= n

    # -- mask -----------------------------------------------------------
    def pad_mask(self, mask: torch.Tensor, input_size: int) -> torch.Tensor:
        seg = (input_size - 1) // self.tps
        extra = (seg + 1) * self.tps - input_size
        shape = list(mask.shape)
        shape[-1] = extra
        fill = torch.full(shape, torch.finfo(mask.dtype).min, dtype=mask.dtype)
        return torch.cat([mask, fill], dim=-1)

    # -- beam gather ----------------------------------------------------
    def gather(self, beam_idx: torch.Tensor) -> None:
        if self.k is not None:
            self.k = self.k.index_select(0, beam_idx)
            self.v = self.v.index_select(0, beam_idx)

    @property
    def capacity(self) -> int:
        return 0 if self.k is None else self.k.size(self.axis)


class GrowingCacheRef:
    """One layer's cache under the DYNAMIC policy (concatenate every step)."""

    policy = "dynamic"

    def __init__(self, max_seq_length: int):
        self.k = None
        self.v = None
        self.seq_len = 0
        self.axis = None
        self.capacity_trace: List[int] = []

    def append(self, k_new, v_new, axis: int):
        if self.axis is None:
            self.axis = axis
        assert self.axis == axis, "concat_dim should be the same for all updates"
        if self.k is None:
            self.k, self.v = k_new, v_new
        else:
            self.k = torch.cat([self.k, k_new], dim=axis)
            self.v = torch.cat([self.v, v_new], dim=axis)
        self.seq_len = int(self.k.size(axis))
        self.capacity_trace.append(self.seq_len)
        return self.k, self.v

    def remove(self, n: int) -> None:
        if self.k is None:
            return
        if n > self.seq_len:
            raise ValueError(OVER_REMOVE_MSG)
        self.seq_len -= n
        self.k = self.k.narrow(self.axis, 0, self.seq_len)
        self.v = self.v.narrow(self.axis, 0, self.seq_len)

    def pad_mask(self, mask, input_size):
        return mask

    gather = SegmentedCacheRef.gather

    @property
    def capacity(self) -> int:
        return self.seq_len


def cache_class_for(policy: str):
    if policy == "bmc":
        return SegmentedCacheRef
    if policy == "dynamic":
        return GrowingCacheRef
    raise ValueError(f"Invalid cache type: {policy}")


class CacheManagerRef:
    """Per-layer fan-out with the manager's surface (cache.py:48-123)."""

    def __init__(self, num_layers: int, max_seq_length: int, policy: str):
        cls = cache_class_for(policy)
        self.layers = [cls(max_seq_length) for _ in range(num_layers)]

    def __len__(self) -> int:
        return int(self.layers[0].seq_len)

    def __getitem__(self, i):
        return self.layers[i]

    def pad_mask(self, mask, input_size):
        return self.layers[0].pad_mask(mask, input_size)

    def remove(self, n: int) -> None:
        for c in self.layers:
            c.remove(n)

    def gather(self, beam_idx) -> None:
        for c in self.layers:
            c.gather(beam_idx)


def replay_trace(ops: List[Tuple], max_seq_length: int, policy: str, tps_env=None):
    """Integer-only replay of an append/remove script.

    ``ops`` is a list of ("append", n) / ("remove", n).  Returns the list of
    (seq_len, capacity) after every op; over-removal yields ("error",).
    This is what slot indices, block tables and rollback lengths are compared
    with bit-exactly.
    """
    tps = bmc_tokens_per_split(max_seq_length) if policy == "bmc" else 1
    seq_len, cap, started = 0, 0, False
    out = []
    for kind, n in ops:
        if kind == "append":
            if policy == "bmc":
                cap = bmc_capacity_after(cap if started else 0, seq_len, n, tps)
            seq_len += n
            if policy != "bmc":
                cap = seq_len
            started = True
            out.append((seq_len, cap))
        elif kind == "remove":
            if not started:
                out.append((seq_len, cap))
            elif n > seq_len:
                out.append(("error",))
            else:
                seq_len -= n
                if policy != "bmc":
                    cap = seq_len
                out.append((seq_len, cap))
        else:
            raise ValueError(kind)
    return out
