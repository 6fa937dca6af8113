"""KV-cache manager and per-layer cache objects on a device-resident paged pool.

Drop-in for the reference's pace/llm/cache.py (same class and method names, same
argument meaning, same errors):

    KVCacheType, get_kv_cache_class            cache.py:18-45
    KVCacheManager                             cache.py:48-123
    BMCKVCache / DynamicKVCache                cache.py:170-400

What differs underneath: K/V live in one paged pool per manager
(``[layer][K|V][page][kv_head][page_tokens][head_dim]`` bf16 in HBM) with the block
table, lengths and free list in device memory; append / rollback / beam gather are
CUDA kernels (csrc/kv_pool.cu) and the latter two move no K/V bytes.  ``capacity``
follows the reference's BMC growth trace exactly (whole ``tokens_per_split`` segments);
it is bookkeeping on top of the physical pages, which are 64 tokens by default.  ``update_cache`` returns handles (``PagedKV``) instead of
dense tensors; ``MultiHeadAttention`` consumes them directly.  The host keeps
integer mirrors of lengths and capacities because the reference API is
synchronous about them (``len(manager)``, ``ValueError`` on over-removal).

Extensions the reference does not have (its batch shares one length): ragged
per-sequence appends and rollbacks (``n_new_per_seq=``, list-valued
``remove_cache``), a shared long-lived pool (``pool=``) and deferred decode appends
(``defer_appends``): a one-token ``update_cache`` then only stages the new row, the
attention op reads it from the staging buffer as the newest key, and ``commit()`` stores
the staged rows of all layers with one kernel after the step's last layer.
"""
import ctypes as C
import math
import os
from abc import ABC, abstractmethod
from enum import Enum
from typing import List, Optional, Sequence, Tuple, Union

import torch

from pace_b200 import _C
from pace_b200 import torch_ops  # noqa: F401  (defines torch.ops.pace_b200.*)

OVER_REMOVE_MSG = "Cannot remove more tokens than available in cache."
KV_PAGE_TOKENS = 64


def physical_page_tokens(tokens_per_split: Optional[int]) -> int:
    """Tokens per physical page of the pool.

    64 by default: one page is then exactly one full K/V chunk of the attention kernels (one TMA box
    of 64 rows per 128-byte column block), whatever the BMC segment size.  The reference's capacity
    (a multiple of ``tokens_per_split``) is bookkeeping on top of the pages and does not depend on
    their size.  ``PACE_KV_PAGE_TOKENS=tps`` makes a page one BMC segment instead, an integer forces a size.
    """
    v = os.getenv("PACE_KV_PAGE_TOKENS", "")
    if v == "tps" and tokens_per_split:
        return int(tokens_per_split)
    if v.isdigit() and int(v) > 0:
        return int(v)
    return KV_PAGE_TOKENS


class KVCacheType(Enum):
    """Cache policies, as in the reference (cache.py:18-33)."""

    DYNAMIC = "dynamic"
    BMC = "bmc"

    @staticmethod
    def get_kv_cache_type(cache_type: Union[str, "KVCacheType"]) -> "KVCacheType":
        if isinstance(cache_type, str):
            return KVCacheType(cache_type)
        return cache_type


def get_kv_cache_class(cache_type: Union[str, KVCacheType]):
    cache_type = KVCacheType.get_kv_cache_type(cache_type)
    if cache_type == KVCacheType.DYNAMIC:
        return DynamicKVCache
    if cache_type == KVCacheType.BMC:
        return BMCKVCache
    raise ValueError(f"Invalid cache type: {cache_type}")


def bmc_tokens_per_split(max_seq_length: int) -> int:
    """Segment size of the BMC policy; honours PACE_BMC_NUM_SPLITS (cache.py:177-181)."""
    num_splits = int(os.getenv("PACE_BMC_NUM_SPLITS", int(math.sqrt(max_seq_length))))
    return max_seq_length // num_splits


def _stream_ptr(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_OPS = torch.ops.pace_b200   # every device-side step of this module goes through the dispatcher ops


class KVPool:
    """Device memory + descriptor of one paged pool (C struct pace_kv_pool_t)."""

    def __init__(self, n_layers: int, n_kv_heads: int, head_dim: int, page_tokens: int, n_pages: int,
                 max_seqs: int, max_pages_per_seq: int, device):
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("pace_b200 KV pools live in CUDA memory; got device " + str(device))
        self.device = device
        self.desc = _C.KVPoolStruct(n_layers=n_layers, n_kv_heads=n_kv_heads, head_dim=head_dim,
                                    page_tokens=page_tokens, n_pages=n_pages, max_seqs=max_seqs,
                                    max_pages_per_seq=max_pages_per_seq)
        pb, mb = C.c_uint64(), C.c_uint64()
        _C.check(_C.lib.pace_kv_pool_bytes(C.byref(self.desc), C.byref(pb), C.byref(mb)), "pace_kv_pool_bytes")
        # zero-filled like the reference's fresh segments (cache.py:255-256)
        self.pages = torch.zeros(pb.value, dtype=torch.uint8, device=device)
        self.meta = torch.zeros(mb.value, dtype=torch.uint8, device=device)
        _C.check(_C.lib.pace_kv_pool_bind(C.byref(self.desc), self.pages.data_ptr(), self.meta.data_ptr()),
                 "pace_kv_pool_bind")
        with torch.cuda.device(device):
            _C.check(_C.lib.pace_kv_pool_reset(C.byref(self.desc), _stream_ptr(device)), "pace_kv_pool_reset")
        self.n_layers, self.n_kv_heads, self.head_dim = n_layers, n_kv_heads, head_dim
        self.page_tokens, self.n_pages = page_tokens, n_pages
        self.max_seqs, self.max_pages_per_seq = max_seqs, max_pages_per_seq
        self._free_slots = list(range(max_seqs - 1, -1, -1))
        self.host_pages = [0] * max_seqs          # host mirror of seq_pages (admission control)
        self.host_free_pages = n_pages
        self.shared_pages = False                 # set by a beam gather: appends may copy-on-write

    @property
    def ref(self):
        return C.byref(self.desc)

    @property
    def handle(self) -> int:
        """The pool as the ``torch.ops.pace_b200`` ops name it: the address of its descriptor."""
        return C.addressof(self.desc)

    # -- slots -------------------------------------------------------------
    def alloc_slots(self, n: int) -> List[int]:
        if n > len(self._free_slots):
            raise RuntimeError(f"KV pool has {len(self._free_slots)} free sequence slots, {n} requested")
        return [self._free_slots.pop() for _ in range(n)]

    def release_slots(self, slots: Sequence[int], slots_dev: Optional[torch.Tensor] = None) -> None:
        if not slots:
            return
        if slots_dev is None:
            slots_dev = torch.tensor(list(slots), dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            _C.check(_C.lib.pace_kv_seq_release(self.ref, slots_dev.data_ptr(), len(slots), _stream_ptr(self.device)),
                     "pace_kv_seq_release")
        for s in slots:
            if not self.shared_pages:
                self.host_free_pages += self.host_pages[s]
            self.host_pages[s] = 0
            self._free_slots.append(s)

    # -- status ------------------------------------------------------------
    def query(self) -> Tuple[int, int]:
        """(sticky status bits, free pages); synchronises the current stream."""
        out = (C.c_int32 * 4)()
        with torch.cuda.device(self.device):
            _C.check(_C.lib.pace_kv_pool_query(self.ref, C.byref(out), _stream_ptr(self.device)), "pace_kv_pool_query")
        return int(out[0]), int(out[1])

    def check_status(self) -> None:
        bits, _ = self.query()
        if bits:
            raise _C.PaceError("KV pool device status: " + _C.describe_status(bits))

    def clear_status(self) -> None:
        with torch.cuda.device(self.device):
            _C.check(_C.lib.pace_kv_pool_clear_status(self.ref, _stream_ptr(self.device)), "pace_kv_pool_clear_status")

    # raw views for tests / debugging (device tensors, no copies)
    def _meta_view(self, ptr: int, n: int) -> torch.Tensor:
        off = ptr - self.meta.data_ptr()
        return self.meta[off: off + 4 * n].view(torch.int32)

    def block_table(self) -> torch.Tensor:
        return self._meta_view(self.desc.block_table, self.max_seqs * self.max_pages_per_seq).view(
            self.max_seqs, self.max_pages_per_seq)

    def seq_len(self) -> torch.Tensor:
        return self._meta_view(self.desc.seq_len, self.n_layers * self.max_seqs).view(self.n_layers, self.max_seqs)

    def seq_pages(self) -> torch.Tensor:
        return self._meta_view(self.desc.seq_pages, self.max_seqs)

    def page_ref(self) -> torch.Tensor:
        return self._meta_view(self.desc.page_ref, self.n_pages)


class PagedKV:
    """What ``update_cache`` returns for K (or V): a view of one layer of the pool.

    Quacks like the dense ``[B, H, capacity, D]`` tensor the reference returns
    (cache.py:326) as far as shape queries go; ``dense()`` materialises it.
    """

    def __init__(self, cache: "KVCacheBase", which: str):
        self.cache = cache
        self.which = which

    @property
    def shape(self) -> torch.Size:
        return self.cache._reported_shape()

    def size(self, dim: Optional[int] = None):
        return self.shape if dim is None else self.shape[dim]

    def dim(self) -> int:
        return len(self.shape)

    @property
    def dtype(self):
        return torch.bfloat16

    @property
    def device(self):
        return self.cache.pool.device

    def contiguous(self):
        return self

    def dense(self) -> torch.Tensor:
        k, v = self.cache.read_dense()
        return k if self.which == "k" else v

    def __repr__(self):
        return f"PagedKV({self.which}, layer={self.cache.layer}, shape={tuple(self.shape)})"


class KVCacheManager:
    """One cache object per layer over a shared pool (reference: cache.py:48-123)."""

    def __init__(self, config, max_seq_length: int, cache_type: KVCacheType, pool: Optional[KVPool] = None,
                 extra_tokens: int = 0):
        self.num_layers = config.num_hidden_layers
        self.cache_type = KVCacheType.get_kv_cache_type(cache_type)
        self.kv_cache_class = get_kv_cache_class(self.cache_type)
        self.max_seq_length = max_seq_length
        self.extra_tokens = extra_tokens
        self.pool: Optional[KVPool] = pool
        self._owns_pool = pool is None
        self.slots: Optional[List[int]] = None
        self.slots_dev: Optional[torch.Tensor] = None
        self.identity_slots = False
        self.static_launch = False   # frozen launch sequence (CUDA graphs): layer 0 always reserves
        self.capturing = False       # launches are being recorded, not executed: leave the mirror alone
        self.skip_reserve = False    # with static_launch: record the step without its page reservation
        # Deferred decode appends: a one-token update_cache only stages its row (nothing is launched when
        # the caller already wrote it into the staging buffer), attention takes it as a pending key, and
        # commit() appends every layer's row in one launch.  Off by default: update_cache then appends
        # at once, as the reference does.
        self.defer_appends = False
        self._stage_k: Optional[torch.Tensor] = None   # [layers, B, H, 1, D] views of the staging buffer
        self._stage_v: Optional[torch.Tensor] = None
        self._pending: set = set()                     # layers whose newest row is staged, not yet committed
        self._row_stored: set = set()                  # ... and of those, the layers whose row an attention launch has stored
        # Device-resident counts: appends and rollbacks whose per-sequence counts are CUDA tensors (the
        # output of a kernel, e.g. PARD acceptance) are launched without the host ever seeing the numbers.
        # The host mirror of lengths is then out of date until sync_host_mirror() reads the device's back.
        self.host_mirror_stale = False
        self.cache_objects: List[KVCacheBase] = [
            self.kv_cache_class(max_seq_length, manager=self, layer=i) for i in range(self.num_layers)
        ]

    # -- pool creation on first use (shapes are only known then) -----------------
    def _ensure_pool(self, batch: int, n_kv_heads: int, head_dim: int, device) -> None:
        if self.slots is not None:
            return
        page_tokens = self.cache_objects[0].page_tokens
        if self.pool is None:
            # capacity can exceed max_seq_length by up to one segment (cache.py:300-313), PARD adds drafts
            max_tokens = self.max_seq_length + self.extra_tokens + 2 * page_tokens
            max_pages = (max_tokens + page_tokens - 1) // page_tokens + 1
            self.pool = KVPool(self.num_layers, n_kv_heads, head_dim, page_tokens, n_pages=batch * max_pages + batch,
                               max_seqs=batch, max_pages_per_seq=max_pages, device=device)
        else:
            p = self.pool
            if (p.n_layers, p.n_kv_heads, p.head_dim, p.page_tokens) != (self.num_layers, n_kv_heads, head_dim,
                                                                        page_tokens):
                raise ValueError("shared KV pool geometry does not match this manager")
        self.slots = self.pool.alloc_slots(batch)
        self.slots_dev = torch.tensor(self.slots, dtype=torch.int32, device=self.pool.device)
        self.identity_slots = self.slots == list(range(batch))

    def __len__(self) -> int:
        return int(self.cache_objects[0].seq_len)

    # -- deferred decode appends ---------------------------------------------------------------
    def adopt_staging(self, k_all: torch.Tensor, v_all: torch.Tensor) -> None:
        """Use the caller's buffers as the staging area of deferred appends: bf16 ``[layers, B, H, 1, D]``
        tensors (views with any uniform strides, D contiguous, rows 16-byte aligned) that hold every
        layer's new K and V row when the step runs - typically the output buffer of the projections.
        ``update_cache(k_all[l], v_all[l], 2)`` then stages without launching anything."""
        for x in (k_all, v_all):
            if x.dtype != torch.bfloat16 or x.dim() != 5 or x.shape[0] != self.num_layers or x.shape[3] != 1:
                raise ValueError("staging tensors must be bf16 [layers, B, H, 1, D]")
            if x.stride(4) != 1 or any(st % 8 for st in x.stride()[:4]) or x.data_ptr() % 16:
                raise ValueError("staging rows must be contiguous in D and 16-byte aligned")
        if k_all.shape != v_all.shape or k_all.stride() != v_all.stride():
            raise ValueError("K and V staging tensors must have the same shape and strides")
        self.commit()
        self._stage_k, self._stage_v = k_all, v_all

    def staging(self, layer: int) -> Tuple[torch.Tensor, torch.Tensor]:
        """Where layer ``layer``'s next K and V row go in deferred mode: ``[B, H, 1, D]`` views."""
        if self._stage_k is None:
            pool = self.pool
            if pool is None or self.slots is None:
                raise RuntimeError("the staging buffer is sized on the first update_cache")
            buf = torch.zeros(self.num_layers, 2, len(self.slots), pool.n_kv_heads, 1, pool.head_dim,
                              dtype=torch.bfloat16, device=pool.device)
            self._stage_k, self._stage_v = buf[:, 0], buf[:, 1]
        return self._stage_k[layer], self._stage_v[layer]

    def commit(self) -> None:
        """Stores every staged row in the pool and advances the device lengths: one kernel per run of
        consecutive layers (one kernel for a whole decode step).  Called by whatever needs the pool
        itself up to date (rollback, gather, read-back, a multi-token append or attention call); a
        step that only decodes calls it once, after its last layer."""
        if not self._pending:
            return
        layers = sorted(self._pending)
        pool, k_all, v_all = self.pool, self._stage_k, self._stage_v
        lo = 0
        while lo < len(layers):
            hi = lo
            while hi + 1 < len(layers) and layers[hi + 1] == layers[hi] + 1:
                hi += 1
            a, b = layers[lo], layers[hi] + 1
            # rows that the layers' decode launches have stored themselves need no second copy
            stored = all(l in self._row_stored for l in range(a, b))
            _OPS.kv_append_layers(pool.handle, pool.pages, pool.meta, a, b, self.slots_dev,
                                  None if stored else k_all[a:b], None if stored else v_all[a:b])
            lo = hi + 1
        self._pending.clear()
        self._row_stored.clear()

    def __getitem__(self, idx: int) -> "KVCacheBase":
        return self.cache_objects[idx]

    def update_mask(self, attn_mask: torch.Tensor, input_size: int) -> torch.Tensor:
        return self.cache_objects[0].update_mask(attn_mask, input_size)

    def advance_host_mirror(self, n: int) -> bool:
        """Every layer appends ``n`` tokens to every sequence (a replayed decode step): advances the
        host mirror of pages, lengths and capacities without touching the device.  Returns True when
        some sequence needs new pages.  The layers of a manager move in lockstep, so the page
        arithmetic is done once, not once per layer."""
        counts = [n] * len(self.slots)
        first = self.cache_objects[0]
        grow = first._host_account(counts)
        for c in self.cache_objects[1:]:
            if len(c._lens) != len(first._lens):
                grow |= c._host_account(counts)
                continue
            c._lens = [x + n for x in c._lens]
            c._capacity = c._capacity_after(max(c._lens))
        return grow

    def update_cache_with_beam_indices(self, beam_idx: torch.Tensor) -> None:
        """Beam gather (cache.py:106-116): ONE index-only kernel for all layers."""
        if self.slots is None:
            return
        self.commit()
        pool = self.pool
        idx = beam_idx.to(device=pool.device, dtype=torch.int64).contiguous()
        if idx.numel() != len(self.slots):
            raise ValueError("beam_idx must have one entry per cached sequence")
        _OPS.kv_gather(pool.handle, pool.meta, self.slots_dev, idx)
        pool.shared_pages = True
        order = beam_idx.tolist()
        pages = [pool.host_pages[self.slots[j]] for j in order]
        for i, s in enumerate(self.slots):
            pool.host_pages[s] = pages[i]
        for c in self.cache_objects:
            if c._lens:
                c._lens = [c._lens[j] for j in order]

    def sync_host_mirror(self) -> None:
        """Reads the device's lengths and page counts back (one synchronisation) after appends or
        rollbacks with device-resident counts.  The reported BMC capacity is re-derived from the
        lengths as they are now (the reference's capacity never shrinks on a rollback; a caller that
        needs that history keeps its counts on the host)."""
        if self.slots is None:
            return
        self.commit()
        pool = self.pool
        lens = pool.seq_len()[:, self.slots_dev.long()].cpu().tolist()
        pages = pool.seq_pages()[self.slots_dev.long()].cpu().tolist()
        for c, row in zip(self.cache_objects, lens):
            c._lens = [int(x) for x in row]
            c._capacity = max(c._capacity, c._capacity_after(max(c._lens))) if c._lens else 0
        for s_, n in zip(self.slots, pages):
            pool.host_pages[s_] = int(n)
        pool.host_free_pages = pool.query()[1]
        self.host_mirror_stale = False

    def remove_cache(self, remove_len) -> None:
        """Rollback on every layer (cache.py:118-123): one kernel, no K/V bytes moved.  A CUDA int32
        tensor of per-sequence counts is consumed on the device (no host check: over-removal raises the
        pool's PACE_DEV_OVER_REMOVE bit instead of the ValueError)."""
        live = [c for c in self.cache_objects if c.key is not None]
        if not live:
            return
        self.commit()
        if isinstance(remove_len, torch.Tensor) and remove_len.is_cuda:
            if remove_len.dtype != torch.int32 or remove_len.numel() != len(self.slots):
                raise ValueError("device-resident remove counts must be an int32 tensor with one entry per sequence")
            _OPS.kv_truncate(self.pool.handle, self.pool.meta, 0, self.num_layers, self.slots_dev, 0, remove_len)
            self.host_mirror_stale = True
            return
        per_seq = live[0]._normalise_remove(remove_len)
        for c in live:
            c._check_remove(per_seq)
        pool = self.pool
        if len(live) == self.num_layers:
            scalar, dev = live[0]._remove_args(per_seq)
            _OPS.kv_truncate(pool.handle, pool.meta, 0, self.num_layers, self.slots_dev, scalar, dev)
            for c in live:
                c._apply_remove(per_seq)
        else:
            for c in live:
                c.remove_cache(remove_len)

    def recycle(self, batch_indices: Sequence[int]) -> None:
        """Ends the sequences at these batch positions: their pages go back to the pool and their
        lengths to zero on every layer, while the slots stay with this manager and can take the next
        requests (continuous batching; the reference only drops whole managers, generator.py:396-410)."""
        idx = sorted(set(int(b) for b in batch_indices))
        if not idx or self.slots is None:
            return
        self.commit()
        pool = self.pool
        slots = [self.slots[b] for b in idx]
        dev = torch.tensor(slots, dtype=torch.int32, device=pool.device)
        with torch.cuda.device(pool.device):
            _C.check(_C.lib.pace_kv_seq_release(pool.ref, dev.data_ptr(), len(slots), _stream_ptr(pool.device)),
                     "pace_kv_seq_release")
        for s in slots:
            if not pool.shared_pages:
                pool.host_free_pages += pool.host_pages[s]
            pool.host_pages[s] = 0
        for c in self.cache_objects:
            if c._lens:
                for b in idx:
                    c._lens[b] = 0

    def release(self) -> None:
        if self.pool is not None and self.slots is not None:
            self._pending.clear()   # staged rows of sequences that are being dropped
            self._row_stored.clear()
            if not self._owns_pool:
                self.pool.release_slots(self.slots, self.slots_dev)
            self.slots = None
            self.slots_dev = None
        if self._owns_pool:
            self.pool = None

    def __del__(self):
        try:
            self.release()
        except Exception:
            pass


class KVCacheBase(ABC):
    """Common machinery of the two policies (reference: cache.py:126-167)."""

    policy_page_tokens: int

    def __init__(self, max_seq_length: int, manager: Optional[KVCacheManager] = None, layer: int = 0):
        if manager is None:  # a free-standing layer cache, as the reference's tests build them
            class _Cfg:
                num_hidden_layers = 1
            manager = KVCacheManager.__new__(KVCacheManager)
            manager.num_layers, manager.cache_type = 1, None
            manager.max_seq_length, manager.extra_tokens = max_seq_length, 0
            manager.pool, manager._owns_pool, manager.slots, manager.slots_dev = None, True, None, None
            manager.static_launch = manager.capturing = manager.skip_reserve = False
            manager.identity_slots = False
            manager.defer_appends, manager._stage_k, manager._stage_v, manager._pending = False, None, None, set()
            manager._row_stored = set()
            manager.host_mirror_stale = False
            manager.cache_objects = [self]
        self.manager = manager
        self.layer = layer
        self.key: Optional[PagedKV] = None
        self.value: Optional[PagedKV] = None
        self.concat_dim: Optional[int] = None
        self._lens: List[int] = []        # host mirror, one entry per batch row
        self._capacity = 0                # tokens, as the reference's buffer size along concat_dim
        self._ndim = 4

    # -- reference attributes --------------------------------------------------
    @property
    def pool(self) -> KVPool:
        return self.manager.pool

    @property
    def seq_len(self) -> int:
        if not self._lens:
            return 0
        return self._lens[0] if len(set(self._lens)) == 1 else max(self._lens)

    @property
    def seq_lens(self) -> List[int]:
        return list(self._lens)

    @property
    def capacity(self) -> int:
        return self._capacity

    @abstractmethod
    def _capacity_after(self, updated: int) -> int:
        ...

    def _reported_shape(self) -> torch.Size:
        b, h, d = len(self._lens), self.pool.n_kv_heads, self.pool.head_dim
        if self._ndim == 3:
            return torch.Size((b, self._capacity, d))
        return torch.Size((b, h, self._capacity, d))

    def update_mask(self, attn_mask: torch.Tensor, input_size: int) -> torch.Tensor:
        return attn_mask

    # -- append ------------------------------------------------------------------
    def _begin_append(self, B: int, H: int, n: int, D: int, device, n_new_per_seq):
        """Host accounting and page reservation shared by the two append entry points.  Returns the
        pool, the manager, the device pointer of the ragged counts (or None), the stream pointer and
        the tensor that keeps those counts alive."""
        mgr = self.manager
        mgr._ensure_pool(B, H, D, device)
        pool = self.pool
        if (H, D) != (pool.n_kv_heads, pool.head_dim) or B != len(mgr.slots):
            raise ValueError(f"update_cache got [B={B},H={H},D={D}], the cache holds "
                             f"[B={len(mgr.slots)},H={pool.n_kv_heads},D={pool.head_dim}]")
        if not self._lens:
            self._lens = [0] * B
        counts = [n] * B if n_new_per_seq is None else [int(x) for x in n_new_per_seq]
        if len(counts) != B or any(c < 0 or c > n for c in counts):
            raise ValueError("n_new_per_seq must hold B counts in [0, n]")
        n_dev = None
        if n_new_per_seq is not None:
            n_dev = torch.tensor(counts, dtype=torch.int32, device=pool.device)
        static = mgr.static_launch
        grow = self._host_account(counts, dry_run=mgr.capturing)
        sp = _stream_ptr(pool.device)
        nptr = n_dev.data_ptr() if n_dev is not None else None
        with torch.cuda.device(pool.device):
            # after a beam gather pages may be shared: the first layer's reserve un-shares (copies on
            # write) whatever this append is about to write into, for all layers at once.  Under a
            # CUDA graph the launch sequence is frozen, so the first layer always reserves.
            # (skip_reserve: the step is being recorded a second time, for replays the host mirror knows to
            # need no new page)
            need_reserve = ((self.layer == 0 and not mgr.skip_reserve) if static
                            else (grow or (pool.shared_pages and self.layer == 0)))
            if need_reserve:
                _OPS.kv_reserve(pool.handle, pool.meta, self.layer, mgr.slots_dev, n, n_dev)
        return pool, mgr, nptr, sp, n_dev

    def update_cache_rope(self, query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, table_row: torch.Tensor,
                          rope, n_new_per_seq: Optional[Sequence[int]] = None,
                          query_out: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, PagedKV, PagedKV]:
        """RoPE and append in one kernel: the three calls between the projections and the attention
        op of a decoder layer (reference pace/llm/models/llama.py:130-165: view as heads, rotate q and
        k, ``update_cache``).  ``query`` / ``key`` / ``value`` are the projection outputs viewed as
        ``[B, n, heads, D]`` (no transpose), ``table_row`` the int32 ``[B, n]`` rows of the rotary
        tables (``RotaryEmbedding.table_rows(position_ids)``), ``rope`` a
        ``pace_b200.ops.RotaryEmbedding``.  Returns the rotated queries as ``[B, Hq, n, D]`` (a view
        of ``query_out``, by default written over ``query``) and the cache handles."""
        if self.concat_dim is None:
            self.concat_dim = 2
        elif self.concat_dim != 2:
            raise AssertionError("concat_dim should be the same for all updates")
        if query.device.type != "cuda":
            raise RuntimeError("pace_b200 caches take CUDA tensors (there is no CPU path)")
        for name, x in (("query", query), ("key", key), ("value", value)):
            if x.dtype != torch.bfloat16 or x.dim() != 4:
                raise TypeError(f"{name} must be a bf16 [B, n, heads, D] tensor")
            if x.stride(3) != 1 or any(s % 8 for s in x.stride()[:3]) or x.data_ptr() % 16:
                raise ValueError(f"{name}: head_dim must be contiguous and every row 16-byte aligned")
        B, n, Hq, D = query.shape
        H = key.shape[2]
        if key.shape != value.shape or key.shape[:2] != (B, n) or key.shape[3] != D:
            raise ValueError("key and value must be [B, n, kv_heads, D] like the query")
        out = query if query_out is None else query_out
        if out.shape != query.shape or out.dtype != torch.bfloat16 or out.stride(3) != 1 or out.data_ptr() % 16 \
                or any(s % 8 for s in out.stride()[:3]):
            raise ValueError("query_out must be a bf16 [B, n, Hq, D] tensor with 16-byte aligned rows")
        if table_row.shape != (B, n) or table_row.dtype != torch.int32 or table_row.stride(1) != 1:
            raise ValueError("table_row must be an int32 [B, n] tensor")
        self._ndim = 4
        mgr = self.manager
        if isinstance(n_new_per_seq, torch.Tensor):
            # device-resident counts (int32 [B], each <= n): nothing about them reaches the host.  The first
            # layer's reservation provides the pages for all layers (they share the block table).
            if not n_new_per_seq.is_cuda or n_new_per_seq.dtype != torch.int32 or n_new_per_seq.numel() != B:
                raise ValueError("device-resident counts must be a CUDA int32 tensor with one entry per sequence")
            mgr.commit()
            mgr._ensure_pool(B, H, D, query.device)
            pool = self.pool
            if not self._lens:
                self._lens = [0] * B
            if self.layer == 0:
                _OPS.kv_reserve(pool.handle, pool.meta, 0, mgr.slots_dev, n, n_new_per_seq)
            cos, sin = rope.device_tables(pool.device)
            _OPS.kv_append_rope(pool.handle, pool.pages, pool.meta, self.layer, mgr.slots_dev, query, key, value, out,
                                table_row, cos, sin, rope.rotary_dim, not rope.is_neox_style, n_new_per_seq, None, None)
            mgr.host_mirror_stale = True
            if self.key is None:
                self.key, self.value = PagedKV(self, "k"), PagedKV(self, "v")
            return out.transpose(1, 2), self.key, self.value
        staged = mgr.defer_appends and n == 1 and n_new_per_seq is None
        if not staged or self.pending:
            mgr.commit()     # a multi-token append, or a second token for this layer: the pool has to be up to date
        pool, mgr, nptr, sp, n_dev = self._begin_append(B, H, n, D, query.device, n_new_per_seq)
        cos, sin = rope.device_tables(pool.device)
        ks, vs = mgr.staging(self.layer) if staged else (None, None)
        _OPS.kv_append_rope(pool.handle, pool.pages, pool.meta, self.layer, mgr.slots_dev, query, key, value, out,
                            table_row, cos, sin, rope.rotary_dim, not rope.is_neox_style, n_dev, ks, vs)
        if staged:           # the rotated key and the value sit in the staging rows; the decode launch takes them along
            mgr._pending.add(self.layer)
            mgr._row_stored.discard(self.layer)
        if self.key is None:
            self.key, self.value = PagedKV(self, "k"), PagedKV(self, "v")
        return out.transpose(1, 2), self.key, self.value

    def update_cache(self, key_states: torch.Tensor, value_states: torch.Tensor, concat_dim: int,
                     n_new_per_seq: Optional[Sequence[int]] = None) -> Tuple[PagedKV, PagedKV]:
        """Append ``[B, H, n, D]`` new keys/values (cache.py:268-326 / 370-400)."""
        if self.concat_dim is None:
            self.concat_dim = concat_dim
        elif self.concat_dim != concat_dim:
            raise AssertionError("concat_dim should be the same for all updates")
        if key_states.device.type != "cuda":
            raise RuntimeError("pace_b200 caches take CUDA tensors (there is no CPU path)")
        if key_states.dtype != torch.bfloat16 or value_states.dtype != torch.bfloat16:
            raise TypeError("pace_b200 caches hold bf16 keys/values")
        if key_states.shape != value_states.shape:
            raise ValueError("key_states and value_states must have the same shape")
        if key_states.dim() == 3 and concat_dim == 1:      # [B, n, D]: one KV head
            self._ndim = 3
            key_states, value_states = key_states.unsqueeze(1), value_states.unsqueeze(1)
        elif key_states.dim() == 4 and concat_dim == 2:
            self._ndim = 4
        else:
            raise ValueError("expected [B, H, n, D] with concat_dim=2 (or [B, n, D] with concat_dim=1)")
        B, H, n, D = key_states.shape
        if key_states.stride(3) != 1 or value_states.stride(3) != 1 or key_states.stride() != value_states.stride():
            key_states, value_states = key_states.contiguous(), value_states.contiguous()
        if any(s % 8 for s in key_states.stride()[:3]) or key_states.data_ptr() % 16 or value_states.data_ptr() % 16:
            key_states, value_states = key_states.contiguous().clone(), value_states.contiguous().clone()
        mgr = self.manager
        if mgr.defer_appends and n == 1 and n_new_per_seq is None and self._ndim == 4:
            return self._stage_row(key_states, value_states)
        mgr.commit()
        pool, mgr, nptr, sp, n_dev = self._begin_append(B, H, n, D, key_states.device, n_new_per_seq)
        _OPS.kv_append(pool.handle, pool.pages, pool.meta, self.layer, mgr.slots_dev, key_states, value_states, n_dev)
        if self.key is None:
            self.key, self.value = PagedKV(self, "k"), PagedKV(self, "v")
        return self.key, self.value

    @property
    def pending(self) -> bool:
        """True while this layer's newest row is staged (counted in ``seq_len``, not yet in the pool)."""
        return self.layer in self.manager._pending

    def _stage_row(self, key_states: torch.Tensor, value_states: torch.Tensor) -> Tuple[PagedKV, PagedKV]:
        """Deferred form of a one-token append: host accounting and page reservation as usual, the row
        itself only goes to (or already sits in) the manager's staging buffer."""
        mgr = self.manager
        if self.pending:
            mgr.commit()    # a second token for this layer: the first one has to be in the pool
        B, H, _, D = key_states.shape
        self._begin_append(B, H, 1, D, key_states.device, None)
        ks, vs = mgr.staging(self.layer)
        for dst, src in ((ks, key_states), (vs, value_states)):
            if dst.data_ptr() != src.data_ptr() or dst.stride() != src.stride():
                dst.copy_(src)
        mgr._pending.add(self.layer)
        mgr._row_stored.discard(self.layer)
        if self.key is None:
            self.key, self.value = PagedKV(self, "k"), PagedKV(self, "v")
        return self.key, self.value

    def _host_account(self, counts: Sequence[int], dry_run: bool = False) -> bool:
        """Advance the host mirror (pages shared by all layers, lengths, capacity) for an append of
        ``counts[b]`` tokens.  Returns True when some sequence needs new pages.  ``dry_run`` checks
        without recording (a launch being captured into a CUDA graph does not execute)."""
        pool, mgr = self.pool, self.manager
        P = pool.page_tokens
        grow = False
        for b, slot in enumerate(mgr.slots):
            need = (self._lens[b] + counts[b] + P - 1) // P
            if need > pool.max_pages_per_seq:
                raise RuntimeError(f"sequence needs {need} pages, the pool's table rows hold {pool.max_pages_per_seq}")
            if need > pool.host_pages[slot]:
                grow = True
                if not dry_run:
                    pool.host_free_pages -= need - pool.host_pages[slot]
                    pool.host_pages[slot] = need
        if pool.host_free_pages < 0 and not pool.shared_pages:
            raise RuntimeError("KV pool exhausted")
        if not dry_run:
            for b in range(len(self._lens)):
                self._lens[b] += counts[b]
            self._capacity = self._capacity_after(max(self._lens))
        return grow

    # -- rollback ----------------------------------------------------------------
    def _normalise_remove(self, remove_len) -> List[int]:
        if isinstance(remove_len, torch.Tensor):
            remove_len = remove_len.tolist()
        if isinstance(remove_len, (list, tuple)):
            out = [int(x) for x in remove_len]
            if len(out) != len(self._lens):
                raise ValueError("per-sequence remove lengths must match the batch")
            return out
        return [int(remove_len)] * len(self._lens)

    def _check_remove(self, per_seq: List[int]) -> None:
        for r, have in zip(per_seq, self._lens):
            if r > have:
                raise ValueError(OVER_REMOVE_MSG)
            if r < 0:
                raise ValueError("remove_len must be non-negative")

    def _remove_args(self, per_seq: List[int]):
        if len(set(per_seq)) <= 1:
            return (per_seq[0] if per_seq else 0), None
        dev = torch.tensor(per_seq, dtype=torch.int32, device=self.pool.device)
        self._keepalive = dev
        return 0, dev

    def _apply_remove(self, per_seq: List[int]) -> None:
        self._lens = [have - r for have, r in zip(self._lens, per_seq)]
        self._after_remove()

    def _after_remove(self) -> None:
        pass

    def remove_cache(self, remove_len) -> None:
        """Forget the last tokens (cache.py:224-240 / 352-368): lengths only, pages kept."""
        if self.key is None:
            return  # silent no-op on an empty cache, as the reference
        self.manager.commit()
        per_seq = self._normalise_remove(remove_len)
        self._check_remove(per_seq)
        pool, mgr = self.pool, self.manager
        scalar, dev = self._remove_args(per_seq)
        _OPS.kv_truncate(pool.handle, pool.meta, self.layer, self.layer + 1, mgr.slots_dev, scalar, dev)
        self._apply_remove(per_seq)

    # -- gather --------------------------------------------------------------------
    def update_cache_with_beam_indices(self, beam_idx: torch.Tensor) -> None:
        """Per-layer form of the reference API (cache.py:161-167).  The block table is
        shared by all layers, so the gather is done once by the manager; calling it
        on a layer object directly is only valid for a free-standing single layer."""
        if self.key is None:
            return
        if self.manager.num_layers != 1:
            raise RuntimeError("beam gather permutes the table shared by all layers: call it on the manager")
        self.manager.update_cache_with_beam_indices(beam_idx)

    # -- read-back -------------------------------------------------------------------
    def read_dense(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """Dense ``[B, H, capacity, D]`` K and V, i.e. what the reference's update_cache returns."""
        pool, mgr = self.pool, self.manager
        mgr.commit()
        B, cap = len(self._lens), self._capacity
        k = torch.empty(B, pool.n_kv_heads, cap, pool.head_dim, dtype=torch.bfloat16, device=pool.device)
        v = torch.empty_like(k)
        if cap:
            _OPS.kv_read_dense(pool.handle, pool.pages, self.layer, mgr.slots_dev, k, v)
        if self._ndim == 3:
            return k[:, 0], v[:, 0]
        return k, v


class BMCKVCache(KVCacheBase):
    """Segmented growth: capacity rises in whole ``tokens_per_split`` steps (cache.py:170-326)."""

    def __init__(self, max_seq_length: int, manager: Optional[KVCacheManager] = None, layer: int = 0):
        super().__init__(max_seq_length, manager, layer)
        self.tokens_per_split = bmc_tokens_per_split(max_seq_length)
        self.page_tokens = physical_page_tokens(self.tokens_per_split)

    def _capacity_after(self, updated: int) -> int:
        # a fresh buffer is made when none exists or the new length reaches the capacity (cache.py:292-313)
        if self._capacity == 0 or updated >= self._capacity:
            return ((updated - 1) // self.tokens_per_split + 1) * self.tokens_per_split
        return self._capacity

    def update_mask(self, attn_mask: torch.Tensor, input_size: int) -> torch.Tensor:
        """Pad the mask with finfo.min up to the capacity (cache.py:195-222)."""
        segment_idx = (input_size - 1) // self.tokens_per_split
        shape = list(attn_mask.shape)
        shape[-1] = (segment_idx + 1) * self.tokens_per_split - input_size
        pad = torch.full(shape, torch.finfo(attn_mask.dtype).min, dtype=attn_mask.dtype, device=attn_mask.device)
        return torch.cat([attn_mask, pad], dim=-1)


class DynamicKVCache(KVCacheBase):
    """No padding: the reported buffer is exactly the cached length (cache.py:329-400)."""

    def __init__(self, max_seq_length: int, manager: Optional[KVCacheManager] = None, layer: int = 0):
        super().__init__(max_seq_length, manager, layer)
        self.page_tokens = physical_page_tokens(None)

    def _capacity_after(self, updated: int) -> int:
        return updated

    def _after_remove(self) -> None:
        self._capacity = max(self._lens) if self._lens else 0
