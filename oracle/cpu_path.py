"""The reference's per-layer KV-cache path as it runs on the host CPU.  TEST INFRASTRUCTURE ONLY.

One call = what a reference decoder layer does between the RoPE and the output
projection (pace/llm/models/llama.py:152-165): expand GQA heads with repeat_kv,
append to the layer's BMC cache (pace/llm/cache.py:268-326), attend over the whole
padded buffer under the additive mask (NATIVE backend = torch CPU SDPA,
pace/ops/backends/native.py:44-47; or the C restatement of the JIT backend's
four-primitive sequence, csrc/ops/kernels/attention_kernels.cpp:218-257).
Used as the checker in tests and as the timed CPU baseline of bench.py.
"""
import statistics
import time
from typing import List

import torch

from oracle import attention_ref as A
from oracle import ref_loader
from oracle.kv_cache_ref import SegmentedCacheRef


class CpuDecodeLayers:
    """n_layers BMC caches in the reference's layout ([B, Hq, cap, D], heads expanded)."""

    def __init__(self, n_layers: int, batch: int, hq: int, hkv: int, d: int, prompt_len: int, max_len: int,
                 seed: int = 0, flavour: str = "native"):
        g = torch.Generator().manual_seed(seed)
        self.rep = hq // hkv
        self.flavour = flavour
        self.caches: List[SegmentedCacheRef] = []
        for _ in range(n_layers):
            c = SegmentedCacheRef(max_len)
            k = torch.randn(batch, hkv, prompt_len, d, generator=g).bfloat16()
            v = torch.randn(batch, hkv, prompt_len, d, generator=g).bfloat16()
            c.append(A.repeat_kv(k, self.rep), A.repeat_kv(v, self.rep), axis=2)
            self.caches.append(c)
        self.k_new = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
        self.v_new = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
        self.q = torch.randn(batch, hq, 1, d, generator=g).bfloat16()
        self.batch = batch

    def step(self, nthreads: int = 0) -> torch.Tensor:
        out = None
        for c in self.caches:
            K, V = c.append(A.repeat_kv(self.k_new, self.rep), A.repeat_kv(self.v_new, self.rep), axis=2)
            n = c.seq_len
            m2 = torch.ones(self.batch, n, dtype=torch.long)
            m4 = c.pad_mask(A.additive_mask_4d(m2, 1, n, torch.bfloat16), n)
            if self.flavour == "jit_c":
                from oracle import jit_c
                out = jit_c.attention_bf16(self.q, K, V, m4, nthreads=nthreads or torch.get_num_threads())
            else:
                out = A.sdpa_native(self.q, K, V, m4)
        return out


class RefDecodeLayers:
    """The same layers built from the reference's own classes, unmodified (through
    oracle/ref_loader.py): ``BMCKVCache.update_cache`` (pace/llm/cache.py:268-326) on
    ``repeat_kv``-expanded heads (pace/llm/models/llama.py:50-61, 152-158), the mask padded by
    ``update_mask`` (cache.py:195-222) and ``MultiHeadAttention`` on the NATIVE backend
    (pace/ops/backends/native.py:32-47)."""

    def __init__(self, n_layers: int, batch: int, hq: int, hkv: int, d: int, prompt_len: int, max_len: int,
                 seed: int = 0):
        ref = ref_loader.load()
        self.ref = ref
        g = torch.Generator().manual_seed(seed)
        self.rep = hq // hkv
        self.mha = ref.MultiHeadAttention(backend_impl=ref.BackendType.NATIVE, dtype=torch.bfloat16)
        self.caches = []
        for _ in range(n_layers):
            c = ref.BMCKVCache(max_len)
            k = torch.randn(batch, hkv, prompt_len, d, generator=g).bfloat16()
            v = torch.randn(batch, hkv, prompt_len, d, generator=g).bfloat16()
            c.update_cache(ref.repeat_kv(k, self.rep), ref.repeat_kv(v, self.rep), concat_dim=2)
            self.caches.append(c)
        self.k_new = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
        self.v_new = torch.randn(batch, hkv, 1, d, generator=g).bfloat16()
        self.q = torch.randn(batch, hq, 1, d, generator=g).bfloat16()
        self.batch = batch

    def step(self, nthreads: int = 0) -> torch.Tensor:
        ref, out = self.ref, None
        for c in self.caches:
            K, V = c.update_cache(ref.repeat_kv(self.k_new, self.rep), ref.repeat_kv(self.v_new, self.rep), concat_dim=2)
            n = c.seq_len
            m2 = torch.ones(self.batch, n, dtype=torch.long)
            m4 = c.update_mask(A.additive_mask_4d(m2, 1, n, torch.bfloat16), n)
            out = self.mha(self.q, K, V, attention_mask=m4)
        return out


def time_decode_tokens_per_s(model_layers: int, sample_layers: int, batch: int, hq: int, hkv: int, d: int,
                             prompt_len: int, max_len: int, steps: int, warmup: int, flavour: str = "native"):
    """Times `steps` decode steps over `sample_layers` layers and scales to `model_layers`.

    Runs the reference's own classes when a reference tree is at hand (``kind`` "reference"), else
    the restatement above ("port").  The step time is the MEDIAN over the timed steps: a step in
    which a BMC segment is added re-allocates every layer's buffers and takes several times as long,
    and how many of those fall into the timed window depends on the step count.
    Returns (tokens/s, seconds per model step, kind)."""
    kind = "reference" if (flavour == "native" and ref_loader.available()) else "port"
    if kind == "reference":
        w = RefDecodeLayers(sample_layers, batch, hq, hkv, d, prompt_len, max_len)
    else:
        w = CpuDecodeLayers(sample_layers, batch, hq, hkv, d, prompt_len, max_len, flavour=flavour)
    for _ in range(warmup):
        w.step()
    times = []
    for _ in range(steps):
        t0 = time.perf_counter()
        w.step()
        times.append(time.perf_counter() - t0)
    dt = statistics.median(times)                    # seconds per step over sample_layers
    per_model_step = dt * model_layers / sample_layers
    return batch / per_model_step, per_model_step, kind
