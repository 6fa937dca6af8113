"""Serving loops over one shared KV pool (one model instance on one GPU): wave admission and
continuous batching.

The reference serves static batches: the router collects requests for a time window and the server
runs ``generate`` on the padded batch (pace/server/router.py:112-191, server.py:74-100); continuous
batching is on its roadmap only (docs/LLM.md:24-25).  The multi-instance benchmark needs more than a
padded batch: 256 concurrent requests per GPU with prompts from 256 to 32768 tokens do not fit the
pool at once (about 229 GB of K/V for an 8B-shaped model), so requests are admitted in waves as the
pool's free pages allow, prefilled in 512-token chunks with ragged lengths, decoded together, and
their pages released.  Nothing here is a kernel: it is the caller that exercises chunked append,
prefill tiles, decode attention and page recycling on a long-lived pool.
"""
import time
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from pace_b200.llm.cache import KVCacheManager, KVCacheType, KVPool, physical_page_tokens


@dataclass
class WaveStats:
    waves: int = 0
    prompt_tokens: int = 0
    output_tokens: int = 0
    prefill_s: float = 0.0
    decode_s: float = 0.0
    wave_sizes: List[int] = field(default_factory=list)


class WaveServer:
    def __init__(self, model, pool_tokens: int, max_batch: int, max_seq_len: int, prefill_chunk: int = 512,
                 cache_type: KVCacheType = KVCacheType.BMC):
        self.model = model
        cfg = model.config
        self.device = next(model.parameters()).device
        self.page_tokens = physical_page_tokens(None)
        self.prefill_chunk = prefill_chunk
        self.cache_type = cache_type
        self.max_batch = max_batch
        head_dim = cfg.hidden_size // cfg.num_attention_heads
        n_pages = max(1, pool_tokens // self.page_tokens)
        max_pages = (max_seq_len + 2 * self.page_tokens) // self.page_tokens + 2
        self.pool = KVPool(cfg.num_hidden_layers, cfg.num_key_value_heads, head_dim, self.page_tokens, n_pages,
                           max_seqs=max_batch, max_pages_per_seq=max_pages, device=self.device)

    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_tokens - 1) // self.page_tokens + 1

    def admit(self, lengths: Sequence[int], max_new: int) -> int:
        """How many of the next requests fit the pool together (at least one if any fits at all)."""
        free, n = self.pool.host_free_pages, 0
        for L in lengths[: self.max_batch]:
            need = self._pages_for(L + max_new)
            if need > free:
                break
            free -= need
            n += 1
        return n

    @torch.inference_mode()
    def run(self, prompts: List[torch.Tensor], max_new: int, pad_id: int = 0):
        """Serves every prompt (1-D token tensors) greedily for ``max_new`` tokens.  Returns the
        generated tokens per request and the timing / wave statistics."""
        stats = WaveStats()
        outputs: List[Optional[List[int]]] = [None] * len(prompts)
        todo = list(range(len(prompts)))
        while todo:
            n = self.admit([len(prompts[i]) for i in todo], max_new)
            if n == 0:
                raise RuntimeError(f"request of {len(prompts[todo[0]])} tokens does not fit the KV pool")
            wave, todo = todo[:n], todo[n:]
            lens = [len(prompts[i]) for i in wave]
            mgr = KVCacheManager(self.model.config, max(lens) + max_new, self.cache_type, pool=self.pool)
            torch.cuda.synchronize(self.device)
            t0 = time.perf_counter()
            # ---- chunked prefill, ragged: every sequence feeds up to prefill_chunk tokens per pass ----
            done = [0] * n
            last_logits = [None] * n
            while any(d < L for d, L in zip(done, lens)):
                counts = [min(self.prefill_chunk, L - d) for d, L in zip(done, lens)]
                width = max(counts)
                new = torch.full((n, width), pad_id, dtype=torch.long)
                for b, i in enumerate(wave):
                    if counts[b]:
                        new[b, : counts[b]] = prompts[i][done[b]: done[b] + counts[b]]
                logits = self.model.forward_ragged(new.to(self.device), counts, mgr).logits
                for b in range(n):
                    if counts[b]:
                        done[b] += counts[b]
                        if done[b] == lens[b]:
                            last_logits[b] = logits[b, counts[b] - 1].float()
            nxt = torch.stack(last_logits).argmax(dim=-1)
            torch.cuda.synchronize(self.device)
            t1 = time.perf_counter()
            # ---- decode ----
            gen = [nxt]
            for _ in range(max_new - 1):
                logits = self.model.forward_ragged(nxt.unsqueeze(1), [1] * n, mgr).logits
                nxt = logits[:, 0].float().argmax(dim=-1)
                gen.append(nxt)
            toks = torch.stack(gen, dim=1).cpu()
            torch.cuda.synchronize(self.device)
            t2 = time.perf_counter()
            self.pool.check_status()
            mgr.release()
            for b, i in enumerate(wave):
                outputs[i] = toks[b].tolist()
            stats.waves += 1
            stats.wave_sizes.append(n)
            stats.prompt_tokens += sum(lens)
            stats.output_tokens += n * max_new
            stats.prefill_s += t1 - t0
            stats.decode_s += t2 - t1
        return outputs, stats


# ---------------------------------------------------------------------------------------------------
# Continuous batching
# ---------------------------------------------------------------------------------------------------
@dataclass
class _Running:
    request: int
    prompt: torch.Tensor
    max_new: int
    fed: int = 0                      # prompt tokens already in the cache
    out: List[int] = field(default_factory=list)
    next_token: Optional[int] = None  # generated, not yet fed back


@dataclass
class BatchStats:
    steps: int = 0
    prompt_tokens: int = 0
    output_tokens: int = 0
    seconds: float = 0.0
    max_running: int = 0
    padded_tokens: int = 0            # token rows that went through the model in total
    kv_bytes_read: int = 0            # K/V bytes the attention launches had to read (every layer, GQA, bf16)
    kv_bytes_written: int = 0         # K/V bytes appended
    admissions: int = 0               # steps in which at least one waiting request took a free slot


class ContinuousBatcher:
    """Iteration-level scheduling over a fixed set of cache slots (the reference names continuous
    batching as future work, docs/LLM.md:24-25; its router batches statically,
    pace/server/router.py:112-191).

    Every step feeds each running sequence what it needs next - up to ``prefill_chunk`` prompt tokens
    or its one newest generated token - through one forward pass over the packed tokens; a sequence that finishes
    gives its pages back at once (``KVCacheManager.recycle``) and the next waiting request takes its
    slot in the same step, provided the pool has the pages for its prompt and its ``max_new`` tokens.
    What makes this cheap on this cache: ragged appends and ragged attention are single launches,
    and admitting or retiring a sequence moves no K/V bytes, only block-table rows.
    """

    def __init__(self, model, pool_tokens: int, max_batch: int, max_seq_len: int, prefill_chunk: int = 256,
                 cache_type: KVCacheType = KVCacheType.BMC, max_step_tokens: int = 1024):
        self.model = model
        cfg = model.config
        self.device = next(model.parameters()).device
        self.page_tokens = physical_page_tokens(None)
        self.prefill_chunk = prefill_chunk
        self.max_batch = max_batch
        # A step's tokens go through the model packed back to back (``forward_packed``), at most this
        # many: every decoding sequence's one token first, prompt chunks with what is left.
        self.max_step_tokens = max(max_step_tokens, max_batch)
        head_dim = cfg.hidden_size // cfg.num_attention_heads
        n_pages = max(1, pool_tokens // self.page_tokens)
        max_pages = (max_seq_len + 2 * self.page_tokens) // self.page_tokens + 2
        self.pool = KVPool(cfg.num_hidden_layers, cfg.num_key_value_heads, head_dim, self.page_tokens, n_pages,
                           max_seqs=max_batch, max_pages_per_seq=max_pages, device=self.device)
        self.manager = KVCacheManager(cfg, max_seq_len, cache_type, pool=self.pool)
        self.slots: List[Optional[_Running]] = [None] * max_batch
        self.reserved_pages = 0        # pages promised to running sequences (prompt + max_new each)

    def _pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_tokens - 1) // self.page_tokens + 1

    def _admit(self, waiting: List[_Running]) -> None:
        total = self.pool.n_pages
        for b in range(self.max_batch):
            if not waiting:
                return
            if self.slots[b] is not None:
                continue
            need = self._pages_for(len(waiting[0].prompt) + waiting[0].max_new)
            if need > total:
                raise RuntimeError(f"request of {len(waiting[0].prompt)} tokens does not fit the KV pool")
            if self.reserved_pages + need > total:
                return                  # first come, first served: nobody overtakes the head of the queue
            self.reserved_pages += need
            self.slots[b] = waiting.pop(0)

    @torch.inference_mode()
    def run(self, prompts: List[torch.Tensor], max_new: int, pad_id: int = 0):
        """Serves every prompt (1-D token tensors) greedily for ``max_new`` tokens.  Returns the generated
        tokens per request and the statistics."""
        stats = BatchStats()
        outputs: List[Optional[List[int]]] = [None] * len(prompts)
        waiting = [_Running(i, p, max_new) for i, p in enumerate(prompts)]
        B = self.max_batch
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        # the manager's batch is every slot, from the first pass on
        cfg = self.model.config
        row_bytes = cfg.num_hidden_layers * 2 * cfg.num_key_value_heads * (cfg.hidden_size // cfg.num_attention_heads) * 2
        while waiting or any(s is not None for s in self.slots):
            n_wait = len(waiting)
            self._admit(waiting)
            stats.admissions += int(len(waiting) < n_wait)
            counts = [0] * B
            budget = self.max_step_tokens
            for b, s in enumerate(self.slots):          # decoding sequences first: one token each
                if s is not None and s.fed >= len(s.prompt):
                    counts[b] = 1
                    budget -= 1
            for b, s in enumerate(self.slots):          # prompt chunks share what is left
                if s is not None and s.fed < len(s.prompt) and budget > 0:
                    counts[b] = min(self.prefill_chunk, len(s.prompt) - s.fed, budget)
                    budget -= counts[b]
            if sum(counts) == 0:
                raise RuntimeError("nothing admitted and nothing running")
            pieces = []
            for b, s in enumerate(self.slots):
                if s is None or counts[b] == 0:
                    continue
                if s.fed < len(s.prompt):
                    pieces.append(s.prompt[s.fed: s.fed + counts[b]])
                else:
                    pieces.append(torch.tensor([s.next_token]))
            tokens = torch.cat(pieces).to(self.device)
            # a sequence's launch reads every cached row up to and including the step's own tokens, once
            for b, s in enumerate(self.slots):
                if s is not None and counts[b]:
                    cached = s.fed if s.fed < len(s.prompt) else len(s.prompt) + len(s.out) - 1
                    stats.kv_bytes_read += row_bytes * (cached + counts[b])
                    stats.kv_bytes_written += row_bytes * counts[b]
            logits = self.model.forward_packed(tokens, counts, self.manager).logits
            picked = logits.float().argmax(dim=-1).tolist()
            done = []
            for b, s in enumerate(self.slots):
                if s is None or counts[b] == 0:
                    continue
                if s.fed < len(s.prompt):
                    s.fed += counts[b]
                    stats.prompt_tokens += counts[b]
                    if s.fed < len(s.prompt):
                        continue        # still prefilling: this pass's logits are not sampled
                s.next_token = picked[b]
                s.out.append(picked[b])
                stats.output_tokens += 1
                if len(s.out) >= s.max_new:
                    done.append(b)
            if done:
                self.manager.recycle(done)
                for b in done:
                    s = self.slots[b]
                    outputs[s.request] = s.out
                    self.reserved_pages -= self._pages_for(len(s.prompt) + s.max_new)
                    self.slots[b] = None
            stats.steps += 1
            stats.padded_tokens += sum(counts)
            stats.max_running = max(stats.max_running, sum(s is not None for s in self.slots) + len(done))
        torch.cuda.synchronize(self.device)
        stats.seconds = time.perf_counter() - t0
        self.pool.check_status()
        return outputs, stats
