"""Wave-admission serving loop over one shared KV pool (one model instance on one GPU).

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
