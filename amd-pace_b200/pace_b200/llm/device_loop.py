"""Greedy decode loop that stays on the device: one CUDA graph per generated token, no host
synchronisation between tokens.

The reference's step loop (pace/llm/generator.py:715-818) returns to Python after every token: the
sampler's argmax (sampler.py:215-260), the stopping criteria (stopping_criteria.py:73-127: an EOS id
or the length limit ends a sequence) and the attention-mask bookkeeping all run on the host, which
on a GPU costs more than the kernels of a small batch.  Here the whole step - embedding, every
layer's projections, fused RoPE + append, decode attention, MLP, the LM head, argmax, the EOS flags,
the write of the new token into the output buffer and into the next step's input, the position
increment - is recorded once (``StepGraph``) and replayed; lengths, block tables, positions, the
step counter and the finished flags are device tensors that the recorded kernels advance.  The
host looks at the flags only every ``poll_every`` tokens.

Greedy only (the benchmark configurations decode greedily); ragged PARD acceptance needs
data-dependent launch shapes and stays in ``Generator``.
"""
from typing import List, Optional, Sequence

import torch

from pace_b200.llm.cache import KVCacheManager
from pace_b200.llm.graph import StepGraph


class GreedyDeviceLoop:
    """Continues greedy decoding of ``model`` over ``manager``'s caches.

    ``last_tokens`` [B] are the newest tokens (not yet fed to the model), ``positions`` [B] their
    position ids, ``kv_start`` the left-pad counts (or None).  ``eos_token_ids`` end a sequence:
    the EOS token itself is kept, everything after it is ``pad_token_id`` (reference
    stopping_criteria.py:73-104, generator.py:788-806).  ``keep_logits`` leaves every step's last-position
    logits in ``self.logits`` ([B, vocab] fp32, overwritten by the next step): what a test compares with a
    recorded run of the reference model."""

    def __init__(self, model, manager: KVCacheManager, last_tokens: torch.Tensor, positions: torch.Tensor,
                 max_new_tokens: int, kv_start: Optional[torch.Tensor] = None,
                 eos_token_ids: Optional[Sequence[int]] = None, pad_token_id: int = 0, keep_logits: bool = False):
        dev = last_tokens.device
        B = last_tokens.shape[0]
        self.model, self.manager, self.max_new = model, manager, max_new_tokens
        self.cur = last_tokens.reshape(B, 1).clone()
        self.pos = positions.reshape(B, 1).clone()
        self.tokens = torch.full((B, max_new_tokens), pad_token_id, dtype=torch.long, device=dev)
        self.step = torch.zeros(1, dtype=torch.long, device=dev)          # tokens produced so far
        self.finished = torch.zeros(B, dtype=torch.bool, device=dev)
        self.produced = 0
        self._eos = set(int(t) for t in (eos_token_ids or []))
        eos = torch.tensor(list(eos_token_ids) if eos_token_ids else [], dtype=torch.long, device=dev)
        pad = torch.full((B,), pad_token_id, dtype=torch.long, device=dev)
        self.logits = torch.zeros(B, model.vocab_size, dtype=torch.float32, device=dev) if keep_logits else None

        def one_token():
            hidden = model.model.forward_tokens(self.cur, manager, self.pos, kv_start)
            last = model.lm_head(hidden)[:, -1].float()
            if self.logits is not None:
                self.logits.copy_(last)
            nxt = last.argmax(dim=-1)
            nxt = torch.where(self.finished, pad, nxt)
            col = self.step.clamp(max=max_new_tokens - 1).expand(B, 1)
            self.tokens.scatter_(1, col, nxt.unsqueeze(1))
            if eos.numel():
                self.finished.logical_or_(torch.isin(nxt, eos))
            self.step.add_(1)
            self.cur.copy_(nxt.unsqueeze(1))
            self.pos.add_(1)
            return self.tokens

        # one token per sequence and step: the appends are deferred (the rotated key and the value are staged
        # by the RoPE kernel, ride along with the layer's decode launch and are committed once per step)
        manager.defer_appends = True
        with torch.inference_mode():
            self.graph = StepGraph(manager, one_token, n_new=1, warmup=1)   # the warm-up step is token 0
        self.produced = 1

    @torch.inference_mode()
    def run(self, poll_every: int = 16) -> torch.Tensor:
        """Decodes until ``max_new_tokens`` or until every sequence has met an EOS id; returns the
        ``[B, max_new_tokens]`` token buffer (device)."""
        while self.produced < self.max_new:
            n = min(poll_every, self.max_new - self.produced)
            for _ in range(n):
                self.graph.replay()
            self.produced += n
            if bool(self.finished.all()):           # the only host synchronisation, once per poll
                break
        self.manager.pool.check_status()
        return self.tokens

    def lengths(self) -> List[int]:
        """Generated tokens per sequence, the EOS token included."""
        toks = self.tokens.cpu()
        n = min(self.produced, self.max_new)
        out = []
        for b in range(toks.shape[0]):
            row = toks[b, :n].tolist()
            out.append(next((i + 1 for i, t in enumerate(row) if t in self._eos), n))
        return out
