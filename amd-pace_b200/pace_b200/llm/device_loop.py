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
from pace_b200.ops.linear import linear


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
            last = linear(hidden, model.lm_head.weight)[:, -1].float()
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


class PardDeviceLoop:
    """PARD speculative decoding whose steps never come back to the host.

    The reference's step (pace/llm/generator.py:638-713, 745-749) - draft pass over history + d - 1
    placeholders, target pass over history + d drafts, acceptance, rollback of both caches - returns to
    Python for every decision; ``Generator`` of this package does the same per sequence with
    ``.tolist()`` calls.  Here every quantity a step produces stays on the device: the token history and
    its lengths are tensors, the ragged counts of both passes are computed from the lengths the pools
    hold, ``pace_pard_accept`` turns drafts and target tokens into keep counts, rollback counts and kept
    tokens, and ``pace_kv_truncate`` consumes the rollback counts directly.  Shapes are fixed (every
    sequence is padded to the most tokens a pass can need), so a step is a fixed launch sequence.

    The prompt pass has the same form with wider shapes and runs first (``prime()``).  ``forced`` is an
    optional uint8 ``[steps, B, d - 1]`` tensor of acceptance draws (the benchmark's seeded Bernoulli, or a
    recorded run's decisions); without it drafts are accepted while they equal the target's tokens.
    ``log`` keeps every step's keep counts and both caches' lengths after the rollback, on the device.
    """

    def __init__(self, target, draft, target_mgr: KVCacheManager, draft_mgr: KVCacheManager, prompts: torch.Tensor,
                 d: int, max_steps: int, pard_token: int = 1, forced: Optional[torch.Tensor] = None):
        dev = next(target.parameters()).device
        B, P = prompts.shape
        self.target, self.draft, self.tm, self.dm, self.d = target, draft, target_mgr, draft_mgr, d
        self.B, self.P, self.max_steps, self.dev = B, P, max_steps, dev
        self.cap = P + max_steps * d + d + 1
        self.hist = torch.zeros(B, self.cap, dtype=torch.long, device=dev)
        self.hist[:, :P] = prompts.to(dev)
        self.n = torch.full((B,), P, dtype=torch.int32, device=dev)          # tokens of the running history
        self.pard = torch.full((1, 1), pard_token, dtype=torch.long, device=dev)
        self.forced = forced.to(dev).contiguous() if forced is not None else None
        self.step_idx = 0
        self.keep = torch.zeros(B, dtype=torch.int32, device=dev)
        self.t_rm = torch.zeros(B, dtype=torch.int32, device=dev)
        self.d_rm = torch.zeros(B, dtype=torch.int32, device=dev)
        self.kept = torch.zeros(B, d, dtype=torch.long, device=dev)
        self.log_keep = torch.zeros(max_steps, B, dtype=torch.int32, device=dev)
        self.log_t_len = torch.zeros(max_steps, B, dtype=torch.int32, device=dev)
        self.log_d_len = torch.zeros(max_steps, B, dtype=torch.int32, device=dev)
        self.log_t_app = torch.zeros(max_steps, B, dtype=torch.int32, device=dev)
        self.log_d_app = torch.zeros(max_steps, B, dtype=torch.int32, device=dev)
        self._ar = {}
        self._zero = torch.zeros(B, dtype=torch.int32, device=dev)

    def _arange(self, n: int) -> torch.Tensor:
        if n not in self._ar:
            self._ar[n] = torch.arange(n, device=self.dev, dtype=torch.long).unsqueeze(0)
        return self._ar[n]

    def _cached(self, mgr: KVCacheManager) -> torch.Tensor:
        if mgr.pool is None or mgr.slots_dev is None:
            return self._zero
        return mgr.pool.seq_len()[0].index_select(0, mgr.slots_dev.long())

    def _pass(self, model, mgr, tail: torch.Tensor, tail_len: int, width: int, first: bool):
        """Feeds every sequence what its cache lacks of history + tail (``tail`` [B, tail_len]); returns the
        argmax of every fed position [B, width] and the counts [B] (device)."""
        cached = self._cached(mgr).long()
        h = self.n.long() - cached                                      # history tokens the cache lacks
        counts = (h + tail_len).to(torch.int32)
        j = self._arange(width)
        src = (cached.unsqueeze(1) + j).clamp_(max=self.cap - 1)
        from_hist = self.hist.gather(1, src)
        tj = (j - h.unsqueeze(1)).clamp_(0, tail_len - 1)
        ids = torch.where(j < h.unsqueeze(1), from_hist, tail.gather(1, tj))
        if first:   # the prompt pass creates the pool: counts are the same for every sequence and known to the host
            out = model.forward_ragged(ids, [self.P + tail_len] * self.B, mgr)
        else:
            out = model.forward_device_ragged(ids, counts, mgr)
        return out.logits.float().argmax(dim=-1), counts

    @torch.inference_mode()
    def step(self) -> None:
        d, B = self.d, self.B
        first = self.step_idx == 0
        wd = self.P + d - 1 if first else 2 * d - 1
        wt = self.P + d if first else d + 1
        i = self.step_idx
        # draft pass: history + (d - 1) placeholders; the drafts are the last d positions' argmax
        am, cnt_d = self._pass(self.draft, self.dm, self.pard.expand(B, d - 1), d - 1, wd, first)
        rows = (cnt_d.long() - d).unsqueeze(1) + self._arange(d)
        drafts = am.gather(1, rows.clamp_(0, wd - 1))
        # target pass: history + the d drafts; its last min(d + 1, fed) positions are the target's tokens
        am_t, cnt_t = self._pass(self.target, self.tm, drafts, d, wt, first)
        take = cnt_t.clamp(max=d + 1)
        rows_t = (cnt_t.long() - take.long()).unsqueeze(1) + self._arange(d + 1)
        target_next = am_t.gather(1, rows_t.clamp_(0, wt - 1))
        forced = self.forced[i] if self.forced is not None else None
        torch.ops.pace_b200.pard_accept(drafts, target_next, take, forced, self.keep, self.t_rm, self.d_rm, self.kept)
        # the kept tokens join the history
        pos = (self.n.long().unsqueeze(1) + self._arange(d)).clamp_(max=self.cap - 1)
        live = self._arange(d) < self.keep.long().unsqueeze(1)
        self.hist.scatter_(1, pos, torch.where(live, self.kept, self.hist.gather(1, pos)))
        self.n.add_(self.keep)
        # rollback, counts straight from the acceptance kernel
        self.tm.remove_cache(self.t_rm)
        self.dm.remove_cache(self.d_rm)
        self.log_keep[i].copy_(self.keep)
        self.log_t_app[i].copy_(cnt_t)
        self.log_d_app[i].copy_(cnt_d)
        self.log_t_len[i].copy_(self._cached(self.tm))
        self.log_d_len[i].copy_(self._cached(self.dm))
        self.step_idx += 1

    def run(self, steps: int) -> None:
        for _ in range(steps):
            self.step()

    def finish(self):
        """One synchronisation: host mirrors of both caches, the history as lists."""
        self.tm.sync_host_mirror()
        self.dm.sync_host_mirror()
        self.tm.pool.check_status()
        self.dm.pool.check_status()
        n = self.n.tolist()
        hist = self.hist.cpu()
        return [hist[b, : n[b]].tolist() for b in range(self.B)]
