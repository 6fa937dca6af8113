"""Generation loop: greedy decoding and PARD speculative decoding over the B200 KV-cache path.

Re-hosts the part of the reference's ``Generator`` (pace/llm/generator.py) that drives the hot path:

  _prepare_kv_cache                    generator.py:396-410   one manager per model, max_new + prompt
  _prepare_for_pard                    generator.py:412-449   second manager for the draft model
  _speculate_tokens                    generator.py:638-667   one draft pass over history + (d-1) placeholders
  _postprocess_speculated_tokens       generator.py:669-713   accept / rollback
  _generate                            generator.py:715-818   the step loop
  _beam_search                         generator.py:517-636   beams re-ordered every step, the cache with them

What each step does to the caches follows the reference exactly: the draft cache takes
history + d - 1 tokens and always gives d - 1 back; the target cache takes history + d tokens and
gives back d - keep + 1 of them unless every compared draft matched (keep == d), in which case nothing
is removed and the unverified last draft row stays (generator.py:696-706).

Beyond the reference (which asserts batch size 1 for PARD, generator.py:427-430): a batch of
sequences, each with its own acceptance, so appends and rollbacks are ragged per sequence; and
acceptance forced by a seeded Bernoulli draw per draft token instead of the token comparison, which
is how the speculative configuration of the benchmark exercises rollback with random weights.
"""
from typing import List, Optional

import torch

from pace_b200.llm.cache import KVCacheManager, KVCacheType
from pace_b200.llm.configs import PardSpecDecodeConfig, SamplingConfig
from pace_b200.llm.outputs import GeneratorOutput, SpeculativeStats


class Generator:
    def __init__(self, model, pard_model=None, pard_config: Optional[PardSpecDecodeConfig] = None,
                 kv_cache_type: KVCacheType = KVCacheType.BMC):
        self.model = model
        self.pard_model = pard_model
        self.pard_config = pard_config if pard_model is not None else None
        self.kv_cache_type = kv_cache_type
        self.device = next(model.parameters()).device
        self.trace: List[list] = []        # (cache, op, n per sequence) - what the tests compare with the reference

    # -- preparation --------------------------------------------------------------------------
    def _prepare_kv_cache(self, kv_cache_type, input_prompts: torch.Tensor) -> None:
        max_seq_length = self.sampling_config.max_new_tokens + input_prompts.size(-1)
        extra = self.pard_config.num_speculative_tokens + 1 if self.pard_config else 0
        self.kv_cache_manager = KVCacheManager(self.model.config, max_seq_length, kv_cache_type, extra_tokens=extra)
        # one-token decode steps stage their rows and commit once per step; prompt, verify and ragged passes
        # append several tokens per sequence and are not affected
        self.kv_cache_manager.defer_appends = True

    def _prepare_for_pard(self, input_prompts: torch.Tensor) -> None:
        if self.pard_config is None:
            self.draft_size = 0
            return
        self.draft_size = self.pard_config.num_speculative_tokens
        self.total_speculated_tokens: List[int] = []
        self.pard_kv_cache_manager = KVCacheManager(
            self.pard_model.config, self.sampling_config.max_new_tokens + input_prompts.size(-1), self.kv_cache_type,
            extra_tokens=self.draft_size + 1)
        self._accept_rng = None
        if self.pard_config.forced_accept_prob is not None:
            self._accept_rng = torch.Generator().manual_seed(self.pard_config.forced_accept_seed)

    def prepare_for_generate(self, prompts: torch.Tensor, sampling_config: Optional[SamplingConfig] = None):
        self.sampling_config = sampling_config or SamplingConfig()
        self._prepare_kv_cache(self.kv_cache_type, prompts)
        self._prepare_for_pard(prompts)
        self.trace = []
        return prompts

    # -- helpers --------------------------------------------------------------------------------
    def _run_ragged(self, model, manager, tag: str, history: List[List[int]], tail: List[List[int]]):
        """Feeds every sequence the part of history + tail its cache does not hold yet."""
        cached = manager[0].seq_lens if manager[0].seq_lens else [0] * len(history)
        rows = [(history[b] + tail[b])[cached[b]:] for b in range(len(history))]
        counts = [len(r) for r in rows]
        n_max = max(counts)
        new = torch.full((len(rows), n_max), self.sampling_config.pad_token_id, dtype=torch.long)
        for b, r in enumerate(rows):
            new[b, : len(r)] = torch.tensor(r, dtype=torch.long)
        out = model.forward_ragged(new.to(self.device), counts, manager)
        self.trace.append([tag, "append", counts])
        return out.logits, counts

    def _speculate_tokens(self, history: List[List[int]]) -> List[List[int]]:
        d = self.draft_size
        if self.pard_config is None:
            return [[] for _ in history]
        tail = [[self.pard_config.pard_token] * (d - 1) for _ in history]
        logits, counts = self._run_ragged(self.pard_model, self.pard_kv_cache_manager, "draft", history, tail)
        drafts = []
        for b, n in enumerate(counts):
            drafts.append(logits[b, n - d: n].argmax(dim=-1).tolist())
        return drafts

    def _postprocess_speculated_tokens(self, next_tokens: List[List[int]], drafts: List[List[int]]) -> List[List[int]]:
        """Accept leading matches among the first d-1 drafts, always keep one target token, roll the
        caches back (generator.py:684-706) - per sequence."""
        if self.pard_config is None:
            return next_tokens
        d = self.draft_size
        kept, target_rm, draft_rm = [], [], []
        for b in range(len(drafts)):
            if self._accept_rng is not None:
                draws = (torch.rand(d - 1, generator=self._accept_rng) < self.pard_config.forced_accept_prob).tolist()
            else:
                draws = [i < len(next_tokens[b]) and next_tokens[b][i] == drafts[b][i] for i in range(d - 1)]
            keep = 0
            for ok in draws:
                if not ok:
                    break
                keep += 1
            keep += 1                                   # the target's own token is always kept
            toks = (drafts[b][: keep - 1] if self._accept_rng is not None else next_tokens[b][: keep - 1])
            toks = toks + [next_tokens[b][min(keep - 1, len(next_tokens[b]) - 1)]]
            kept.append(toks)
            target_rm.append(d - keep + 1 if d - keep > 0 else 0)
            draft_rm.append(d - 1)
            self.total_speculated_tokens.append(keep)
        if any(target_rm):
            self.kv_cache_manager.remove_cache(target_rm)
        self.trace.append(["target", "remove", target_rm])
        self.pard_kv_cache_manager.remove_cache(draft_rm)
        self.trace.append(["draft", "remove", draft_rm])
        return kept

    # -- the loop ----------------------------------------------------------------------------------
    @torch.inference_mode()
    def _generate(self, inputs: torch.Tensor) -> GeneratorOutput:
        history = [row.tolist() for row in inputs]
        prompt_len = inputs.shape[1]
        max_len = prompt_len + self.sampling_config.max_new_tokens
        d = self.draft_size
        while min(len(h) for h in history) < max_len:
            drafts = self._speculate_tokens(history)
            logits, counts = self._run_ragged(self.model, self.kv_cache_manager, "target", history, drafts)
            next_tokens = []
            for b, n in enumerate(counts):
                take = min(d + 1, n)
                next_tokens.append(logits[b, n - take: n].float().argmax(dim=-1).tolist())
            kept = self._postprocess_speculated_tokens(next_tokens, drafts)
            for b in range(len(history)):
                if len(history[b]) < max_len or self.pard_config is not None:
                    history[b] = history[b] + kept[b]
        lengths = [len(h) for h in history]
        out = torch.full((len(history), max(lengths)), self.sampling_config.pad_token_id, dtype=torch.long)
        for b, h in enumerate(history):
            out[b, : len(h)] = torch.tensor(h)
        stats = None
        if self.pard_config is not None:
            stats = SpeculativeStats(total_speculated_tokens=sum(self.total_speculated_tokens),
                                     mean_accepted_tokens=sum(self.total_speculated_tokens) / len(self.total_speculated_tokens))
        self.kv_cache_manager.pool.check_status()
        return GeneratorOutput(output_token_ids=out, lengths=lengths, speculative_stats=stats)

    # -- beam search -----------------------------------------------------------------------------
    @staticmethod
    def beam_step(logits: torch.Tensor, beam_scores: torch.Tensor, num_beams: int):
        """One re-ranking step on the last position's logits ``[B * beams, V]``: every beam's continuations
        are scored by summed log-probabilities and the best ``beams`` per prompt survive.  Returns
        ``(beam_idx [B * beams], next_tokens [B * beams], new beam_scores)``; ``beam_idx[i]`` is the row of
        the batch that row i continues - what the reference hands to
        ``update_cache_with_beam_indices`` (generator.py:585-610).  Scoring is the length-penalty-free
        core of the reference's sampler + ``BeamSearchScorer`` pair; EOS handling is not part of it."""
        n, vocab = logits.shape
        batch = n // num_beams
        logp = torch.log_softmax(logits.float(), dim=-1) + beam_scores.view(n, 1)
        top, flat = logp.view(batch, num_beams * vocab).topk(num_beams, dim=-1)
        src = torch.div(flat, vocab, rounding_mode="floor")
        beam_idx = (src + torch.arange(batch, device=logits.device).unsqueeze(1) * num_beams).view(n)
        return beam_idx, (flat % vocab).view(n), top.reshape(n)

    @torch.inference_mode()
    def _beam_search(self, inputs: torch.Tensor) -> GeneratorOutput:
        """Beam search over the paged cache (reference: generator.py:517-636).  Every step the surviving
        beams are re-ordered and ``KVCacheManager.update_cache_with_beam_indices`` makes the cache follow:
        on the paged pool that is an index-only kernel (block-table rows and lengths are permuted, pages
        shared by several beams are reference-counted and copied on the next write), where the reference
        moves every layer's whole K and V with ``index_select`` (cache.py:161-167)."""
        nb = self.sampling_config.num_beams
        ids = inputs.to(self.device).repeat_interleave(nb, dim=0)
        batch = inputs.shape[0]
        mask = torch.ones_like(ids)
        scores = torch.zeros(batch, nb, dtype=torch.float32, device=self.device)
        scores[:, 1:] = -1e9                      # all beams of a prompt start out identical: only one may win
        scores = scores.view(-1)
        for _ in range(self.sampling_config.max_new_tokens):
            logits = self.model(ids, kv_cache=self.kv_cache_manager, attention_mask=mask).logits[:, -1]
            beam_idx, tokens, scores = self.beam_step(logits, scores, nb)
            ids = torch.cat([ids[beam_idx], tokens.unsqueeze(-1)], dim=-1)
            mask = torch.cat([mask, mask.new_ones(mask.shape[0], 1)], dim=-1)
            self.kv_cache_manager.update_cache_with_beam_indices(beam_idx)
            self.trace.append(["target", "gather", beam_idx.tolist()])
        best = scores.view(batch, nb).argmax(dim=-1) + torch.arange(batch, device=self.device) * nb
        out = ids[best].cpu()
        self.kv_cache_manager.pool.check_status()
        return GeneratorOutput(output_token_ids=out, lengths=[out.shape[1]] * batch, speculative_stats=None)

    def generate(self, inputs: torch.Tensor, sampling_config: Optional[SamplingConfig] = None) -> GeneratorOutput:
        self.prepare_for_generate(inputs, sampling_config)
        if self.sampling_config.num_beams > 1:
            if self.pard_config is not None:
                raise ValueError("beam search and PARD speculative decoding do not combine")
            return self._beam_search(inputs)
        return self._generate(inputs)
