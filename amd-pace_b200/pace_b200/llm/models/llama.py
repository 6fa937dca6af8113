"""Llama decoder re-hosted on CUDA tensors around the B200 KV-cache path.

The caller of the hot path, kept in the reference's shape (pace/llm/models/llama.py): per layer
q/k/v projection -> RoPE -> ``kv_cache.update_cache`` -> ``MultiHeadAttention`` -> o_proj
(llama.py:111-170), model forward slicing off what is already cached (llama.py:270-318).
Parameter names match the reference's state dict, so its weights load unchanged.

Differences that come from the path being on the GPU:
  * no ``repeat_kv``: the cache holds the KV heads, the attention kernels are GQA-native;
  * no 4-D additive mask: causality and left padding reach the kernels as per-sequence integers
    (``kv_start`` = padded positions, the causal tail follows from the cached lengths);
  * RoPE is fused into the append kernel (``update_cache_rope``); projections, norms and the MLP
    are stock torch CUDA ops (they are not part of the path);
  * ``forward_tokens`` takes only the NEW tokens and allows ragged counts per sequence, which
    batched speculative decoding needs; ``forward`` is the reference signature on top of it.
"""
import math
from typing import List, Optional, Sequence

import torch
import torch.nn.functional as F
from torch import nn

from pace_b200.llm.cache import KVCacheBase, KVCacheManager
from pace_b200.llm.outputs import ModelOutput
from pace_b200.ops import MultiHeadAttention, RotaryEmbedding
from pace_b200.ops.linear import linear


def _lin(module: nn.Linear, x: torch.Tensor) -> torch.Tensor:
    """``module(x)``; a decode step's few token rows take the weight-streaming kernel (ops/linear.py)."""
    return linear(x, module.weight, module.bias)


class _FusedLinear(nn.Module):
    """Holds ``linear.weight`` like the reference's fused linear + activation operators."""

    def __init__(self, in_features: int, out_features: int):
        super().__init__()
        self.linear = nn.Linear(in_features, out_features, bias=False)


class RMSNorm(nn.Module):
    def __init__(self, hidden: int, eps: float):
        super().__init__()
        self.weight = nn.Parameter(torch.ones(hidden))
        self.eps = eps

    def forward(self, x):
        return F.rms_norm(x, (x.shape[-1],), self.weight, self.eps)


class LlamaMLP(nn.Module):
    """down(up(x) * silu(gate(x))) (reference MergedMLP with gate, pace/ops/mlp.py:73-79)."""

    def __init__(self, hidden: int, inter: int):
        super().__init__()
        self.up_proj = _FusedLinear(hidden, inter)
        self.gate_proj = _FusedLinear(hidden, inter)
        self.down_proj = nn.Linear(inter, hidden, bias=False)

    def forward(self, x):
        return _lin(self.down_proj, _lin(self.up_proj.linear, x) * F.silu(_lin(self.gate_proj.linear, x)))


class FusedRope:
    """What a decoder layer needs to rotate and append in one kernel: the operator (tables) and the
    table row of every new token."""

    def __init__(self, op: RotaryEmbedding, table_row: torch.Tensor):
        self.op, self.table_row = op, table_row


FUSED_ROPE = True     # RoPE fused into the append kernel; False keeps it as separate elementwise ops (tests compare the two)


class LlamaAttention(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.hidden_size = config.hidden_size
        self.num_heads = config.num_attention_heads
        self.head_dim = self.hidden_size // self.num_heads
        self.num_key_value_heads = config.num_key_value_heads
        self.q_proj = nn.Linear(self.hidden_size, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(self.hidden_size, self.num_key_value_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.hidden_size, self.hidden_size, bias=False)
        self.attention = MultiHeadAttention()

    def forward(self, hidden_states, position_embeddings, kv_cache: KVCacheBase, kv_start=None, n_new=None,
                q_lens=None):
        bsz, q_len, _ = hidden_states.size()
        q = _lin(self.q_proj, hidden_states).view(bsz, q_len, self.num_heads, self.head_dim)
        k = _lin(self.k_proj, hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim)
        v = _lin(self.v_proj, hidden_states).view(bsz, q_len, self.num_key_value_heads, self.head_dim)
        # the hot path: rotate, append, then attend over the cache (llama.py:146-165)
        if isinstance(position_embeddings, FusedRope):
            q, key_h, value_h = kv_cache.update_cache_rope(q, k, v, position_embeddings.table_row,
                                                           position_embeddings.op, n_new_per_seq=n_new)
        else:
            q, k = position_embeddings(query=q.transpose(1, 2), key=k.transpose(1, 2))
            key_h, value_h = kv_cache.update_cache(k, v.transpose(1, 2), concat_dim=2, n_new_per_seq=n_new)
        out = self.attention(q, key_h, value_h, attention_mask=None, kv_start=kv_start, q_lens=q_lens)
        out = out.transpose(1, 2).reshape(bsz, q_len, -1)
        return _lin(self.o_proj, out)

    def forward_packed(self, hidden: torch.Tensor, pk: "Packed", kv_cache: KVCacheBase) -> torch.Tensor:
        """``hidden`` [T, hidden]: the step's tokens of all sequences, back to back."""
        T = hidden.shape[0]
        pk.q[pk.bidx, pk.tidx] = self.q_proj(hidden).view(T, self.num_heads, self.head_dim)
        pk.k[pk.bidx, pk.tidx] = self.k_proj(hidden).view(T, self.num_key_value_heads, self.head_dim)
        pk.v[pk.bidx, pk.tidx] = self.v_proj(hidden).view(T, self.num_key_value_heads, self.head_dim)
        q, key_h, value_h = kv_cache.update_cache_rope(pk.q, pk.k, pk.v, pk.rope.table_row, pk.rope.op,
                                                       n_new_per_seq=pk.counts)
        out = self.attention(q, key_h, value_h, attention_mask=None, q_lens=pk.q_lens)
        return self.o_proj(out.transpose(1, 2)[pk.bidx, pk.tidx].reshape(T, -1))


class Packed:
    """One scheduler step's tokens without padding: token i of the flat list is token ``tidx[i]`` of the
    new tokens of sequence ``bidx[i]``.  The projections, norms and the MLP run on the flat list; only
    around the cache and the attention kernels (which address a sequence's rows by a batch stride)
    q, k and v are scattered into ``[B, n_max, heads, D]`` staging buffers shared by all layers."""

    def __init__(self, counts: Sequence[int], cached: Sequence[int], rope: RotaryEmbedding, cfg, device,
                 max_positions: int):
        self.counts = [int(c) for c in counts]
        B, n_max = len(self.counts), max(self.counts)
        self.n_max = n_max
        bidx = [b for b, c in enumerate(self.counts) for _ in range(c)]
        tidx = [t for c in self.counts for t in range(c)]
        self.bidx = torch.tensor(bidx, dtype=torch.long, device=device)
        self.tidx = torch.tensor(tidx, dtype=torch.long, device=device)
        base = torch.tensor(list(cached), dtype=torch.long, device=device).unsqueeze(1)
        pos = (base + torch.arange(n_max, device=device).unsqueeze(0)).clamp_(max=max_positions - 1)
        self.rope = FusedRope(rope, rope.table_rows(pos))
        self.q_lens = torch.tensor(self.counts, dtype=torch.int32, device=device)
        last, off = [], 0
        for c in self.counts:
            off += c
            if c:
                last.append(off - 1)
        self.last_rows = torch.tensor(last, dtype=torch.long, device=device)   # flat index of every live sequence's last token
        self.live = [b for b, c in enumerate(self.counts) if c]
        D = cfg.hidden_size // cfg.num_attention_heads
        self.q = torch.zeros(B, n_max, cfg.num_attention_heads, D, dtype=torch.bfloat16, device=device)
        self.k = torch.zeros(B, n_max, cfg.num_key_value_heads, D, dtype=torch.bfloat16, device=device)
        self.v = torch.zeros_like(self.k)


class LlamaDecoderLayer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.input_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)
        self.self_attn = LlamaAttention(config)
        self.mlp = LlamaMLP(config.hidden_size, config.intermediate_size)
        self.post_attention_layernorm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward(self, hidden_states, position_embeddings, kv_cache, kv_start=None, n_new=None, q_lens=None):
        h = hidden_states + self.self_attn(self.input_layernorm(hidden_states), position_embeddings, kv_cache,
                                           kv_start, n_new, q_lens)
        return h + self.mlp(self.post_attention_layernorm(h))

    def forward_packed(self, hidden, pk, kv_cache):
        h = hidden + self.self_attn.forward_packed(self.input_layernorm(hidden), pk, kv_cache)
        return h + self.mlp(self.post_attention_layernorm(h))


class LlamaModel(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size, getattr(config, "pad_token_id", None))
        self.layers = nn.ModuleList([LlamaDecoderLayer(config) for _ in range(config.num_hidden_layers)])
        self.rotary_emb = RotaryEmbedding(getattr(config, "rope_scaling", None),
                                          config.hidden_size // config.num_attention_heads,
                                          config.max_position_embeddings, config.rope_theta)
        self.norm = RMSNorm(config.hidden_size, config.rms_norm_eps)

    def forward_tokens(self, new_ids: torch.Tensor, kv_cache: KVCacheManager, position_ids: torch.Tensor,
                       kv_start: Optional[torch.Tensor] = None, n_new: Optional[Sequence[int]] = None):
        hidden = self.embed_tokens(new_ids)
        if FUSED_ROPE and hidden.dtype == torch.bfloat16:
            rope = FusedRope(self.rotary_emb, self.rotary_emb.table_rows(position_ids))
        else:
            rope = self.rotary_emb(hidden, position_ids)
        q_lens = None
        if isinstance(n_new, torch.Tensor):
            q_lens = n_new           # device-resident counts: used as they are, by the append and by the attention
        elif n_new is not None:
            q_lens = torch.tensor(list(n_new), dtype=torch.int32, device=new_ids.device)
        for idx, layer in enumerate(self.layers):
            hidden = layer(hidden, rope, kv_cache[idx], kv_start, n_new, q_lens)
        kv_cache.commit()        # deferred decode appends: one launch advances every layer (a no-op otherwise)
        return self.norm(hidden)

    def forward_packed(self, tokens: torch.Tensor, pk: "Packed", kv_cache: KVCacheManager) -> torch.Tensor:
        hidden = self.embed_tokens(tokens)
        for idx, layer in enumerate(self.layers):
            hidden = layer.forward_packed(hidden, pk, kv_cache[idx])
        kv_cache.commit()
        return self.norm(hidden)


class LlamaForCausalLM(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.model = LlamaModel(config)
        self.vocab_size = config.vocab_size
        self.lm_head = nn.Linear(config.hidden_size, config.vocab_size, bias=False)

    # -- the reference signature (llama.py:428-440) -----------------------------------------
    def forward(self, input_ids: torch.LongTensor, kv_cache: KVCacheManager, attention_mask: torch.Tensor,
                inputs_embeds=None) -> ModelOutput:
        """``input_ids`` is the whole history; what the cache already holds is sliced off
        (llama.py:284-286).  ``attention_mask`` is the 2-D 0/1 mask; zeros on the left are padding."""
        if inputs_embeds is not None:
            raise NotImplementedError("inputs_embeds is not supported")
        past = len(kv_cache)
        new_ids = input_ids[:, past:]
        mask = attention_mask.to(input_ids.device)
        position_ids = mask.long().cumsum(-1) - 1
        position_ids.masked_fill_(mask == 0, 1)
        position_ids = position_ids[:, past: past + new_ids.shape[1]]
        kv_start = None
        if bool((mask == 0).any()):
            kv_start = (mask.cumsum(-1) == 0).sum(-1).to(torch.int32)
        hidden = self.model.forward_tokens(new_ids, kv_cache, position_ids, kv_start)
        return ModelOutput(logits=_lin(self.lm_head, hidden))

    # -- ragged form used by batched speculative decoding ---------------------------------------
    def forward_ragged(self, new_ids: torch.Tensor, n_new: Sequence[int], kv_cache: KVCacheManager) -> ModelOutput:
        """``new_ids`` [B, n_max] holds, left-aligned, ``n_new[b]`` new tokens of sequence b; positions
        continue from each sequence's cached length."""
        cached = kv_cache[0].seq_lens if kv_cache[0].seq_lens else [0] * new_ids.shape[0]
        base = torch.tensor(cached, dtype=torch.long, device=new_ids.device).unsqueeze(1)
        position_ids = base + torch.arange(new_ids.shape[1], device=new_ids.device).unsqueeze(0)
        position_ids.clamp_(max=self.config.max_position_embeddings - 1)
        ragged = None if all(n == new_ids.shape[1] for n in n_new) else list(n_new)
        hidden = self.model.forward_tokens(new_ids, kv_cache, position_ids, None, ragged)
        return ModelOutput(logits=_lin(self.lm_head, hidden))


    def forward_device_ragged(self, new_ids: torch.Tensor, n_new: torch.Tensor, kv_cache: KVCacheManager,
                              slots: Optional[torch.Tensor] = None) -> ModelOutput:
        """``forward_ragged`` with the counts on the device: ``n_new`` is a CUDA int32 ``[B]`` tensor (the
        output of a kernel), positions continue from the lengths the device holds, and nothing is read
        back - the host never learns how many tokens each sequence took.  The cache must exist already
        (a prompt pass has run)."""
        pool = kv_cache.pool
        base = pool.seq_len()[0].index_select(0, kv_cache.slots_dev.long()).long().unsqueeze(1)
        position_ids = base + torch.arange(new_ids.shape[1], device=new_ids.device).unsqueeze(0)
        position_ids.clamp_(max=self.config.max_position_embeddings - 1)
        hidden = self.model.forward_tokens(new_ids, kv_cache, position_ids, None, n_new)
        return ModelOutput(logits=_lin(self.lm_head, hidden))

    # -- packed form used by continuous batching ----------------------------------------------------
    def forward_packed(self, tokens: torch.Tensor, counts: Sequence[int], kv_cache: KVCacheManager) -> ModelOutput:
        """``tokens`` [T] holds the new tokens of every sequence back to back, ``counts[b]`` of them for
        sequence b (zero for a sequence that sits this step out); positions continue from each
        sequence's cached length.  Returns the logits of the LAST new token of every sequence that had
        any, as ``[B, vocab]`` (rows of idle sequences are zero): the LM head runs on those rows only."""
        B = len(counts)
        cached = kv_cache[0].seq_lens if kv_cache[0].seq_lens else [0] * B
        pk = Packed(counts, cached, self.model.rotary_emb, self.config, tokens.device,
                    self.config.max_position_embeddings)
        hidden = self.model.forward_packed(tokens, pk, kv_cache)
        logits = torch.zeros(B, self.vocab_size, dtype=hidden.dtype, device=hidden.device)
        logits[torch.tensor(pk.live, device=hidden.device)] = self.lm_head(hidden[pk.last_rows])
        return ModelOutput(logits=logits)


def random_init_(model: nn.Module, seed: int, std: float = 0.02) -> nn.Module:
    """N(0, std) weights from a seed (norm weights stay at one): the BASELINE configs' synthetic models."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() >= 2:
                p.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))
    return model
