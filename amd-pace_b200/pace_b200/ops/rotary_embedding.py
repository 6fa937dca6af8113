"""RotaryEmbedding operator: the reference's front end (pace/ops/rotary_embedding.py:202-485) with
the same constructor arguments, buffers and ``forward`` contract, plus what the fused CUDA path
needs: the table row of every position as an int32 tensor and the fp32 tables on the device.

On the hot path the rotation is not done here: ``KVCacheBase.update_cache_rope`` hands the tables to
``pace_kv_append_rope``, which rotates q and k while it appends k and v (one kernel instead of the
reference's index_select + eight elementwise ops + the append).  ``forward`` keeps the reference's
two return forms for callers that rotate outside the cache.
"""
import math
from functools import partial
from typing import Any, Callable, Dict, Optional, Tuple, Union

import torch
from torch import nn


def _frequencies(theta: float, rotary_dim: int, divide_by=None) -> torch.Tensor:
    exponents = torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim
    freq = theta ** exponents
    if divide_by:
        freq = torch.tensor(divide_by, dtype=torch.float32) * freq
    return 1.0 / freq


def _tables(freq: torch.Tensor, n_rows, gain: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    angle = torch.einsum("i,j -> ij", torch.arange(n_rows, dtype=torch.float), freq)
    return angle.cos() * gain, angle.sin() * gain


class RotaryEmbedding(nn.Module):
    """``rope_scaling`` selects the variant through ``rope_type`` (or the older ``type``) key:
    ``default``, ``linear`` (``scaling_factor``), ``dynamic`` (NTK, ``scaling_factor``), ``llama3``
    (``factor``, ``low_freq_factor``, ``high_freq_factor``, ``original_max_position_embeddings``) and
    ``longrope`` (``short_factor``, ``long_factor``, optional ``attention_factor``; keyword
    ``original_max_position_embeddings``).  Tables are fp32 ``[rows, rotary_dim / 2]``."""

    def __init__(self, rope_scaling: Optional[Dict[str, Any]], rotary_dim: int, max_position_embeddings: int,
                 rope_theta: float, partial_rotary_factor: float = 1.0, dtype: Optional[torch.dtype] = None,
                 backend_impl=None, is_neox_style: bool = True, **rope_kwargs):
        super().__init__()
        if partial_rotary_factor < 1.0:
            rotary_dim = int(rotary_dim * partial_rotary_factor)
        self.rotary_dim = rotary_dim
        self.partial_rotary_factor = partial_rotary_factor
        self.rope_kwargs = rope_kwargs
        self.rope_scaling = rope_scaling
        self.rope_type = "default" if rope_scaling is None else rope_scaling.get("rope_type", rope_scaling.get("type"))
        self.max_position_embeddings = max_position_embeddings
        self.rope_theta = rope_theta
        self.is_neox_style = is_neox_style
        self.original_max_position_embeddings = None
        kind, R, N = self.rope_type, rotary_dim, max_position_embeddings
        if kind == "default":
            cos, sin = _tables(_frequencies(rope_theta, R), N)
        elif kind == "linear":
            # (the reference scales cos and sin themselves by the factor, rotary_embedding.py:124-136)
            cos, sin = _tables(_frequencies(rope_theta, R), N, rope_scaling["scaling_factor"])
        elif kind == "dynamic":
            f = rope_scaling["scaling_factor"]
            rows = N * f
            theta = rope_theta * ((f * rows / N) - (f - 1)) ** (R / (R - 2))
            cos, sin = _tables(_frequencies(theta, R), rows)
        elif kind == "llama3":
            f, lo, hi = rope_scaling["factor"], rope_scaling["low_freq_factor"], rope_scaling["high_freq_factor"]
            window = rope_scaling["original_max_position_embeddings"]
            base = _frequencies(rope_theta, R)
            wavelength = 2 * math.pi / base
            blend = (window / wavelength - lo) / (hi - lo) if lo != hi else 0
            mixed = (1 - blend) * base / f + blend * base
            freq = torch.where(wavelength < window / hi, base, torch.where(wavelength > window / lo, base / f, mixed))
            cos, sin = _tables(freq, N)
        elif kind == "longrope":
            window = rope_kwargs.get("original_max_position_embeddings", N)
            self.original_max_position_embeddings = window
            ratio = N / window
            gain = 1.0 if ratio <= 1.0 else math.sqrt(1 + math.log(ratio) / math.log(window))
            if rope_scaling.get("attention_factor") is not None:
                gain = rope_scaling["attention_factor"]
            short = _tables(_frequencies(rope_theta, R, rope_scaling["short_factor"]), window, gain)
            long = _tables(_frequencies(rope_theta, R, rope_scaling["long_factor"]), N, gain)
            cos, sin = torch.cat([short[0], long[0]]), torch.cat([short[1], long[1]])
        else:
            raise ValueError(f"Unsupported RoPE type: {kind}")
        self.register_buffer("cos_cache", cos.contiguous(), persistent=False)
        self.register_buffer("sin_cache", sin.contiguous(), persistent=False)
        self._device_tables = {}

    # ---- what the fused kernel takes ----------------------------------------------------------
    def table_rows(self, position_ids: torch.Tensor, offsets: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Row of the tables each position reads, int32 and contiguous (rotary_embedding.py:382-396:
        longrope moves every index to the long table as soon as one position leaves the original window)."""
        idx = position_ids
        if self.rope_type == "longrope":
            k = self.original_max_position_embeddings
            idx = idx + (torch.any(position_ids > k).to(idx.dtype) * k)
            if offsets is not None:
                idx = idx + offsets
        return idx.to(torch.int32).contiguous()

    def device_tables(self, device) -> Tuple[torch.Tensor, torch.Tensor]:
        key = str(torch.device(device))
        if key not in self._device_tables:
            self._device_tables[key] = (self.cos_cache.to(device=device, dtype=torch.float32).contiguous(),
                                        self.sin_cache.to(device=device, dtype=torch.float32).contiguous())
        return self._device_tables[key]

    # ---- the reference's forward contract -------------------------------------------------------
    def forward(self, x: torch.Tensor, position_ids: torch.Tensor, return_cos_sin: bool = False,
                offsets: Optional[torch.Tensor] = None) -> Union[Callable, Tuple[torch.Tensor, torch.Tensor]]:
        rows = self.table_rows(position_ids, offsets).long().flatten()
        cos = self.cos_cache.to(x.device).index_select(0, rows).unflatten(0, position_ids.shape).to(x.dtype)
        sin = self.sin_cache.to(x.device).index_select(0, rows).unflatten(0, position_ids.shape).to(x.dtype)
        if return_cos_sin:
            return cos, sin
        return partial(self.apply_rotary_emb, cos=cos, sin=sin, unsqueeze_dim=1)

    def _rotate(self, x, cos, sin, unsqueeze_dim, is_neox_style):
        cos, sin = cos.unsqueeze(unsqueeze_dim), sin.unsqueeze(unsqueeze_dim)
        R = self.rotary_dim
        turn, keep = x[..., :R], x[..., R:]
        if is_neox_style:
            a, b = turn[..., : R // 2], turn[..., R // 2:]
        else:
            a, b = turn[..., ::2], turn[..., 1::2]
        ra, rb = a * cos - b * sin, b * cos + a * sin
        turned = torch.cat((ra, rb), dim=-1) if is_neox_style else torch.stack((ra, rb), dim=-1).flatten(-2)
        return torch.cat((turned, keep), dim=-1) if keep.shape[-1] else turned

    def apply_rotary_emb(self, query, key, cos, sin, unsqueeze_dim: int = 1, is_neox_style: Optional[bool] = None):
        """query / key ``[B, heads, S, D]``, cos / sin ``[B, S, rotary_dim / 2]`` in their dtype."""
        style = self.is_neox_style if is_neox_style is None else is_neox_style
        return self._rotate(query, cos, sin, unsqueeze_dim, style), self._rotate(key, cos, sin, unsqueeze_dim, style)

    def extra_repr(self):
        return (f"rope_type={self.rope_type}, rotary_dim={self.rotary_dim}, "
                f"max_position_embeddings={self.max_position_embeddings}, rope_theta={self.rope_theta}")
