"""CPU restatement of the reference's rotary position embedding (RoPE) for the step in front of
the K/V append.  TEST INFRASTRUCTURE ONLY: imported by tests/, __graft_entry__.smoke() and the CPU
baseline leg of bench.py, never by the product path.

Follows pace/ops/rotary_embedding.py of the reference:
  * cos/sin tables are fp32, one row per position, rotary_dim / 2 columns         (:88-107)
  * "default"  inv_freq = 1 / theta^(2i / rotary_dim)                              (:65-85, :110-121)
  * "linear"   same frequencies, cos and sin multiplied by the scaling factor      (:124-136)
  * "dynamic"  NTK: theta rescaled for a window of max_pos * factor positions      (:139-155)
  * "llama3"   per-frequency interpolation between f and f / factor                (:158-193)
  * "longrope" per-frequency rescale factors, a short and a long table stacked     (:196-206, :324-361)
  * forward: rows picked by position id (longrope: shifted to the long table when any position
    lies beyond the original window), cast to the activations' dtype                (:375-404)
  * application in the activations' dtype, NeoX halves or GPT-J pairs; every product and every
    sum is rounded to that dtype, as torch's bf16 elementwise ops do               (:413-441)

Pinned by tests/golden/rope_cases.pt (outputs of the reference operator itself).
"""
import math
from typing import Dict, Optional, Tuple

import torch


def inv_freq(theta: float, rotary_dim: int, rescale=None) -> torch.Tensor:
    r = torch.tensor(rescale, dtype=torch.float32) if rescale else 1
    return 1.0 / (r * (theta ** (torch.arange(0, rotary_dim, 2, dtype=torch.float) / rotary_dim)))


def tables_from(freq: torch.Tensor, rows, factor: float = 1.0) -> Tuple[torch.Tensor, torch.Tensor]:
    t = torch.arange(rows, dtype=torch.float)
    ang = torch.einsum("i,j -> ij", t, freq)
    return ang.cos() * factor, ang.sin() * factor


def build_tables(rope_scaling: Optional[Dict], rotary_dim: int, max_pos: int, theta: float,
                 partial_rotary_factor: float = 1.0, **kwargs):
    """Returns (cos, sin, rotary_dim, rope_type, original_window) as the reference's constructor
    leaves them (rotary_embedding.py:256-368)."""
    if partial_rotary_factor < 1.0:
        rotary_dim = int(rotary_dim * partial_rotary_factor)
    kind = "default" if rope_scaling is None else rope_scaling.get("rope_type", rope_scaling.get("type"))
    window = None
    if kind == "default":
        cos, sin = tables_from(inv_freq(theta, rotary_dim), max_pos)
    elif kind == "linear":
        cos, sin = tables_from(inv_freq(theta, rotary_dim), max_pos, rope_scaling["scaling_factor"])
    elif kind == "dynamic":
        f = rope_scaling["scaling_factor"]
        max_len = max_pos * f
        base = theta * ((f * max_len / max_pos) - (f - 1)) ** (rotary_dim / (rotary_dim - 2))
        cos, sin = tables_from(inv_freq(base, rotary_dim), max_len)
    elif kind == "llama3":
        f, lo, hi = rope_scaling["factor"], rope_scaling["low_freq_factor"], rope_scaling["high_freq_factor"]
        orig = rope_scaling["original_max_position_embeddings"]
        fr = inv_freq(theta, rotary_dim)
        wave = 2 * math.pi / fr
        smooth = (orig / wave - lo) / (hi - lo) if lo != hi else 0
        fr = torch.where(wave < orig / hi, fr,
                         torch.where(wave > orig / lo, fr / f, (1 - smooth) * fr / f + smooth * fr))
        cos, sin = tables_from(fr, max_pos)
    elif kind == "longrope":
        window = kwargs.get("original_max_position_embeddings", max_pos)
        scale = max_pos / window
        factor = 1.0 if scale <= 1.0 else math.sqrt(1 + math.log(scale) / math.log(window))
        if rope_scaling.get("attention_factor") is not None:
            factor = rope_scaling["attention_factor"]
        sc, ss = tables_from(inv_freq(theta, rotary_dim, rope_scaling["short_factor"]), window, factor)
        lc, ls = tables_from(inv_freq(theta, rotary_dim, rope_scaling["long_factor"]), max_pos, factor)
        cos, sin = torch.cat([sc, lc]), torch.cat([ss, ls])
    else:
        raise ValueError(f"unsupported rope type {kind}")
    return cos, sin, rotary_dim, kind, window


def table_rows(position_ids: torch.Tensor, kind: str, window: Optional[int]) -> torch.Tensor:
    """Row of the table each position reads (rotary_embedding.py:382-396)."""
    if kind == "longrope":
        shift = (torch.any(position_ids > window).float() * torch.full_like(position_ids, window)).long()
        return position_ids + shift
    return position_ids


def apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary_dim: int, neox: bool = True) -> torch.Tensor:
    """x [B, H, S, D]; cos/sin [B, S, rotary_dim / 2] already in x's dtype.  Each elementwise op
    rounds to x's dtype (rotary_embedding.py:406-441)."""
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    rot, rest = x[..., :rotary_dim], x[..., rotary_dim:]
    if neox:
        x1, x2 = rot[..., : rotary_dim // 2], rot[..., rotary_dim // 2:]
    else:
        x1, x2 = rot[..., ::2], rot[..., 1::2]
    o1 = x1 * c - x2 * s
    o2 = x2 * c + x1 * s
    out = torch.cat((o1, o2), dim=-1) if neox else torch.stack((o1, o2), dim=-1).flatten(-2)
    return torch.cat((out, rest), dim=-1)


def rotate(q: torch.Tensor, k: torch.Tensor, position_ids: torch.Tensor, cos_t: torch.Tensor, sin_t: torch.Tensor,
           rotary_dim: int, kind: str = "default", window: Optional[int] = None, neox: bool = True):
    rows = table_rows(position_ids, kind, window).flatten()
    cos = cos_t.index_select(0, rows).unflatten(0, position_ids.shape).to(q.dtype)
    sin = sin_t.index_select(0, rows).unflatten(0, position_ids.shape).to(q.dtype)
    return apply(q, cos, sin, rotary_dim, neox), apply(k, cos, sin, rotary_dim, neox)
