"""Generates tests/golden/rope_cases.pt by running the reference's own RotaryEmbedding operator
(pace/ops/rotary_embedding.py) on seeded inputs: its cos/sin caches for every rope_type it
supports and the rotated query/key tensors for NeoX and GPT-J pairing.

Run where the reference tree exists:  python tests/golden/make_golden_rope.py
TEST INFRASTRUCTURE: the vectors pin oracle/rope_ref.py and, through it, the CUDA kernel.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))

from oracle import ref_loader  # noqa: E402

CASES = [
    # name, rope_scaling, head_dim, max_pos, theta, partial_rotary_factor, extra kwargs
    ("default", {"rope_type": "default"}, 64, 160, 10000.0, 1.0, {}),
    ("default_theta5e5_d128", None, 128, 96, 500000.0, 1.0, {}),
    ("linear", {"rope_type": "linear", "scaling_factor": 2.0}, 64, 128, 10000.0, 1.0, {}),
    ("dynamic", {"rope_type": "dynamic", "scaling_factor": 2.0}, 64, 64, 10000.0, 1.0, {}),
    ("llama3", {"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                "original_max_position_embeddings": 64}, 128, 256, 500000.0, 1.0, {}),
    ("longrope", {"rope_type": "longrope", "short_factor": [1.0 + 0.05 * i for i in range(12)],
                  "long_factor": [1.0 + 0.4 * i for i in range(12)]}, 32, 128, 10000.0, 0.75,
     {"original_max_position_embeddings": 48}),
    # partial rotation (48 of 64 elements) on a head size the paged cache holds
    ("longrope_d64", {"rope_type": "longrope", "short_factor": [1.0 + 0.03 * i for i in range(24)],
                      "long_factor": [1.0 + 0.25 * i for i in range(24)], "attention_factor": 1.1}, 64, 96, 10000.0,
     0.75, {"original_max_position_embeddings": 40}),
]


def main():
    ref_loader.load()
    from pace.ops.rotary_embedding import RotaryEmbedding
    out = {}
    for name, scaling, head_dim, max_pos, theta, partial, extra in CASES:
        g = torch.Generator().manual_seed(len(name) * 131 + head_dim)
        rope = RotaryEmbedding(scaling, head_dim, max_pos, theta, partial_rotary_factor=partial, **extra)
        B, S, Hq, Hkv = 2, 5, 4, 2
        q = torch.randn(B, Hq, S, head_dim, generator=g).bfloat16()
        k = torch.randn(B, Hkv, S, head_dim, generator=g).bfloat16()
        rows = rope.cos_cache.shape[0]
        longrope = name.startswith("longrope")
        limit = max_pos if not longrope else extra["original_max_position_embeddings"]
        sets = {"short": torch.stack([torch.arange(S) + 3, torch.arange(S) + limit - S - 1])}
        if longrope:   # a position beyond the original window switches every index to the long table
            sets["long"] = torch.stack([torch.arange(S) + limit - 8, torch.arange(S) + limit + 12])
        case = {"rope_scaling": scaling, "head_dim": head_dim, "max_position_embeddings": max_pos, "rope_theta": theta,
                "partial_rotary_factor": partial, "kwargs": extra, "rotary_dim": rope.rotary_dim,
                "cos_cache": rope.cos_cache.clone(), "sin_cache": rope.sin_cache.clone(), "cache_rows": rows,
                "q": q, "k": k, "applied": {}}
        for tag, pos in sets.items():
            cos, sin = rope(q, pos, return_cos_sin=True)
            styles = [True] if longrope else [True, False]
            for neox in styles:
                qr, kr = rope.apply_rotary_emb(q, k, cos, sin, unsqueeze_dim=1, is_neox_style=neox)
                case["applied"][f"{tag}_{'neox' if neox else 'gptj'}"] = {
                    "position_ids": pos, "cos": cos, "sin": sin, "q_rot": qr, "k_rot": kr}
        out[name] = case
    torch.save(out, os.path.join(HERE, "rope_cases.pt"))
    print("wrote rope_cases.pt:", {k: tuple(v["cos_cache"].shape) for k, v in out.items()})


if __name__ == "__main__":
    main()
