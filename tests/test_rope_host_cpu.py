"""Host side of the fused RoPE + append: the RotaryEmbedding operator's tables, table rows and
torch-level rotation against the vectors recorded from the reference operator (no GPU needed)."""
import os

import torch

G_DIR = os.path.join(os.path.dirname(__file__), "golden")


def _cases():
    return torch.load(os.path.join(G_DIR, "rope_cases.pt"))


def _build(c):
    from pace_b200.ops import RotaryEmbedding
    return RotaryEmbedding(c["rope_scaling"], c["head_dim"], c["max_position_embeddings"], c["rope_theta"],
                           partial_rotary_factor=c["partial_rotary_factor"], **c["kwargs"])


def test_operator_tables_equal_the_reference_tables():
    for name, c in _cases().items():
        rope = _build(c)
        assert rope.rotary_dim == c["rotary_dim"], name
        assert torch.equal(rope.cos_cache, c["cos_cache"]) and torch.equal(rope.sin_cache, c["sin_cache"]), name


def test_operator_forward_contract_and_table_rows():
    for name, c in _cases().items():
        rope = _build(c)
        for tag, a in c["applied"].items():
            pos = a["position_ids"]
            cos, sin = rope(c["q"], pos, return_cos_sin=True)
            assert torch.equal(cos, a["cos"]) and torch.equal(sin, a["sin"]), (name, tag)
            rows = rope.table_rows(pos)
            assert rows.dtype == torch.int32 and rows.shape == pos.shape
            assert torch.equal(rope.cos_cache.index_select(0, rows.long().flatten()).to(torch.bfloat16),
                               a["cos"].flatten(0, 1)), (name, tag)
            q, k = rope(c["q"], pos)(query=c["q"], key=c["k"]) if tag.endswith("neox") else \
                rope.apply_rotary_emb(c["q"], c["k"], cos, sin, is_neox_style=False)
            assert torch.equal(q, a["q_rot"]) and torch.equal(k, a["k_rot"]), (name, tag)


def test_longrope_switches_tables_only_beyond_the_original_window():
    c = _cases()["longrope_d64"]
    rope = _build(c)
    k = c["kwargs"]["original_max_position_embeddings"]
    inside = torch.tensor([[0, 5, k]])
    assert torch.equal(rope.table_rows(inside), inside.to(torch.int32))
    beyond = torch.tensor([[0, 5, k + 1]])
    assert torch.equal(rope.table_rows(beyond), (beyond + k).to(torch.int32))
