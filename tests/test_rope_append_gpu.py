"""RoPE fused into the K/V append (pace_kv_append_rope) against the CPU oracle, bit for bit."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

G_DIR = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _build(case):
    from pace_b200.ops import RotaryEmbedding
    return RotaryEmbedding(case["rope_scaling"], case["head_dim"], case["max_position_embeddings"], case["rope_theta"],
                           partial_rotary_factor=case["partial_rotary_factor"], **case["kwargs"])


def test_fused_rope_append_matches_reference_golden():
    """Every rope_type of the reference operator, NeoX and GPT-J pairing: the rotated queries the
    kernel returns and the rotated keys it stored equal the reference's outputs exactly."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    cases = torch.load(os.path.join(G_DIR, "rope_cases.pt"))
    assert any(n.startswith("longrope") and c["head_dim"] in (64, 128) for n, c in cases.items())
    for name, c in cases.items():
        if c["head_dim"] not in (64, 128):     # head sizes the paged cache does not hold
            continue
        for tag, a in c["applied"].items():
            rope = _build(c)
            rope.is_neox_style = tag.endswith("neox")
            q = c["q"].transpose(1, 2).contiguous().to(DEV)          # [B, S, Hq, D] as a projection leaves it
            k = c["k"].transpose(1, 2).contiguous().to(DEV)
            v = torch.randn_like(k)
            mgr = KVCacheManager(Cfg(1), 64, KVCacheType.BMC)
            rows = rope.table_rows(a["position_ids"]).to(DEV)
            q_rot, K, V = mgr[0].update_cache_rope(q.clone(), k, v, rows, rope)
            assert torch.equal(q_rot.cpu(), a["q_rot"]), (name, tag)
            dk, dv = mgr[0].read_dense()
            S = k.shape[1]
            assert torch.equal(dk[:, :, :S].cpu(), a["k_rot"]), (name, tag)
            assert torch.equal(dv[:, :, :S].cpu(), v.transpose(1, 2).cpu()), (name, tag)
            mgr.pool.check_status()


@pytest.mark.parametrize("B,S,Hq,Hkv,D,past", [(32, 1, 32, 8, 128, 519), (3, 17, 8, 2, 128, 40), (2, 70, 4, 4, 64, 0)])
def test_fused_rope_append_matches_oracle_with_history_and_ragged_counts(B, S, Hq, Hkv, D, past):
    """Appends behind an existing history, ragged counts per sequence, strided (fused-QKV) inputs."""
    from oracle import rope_ref
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import RotaryEmbedding
    g = torch.Generator().manual_seed(B * 7 + S)
    rope = RotaryEmbedding({"rope_type": "llama3", "factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                            "original_max_position_embeddings": 256}, D, 1024, 500000.0)
    mgr = KVCacheManager(Cfg(2), past + S + 8, KVCacheType.BMC)
    if past:
        old = torch.randn(B, Hkv, past, D, generator=g).bfloat16().to(DEV)
        mgr[1].update_cache(old, old.flip(1), concat_dim=2)
    counts = [max(1, S - (b % 3)) for b in range(B)]
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, generator=g).bfloat16().to(DEV)       # one fused projection output
    q = qkv[..., : Hq * D].view(B, S, Hq, D)
    k = qkv[..., Hq * D: (Hq + Hkv) * D].view(B, S, Hkv, D)
    v = qkv[..., (Hq + Hkv) * D:].view(B, S, Hkv, D)
    pos = torch.stack([torch.arange(S) + past - (b % 2) for b in range(B)]).clamp_(min=0)     # left-pad style shifts
    q_out = torch.empty(B, S, Hq, D, dtype=torch.bfloat16, device=DEV)
    q_rot, K, V = mgr[1].update_cache_rope(q, k, v, rope.table_rows(pos).to(DEV), rope, n_new_per_seq=counts,
                                           query_out=q_out)
    want_q, want_k = rope_ref.rotate(q.cpu().transpose(1, 2), k.cpu().transpose(1, 2), pos, rope.cos_cache,
                                     rope.sin_cache, rope.rotary_dim)
    dk, dv = mgr[1].read_dense()
    for b in range(B):
        n = counts[b]
        assert torch.equal(q_rot[b, :, :n].cpu(), want_q[b, :, :n])
        assert torch.equal(dk[b, :, past: past + n].cpu(), want_k[b, :, :n])
        assert torch.equal(dv[b, :, past: past + n].cpu(), v[b, :n].transpose(0, 1).cpu())
        if past:
            assert torch.equal(dk[b, :, :past], old[b])
    assert list(mgr[1].seq_lens) == [past + n for n in counts]
    mgr.pool.check_status()


def test_fused_rope_error_surface():
    from pace_b200 import _C
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import RotaryEmbedding
    rope = RotaryEmbedding(None, 128, 64, 10000.0)
    mgr = KVCacheManager(Cfg(1), 32, KVCacheType.BMC)
    q = torch.zeros(1, 2, 4, 128, dtype=torch.bfloat16, device=DEV)
    k = torch.zeros(1, 2, 2, 128, dtype=torch.bfloat16, device=DEV)
    rows = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    with pytest.raises(TypeError):
        mgr[0].update_cache_rope(q.float(), k, k, rows, rope)
    with pytest.raises(ValueError):
        mgr[0].update_cache_rope(q, k, k, rows.long(), rope)
    with pytest.raises(ValueError):
        mgr[0].update_cache_rope(q[..., 1:], k, k, rows, rope)          # rows no longer 16-byte aligned
    # a table row outside the table: sticky device status, the token passes through unrotated
    bad = torch.tensor([[0, 64]], dtype=torch.int32, device=DEV)
    q1 = torch.randn(1, 2, 4, 128, device=DEV).bfloat16()
    out, _, _ = mgr[0].update_cache_rope(q1.clone(), k, k, bad, rope)
    assert torch.equal(out[0, :, 1], q1[0, 1])
    with pytest.raises(_C.PaceError):
        mgr.pool.check_status()


def test_back_to_back_appends_to_different_layers_keep_their_lengths():
    """Appends to different layers launched with nothing in between may overlap on the GPU
    (programmatic dependent launch); every layer must still advance its own lengths exactly once."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import RotaryEmbedding
    L, B, Hq, Hkv, D = 8, 32, 32, 8, 128
    rope = RotaryEmbedding(None, D, 4096, 10000.0)
    mgr = KVCacheManager(Cfg(L), 600, KVCacheType.BMC)
    q = torch.randn(B, 1, Hq, D, device=DEV).bfloat16()
    k = torch.randn(B, 1, Hkv, D, device=DEV).bfloat16()
    for step in range(40):
        rows = torch.full((B, 1), step, dtype=torch.int32, device=DEV)
        for l in range(L):
            if step % 2:
                mgr[l].update_cache_rope(q, k, k, rows, rope, query_out=torch.empty_like(q))
            else:
                mgr[l].update_cache(k.transpose(1, 2), k.transpose(1, 2), concat_dim=2)
    torch.cuda.synchronize()
    mgr.pool.check_status()
    lens = mgr.pool.seq_len().cpu()
    assert bool((lens[:L, :B] == 40).all()), lens[:L, :B]
