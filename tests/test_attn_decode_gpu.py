"""Decode attention (one query token) over the paged cache vs the CPU oracle."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3          # parity budget for bf16 caches


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _fill(mgr, layer, ks, vs):
    """Ragged fill: ks[b] is [Hkv, L_b, D]."""
    B = len(ks)
    Lmax = max(k.shape[1] for k in ks)
    H, D = ks[0].shape[0], ks[0].shape[2]
    kp = torch.zeros(B, H, Lmax, D, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    for b in range(B):
        kp[b, :, : ks[b].shape[1]] = ks[b]
        vp[b, :, : vs[b].shape[1]] = vs[b]
    return mgr[layer].update_cache(kp, vp, concat_dim=2, n_new_per_seq=[k.shape[1] for k in ks])


def _oracle(q, ks, vs, left_pad=None, flavour="native"):
    from oracle.attention_ref import attend_over_cache
    outs = []
    for b in range(len(ks)):
        L = ks[b].shape[1]
        outs.append(attend_over_cache(q[b:b + 1].cpu(), ks[b][None].cpu(), vs[b][None].cpu(), L,
                                      0 if left_pad is None else left_pad[b], flavour)[0])
    return torch.stack(outs).float()


def _check(got, want):
    err = (got.float().cpu() - want).abs()
    assert err.max().item() < MAX_ABS, f"max-abs {err.max().item()}"
    assert err.mean().item() < MEAN_ABS, f"mean-abs {err.mean().item()}"


def test_decode_matches_reference_golden():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    case = torch.load(os.path.join(G, "decode_case.pt"))
    B = case["B"]
    mgr = KVCacheManager(Cfg(1), case["max_len"], KVCacheType.BMC)
    ks = [case["k_cache"][b][:, : case["lens"][b]].to(DEV) for b in range(B)]
    vs = [case["v_cache"][b][:, : case["lens"][b]].to(DEV) for b in range(B)]
    _fill(mgr, 0, ks, vs)
    k_new = torch.stack(case["k_new"]).to(DEV)
    v_new = torch.stack(case["v_new"]).to(DEV)
    K, V = mgr[0].update_cache(k_new, v_new, concat_dim=2)
    q = torch.stack(case["q"]).to(DEV)
    out = MultiHeadAttention()(q, K, V)
    assert out.shape == q.shape and out.dtype == torch.bfloat16
    _check(out, torch.stack(case["out"]).float())
    dk, dv = mgr[0].read_dense()
    for b in range(B):
        n = case["lens"][b] + 1
        assert torch.equal(dk[b, :, :n].cpu(), case["k_cache"][b][:, :n])
        assert torch.equal(dv[b, :, :n].cpu(), case["v_cache"][b][:, :n])
    mgr.pool.check_status()


CASES = [
    # B, Hq, Hkv, D, max_len, lens
    (4, 32, 8, 128, 1025, [128, 1024, 577, 300]),          # config-1 shape
    (1, 32, 8, 128, 64, [1]),                               # a single cached token
    (3, 8, 2, 128, 100, [9, 10, 11]),                       # page_tokens 10: one under / at / over a page
    (2, 8, 8, 64, 300, [250, 33]),                          # MHA (G=1), D=64
    (2, 16, 8, 64, 90, [64, 65]),                           # G=2
    (2, 32, 4, 128, 500, [200, 437]),                       # G=8
    (37, 8, 2, 64, 130, [1 + (7 * i) % 120 for i in range(37)]),   # more units than a CTA range holds
    (1, 8, 2, 128, 40000, [33000]),                         # one long sequence: every CTA gets a slice of it
    (2, 32, 8, 128, 9000, [8190, 4097]),                    # page_tokens 95 > 64: sub-page chunks
]


@pytest.mark.parametrize("B,Hq,Hkv,D,max_len,lens", CASES)
def test_decode_matches_oracle(B, Hq, Hkv, D, max_len, lens):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(B * 1000 + Hq + D + len(lens))
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(2), max_len, KVCacheType.BMC)
    K, V = _fill(mgr, 1, ks, vs)                      # layer 1 of 2: layer offsets are exercised
    mha = MultiHeadAttention()
    out = mha(q, K, V)
    _check(out, _oracle(q, ks, vs))
    out2 = mha(q, K, V)                               # second launch: arrival counters were reset
    assert torch.equal(out, out2)
    mgr.pool.check_status()


def test_decode_left_padding_and_transposed_query():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(5)
    B, Hq, Hkv, D = 3, 8, 2, 128
    lens, pads = [70, 70, 70], [0, 13, 69]
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    # the layout a model produces: [B, S, Hq, D] viewed as [B, Hq, S, D]
    q = torch.randn(B, 1, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(1), 128, KVCacheType.DYNAMIC)
    K, V = _fill(mgr, 0, ks, vs)
    kv_start = torch.tensor(pads, dtype=torch.int32, device=DEV)
    out = MultiHeadAttention()(q, K, V, kv_start=kv_start)
    _check(out, _oracle(q, ks, vs, left_pad=pads))
    # the same padding given the reference's way, as an additive 4-D mask
    from oracle.attention_ref import additive_mask_4d
    m2 = torch.ones(B, 70, dtype=torch.long)
    for b, p in enumerate(pads):
        m2[b, :p] = 0
    m4 = additive_mask_4d(m2, 1, 70, torch.bfloat16).to(DEV)
    out_m = MultiHeadAttention()(q, K, V, attention_mask=m4)
    assert torch.equal(out, out_m)
    mgr.pool.check_status()


def test_decode_after_rollback_ignores_stale_rows():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(6)
    B, Hq, Hkv, D, L = 2, 8, 2, 64, 50
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for _ in range(B)]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for _ in range(B)]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 100, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    mgr.remove_cache(8)
    out = MultiHeadAttention()(q, K, V)
    _check(out, _oracle(q, [k[:, :42] for k in ks], [v[:, :42] for v in vs]))
    mgr.pool.check_status()
