"""Tensor-core attention (verify / prefill / dense op / packed-GQA decode) vs the CPU oracle."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

G_DIR = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3          # parity budget for bf16 caches


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _fill(mgr, layer, ks, vs):
    B = len(ks)
    Lmax = max(k.shape[1] for k in ks)
    H, D = ks[0].shape[0], ks[0].shape[2]
    kp = torch.zeros(B, H, Lmax, D, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    for b in range(B):
        kp[b, :, : ks[b].shape[1]] = ks[b]
        vp[b, :, : vs[b].shape[1]] = vs[b]
    return mgr[layer].update_cache(kp, vp, concat_dim=2, n_new_per_seq=[k.shape[1] for k in ks])


def _oracle(q, ks, vs, left_pad=None, q_lens=None):
    """q [B,Hq,S,D]; the S (or q_lens[b]) newest cached tokens are the queries' own."""
    from oracle.attention_ref import attend_over_cache
    outs = []
    for b in range(len(ks)):
        L = ks[b].shape[1]
        s = q.shape[2] if q_lens is None else q_lens[b]
        o = attend_over_cache(q[b:b + 1, :, :s].cpu(), ks[b][None].cpu(), vs[b][None].cpu(), L,
                              0 if left_pad is None else left_pad[b], "native")[0].float()
        outs.append(o)
    return outs


def _check(got, want):
    err = (got.float().cpu() - want).abs()
    assert err.max().item() < MAX_ABS, f"max-abs {err.max().item()}"
    assert err.mean().item() < MEAN_ABS, f"mean-abs {err.mean().item()}"


def test_verify_matches_reference_golden():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    case = torch.load(os.path.join(G_DIR, "verify_case.pt"))
    B, S = case["B"], case["S"]
    mgr = KVCacheManager(Cfg(1), case["max_len"], KVCacheType.BMC)
    ks = [case["k_cache"][b][:, : case["lens"][b]].to(DEV) for b in range(B)]
    vs = [case["v_cache"][b][:, : case["lens"][b]].to(DEV) for b in range(B)]
    _fill(mgr, 0, ks, vs)
    K, V = mgr[0].update_cache(torch.stack(case["k_new"]).to(DEV), torch.stack(case["v_new"]).to(DEV), concat_dim=2)
    q = torch.stack(case["q"]).to(DEV)
    kv_start = torch.tensor(case["left_pad"], dtype=torch.int32, device=DEV)
    out = MultiHeadAttention()(q, K, V, kv_start=kv_start)
    assert out.shape == q.shape
    _check(out, torch.stack(case["out"]).float())
    dk, dv = mgr[0].read_dense()
    for b in range(B):
        n = case["lens"][b] + S
        assert torch.equal(dk[b, :, :n].cpu(), case["k_cache"][b][:, :n])
    mgr.pool.check_status()


CASES = [
    # B, Hq, Hkv, D, max_len, lens (query tokens included), S
    (16, 32, 8, 128, 1200, [1033] * 16, 9),                 # PARD verify, config-4 target shape
    (4, 32, 8, 64, 1200, [1033, 900, 77, 9], 9),            # draft-model head_dim
    (2, 8, 2, 128, 300, [5, 250], 5),                       # M = 20: 2 x 4 warp grid
    (2, 8, 2, 128, 300, [2, 250], 2),                       # M = 8: packed into one tile
    (3, 8, 8, 64, 200, [40, 13, 199], 13),                  # MHA (G = 1)
    (2, 16, 2, 128, 400, [130, 399], 33),                   # M = 264: several query tiles
    (2, 32, 8, 128, 2100, [512, 1536], 512),                # a 512-token prefill chunk (first chunk / with past)
    (1, 8, 2, 64, 700, [601], 130),                         # prefill, D = 64
    (1, 8, 2, 128, 40000, [20000], 9),                      # long context: unit split over many CTAs
    (2, 32, 8, 128, 9000, [8190, 4097], 9),                 # page_tokens 94 > 64: sub-page chunks
    # 128-row tiles (tcgen05 variant): unit parts of one and two chunks, a last tile of 24 live rows
    (1, 32, 8, 128, 300, [70], 70),
    (2, 16, 16, 64, 1500, [1400, 129], 128),                # MHA, D = 64, exactly one full tile per head
    (1, 8, 2, 128, 20000, [16000], 64),                     # two tiles over a long cache: units cut across many CTAs
    (3, 32, 8, 128, 700, [640, 65, 300], 65),               # 260 rows: three tiles, lengths around chunk boundaries
]


@pytest.mark.parametrize("B,Hq,Hkv,D,max_len,lens,S", CASES)
def test_multi_query_matches_oracle(B, Hq, Hkv, D, max_len, lens, S):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(B * 1000 + Hq + D + S)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    # model layout: [B, S, Hq, D] storage viewed as [B, Hq, S, D]
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(2), max_len, KVCacheType.BMC)
    K, V = _fill(mgr, 1, ks, vs)
    mha = MultiHeadAttention()
    out = mha(q, K, V)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    assert torch.equal(out, mha(q, K, V))
    mgr.pool.check_status()


def test_ragged_query_counts_and_left_padding():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(77)
    B, Hq, Hkv, D, S = 3, 8, 2, 128, 9
    lens, q_lens, pads = [100, 64, 37], [9, 4, 1], [0, 11, 30]
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, S, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 128, KVCacheType.DYNAMIC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, kv_start=torch.tensor(pads, dtype=torch.int32, device=DEV),
                               q_lens=torch.tensor(q_lens, dtype=torch.int32, device=DEV))
    want = _oracle(q, ks, vs, left_pad=pads, q_lens=q_lens)
    for b in range(B):
        _check(out[b, :, : q_lens[b]], want[b])
    mgr.pool.check_status()


def test_large_tiles_ragged_counts_and_left_padding():
    """Ragged query counts and left pads on 128-row tiles (the tcgen05 variant's masking paths)."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(78)
    B, Hq, Hkv, D, S = 3, 16, 4, 128, 48                      # 192 rows per kv head
    lens, q_lens, pads = [300, 64, 140], [48, 17, 1], [0, 11, 70]
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(1), 320, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, kv_start=torch.tensor(pads, dtype=torch.int32, device=DEV),
                               q_lens=torch.tensor(q_lens, dtype=torch.int32, device=DEV))
    want = _oracle(q, ks, vs, left_pad=pads, q_lens=q_lens)
    for b in range(B):
        _check(out[b, :, : q_lens[b]], want[b])
    mgr.pool.check_status()


@pytest.mark.parametrize("D,Hq,Hkv,S,lens,q_lens,pads", [
    # 256-row units (two 128-row tiles share every K/V chunk): ragged query counts, left pads, a last unit whose
    # second tile is empty (q_len 70 x G 4 = 280 rows), a sequence with a single query token
    (128, 16, 4, 160, [700, 170, 330, 160], [160, 70, 1, 160], [0, 23, 100, 0]),
    # head_dim 64, G = 8: 130 tokens = 1040 rows = four full units and 16 rows
    (64, 16, 2, 130, [600, 131], [130, 97], [5, 0]),
    # MHA (G = 1), exactly 256 rows, lengths at chunk boundaries
    (128, 4, 4, 256, [256, 320, 1024], [256, 256, 64], [0, 64, 0]),
])
def test_wide_units_ragged_counts_and_left_padding(D, Hq, Hkv, S, lens, q_lens, pads):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(D + S + Hq)
    B = len(lens)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(1), max(lens) + 64, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    mha = MultiHeadAttention()
    kw = dict(kv_start=torch.tensor(pads, dtype=torch.int32, device=DEV),
              q_lens=torch.tensor(q_lens, dtype=torch.int32, device=DEV))
    out = mha(q, K, V, **kw)
    want = _oracle(q, ks, vs, left_pad=pads, q_lens=q_lens)
    for b in range(B):
        _check(out[b, :, : q_lens[b]], want[b])
    # the same launch on a share of the GPU (units cut across few thread blocks, the cross-block merge of
    # 256-row records) gives the same numbers within the parity budget
    for ctas in (1, 5, 37):
        part = mha(q, K, V, max_ctas=ctas, **kw)
        for b in range(B):
            _check(part[b, :, : q_lens[b]], want[b])
    mgr.pool.check_status()


def test_batch_larger_than_one_launch_on_unlisted_slots():
    """260 sequences x 5 query tiles are more work items than one launch takes: the batch goes out in two
    launches, and on a manager that owns its pool (slots 0..B-1, no slot list is passed) the second
    launch has to start at slot 204, not at slot 0."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    B, Hq, Hkv, D, S = 260, 8, 2, 128, 160
    g = torch.Generator().manual_seed(260)
    lens = [S + (7 * b) % 60 for b in range(B)]
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(1), 256, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    assert mgr.identity_slots
    out = MultiHeadAttention()(q, K, V)
    for b in (0, 1, 203, 204, 205, 259):
        _check(out[b], _oracle(q[b:b + 1], ks[b:b + 1], vs[b:b + 1])[0])
    mgr.pool.check_status()


@pytest.mark.parametrize("grid", [1, 5, 37])
def test_prefill_tiles_under_other_partitions(grid):
    """The same prefill chunk with the chunk stream cut for 1, 5 and 37 CTAs (cut units, partial
    merges across CTAs) on 128-row tiles."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(grid)
    B, Hq, Hkv, D, S = 2, 16, 4, 128, 96
    lens = [777, 96]
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, S, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
    mgr = KVCacheManager(Cfg(1), 800, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, max_ctas=grid)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


@pytest.mark.parametrize("impl", ["mma", "cuda"])
@pytest.mark.parametrize("B,Hq,Hkv,D,max_len,lens", [
    (4, 32, 8, 128, 1025, [128, 1024, 577, 300]),
    (32, 32, 8, 128, 768, [513 + i for i in range(32)]),
    (3, 8, 2, 64, 100, [9, 10, 11]),
    (1, 8, 2, 128, 40000, [33000]),
    (2, 32, 4, 128, 500, [200, 437]),
])
def test_decode_kernels_agree_with_oracle(impl, B, Hq, Hkv, D, max_len, lens):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator().manual_seed(B + Hq + D)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), max_len, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, decode_kernel=impl)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


@pytest.mark.parametrize("Hq,Hkv,D", [(24, 8, 128), (12, 2, 64), (32, 2, 128), (64, 2, 64), (6, 2, 128)])
@pytest.mark.parametrize("tps", [False, True])
def test_decode_group_sizes_without_a_cuda_core_kernel(monkeypatch, Hq, Hkv, D, tps):
    """Groups of 3, 6, 16 and 32 query heads per KV head (the CUDA-core kernel is built for 1, 2, 4
    and 8 only): pace_attn_decode sends them to the tensor-core kernels, 17 and more rows as several
    16-row tiles.  Both page modes."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    if tps:
        monkeypatch.setenv("PACE_KV_PAGE_TOKENS", "tps")
    lens = [5, 64, 333, 130]
    B = len(lens)
    g = torch.Generator().manual_seed(Hq * 7 + D)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 400, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


@pytest.mark.parametrize("lens", [[128, 1024, 577, 300], [40 + 17 * i for i in range(48)]])
def test_decode_whole_units_flag_on_ragged_lengths(lens):
    """PACE_ATTN_WHOLE_UNITS only changes the schedule: forced on a ragged batch (where the host
    would not set it) the result is the oracle's."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    B, Hq, Hkv, D = len(lens), 32, 8, 128
    g = torch.Generator().manual_seed(B)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), max(lens) + 1, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, whole_units=True)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


def test_decode_early_copies_short_and_empty_sequences():
    """Whole-unit decode on 64-token pages sends the copies of a unit's first pages before it knows the
    length: sequences of less than that many pages (copies received and dropped), of exactly a page,
    and sequences rolled back to nothing (zeros out) all give the oracle's rows."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    lens = [1, 63, 64, 65, 128, 129, 191, 192, 300, 2]
    B, Hq, Hkv, D = len(lens), 32, 8, 128
    g = torch.Generator().manual_seed(11)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 4096, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    assert mgr.pool.page_tokens == 64
    mha = MultiHeadAttention()
    out = mha(q, K, V, whole_units=True)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    # roll two sequences back to nothing: their rows come out as zeros, the others are unchanged
    mgr.remove_cache([1, 0, 0, 0, 0, 0, 0, 0, 0, 2])
    out2 = mha(q, K, V, whole_units=True)
    torch.cuda.synchronize()
    assert torch.count_nonzero(out2[0]) == 0 and torch.count_nonzero(out2[9]) == 0
    for b in range(1, 9):
        assert torch.equal(out2[b], out[b])
    mgr.pool.check_status()


def test_decode_eight_warp_ctas():
    """PACE_ATTN_ONE_CTA_PER_SM: decode on eight-warp thread blocks, one per SM (the form used when the
    workspace or the shared memory has no room for two four-warp blocks per SM)."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    lens = [513 + 3 * i for i in range(32)]
    B, Hq, Hkv, D = len(lens), 32, 8, 128
    g = torch.Generator().manual_seed(77)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 768, KVCacheType.BMC)
    K, V = _fill(mgr, 0, ks, vs)
    out = MultiHeadAttention()(q, K, V, one_cta_per_sm=True)
    want = _oracle(q, ks, vs)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


def test_layers_alternating_whole_units_and_cut_units(monkeypatch):
    """[append, decode attention] for layer after layer with nothing between the launches, every
    other attention launch told to keep units whole: the append behind such a launch does not wait
    for it, the one behind a launch that may use the workspace does.  Every layer's output over
    several steps is the oracle's."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    from pace_b200.ops.backends import b200
    L, B, Hq, Hkv, D, steps = 6, 8, 32, 8, 128, 5
    lens = [300 + 40 * b for b in range(B)]
    g = torch.Generator().manual_seed(5)
    ks = [[torch.randn(Hkv, n, D, generator=g).bfloat16().to(DEV) for n in lens] for _ in range(L)]
    vs = [[torch.randn(Hkv, n, D, generator=g).bfloat16().to(DEV) for n in lens] for _ in range(L)]
    mgr = KVCacheManager(Cfg(L), max(lens) + steps + 1, KVCacheType.BMC)
    for l in range(L):
        _fill(mgr, l, ks[l], vs[l])
    new = torch.randn(steps, L, B, 2 * Hkv + Hq, 1, D, generator=g).bfloat16().to(DEV)
    outs = torch.empty(steps, L, B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    mha = MultiHeadAttention()
    flip = {"n": 0}

    def every_other(*a, **k):
        flip["n"] += 1
        return flip["n"] % 2 == 1

    monkeypatch.setattr(b200, "even_lengths", every_other)
    for t in range(steps):
        for l in range(L):
            K, V = mgr[l].update_cache(new[t, l, :, :Hkv], new[t, l, :, Hkv:2 * Hkv], concat_dim=2)
            mha(new[t, l, :, 2 * Hkv:], K, V, out=outs[t, l])
    torch.cuda.synchronize()
    mgr.pool.check_status()
    for l in (0, 3, 5):
        kk = [torch.cat([ks[l][b]] + [new[t, l, b, :Hkv, 0][:, None] for t in range(steps)], dim=1) for b in range(B)]
        vv = [torch.cat([vs[l][b]] + [new[t, l, b, Hkv:2 * Hkv, 0][:, None] for t in range(steps)], dim=1) for b in range(B)]
        for t in (0, steps - 1):
            n_t = [lens[b] + t + 1 for b in range(B)]
            want = _oracle(new[t, l, :, 2 * Hkv:], [kk[b][:, :n_t[b]] for b in range(B)], [vv[b][:, :n_t[b]] for b in range(B)])
            for b in range(B):
                _check(outs[t, l, b], want[b])


# ---- the dense form: the reference custom op's operands (reference tests/ops/test_sdpa.py:79-127) ----
@pytest.mark.parametrize("B,N,S,H,L", [(1, 1, 1, 64, 1), (2, 16, 1, 128, 512), (2, 16, 128, 64, 512),
                                       (1, 32, 128, 128, 2048), (3, 4, 7, 128, 33), (32, 1, 1, 64, 512)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_dense_op_matches_reference_restatements(B, N, S, H, L, dtype):
    from pace_b200.ops import MultiHeadAttention
    from oracle.attention_ref import sdpa_native, sdpa_jit_restated
    g = torch.Generator().manual_seed(B + N + S + H + L)
    q = torch.randn(B, N, S, H, generator=g).to(dtype)
    k = torch.randn(B, N, L, H, generator=g).to(dtype)
    v = torch.randn(B, N, L, H, generator=g).to(dtype)
    m = torch.randn(B, 1, 1, L, generator=g).to(dtype)
    out = MultiHeadAttention()(q.to(DEV), k.to(DEV), v.to(DEV), attention_mask=m.to(DEV))
    assert out.dtype == dtype and out.shape == q.shape
    # bf16 inputs are what the kernel computes on, so the fp32 case is compared at bf16 precision.
    # Against NATIVE (fp32 accumulation over bf16 operands, the arithmetic of this kernel): the parity
    # budget of the paged tests, 2e-2 / 2e-3.
    qb, kb, vb, mb = (t.bfloat16() for t in (q, k, v, m))
    _check(out, sdpa_native(qb, kb, vb, mb).float())
    # Against the restatement of the JIT flavour, which rounds the [S, L] scores and the probabilities to bf16
    # as that back end's four primitives do (attention_kernels.cpp:218-257): those two roundings alone put it
    # up to 2e-2 away from NATIVE, so the budget is the sum.  (The reference pins its own op at 1e-1 against
    # both, test_sdpa.py:113-127.)
    err = (out.float().cpu() - sdpa_jit_restated(qb, kb, vb, mb).float()).abs()
    assert err.max().item() < 4e-2 and err.mean().item() < 4e-3, (err.max().item(), err.mean().item())


def test_dense_op_full_mask_rows_and_gqa():
    from pace_b200.ops import MultiHeadAttention
    from oracle.attention_ref import sdpa_native, repeat_kv, additive_mask_4d
    g = torch.Generator().manual_seed(9)
    B, N, Nkv, S, H, L = 2, 8, 2, 6, 128, 70
    q = torch.randn(B, N, S, H, generator=g).bfloat16()
    k = torch.randn(B, Nkv, L, H, generator=g).bfloat16()
    v = torch.randn(B, Nkv, L, H, generator=g).bfloat16()
    m2 = torch.ones(B, L, dtype=torch.long)
    m2[1, :9] = 0
    m4 = additive_mask_4d(m2, S, L, torch.bfloat16)          # [B,1,S,L] causal + padding, as the model builds it
    out = MultiHeadAttention()(q.to(DEV), k.to(DEV), v.to(DEV), attention_mask=m4.to(DEV))
    want = sdpa_native(q, repeat_kv(k, 4), repeat_kv(v, 4), m4)
    _check(out, want.float())


def test_dense_op_error_surface():
    # messages the reference's tests look for (tests/ops/test_sdpa.py:129-208)
    from pace_b200.ops import MultiHeadAttention
    mha = MultiHeadAttention()
    q = torch.randn(2, 4, 8, 64, device=DEV).bfloat16()
    k = torch.randn(2, 4, 16, 64, device=DEV).bfloat16()
    m = torch.randn(2, 1, 1, 16, device=DEV).bfloat16()
    with pytest.raises(RuntimeError, match="attention requires 4D inputs"):
        mha(q.view(8, 8, 64), k, k, attention_mask=m)
    with pytest.raises(RuntimeError, match="attention requires 4D inputs"):
        mha(q, k, k, attention_mask=m.view(2, 16))
    with pytest.raises(RuntimeError, match="only support the dtypes Float and BF16 types for input"):
        mha(q.to(torch.int8), k.to(torch.int8), k.to(torch.int8), attention_mask=m)
    with pytest.raises(RuntimeError, match="no CPU path"):
        mha(q.cpu(), k.cpu(), k.cpu(), attention_mask=m.cpu())


def test_torch_ops_pace_attention_schema_on_cuda():
    # the reference's custom-op entry (csrc/ops/attention.cpp:104-108), same call as its tests make
    import pace_b200.ops  # noqa: F401
    from oracle.attention_ref import sdpa_native
    g = torch.Generator().manual_seed(11)
    q = torch.randn(2, 16, 1, 128, generator=g).bfloat16()
    k = torch.randn(2, 16, 300, 128, generator=g).bfloat16()
    v = torch.randn(2, 16, 300, 128, generator=g).bfloat16()
    m = torch.randn(2, 1, 1, 300, generator=g).bfloat16()
    for use_kq in (0, 1, False):
        out = torch.ops.pace.attention(q.to(DEV), k.to(DEV), v.to(DEV), m.to(DEV), use_kq)
        _check(out, sdpa_native(q, k, v, m).float())
    with pytest.raises(RuntimeError, match="attention requires use_KQ to be 0 or 1"):
        torch.ops.pace.attention(q.to(DEV), k.to(DEV), v.to(DEV), m.to(DEV), 7)
    with pytest.raises(RuntimeError, match="attention requires 4D inputs"):
        torch.ops.pace.attention(q.to(DEV), k.to(DEV).view(32, 300, 128), v.to(DEV), m.to(DEV), 0)
