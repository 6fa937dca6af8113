"""Parity of the paged CUDA cache with the reference's cache bookkeeping (bit-exact)."""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

G = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _traces():
    with open(os.path.join(G, "cache_traces.json")) as f:
        return json.load(f)


def test_reference_known_answers_on_device():
    # reference tests/llm_infra/test_cache.py:53-64,76-80 with CUDA bf16 tensors
    from pace_b200.llm.cache import BMCKVCache, DynamicKVCache, KVCacheManager, KVCacheType
    k = torch.rand(2, 10, 64, device=DEV).bfloat16()
    c = BMCKVCache(128)
    key, value = c.update_cache(k, k.clone(), concat_dim=1)
    assert key.shape[1] == 11 and value.shape[1] == 11
    assert c.update_mask(torch.ones(2, 10), 10).shape == (2, 11)
    dk, dv = c.read_dense()
    assert dk.shape == (2, 11, 64)
    assert torch.equal(dk[:, :10], k) and torch.count_nonzero(dk[:, 10:]) == 0
    d = DynamicKVCache(128)
    key, value = d.update_cache(k, k.clone(), concat_dim=1)
    assert key.shape[1] == 10
    m = KVCacheManager(Cfg(2), 128, KVCacheType.DYNAMIC)
    assert len(m.cache_objects) == 2 and isinstance(m[0], DynamicKVCache)
    assert m.update_mask(torch.ones(2, 10), 10).shape == (2, 10)
    c.pool.check_status()


@pytest.mark.parametrize("name", sorted(k for k in _traces() if not k.startswith("test_cache_py")))
def test_length_and_capacity_traces(name):
    from pace_b200.llm.cache import get_kv_cache_class
    e = _traces()[name]
    policy = name.split("/")[1]
    c = get_kv_cache_class(policy)(e["max_len"])
    torch.manual_seed(0)
    for (kind, n), want in zip(e["ops"], e["trace"]):
        if kind == "append":
            x = torch.randn(1, 2, n, 64, device=DEV).bfloat16()
            k, _ = c.update_cache(x, x.clone(), concat_dim=2)
            assert [c.seq_len, k.shape[2]] == want
        elif want[0] == "error":
            with pytest.raises(ValueError, match="Cannot remove more tokens than available in cache"):
                c.remove_cache(n)
        else:
            c.remove_cache(n)
            assert [c.seq_len, c.capacity] == want
        if c.key is not None:
            # the device-resident length and page count agree with the host mirror and the reference
            assert int(c.pool.seq_len()[0, c.manager.slots[0]]) == c.seq_len
            if policy == "bmc":
                assert int(c.pool.seq_pages()[c.manager.slots[0]]) * c.page_tokens >= c.seq_len
    if policy == "bmc":
        assert c.tokens_per_split == e["tokens_per_split"]
        for n, w in e["mask_width"].items():
            assert c.update_mask(torch.ones(2, int(n)), int(n)).shape[-1] == w
    if c.key is not None:
        c.pool.check_status()


def test_cache_contents_match_reference_after_append():
    from pace_b200.llm.cache import BMCKVCache
    case = torch.load(os.path.join(G, "decode_case.pt"))
    for b in range(case["B"]):
        L = case["lens"][b]
        kc, vc = case["k_cache"][b].to(DEV), case["v_cache"][b].to(DEV)
        c = BMCKVCache(case["max_len"])
        c.update_cache(kc[None, :, :L], vc[None, :, :L], concat_dim=2)   # strided views, no copy
        K, V = c.update_cache(case["k_new"][b][None].to(DEV), case["v_new"][b][None].to(DEV), concat_dim=2)
        assert K.shape[2] == case["capacity"][b]
        dk, dv = c.read_dense()
        assert torch.equal(dk[0], kc) and torch.equal(dv[0], vc)   # incl. the zero padding rows
        c.pool.check_status()


def test_ragged_append_and_per_sequence_rollback():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from oracle.kv_cache_ref import SegmentedCacheRef
    torch.manual_seed(1)
    B, H, D, n = 3, 2, 64, 9
    m = KVCacheManager(Cfg(2), 200, KVCacheType.BMC)
    refs = [[SegmentedCacheRef(200) for _ in range(B)] for _ in range(2)]
    script = [("a", [9, 4, 7]), ("a", [1, 1, 1]), ("r", [3, 0, 8]), ("a", [9, 9, 2]), ("r", [1, 1, 1]), ("a", [5, 0, 9])]
    for kind, per in script:
        if kind == "a":
            for layer in range(2):
                k = torch.randn(B, H, n, D, device=DEV).bfloat16()
                v = torch.randn(B, H, n, D, device=DEV).bfloat16()
                m[layer].update_cache(k, v, concat_dim=2, n_new_per_seq=per)
                for b in range(B):
                    if per[b]:
                        refs[layer][b].append(k[b:b + 1, :, :per[b]].cpu(), v[b:b + 1, :, :per[b]].cpu(), axis=2)
        else:
            m.remove_cache(per)
            for layer in range(2):
                for b in range(B):
                    refs[layer][b].remove(per[b])
        for layer in range(2):
            assert m[layer].seq_lens == [refs[layer][b].seq_len for b in range(B)]
            assert m.pool.seq_len()[layer, :B].tolist() == m[layer].seq_lens
    for layer in range(2):
        dk, dv = m[layer].read_dense()
        for b in range(B):
            L = refs[layer][b].seq_len
            assert torch.equal(dk[b, :, :L].cpu(), refs[layer][b].k[0, :, :L])
            assert torch.equal(dv[b, :, :L].cpu(), refs[layer][b].v[0, :, :L])
    with pytest.raises(ValueError, match="Cannot remove more tokens"):
        m.remove_cache([1, 500, 1])
    m.pool.check_status()


def test_rollback_keeps_data_and_pages():
    from pace_b200.llm.cache import BMCKVCache
    torch.manual_seed(2)
    c = BMCKVCache(100)            # tokens_per_split = 10
    k = torch.randn(2, 2, 25, 64, device=DEV).bfloat16()
    c.update_cache(k, k.clone(), concat_dim=2)
    pages_before = c.pool.seq_pages()[:2].tolist()
    table_before = c.pool.block_table()[:2].clone()
    c.remove_cache(8)
    assert c.seq_len == 17 and c.capacity == 30
    assert c.pool.seq_pages()[:2].tolist() == pages_before          # capacity kept (reference cache.py:240)
    assert torch.equal(c.pool.block_table()[:2], table_before)
    dk, _ = c.read_dense()
    assert torch.equal(dk[:, :, :25], k)                             # stale rows stay, as in the reference
    k2 = torch.randn(2, 2, 3, 64, device=DEV).bfloat16()
    c.update_cache(k2, k2.clone(), concat_dim=2)
    dk, _ = c.read_dense()
    assert torch.equal(dk[:, :, 17:20], k2) and torch.equal(dk[:, :, 20:25], k[:, :, 20:25])
    c.pool.check_status()


def test_beam_gather_is_index_only_and_matches_reference():
    from pace_b200.llm.cache import BMCKVCache
    case = torch.load(os.path.join(G, "beam_case.pt"))
    c = BMCKVCache(case["max_len"])
    # head_dim 16 in the reference vector; the pool holds 64-wide rows: embed into 64 columns
    def widen(x):
        out = torch.zeros(*x.shape[:-1], 64, dtype=x.dtype)
        out[..., :16] = x
        return out.to(DEV)
    c.update_cache(widen(case["k"]), widen(case["v"]), concat_dim=2)
    pages = c.pool.pages.clone()
    c.update_cache_with_beam_indices(case["idx"])
    assert torch.equal(c.pool.pages, pages)                         # no K/V byte moved
    c.update_cache(widen(case["k2"]), widen(case["v2"]), concat_dim=2)
    c.update_cache_with_beam_indices(case["idx2"])
    assert c.seq_len == case["seq_len"]
    dk, dv = c.read_dense()
    assert torch.equal(dk[..., :16].cpu(), case["K"]) and torch.equal(dv[..., :16].cpu(), case["V"])
    # reference counts: every page owned by some row, shared pages counted once per owner
    refs = c.pool.page_ref()
    table = c.pool.block_table()[:4]
    owned = table[table >= 0]
    assert int(refs.sum()) == owned.numel()
    c.pool.check_status()


def test_pool_exhaustion_is_reported_not_fatal():
    from pace_b200.llm.cache import KVPool
    from pace_b200 import _C
    import ctypes as C
    pool = KVPool(1, 2, 64, 8, n_pages=3, max_seqs=2, max_pages_per_seq=4, device=DEV)
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    s = torch.cuda.current_stream().cuda_stream
    assert _C.lib.pace_kv_reserve(pool.ref, 0, slots.data_ptr(), 2, 16, None, s) == 0   # needs 4 pages, has 3
    bits, free = pool.query()
    assert bits & _C.DEV_POOL_EXHAUSTED and free == 0
    pool.clear_status()
    assert _C.lib.pace_kv_seq_release(pool.ref, slots.data_ptr(), 2, s) == 0
    bits, free = pool.query()
    assert bits == 0 and free == 3
    # device-side over-removal raises the status bit and leaves the length alone
    assert _C.lib.pace_kv_truncate(pool.ref, 0, 1, slots.data_ptr(), 2, 5, None, s) == 0
    bits, _ = pool.query()
    assert bits & _C.DEV_OVER_REMOVE
