"""Size-independent properties of the path at the full size of the decode configuration (batch 32, 32 query /
8 KV heads of 128, 32 layers, 512-token prompts growing to 768): things that must hold whatever the data is,
checked on every sequence, head and layer where the CPU oracle only samples.

* round trip: what was appended (a prompt in chunks, then single tokens through the deferred path, a
  rollback, other tokens in their place) is what the cache holds, bit for bit, and the lengths agree;
* a cache whose value rows are all one vector returns that vector (the softmax weights sum to one);
* doubling every value row doubles the output exactly (a power of two passes through every rounding);
* the result does not depend on how the launch is cut across thread blocks, nor on the order of the cached
  tokens (one query token sees every key), within the parity budget.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3
B, HQ, HKV, D, LAYERS, PROMPT, GROW = 32, 32, 8, 128, 32, 512, 256


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _close(a, b, what):
    err = (a.float() - b.float()).abs()
    assert err.max().item() < MAX_ABS, (what, "max-abs", err.max().item())
    assert err.mean().item() < MEAN_ABS, (what, "mean-abs", err.mean().item())


def test_round_trip_of_every_layer_at_full_size():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator(device=DEV).manual_seed(21)
    mgr = KVCacheManager(Cfg(LAYERS), PROMPT + GROW + 8, KVCacheType.BMC)
    mha = MultiHeadAttention()
    rows = lambda n: torch.randn(B, HKV, n, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()  # noqa: E731
    # the prompt in 128-token chunks, every layer; a running checksum instead of a copy of everything
    want_k = [[] for _ in range(LAYERS)]
    want_v = [[] for _ in range(LAYERS)]
    for c in range(PROMPT // 128):
        for l in range(LAYERS):
            k, v = rows(128), rows(128)
            mgr[l].update_cache(k, v, concat_dim=2)
            if l in (0, 13, LAYERS - 1):
                want_k[l].append(k)
                want_v[l].append(v)
    # single tokens through the deferred path (the decode launch stores the row), all layers, 40 steps
    mgr.defer_appends = True
    q = torch.randn(B, HQ, 1, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    steps = 40
    for t in range(steps):
        for l in range(LAYERS):
            k, v = rows(1), rows(1)
            K, V = mgr[l].update_cache(k, v, concat_dim=2)
            mha(q, K, V)
            if l in (0, 13, LAYERS - 1):
                want_k[l].append(k)
                want_v[l].append(v)
        mgr.commit()
    assert mgr[0].seq_len == PROMPT + steps
    # rollback of 15 tokens, 15 others in their place (one multi-token append per layer)
    mgr.remove_cache(15)
    assert mgr[LAYERS - 1].seq_len == PROMPT + steps - 15
    for l in range(LAYERS):
        k, v = rows(15), rows(15)
        mgr[l].update_cache(k, v, concat_dim=2)
        if l in (0, 13, LAYERS - 1):
            want_k[l] = [torch.cat(want_k[l], dim=2)[:, :, : PROMPT + steps - 15], k]
            want_v[l] = [torch.cat(want_v[l], dim=2)[:, :, : PROMPT + steps - 15], v]
    torch.cuda.synchronize()
    mgr.pool.check_status()
    n = PROMPT + steps
    assert mgr.pool.seq_len()[:, :B].tolist() == [[n] * B for _ in range(LAYERS)]   # every layer, every sequence
    for l in (0, 13, LAYERS - 1):
        dk, dv = mgr[l].read_dense()
        assert torch.equal(dk[:, :, :n], torch.cat(want_k[l], dim=2))
        assert torch.equal(dv[:, :, :n], torch.cat(want_v[l], dim=2))
    mgr.release()


def test_softmax_weights_sum_to_one_and_values_scale_exactly():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator(device=DEV).manual_seed(22)
    L = PROMPT + GROW - 1                                   # 767 cached tokens: the last page is partly filled
    mgr = KVCacheManager(Cfg(3), L + 8, KVCacheType.BMC)
    mha = MultiHeadAttention()
    k = torch.randn(B, HKV, L, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    v = torch.randn(B, HKV, L, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    one = torch.randn(B, HKV, 1, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    q = torch.randn(B, HQ, 1, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    for lo in range(0, L, 256):
        hi = min(L, lo + 256)
        mgr[0].update_cache(k[:, :, lo:hi], v[:, :, lo:hi], concat_dim=2)
        mgr[1].update_cache(k[:, :, lo:hi], (v[:, :, lo:hi].float() * 2).bfloat16(), concat_dim=2)
        mgr[2].update_cache(k[:, :, lo:hi], one.expand(B, HKV, hi - lo, D), concat_dim=2)
    out = mha(q, mgr[0].key, mgr[0].value)
    twice = mha(q, mgr[1].key, mgr[1].value)
    same = mha(q, mgr[2].key, mgr[2].value)
    # every value row is `one`: whatever the scores are, the output is that row (fp32 sum of weights that add
    # up to one, times a bf16 vector, rounded once)
    want = one.repeat_interleave(HQ // HKV, dim=1)          # [B, HQ, 1, D]
    rel = (same.float() - want.float()).abs() / want.float().abs().clamp_min(1e-3)
    assert rel.max().item() < 2.0 ** -7, rel.max().item()
    # values times two: outputs times two, exactly
    assert torch.equal(twice.float(), out.float() * 2)
    mgr.release()


def test_result_does_not_depend_on_the_partition_or_the_order_of_cached_tokens():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator(device=DEV).manual_seed(23)
    lens = [PROMPT + (17 * b) % GROW for b in range(B)]      # ragged, 512 .. 767
    Lmax = max(lens)
    mgr = KVCacheManager(Cfg(2), Lmax + 8, KVCacheType.BMC)
    mha = MultiHeadAttention()
    k = torch.randn(B, HKV, Lmax, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    v = torch.randn(B, HKV, Lmax, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    q = torch.randn(B, HQ, 1, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    kp, vp = k.clone(), v.clone()
    for b in range(B):                                       # the same tokens in another order
        perm = torch.randperm(lens[b], device=DEV, generator=g)
        kp[b, :, : lens[b]] = k[b][:, perm]
        vp[b, :, : lens[b]] = v[b][:, perm]
    mgr[0].update_cache(k, v, concat_dim=2, n_new_per_seq=lens)
    mgr[1].update_cache(kp, vp, concat_dim=2, n_new_per_seq=lens)
    base = mha(q, mgr[0].key, mgr[0].value)
    assert torch.equal(base, mha(q, mgr[0].key, mgr[0].value))          # run to run: bit for bit
    for ctas in (1, 7, 37, 148, 296):
        _close(mha(q, mgr[0].key, mgr[0].value, max_ctas=ctas), base, ("partition", ctas))
    _close(mha(q, mgr[1].key, mgr[1].value), base, "token order")
    # against the oracle on two sequences (the shortest and the longest)
    from oracle.attention_ref import attend_over_cache
    for b in (lens.index(min(lens)), lens.index(max(lens))):
        want = attend_over_cache(q[b:b + 1].cpu(), k[b:b + 1, :, : lens[b]].cpu(), v[b:b + 1, :, : lens[b]].cpu(),
                                 lens[b], 0, "native")[0]
        _close(base[b].cpu(), want, ("oracle", b))
    mgr.pool.check_status()
    mgr.release()


def test_chunked_prefill_equals_one_pass_at_size():
    """Config-3 shape (batch 8, 32 / 8 heads of 128, 512-token chunks): a 1024-token stretch of the prompt
    attended as two chunks of 512 (the second one sees the first through the cache) gives what one pass of
    1024 query tokens gives, and a chunk's first rows do not depend on its later ones (causality) - the wide
    tcgen05 form against itself across different unit boundaries, and against the launch cut over 5 thread
    blocks."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    g = torch.Generator(device=DEV).manual_seed(24)
    Bp, past, S = 8, 1536, 1024
    mgr = KVCacheManager(Cfg(2), past + S + 8, KVCacheType.BMC)
    mha = MultiHeadAttention()
    k = torch.randn(Bp, HKV, past + S, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    v = torch.randn(Bp, HKV, past + S, D, device=DEV, generator=g, dtype=torch.float32).bfloat16()
    q = torch.randn(Bp, S, HQ, D, device=DEV, generator=g, dtype=torch.float32).bfloat16().transpose(1, 2)
    for lo in range(0, past, 512):
        for l in range(2):
            mgr[l].update_cache(k[:, :, lo:lo + 512], v[:, :, lo:lo + 512], concat_dim=2)
    # layer 0: two chunks of 512; layer 1: one pass of 1024
    outs = []
    for c in range(2):
        lo = past + 512 * c
        K, V = mgr[0].update_cache(k[:, :, lo:lo + 512], v[:, :, lo:lo + 512], concat_dim=2)
        outs.append(mha(q[:, :, 512 * c:512 * (c + 1)], K, V))
    K, V = mgr[1].update_cache(k[:, :, past:], v[:, :, past:], concat_dim=2)
    whole = mha(q, K, V)
    _close(torch.cat(outs, dim=2), whole, "two chunks against one pass")
    _close(mha(q, K, V, max_ctas=5), whole, "one pass on 5 thread blocks")
    # causality: the first 300 query tokens alone (ragged count) see exactly what they saw inside the pass
    q_lens = torch.full((Bp,), 300, dtype=torch.int32, device=DEV)
    mgr.remove_cache(S - 300)
    K0, V0 = mgr[1].key, mgr[1].value
    head = mha(q[:, :, :300], K0, V0, q_lens=q_lens)
    _close(head, whole[:, :, :300], "prefix of the pass")
    mgr.pool.check_status()
    mgr.release()
