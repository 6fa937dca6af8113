"""Deferred decode appends: a staged row as the newest key of the decode launch, one batched append
per step.  Contents and lengths must end up bit-identical to per-layer appends; the attention rows
must be the oracle's (reference: llama.py:159-165 does update_cache, then attention, per layer)."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


class Cfg:
    def __init__(self, n):
        self.num_hidden_layers = n


def _fill(mgr, layer, ks, vs):
    B, H, D = len(ks), ks[0].shape[0], ks[0].shape[2]
    Lmax = max(max(k.shape[1] for k in ks), 1)
    kp = torch.zeros(B, H, Lmax, D, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros_like(kp)
    for b in range(B):
        kp[b, :, : ks[b].shape[1]] = ks[b]
        vp[b, :, : vs[b].shape[1]] = vs[b]
    return mgr[layer].update_cache(kp, vp, concat_dim=2, n_new_per_seq=[k.shape[1] for k in ks])


def _oracle(q, ks, vs, left_pad=None):
    from oracle.attention_ref import attend_over_cache
    return [attend_over_cache(q[b:b + 1].cpu(), ks[b][None].cpu(), vs[b][None].cpu(), ks[b].shape[1],
                              0 if left_pad is None else left_pad[b], "native")[0].float() for b in range(len(ks))]


def _check(got, want):
    err = (got.float().cpu() - want).abs()
    assert err.max().item() < MAX_ABS, f"max-abs {err.max().item()}"
    assert err.mean().item() < MEAN_ABS, f"mean-abs {err.mean().item()}"


SHAPES = [
    # Hq, Hkv, D, lens of the cache before the step
    (32, 8, 128, [519, 64, 63, 1, 0, 300]),        # config 2's group of four; an empty cache and page edges
    (32, 8, 64, [1033, 5, 0, 128]),                # the draft model's head_dim
    (8, 8, 128, [70, 0, 129]),                     # groups of one (CUDA-core kernel when nothing is pending)
    (32, 2, 128, [200, 64, 7]),                    # sixteen query heads per KV head: a full 16-row tile
    (64, 2, 64, [90, 0, 257]),                     # thirty-two per KV head: two row tiles
    (24, 8, 128, [31, 333]),                       # three per KV head
]


@pytest.mark.parametrize("schedule", [dict(), dict(whole_units=True), dict(whole_units=False, max_ctas=3),
                                      dict(one_cta_per_sm=True), dict(whole_units=True, one_cta_per_sm=True)])
@pytest.mark.parametrize("Hq,Hkv,D,lens", SHAPES)
@pytest.mark.parametrize("tps", [False, True])
def test_pending_row_decode(monkeypatch, tps, Hq, Hkv, D, lens, schedule):
    """The staged row counts as key number seq_len: outputs equal the oracle's over cache + row, the
    pool's lengths are untouched until commit, and after commit lengths and contents are bit-identical
    to a plain append."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    if tps:
        monkeypatch.setenv("PACE_KV_PAGE_TOKENS", "tps")
    B = len(lens)
    g = torch.Generator().manual_seed(Hq + D + sum(lens))
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    k_new = torch.randn(B, Hkv, 1, D, generator=g).bfloat16().to(DEV)
    v_new = torch.randn(B, Hkv, 1, D, generator=g).bfloat16().to(DEV)
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mha = MultiHeadAttention()

    plain = KVCacheManager(Cfg(1), 1200, KVCacheType.BMC)
    _fill(plain, 0, ks, vs)
    K0, V0 = plain[0].update_cache(k_new, v_new, concat_dim=2)
    out_plain = mha(q, K0, V0, **schedule)

    mgr = KVCacheManager(Cfg(1), 1200, KVCacheType.BMC)
    _fill(mgr, 0, ks, vs)
    mgr.defer_appends = True
    K, V = mgr[0].update_cache(k_new, v_new, concat_dim=2)
    assert mgr[0].pending and mgr[0].seq_lens == [n + 1 for n in lens]
    assert mgr.pool.seq_len()[0, :B].tolist() == lens            # the device has not been told yet
    out = mha(q, K, V, **schedule)
    assert mgr[0].pending                                        # the launch consumed the row in place
    want = _oracle(q, [torch.cat([ks[b], k_new[b]], dim=1) for b in range(B)],
                   [torch.cat([vs[b], v_new[b]], dim=1) for b in range(B)])
    for b in range(B):
        _check(out[b], want[b])
        _check(out_plain[b], want[b])
    _check(out, out_plain.float().cpu())                         # (a bf16 unit in the last place at most)
    mgr.commit()
    assert not mgr[0].pending and mgr.pool.seq_len()[0, :B].tolist() == [n + 1 for n in lens]
    for a, b in zip(mgr[0].read_dense(), plain[0].read_dense()):
        assert torch.equal(a, b)
    # and the committed row is now an ordinary key: a second launch, nothing pending, same rows
    out2 = mha(q, K, V, **schedule)
    assert torch.equal(out2, out_plain)
    mgr.pool.check_status()
    plain.pool.check_status()


def test_pending_row_with_left_padding():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    Hq, Hkv, D, lens, pads = 32, 8, 128, [100, 257, 64], [0, 57, 63]
    B = len(lens)
    g = torch.Generator().manual_seed(3)
    ks = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    vs = [torch.randn(Hkv, L, D, generator=g).bfloat16().to(DEV) for L in lens]
    k_new = torch.randn(B, Hkv, 1, D, generator=g).bfloat16().to(DEV)
    v_new = torch.randn(B, Hkv, 1, D, generator=g).bfloat16().to(DEV)
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    mgr = KVCacheManager(Cfg(1), 400, KVCacheType.BMC)
    _fill(mgr, 0, ks, vs)
    mgr.defer_appends = True
    K, V = mgr[0].update_cache(k_new, v_new, concat_dim=2)
    out = MultiHeadAttention()(q, K, V, kv_start=torch.tensor(pads, dtype=torch.int32, device=DEV))
    want = _oracle(q, [torch.cat([ks[b], k_new[b]], dim=1) for b in range(B)],
                   [torch.cat([vs[b], v_new[b]], dim=1) for b in range(B)], left_pad=pads)
    for b in range(B):
        _check(out[b], want[b])
    mgr.pool.check_status()


@pytest.mark.parametrize("adopt", [False, True])
@pytest.mark.parametrize("use_graph", [False, True])
def test_deferred_steps_equal_per_layer_appends(use_graph, adopt):
    """Many steps over several layers, eagerly and as a replayed CUDA graph, with the manager's own
    staging buffer and with the caller's: lengths, capacities and every layer's K/V contents are
    bit-identical to per-layer appends, attention rows within the parity budget of the oracle."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.llm.graph import StepGraph
    from pace_b200.ops import MultiHeadAttention
    L, B, Hq, Hkv, D, P0, n_steps = 4, 6, 32, 8, 128, 50, 40
    g = torch.Generator().manual_seed(17)
    prompt = [torch.randn(B, Hkv, P0, D, generator=g).bfloat16().to(DEV) for _ in range(L)]
    feeds = [torch.randn(L, B, Hkv + Hkv + Hq, 1, D, generator=g).bfloat16().to(DEV) for _ in range(n_steps)]
    mha = MultiHeadAttention()

    def run(deferred):
        mgr = KVCacheManager(Cfg(L), 120, KVCacheType.BMC)     # tokens_per_split 12: segments are crossed often
        for l in range(L):
            mgr[l].update_cache(prompt[l], prompt[l].flip(1), concat_dim=2)
        buf = torch.empty_like(feeds[0])
        out = torch.empty(L, B, 1, Hq, D, dtype=torch.bfloat16, device=DEV)
        mgr.defer_appends = deferred
        if deferred and adopt:
            mgr.adopt_staging(buf[:, :, :Hkv], buf[:, :, Hkv:2 * Hkv])

        def step():
            for l in range(L):
                K, V = mgr[l].update_cache(buf[l, :, :Hkv], buf[l, :, Hkv:2 * Hkv], 2)
                mha(buf[l, :, 2 * Hkv:], K, V, out=out[l].transpose(1, 2))
            mgr.commit()
            return out

        outs = []
        if use_graph and deferred:
            buf.copy_(feeds[0])
            graph = StepGraph(mgr, step, n_new=1, warmup=1)
            outs.append(out.clone())
            for f in feeds[1:]:
                buf.copy_(f)
                outs.append(graph.replay().clone())
        else:
            for f in feeds:
                buf.copy_(f)
                outs.append(step().clone())
        torch.cuda.synchronize()
        mgr.pool.check_status()
        return outs, mgr

    base, m1 = run(False)
    got, m2 = run(True)
    for l in range(L):
        assert m1[l].seq_lens == m2[l].seq_lens == [P0 + n_steps] * B and m1[l].capacity == m2[l].capacity
        for a, b in zip(m1[l].read_dense(), m2[l].read_dense()):
            assert torch.equal(a, b)
    assert m2.pool.seq_len()[:, :B].tolist() == [[P0 + n_steps] * B] * L
    for t in range(n_steps):
        _check(got[t], base[t].float().cpu())
    # the last step against the oracle, layer 2
    l = 2
    kk = torch.cat([prompt[l]] + [f[l, :, :Hkv] for f in feeds], dim=2)
    vv = torch.cat([prompt[l].flip(1)] + [f[l, :, Hkv:2 * Hkv] for f in feeds], dim=2)
    want = _oracle(feeds[-1][l, :, 2 * Hkv:], [kk[b] for b in range(B)], [vv[b] for b in range(B)])
    for b in range(B):
        _check(got[-1][l, b].transpose(0, 1), want[b])


def test_commit_is_forced_by_what_needs_the_pool():
    """Rollback, a second token, a multi-token append and a read-back all see the staged row."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    B, Hkv, D = 3, 8, 128
    g = torch.Generator().manual_seed(8)
    mgr = KVCacheManager(Cfg(2), 200, KVCacheType.BMC)
    mgr.defer_appends = True
    rows = [torch.randn(B, Hkv, 1, D, generator=g).bfloat16().to(DEV) for _ in range(6)]
    for l in range(2):
        mgr[l].update_cache(rows[0], rows[0], 2)          # staged (first token of an empty cache)
    assert mgr[0].pending and mgr[1].pending
    for l in range(2):
        mgr[l].update_cache(rows[1], rows[1], 2)          # a second token: the first is committed, this one staged
    assert mgr.pool.seq_len()[:, :B].tolist() == [[1] * B] * 2 and len(mgr) == 2
    mgr.remove_cache(1)                                   # commits, then forgets the newest token
    assert not mgr[0].pending and mgr.pool.seq_len()[:, :B].tolist() == [[1] * B] * 2 and len(mgr) == 1
    mgr[0].update_cache(rows[2], rows[2], 2)              # staged on layer 0 only
    k, _ = mgr[0].read_dense()                            # the read-back commits (a run of one layer)
    assert torch.equal(k[:, :, :2], torch.cat([rows[0], rows[2]], dim=2))
    assert mgr.pool.seq_len()[:, :B].tolist() == [[2] * B, [1] * B]
    mgr[1].update_cache(torch.cat([rows[3], rows[4]], dim=2), torch.cat([rows[3], rows[4]], dim=2), 2)   # two tokens: appended at once
    assert not mgr[1].pending and mgr.pool.seq_len()[1, :B].tolist() == [3] * B
    mgr.pool.check_status()


def test_single_layer_pool_append_attend_loop():
    """attn(layer 0), append(layer 0), attn(layer 0) ... with nothing between the launches: the append
    may not overtake the attention launch that reads the same layer's lengths.  Eager calls on a
    free-standing cache object (a one-layer pool), every step against the oracle."""
    from pace_b200.llm.cache import BMCKVCache
    from pace_b200.ops import MultiHeadAttention
    B, Hq, Hkv, D, P0, n_steps = 32, 32, 8, 128, 515, 24
    g = torch.Generator().manual_seed(21)
    cache = BMCKVCache(768)
    k0 = torch.randn(B, Hkv, P0, D, generator=g).bfloat16().to(DEV)
    v0 = torch.randn(B, Hkv, P0, D, generator=g).bfloat16().to(DEV)
    cache.update_cache(k0, v0, 2)
    new = torch.randn(n_steps, B, 2 * Hkv + Hq, 1, D, generator=g).bfloat16().to(DEV)
    outs = torch.empty(n_steps, B, Hq, 1, D, dtype=torch.bfloat16, device=DEV)
    mha = MultiHeadAttention()
    for t in range(n_steps):
        K, V = cache.update_cache(new[t, :, :Hkv], new[t, :, Hkv:2 * Hkv], 2)
        mha(new[t, :, 2 * Hkv:], K, V, out=outs[t])
    torch.cuda.synchronize()
    cache.pool.check_status()
    for t in (0, 7, n_steps - 1):
        kk = torch.cat([k0] + [new[i, :, :Hkv] for i in range(t + 1)], dim=2)
        vv = torch.cat([v0] + [new[i, :, Hkv:2 * Hkv] for i in range(t + 1)], dim=2)
        want = _oracle(new[t, :, 2 * Hkv:], [kk[b] for b in range(B)], [vv[b] for b in range(B)])
        for b in range(0, B, 5):
            _check(outs[t, b], want[b])


def test_append_layers_through_the_c_abi():
    """pace_kv_append_layers on a strided staging tensor with ragged counts, against per-layer
    pace_kv_append calls on a second pool: same pages, same lengths."""
    from pace_b200 import _C
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    L, B, Hkv, D, n = 5, 4, 8, 64, 3
    g = torch.Generator().manual_seed(4)
    stage = torch.randn(L, B, 2 * Hkv, n, D, generator=g).bfloat16().to(DEV)
    counts = [3, 0, 1, 2]
    n_dev = torch.tensor(counts, dtype=torch.int32, device=DEV)
    mgrs = [KVCacheManager(Cfg(L), 300, KVCacheType.BMC) for _ in range(2)]
    seed = torch.randn(B, Hkv, 70, D, generator=g).bfloat16().to(DEV)
    for m in mgrs:
        for l in range(L):
            m[l].update_cache(seed, seed, 2, n_new_per_seq=[70, 1, 64, 33])
    stream = torch.cuda.current_stream().cuda_stream
    a, b = mgrs
    kv = stage[:, :, :Hkv], stage[:, :, Hkv:]
    sl, sb, sh, st, _ = kv[0].stride()
    assert _C.lib.pace_kv_reserve(a.pool.ref, 0, a.slots_dev.data_ptr(), B, n, n_dev.data_ptr(), stream) == 0
    assert _C.lib.pace_kv_append_layers(a.pool.ref, 1, 4, a.slots_dev.data_ptr(), B, n, n_dev.data_ptr(),
                                        kv[0][1].data_ptr(), kv[1][1].data_ptr(), sl, sb, sh, st, stream) == 0
    assert _C.lib.pace_kv_reserve(b.pool.ref, 0, b.slots_dev.data_ptr(), B, n, n_dev.data_ptr(), stream) == 0
    for l in range(1, 4):
        assert _C.lib.pace_kv_append(b.pool.ref, l, b.slots_dev.data_ptr(), B, n, n_dev.data_ptr(),
                                     kv[0][l].data_ptr(), kv[1][l].data_ptr(), sb, sh, st, stream) == 0
    torch.cuda.synchronize()
    assert torch.equal(a.pool.seq_len(), b.pool.seq_len())
    assert a.pool.seq_len()[:, :B].tolist() == [[70, 1, 64, 33]] + [[73, 1, 65, 35]] * 3 + [[70, 1, 64, 33]]
    assert torch.equal(a.pool.pages, b.pool.pages)
    # arguments that cannot be served
    assert _C.lib.pace_kv_append_layers(a.pool.ref, 3, 2, a.slots_dev.data_ptr(), B, n, None, kv[0].data_ptr(),
                                        kv[1].data_ptr(), sl, sb, sh, st, stream) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_kv_append_layers(a.pool.ref, 0, L + 1, a.slots_dev.data_ptr(), B, n, None, kv[0].data_ptr(),
                                        kv[1].data_ptr(), sl, sb, sh, st, stream) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_kv_append_layers(a.pool.ref, 0, L, a.slots_dev.data_ptr(), B, n, None, kv[0].data_ptr() + 2,
                                        kv[1].data_ptr(), sl, sb, sh, st, stream) == _C.PACE_ERR_INVALID
    for m in mgrs:
        m.pool.check_status()


def test_model_decode_with_staged_rope_rows_equals_immediate_appends():
    """The re-hosted Llama decoding token by token: with deferred appends the RoPE kernel stages the rotated
    key and the value, the layer's decode launch takes them along, and one commit per step advances every
    layer.  Same logits (to a bf16 unit) and bit-identical caches as with the append inside every layer."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.llm.models.llama import LlamaForCausalLM, random_init_

    class MC:
        hidden_size, intermediate_size, num_hidden_layers = 512, 512, 3
        num_attention_heads, num_key_value_heads, vocab_size = 8, 2, 200
        max_position_embeddings, rope_theta, rms_norm_eps, pad_token_id = 256, 500000.0, 1e-5, 0
    cfg = MC()
    model = random_init_(LlamaForCausalLM(cfg).to(torch.bfloat16), 7).to(DEV).eval()
    g = torch.Generator().manual_seed(5)
    B, P, steps = 5, 61, 9                       # the decode steps cross a 64-token page boundary
    ids = torch.randint(1, cfg.vocab_size, (B, P + steps), generator=g).to(DEV)
    runs = []
    with torch.inference_mode():
        for deferred in (False, True):
            mgr = KVCacheManager(cfg, P + steps + 1, KVCacheType.BMC)
            mgr.defer_appends = deferred
            logits = []
            mask = torch.ones(B, P, dtype=torch.long, device=DEV)
            for t in range(steps + 1):
                out = model(ids[:, : P + t], kv_cache=mgr, attention_mask=mask)
                logits.append(out.logits[:, -1].float().clone())
                mask = torch.cat([mask, mask.new_ones(B, 1)], dim=-1)
                assert not mgr._pending                                  # the model's forward commits
                assert mgr.pool.seq_len()[:, :B].tolist() == [[P + t] * B] * 3
            runs.append((logits, [mgr[l].read_dense() for l in range(3)], mgr))
    for a, b in zip(runs[0][0], runs[1][0]):
        assert (a - b).abs().max().item() < 2e-2
    for (k0, v0), (k1, v1) in zip(runs[0][1], runs[1][1]):
        assert torch.equal(k0, k1) and torch.equal(v0, v1)
    for r in runs:
        r[2].pool.check_status()
