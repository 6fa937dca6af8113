"""CUDA-graph replay of a decode step gives what eager calls give, with device-resident lengths."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Cfg:
    num_hidden_layers = 3


def _setup(seed):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    g = torch.Generator().manual_seed(seed)
    B, Hq, Hkv, D, P0 = 4, 32, 8, 128, 50
    mgr = KVCacheManager(Cfg(), 120, KVCacheType.BMC)        # tokens_per_split 12: pages are crossed often
    for l in range(3):
        k = torch.randn(B, Hkv, P0, D, generator=g).bfloat16().to(DEV)
        mgr[l].update_cache(k, k.flip(1), concat_dim=2)
    return mgr, (B, Hq, Hkv, D)


def test_graph_replay_equals_eager_steps():
    from pace_b200.llm.graph import StepGraph
    from pace_b200.ops import MultiHeadAttention
    mha = MultiHeadAttention()
    n_steps = 30
    g = torch.Generator().manual_seed(99)
    B, Hq, Hkv, D = 4, 32, 8, 128
    feeds = [torch.randn(3, B, Hkv + Hkv + Hq, D, generator=g).bfloat16().to(DEV) for _ in range(n_steps)]

    def run(use_graph):
        mgr, _ = _setup(5)
        buf = torch.empty_like(feeds[0])
        out = torch.empty(3, B, 1, Hq, D, dtype=torch.bfloat16, device=DEV)

        def step():
            for l in range(3):
                K, V = mgr[l].update_cache(buf[l, :, :Hkv].unsqueeze(2), buf[l, :, Hkv:2 * Hkv].unsqueeze(2), 2)
                mha(buf[l, :, 2 * Hkv:].unsqueeze(2), K, V, out=out[l].transpose(1, 2))
            return out

        outs = []
        if not use_graph:
            for f in feeds:
                buf.copy_(f)
                outs.append(step().clone())
        else:
            buf.copy_(feeds[0])
            graph = StepGraph(mgr, lambda: step(), n_new=1, warmup=1)   # the warm-up step is step 0, run eagerly
            outs.append(out.clone())
            for f in feeds[1:]:
                buf.copy_(f)
                outs.append(graph.replay().clone())
        torch.cuda.synchronize()
        mgr.pool.check_status()
        return outs, mgr

    eager, m1 = run(False)
    replay, m2 = run(True)
    for a, b in zip(eager, replay):
        assert torch.equal(a, b)
    assert m1[0].seq_lens == m2[0].seq_lens == [80] * 4 and m1[0].capacity == m2[0].capacity
    assert m2.pool.seq_len()[:, :4].tolist() == [[80] * 4] * 3
    k1, _ = m1[2].read_dense()
    k2, _ = m2[2].read_dense()
    assert torch.equal(k1, k2)


def test_graph_replay_after_beam_gathers_copies_shared_pages_on_write():
    """A replayed decode step with a beam gather between the replays: the gather permutes block-table
    rows, sequences then share pages, and the step's page reservation (recorded in the graph, run
    whenever pages are shared) copies a shared last page before the appended row lands in it.  Contents
    against a dense index_select / concatenate restatement of the reference's cache (cache.py:161-167,
    268-326), bit for bit; attention rows against the oracle."""
    from oracle.attention_ref import attend_over_cache
    from pace_b200.llm.graph import StepGraph
    from pace_b200.ops import MultiHeadAttention
    mha = MultiHeadAttention()
    g = torch.Generator().manual_seed(123)
    L, B, Hq, Hkv, D, P0, n_steps = 3, 4, 32, 8, 128, 50, 14
    prompt = [torch.randn(B, Hkv, P0, D, generator=g).bfloat16().to(DEV) for _ in range(L)]
    feeds = [torch.randn(L, B, Hkv + Hkv + Hq, D, generator=g).bfloat16().to(DEV) for _ in range(n_steps)]
    perms = [torch.tensor(p) for p in ([0, 0, 1, 1], [2, 0, 0, 3], [1, 1, 1, 1], [0, 1, 2, 3], [3, 3, 0, 2])]

    for deferred in (False, True):
        from pace_b200.llm.cache import KVCacheManager, KVCacheType
        mgr = KVCacheManager(Cfg(), 120, KVCacheType.BMC)
        mgr.defer_appends = deferred
        dense_k = [p.clone() for p in prompt]
        dense_v = [p.flip(1).clone() for p in prompt]
        for l in range(L):
            mgr[l].update_cache(prompt[l], prompt[l].flip(1), concat_dim=2)
        buf = torch.empty_like(feeds[0])
        out = torch.empty(L, B, 1, Hq, D, dtype=torch.bfloat16, device=DEV)

        def step():
            for l in range(L):
                K, V = mgr[l].update_cache(buf[l, :, :Hkv].unsqueeze(2), buf[l, :, Hkv:2 * Hkv].unsqueeze(2), 2)
                mha(buf[l, :, 2 * Hkv:].unsqueeze(2), K, V, out=out[l].transpose(1, 2))
            return out

        buf.copy_(feeds[0])
        graph = StepGraph(mgr, step, n_new=1, warmup=1)
        for l in range(L):
            dense_k[l] = torch.cat([dense_k[l], feeds[0][l, :, :Hkv].unsqueeze(2)], dim=2)
            dense_v[l] = torch.cat([dense_v[l], feeds[0][l, :, Hkv:2 * Hkv].unsqueeze(2)], dim=2)
        for t in range(1, n_steps):
            if t % 3 == 1:                               # a gather before this step
                idx = perms[(t // 3) % len(perms)]
                mgr.update_cache_with_beam_indices(idx.to(DEV))
                for l in range(L):
                    dense_k[l] = dense_k[l].index_select(0, idx.to(DEV))
                    dense_v[l] = dense_v[l].index_select(0, idx.to(DEV))
            buf.copy_(feeds[t])
            got = graph.replay().clone()
            for l in range(L):
                dense_k[l] = torch.cat([dense_k[l], feeds[t][l, :, :Hkv].unsqueeze(2)], dim=2)
                dense_v[l] = torch.cat([dense_v[l], feeds[t][l, :, Hkv:2 * Hkv].unsqueeze(2)], dim=2)
            if t in (2, 7, n_steps - 1):
                l = t % L
                q = feeds[t][l, :, 2 * Hkv:].unsqueeze(2)
                n = dense_k[l].shape[2]
                for b in range(B):
                    want = attend_over_cache(q[b:b + 1].cpu(), dense_k[l][b:b + 1].cpu(), dense_v[l][b:b + 1].cpu(), n)[0]
                    err = (got[l, b].transpose(0, 1).float().cpu() - want.float()).abs()
                    assert err.max().item() < 2e-2 and err.mean().item() < 2e-3, (deferred, t, b, err.max().item())
        torch.cuda.synchronize()
        mgr.pool.check_status()
        assert graph.replays_with_reserve >= 8        # pages stay shared after the first gather: the reserving form runs
        for l in range(L):
            k, v = mgr[l].read_dense()
            n = P0 + n_steps
            assert torch.equal(k[:, :, :n], dense_k[l]) and torch.equal(v[:, :, :n], dense_v[l]), (deferred, l)
