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
