"""BASELINE configurations 3 and 4 at their stated sizes (one or two layers, real head shapes).

Config 3: batch 8, prompt lengths uniform in [1024, 8192], prefill in 512-token chunks written into the
cache and attended chunk by chunk (the tcgen05 tiles, large appends), then 64 decode steps.
Config 4: PARD, batch 16, 8 draft tokens per step, 1024-token prompts, target head_dim 128 / draft
head_dim 64 pools, acceptance forced by a seeded Bernoulli(0.6) per draft token.
Seeded synthetic tensors / token ids of the configurations' shapes stand in for a model's activations.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


class Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _check(got, want, what):
    err = (got.float().cpu() - want.float()).abs()
    assert err.max().item() < MAX_ABS, (what, "max-abs", err.max().item())
    assert err.mean().item() < MEAN_ABS, (what, "mean-abs", err.mean().item())


def test_config3_chunked_prefill_then_decode_at_size():
    from oracle.attention_ref import attend_over_cache
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.ops import MultiHeadAttention
    B, Hq, Hkv, D, CH, n_decode = 8, 32, 8, 128, 512, 64
    g = torch.Generator().manual_seed(3)
    lens = torch.randint(1024, 8193, (B,), generator=g).tolist()
    Lmax = max(lens)
    mgr = KVCacheManager(Cfg(num_hidden_layers=1), Lmax + n_decode + 8, KVCacheType.BMC)
    mha = MultiHeadAttention()
    # the whole prompt's K/V/Q, generated on the host in bf16 (what the oracle reads), moved chunk by chunk
    k_all = torch.randn(B, Hkv, Lmax, D, generator=g).bfloat16()
    v_all = torch.randn(B, Hkv, Lmax, D, generator=g).bfloat16()
    n_chunks = (Lmax + CH - 1) // CH
    picks = {b: {0, (lens[b] // CH) // 2, (lens[b] - 1) // CH} for b in range(B)}   # first, a middle, the last chunk
    for c in range(n_chunks):
        counts = [max(0, min(CH, lens[b] - c * CH)) for b in range(B)]
        kc = k_all[:, :, c * CH:(c + 1) * CH].to(DEV)
        vc = v_all[:, :, c * CH:(c + 1) * CH].to(DEV)
        n = kc.shape[2]
        K, V = mgr[0].update_cache(kc, vc, concat_dim=2, n_new_per_seq=[min(x, n) for x in counts])
        q = torch.randn(B, n, Hq, D, generator=g).bfloat16().to(DEV).transpose(1, 2)
        q_lens = torch.tensor([min(x, n) for x in counts], dtype=torch.int32, device=DEV)
        out = mha(q, K, V, q_lens=q_lens)
        for b in range(B):
            if c in picks[b] and counts[b] > 0:
                have = c * CH + counts[b]
                want = attend_over_cache(q[b:b + 1, :, :counts[b]].cpu(), k_all[b:b + 1, :, :have], v_all[b:b + 1, :, :have],
                                         have, 0, "native")[0]
                _check(out[b, :, :counts[b]], want, ("prefill chunk", c, b))
    assert mgr[0].seq_lens == lens
    assert mgr.pool.seq_len()[0, :B].tolist() == lens
    dk, dv = mgr[0].read_dense()
    for b in range(B):
        assert torch.equal(dk[b, :, :lens[b]].cpu(), k_all[b, :, :lens[b]])
        assert torch.equal(dv[b, :, :lens[b]].cpu(), v_all[b, :, :lens[b]])
    # 64 decode steps on the same cache, with deferred appends (the staged row is the newest key)
    mgr.defer_appends = True
    k_dec = torch.randn(n_decode, B, Hkv, 1, D, generator=g).bfloat16()
    v_dec = torch.randn(n_decode, B, Hkv, 1, D, generator=g).bfloat16()
    q_dec = torch.randn(n_decode, B, Hq, 1, D, generator=g).bfloat16()
    outs = []
    for t in range(n_decode):
        K, V = mgr[0].update_cache(k_dec[t].to(DEV), v_dec[t].to(DEV), concat_dim=2)
        outs.append(mha(q_dec[t].to(DEV), K, V))
        mgr.commit()
    torch.cuda.synchronize()
    mgr.pool.check_status()
    assert mgr.pool.seq_len()[0, :B].tolist() == [n + n_decode for n in lens]
    for t in (0, 31, n_decode - 1):
        for b in range(0, B, 3):
            kk = torch.cat([k_all[b, :, :lens[b]]] + [k_dec[i, b] for i in range(t + 1)], dim=1)[None]
            vv = torch.cat([v_all[b, :, :lens[b]]] + [v_dec[i, b] for i in range(t + 1)], dim=1)[None]
            want = attend_over_cache(q_dec[t, b:b + 1], kk, vv, kk.shape[2], 0, "native")[0]
            _check(outs[t][b], want, ("decode step", t, b))
    dk, dv = mgr[0].read_dense()
    b = B - 1
    assert torch.equal(dk[b, :, lens[b]: lens[b] + n_decode].cpu(), torch.cat([k_dec[i, b] for i in range(n_decode)], dim=1))


def _model(cfg, seed):
    from pace_b200.llm.models.llama import LlamaForCausalLM, random_init_
    return random_init_(LlamaForCausalLM(cfg).to(torch.bfloat16), seed).to(DEV).eval()


def test_config4_pard_at_size():
    """Batch 16, d = 8, 1024-token prompts, Bernoulli(0.6) acceptance with the configuration's seed, more than
    20 speculative steps: every append / rollback length and both caches' final lengths follow the
    reference's rules per sequence (oracle/pard_ref.py restates generator.py:638-713); then a verify launch
    (9 query tokens, ragged) over the target pool as the run left it, and a decode launch over the draft
    pool, against the oracle.  Real head shapes (32 query / 8 KV heads of 128, draft heads of 64), two
    target layers and one draft layer."""
    from oracle.attention_ref import attend_over_cache
    from oracle.pard_ref import length_trace
    from pace_b200.llm.configs import PardSpecDecodeConfig, SamplingConfig
    from pace_b200.llm.generator import Generator
    from pace_b200.ops import MultiHeadAttention
    B, d, P, new = 16, 8, 1024, 80
    mk = lambda layers, hidden, ffn: Cfg(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers,  # noqa: E731
                                         num_attention_heads=32, num_key_value_heads=8, vocab_size=512,
                                         max_position_embeddings=2048, rope_theta=500000.0, rms_norm_eps=1e-5,
                                         pad_token_id=0)
    cfg_t, cfg_d = mk(2, 4096, 512), mk(1, 2048, 512)
    pc = PardSpecDecodeConfig(num_speculative_tokens=d, pard_token=1, forced_accept_prob=0.6, forced_accept_seed=4)
    gen = Generator(_model(cfg_t, 41), _model(cfg_d, 42), pc)
    prompts = torch.randint(2, 512, (B, P), generator=torch.Generator().manual_seed(4))
    out = gen.generate(prompts, SamplingConfig(max_new_tokens=new))
    keeps = gen.total_speculated_tokens
    steps = len(keeps) // B
    assert steps >= 20
    per_seq = [[keeps[s * B + b] for s in range(steps)] for b in range(B)]
    assert all(1 <= k <= d for k in keeps) and len(set(keeps)) > 3
    tmgr, dmgr = gen.kv_cache_manager, gen.pard_kv_cache_manager
    appends_t = [t[2] for t in gen.trace if t[0] == "target" and t[1] == "append"]
    removes_t = [t[2] for t in gen.trace if t[0] == "target" and t[1] == "remove"]
    appends_d = [t[2] for t in gen.trace if t[0] == "draft" and t[1] == "append"]
    for b in range(B):
        tr = length_trace(P, d, per_seq[b])
        assert tmgr[0].seq_lens[b] == tr[-1]["target_len"] and dmgr[0].seq_lens[b] == tr[-1]["draft_len"]
        assert out.lengths[b] == tr[-1]["history"]
        assert [a[b] for a in appends_t] == [s["target_append"] for s in tr]
        assert [r[b] for r in removes_t] == [s["target_remove"] for s in tr]
        assert [a[b] for a in appends_d] == [s["draft_append"] for s in tr]
    for mgr in (tmgr, dmgr):
        for layer in range(mgr.num_layers):
            assert mgr.pool.seq_len()[layer, :B].tolist() == mgr[layer].seq_lens
        mgr.pool.check_status()
    # the pools as the run left them (ragged lengths after 20+ rollbacks): a verify launch on the target pool ...
    g = torch.Generator().manual_seed(9)
    mha = MultiHeadAttention()
    S = d + 1
    lens_t = tmgr[1].seq_lens
    dk, dv = tmgr[1].read_dense()
    q = torch.randn(B, S, 32, 128, generator=g).bfloat16().to(DEV).transpose(1, 2)
    q_lens = [S if b % 3 else S - 2 for b in range(B)]
    got = mha(q, tmgr[1].key, tmgr[1].value, q_lens=torch.tensor(q_lens, dtype=torch.int32, device=DEV))
    for b in range(B):
        n, s = lens_t[b], q_lens[b]
        want = attend_over_cache(q[b:b + 1, :, :s].cpu(), dk[b:b + 1, :, :n].cpu(), dv[b:b + 1, :, :n].cpu(), n, 0, "native")[0]
        _check(got[b, :, :s], want, ("verify", b))
    # ... and a decode launch on the draft pool (head_dim 64)
    lens_d = dmgr[0].seq_lens
    dk, dv = dmgr[0].read_dense()
    q1 = torch.randn(B, 32, 1, 64, generator=g).bfloat16().to(DEV)
    got = mha(q1, dmgr[0].key, dmgr[0].value)
    for b in range(B):
        n = lens_d[b]
        want = attend_over_cache(q1[b:b + 1].cpu(), dk[b:b + 1, :, :n].cpu(), dv[b:b + 1, :, :n].cpu(), n, 0, "native")[0]
        _check(got[b], want, ("draft decode", b))
