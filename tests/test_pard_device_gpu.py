"""PARD speculative decoding with acceptance, rollback and the next step's ragged counts on the device.

Integers are compared exactly: with the reference generator's recorded runs (tests/golden/pard_trace.json)
and with the restatement of its length rules (oracle/pard_ref.py, generator.py:638-713).  Between the
first step and the last nothing may synchronise with the host: the steps run under torch's
synchronisation check in its "error" mode.
"""
import json
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
G_DIR = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


class Cfg:
    def __init__(self, **kw):
        self.__dict__.update(kw)


def _cfg(layers, hidden, heads, kv_heads, ffn, vocab):
    return Cfg(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers, num_attention_heads=heads,
               num_key_value_heads=kv_heads, vocab_size=vocab, max_position_embeddings=512, rope_theta=500000.0,
               rms_norm_eps=1e-5, pad_token_id=0)


def _model(cfg, seed):
    from pace_b200.llm.models.llama import LlamaForCausalLM, random_init_
    return random_init_(LlamaForCausalLM(cfg).to(torch.bfloat16), seed).to(DEV).eval()


def _run_without_host_syncs(loop, steps):
    """Step 0 is the prompt pass (host-sized, creates the pools).  Every later step runs with the
    synchronisation check armed: a .tolist(), .item(), blocking copy or allocation-by-value would raise."""
    loop.step()
    torch.cuda.synchronize()
    torch.cuda.set_sync_debug_mode("error")
    try:
        loop.run(steps - 1)
    finally:
        torch.cuda.set_sync_debug_mode("default")
    torch.cuda.synchronize()


def _managers(cfg_t, cfg_d, P, new, d):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    tm = KVCacheManager(cfg_t, P + new, KVCacheType.BMC, extra_tokens=d + 1)
    dm = KVCacheManager(cfg_d, P + new, KVCacheType.BMC, extra_tokens=d + 1)
    return tm, dm


@pytest.mark.parametrize("name", ["d8_p20", "d4_p9", "d8_p33"])
def test_device_steps_follow_the_reference_trace(name):
    """The reference generator's recorded run (batch 1): its acceptance counts are fed as forced draws, and
    every append / rollback count and every cache length after it must be the recorded one."""
    from pace_b200.llm.device_loop import PardDeviceLoop
    with open(os.path.join(G_DIR, "pard_trace.json")) as f:
        e = json.load(f)[name]
    d, P, keeps = e["d"], e["prompt_len"], list(e["accepted"])
    steps = len(keeps)
    cfg_t, cfg_d = _cfg(2, 128, 2, 1, 256, 96), _cfg(1, 128, 2, 1, 128, 96)
    forced = torch.zeros(steps, 1, d - 1, dtype=torch.uint8)
    for i, k in enumerate(keeps):
        forced[i, 0, : k - 1] = 1
    tm, dm = _managers(cfg_t, cfg_d, P, e["max_new_tokens"] + steps * d, d)
    prompt = torch.randint(2, 96, (1, P), generator=torch.Generator().manual_seed(1))
    loop = PardDeviceLoop(_model(cfg_t, 2), _model(cfg_d, 3), tm, dm, prompt, d, steps, pard_token=1, forced=forced)
    _run_without_host_syncs(loop, steps)
    hist = loop.finish()
    got = []
    t_app, d_app = loop.log_t_app[:, 0].tolist(), loop.log_d_app[:, 0].tolist()
    t_len, d_len, kp = loop.log_t_len[:, 0].tolist(), loop.log_d_len[:, 0].tolist(), loop.log_keep[:, 0].tolist()
    assert kp == keeps
    for i in range(steps):
        t_rm = d - kp[i] + 1 if kp[i] < d else 0
        got += [["draft", "append", d_app[i], d_len[i] + (d - 1)], ["target", "append", t_app[i], t_len[i] + t_rm],
                ["target", "remove", t_rm, t_len[i]], ["draft", "remove", d - 1, d_len[i]]]
    want = [[ev[0], ev[1], ev[2], ev[4]] for ev in e["events"]]
    assert got == want
    assert len(hist[0]) == P + sum(keeps)
    assert tm[0].seq_lens == [t_len[-1]] and dm[0].seq_lens == [d_len[-1]]          # host mirrors after the one sync
    for mgr in (tm, dm):
        assert mgr.pool.seq_len()[:, 0].tolist() == [c.seq_len for c in mgr.cache_objects]


def test_batched_bernoulli_acceptance_on_the_device():
    """Config-4 shape in miniature (the full size is tests/test_configs_at_size_gpu.py): a batch, seeded
    Bernoulli(0.6) draws per draft token, ragged rollback every step.  Keep counts against the draws, all
    lengths against the reference's rules per sequence, and against the host-driven generator on the same draws."""
    from oracle.pard_ref import keep_len_from_matches, length_trace
    from pace_b200.llm.configs import PardSpecDecodeConfig, SamplingConfig
    from pace_b200.llm.device_loop import PardDeviceLoop
    from pace_b200.llm.generator import Generator
    B, d, P, steps = 4, 8, 30, 14
    cfg_t, cfg_d = _cfg(2, 256, 4, 1, 256, 128), _cfg(1, 128, 2, 1, 128, 128)
    target, draft = _model(cfg_t, 4), _model(cfg_d, 5)
    g = torch.Generator().manual_seed(5)
    draws = torch.stack([torch.stack([torch.rand(d - 1, generator=g) < 0.6 for _ in range(B)]) for _ in range(steps)])
    tm, dm = _managers(cfg_t, cfg_d, P, steps * d, d)
    prompts = torch.randint(2, 128, (B, P), generator=torch.Generator().manual_seed(2))
    loop = PardDeviceLoop(target, draft, tm, dm, prompts, d, steps, pard_token=1, forced=draws.to(torch.uint8))
    _run_without_host_syncs(loop, steps)
    hist = loop.finish()
    keeps = loop.log_keep.tolist()
    assert len({k for row in keeps for k in row}) > 2                          # rollback really was ragged
    for b in range(B):
        per_seq = [keeps[i][b] for i in range(steps)]
        assert per_seq == [keep_len_from_matches(draws[i, b].tolist(), d) for i in range(steps)]
        tr = length_trace(P, d, per_seq)
        assert loop.log_t_app[:, b].tolist() == [s["target_append"] for s in tr]
        assert loop.log_d_app[:, b].tolist() == [s["draft_append"] for s in tr]
        assert loop.log_t_len[:, b].tolist() == [s["target_len"] for s in tr]
        assert loop.log_d_len[:, b].tolist() == [s["draft_len"] for s in tr]
        assert len(hist[b]) == tr[-1]["history"] and hist[b][:P] == prompts[b].tolist()
        assert tm[0].seq_lens[b] == tr[-1]["target_len"] and dm[0].seq_lens[b] == tr[-1]["draft_len"]
    for mgr in (tm, dm):
        for layer in range(mgr.num_layers):
            assert mgr.pool.seq_len()[layer, :B].tolist() == mgr[layer].seq_lens
    # the host-driven generator on the same draws (same seed, same order) keeps the same counts
    pc = PardSpecDecodeConfig(num_speculative_tokens=d, pard_token=1, forced_accept_prob=0.6, forced_accept_seed=5)
    gen = Generator(target, draft, pc)
    gen.generate(prompts, SamplingConfig(max_new_tokens=steps))               # runs at least steps / d ... steps steps
    n_host = len(gen.total_speculated_tokens) // B
    assert n_host >= 2
    for i in range(min(n_host, steps)):
        assert gen.total_speculated_tokens[i * B:(i + 1) * B] == keeps[i]


def test_pard_accept_kernel_token_comparison():
    """Without forced draws a draft is accepted while it equals the target's token (generator.py:684-693)."""
    from oracle.pard_ref import keep_len_from_matches, rollback_lengths
    B, d = 6, 5
    g = torch.Generator().manual_seed(0)
    drafts = torch.randint(0, 3, (B, d), generator=g)
    target = torch.randint(0, 3, (B, d + 1), generator=g)
    target[0, : d - 1] = drafts[0, : d - 1]                                      # everything matches
    target[1, 0] = drafts[1, 0] + 1                                              # nothing does
    n_t = torch.tensor([d + 1, d + 1, d, d + 1, 2, d + 1], dtype=torch.int32)
    keep = torch.zeros(B, dtype=torch.int32, device=DEV)
    t_rm, d_rm = torch.zeros_like(keep), torch.zeros_like(keep)
    kept = torch.full((B, d), -1, dtype=torch.long, device=DEV)
    torch.ops.pace_b200.pard_accept(drafts.to(DEV), target.to(DEV), n_t.to(DEV), None, keep, t_rm, d_rm, kept)
    for b in range(B):
        nt = int(n_t[b])
        matches = [i < nt and int(target[b, i]) == int(drafts[b, i]) for i in range(d - 1)]
        k = keep_len_from_matches(matches, d)
        assert int(keep[b]) == k
        assert (int(t_rm[b]), int(d_rm[b])) == rollback_lengths(d, k)
        want = target[b, : k - 1].tolist() + [int(target[b, min(k - 1, nt - 1)])]
        assert kept[b, :k].tolist() == want
