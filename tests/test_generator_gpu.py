"""Generation loop and PARD rollback accounting vs the reference generator's recorded traces."""
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


def test_greedy_decode_lengths_and_cache():
    from pace_b200.llm.generator import Generator
    from pace_b200.llm.configs import SamplingConfig
    cfg = _cfg(2, 128, 2, 1, 256, 64)
    gen = Generator(_model(cfg, 1))
    prompts = torch.randint(1, 64, (3, 17), generator=torch.Generator().manual_seed(0))
    out = gen.generate(prompts, SamplingConfig(max_new_tokens=9))
    assert out.lengths == [26, 26, 26] and torch.equal(out.output_token_ids[:, :17], prompts)
    # the last generated token is never fed back: the cache holds prompt + 8
    assert gen.kv_cache_manager[0].seq_lens == [25, 25, 25]
    assert [t[2] for t in gen.trace if t[1] == "append"] == [[17] * 3] + [[1] * 3] * 8


@pytest.mark.parametrize("name", ["d8_p20", "d4_p9", "d8_p33"])
def test_pard_cache_lengths_follow_the_reference_trace(name):
    """Force, step by step, the acceptance counts the reference run produced and compare every
    append / remove length and the resulting cache length and capacity with its recorded events."""
    from pace_b200.llm.generator import Generator
    from pace_b200.llm.configs import PardSpecDecodeConfig, SamplingConfig
    with open(os.path.join(G_DIR, "pard_trace.json")) as f:
        e = json.load(f)[name]
    d = e["d"]
    cfg_t = _cfg(2, 128, 2, 1, 256, 96)
    cfg_d = _cfg(1, 128, 2, 1, 128, 96)
    gen = Generator(_model(cfg_t, 2), _model(cfg_d, 3), PardSpecDecodeConfig(num_speculative_tokens=d, pard_token=1))
    prompt = torch.randint(2, 96, (1, e["prompt_len"]), generator=torch.Generator().manual_seed(1))
    gen.prepare_for_generate(prompt, SamplingConfig(max_new_tokens=e["max_new_tokens"]))
    # forced acceptance: replay the reference's keep counts exactly
    keeps = list(e["accepted"])

    class Replay:
        def __init__(self):
            self.i = 0
    rep = Replay()
    orig = gen._postprocess_speculated_tokens

    def forced(next_tokens, drafts):
        keep = keeps[rep.i]
        rep.i += 1
        nt = [list(drafts[0][: keep - 1]) + next_tokens[0][keep - 1:]]     # make the first keep-1 drafts "match"
        dr = [list(drafts[0])]
        if keep - 1 < d - 1:
            nt[0][keep - 1] = dr[0][keep - 1] + 1                          # and the next one differ
        return orig(nt, dr)

    gen._postprocess_speculated_tokens = forced
    events = []
    history = [prompt[0].tolist()]
    steps = 0
    with torch.inference_mode():
        while steps < len(keeps):
            drafts = gen._speculate_tokens(history)
            events.append(["draft", "append", gen.trace[-1][2][0], gen.pard_kv_cache_manager[0].seq_len,
                           gen.pard_kv_cache_manager[0].capacity])
            logits, counts = gen._run_ragged(gen.model, gen.kv_cache_manager, "target", history, drafts)
            events.append(["target", "append", counts[0], gen.kv_cache_manager[0].seq_len,
                           gen.kv_cache_manager[0].capacity])
            n = counts[0]
            take = min(d + 1, n)
            nxt = [logits[0, n - take: n].float().argmax(-1).tolist()]
            kept = gen._postprocess_speculated_tokens(nxt, drafts)
            events.append(["target", "remove", gen.trace[-2][2][0], gen.kv_cache_manager[0].seq_len,
                           gen.kv_cache_manager[0].capacity])
            events.append(["draft", "remove", gen.trace[-1][2][0], gen.pard_kv_cache_manager[0].seq_len,
                           gen.pard_kv_cache_manager[0].capacity])
            history[0] = history[0] + kept[0]
            steps += 1
    want = [[ev[0], ev[1], ev[2], ev[4], ev[5]] for ev in e["events"]]
    assert events == want
    # the device-resident lengths agree with the host mirror
    for mgr in (gen.kv_cache_manager, gen.pard_kv_cache_manager):
        assert mgr.pool.seq_len()[:, 0].tolist() == [c.seq_len for c in mgr.cache_objects]
        mgr.pool.check_status()


def test_batched_pard_with_forced_bernoulli_acceptance():
    """Config-4 shape in miniature: batch of sequences, seeded Bernoulli(0.6) acceptance, ragged
    rollback on every step; lengths must follow the reference's rules per sequence."""
    from pace_b200.llm.generator import Generator
    from pace_b200.llm.configs import PardSpecDecodeConfig, SamplingConfig
    from oracle.pard_ref import length_trace
    B, d, P, new = 4, 8, 30, 40
    cfg_t = _cfg(2, 256, 4, 1, 256, 128)        # head_dim 64, G = 4
    cfg_d = _cfg(1, 128, 2, 1, 128, 128)
    pc = PardSpecDecodeConfig(num_speculative_tokens=d, pard_token=1, forced_accept_prob=0.6, forced_accept_seed=5)
    gen = Generator(_model(cfg_t, 4), _model(cfg_d, 5), pc)
    prompts = torch.randint(2, 128, (B, P), generator=torch.Generator().manual_seed(2))
    out = gen.generate(prompts, SamplingConfig(max_new_tokens=new))
    keeps = gen.total_speculated_tokens
    steps = len(keeps) // B
    per_seq = [[keeps[s * B + b] for s in range(steps)] for b in range(B)]
    assert all(1 <= k <= d for k in keeps) and len(set(keeps)) > 2          # rollback really was ragged
    for b in range(B):
        tr = length_trace(P, d, per_seq[b])
        assert gen.kv_cache_manager[0].seq_lens[b] == tr[-1]["target_len"]
        assert gen.pard_kv_cache_manager[0].seq_lens[b] == tr[-1]["draft_len"]
        assert out.lengths[b] == tr[-1]["history"]
    appends_t = [t[2] for t in gen.trace if t[0] == "target" and t[1] == "append"]
    removes_t = [t[2] for t in gen.trace if t[0] == "target" and t[1] == "remove"]
    for b in range(B):
        tr = length_trace(P, d, per_seq[b])
        assert [a[b] for a in appends_t] == [s["target_append"] for s in tr]
        assert [r[b] for r in removes_t] == [s["target_remove"] for s in tr]
    assert gen.kv_cache_manager.pool.seq_len()[0, :B].tolist() == gen.kv_cache_manager[0].seq_lens
    assert 1.0 < out.speculative_stats.mean_accepted_tokens < d


def _golden_model(case):
    from pace_b200.llm.models.llama import LlamaForCausalLM
    cfg = Cfg(**case["cfg"], pad_token_id=0)
    m = LlamaForCausalLM(cfg).to(torch.bfloat16)
    m.load_state_dict(case["state"], strict=True)
    return m.to(DEV).eval(), cfg


def test_beam_loop_follows_the_reference_run():
    """The reference model and the reference cache manager were driven through a 3-beam search on the CPU
    (tests/golden/make_golden_beam.py: the cache follows the beams by index_select of every layer's K/V).
    Teacher-forced with its token ids and beam indices, the paged cache - where the gather only permutes
    block-table rows and the shared pages are copied on the next write - gives the same logits step by
    step and ends with the same contents."""
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    case = torch.load(os.path.join(G_DIR, "beam_loop_case.pt"))
    model, cfg = _golden_model(case)
    steps, nb = case["steps"], case["num_beams"]
    P = case["prompts"].shape[1]
    mgr = KVCacheManager(cfg, P + steps, KVCacheType.BMC)
    shared_seen = 0
    with torch.inference_mode():
        for t in range(steps):
            ids = case["ids"][t].to(DEV)
            out = model(ids, kv_cache=mgr, attention_mask=torch.ones_like(ids))
            got = out.logits[:, -1].float().cpu()
            err = (got - case["logits"][t]).abs()
            assert err.max().item() < 2e-2 and err.mean().item() < 2e-3, (t, err.max().item(), err.mean().item())
            mgr.update_cache_with_beam_indices(case["beam_idx"][t].to(DEV))
            shared_seen = max(shared_seen, int(mgr.pool.page_ref().max().item()))
    assert mgr.pool.shared_pages and shared_seen > 1            # beams did share pages, appends did copy on write
    assert len(mgr) == case["seq_len"]
    n = case["seq_len"]
    for layer in range(2):
        dk, dv = mgr[layer].read_dense()
        assert (dk[:, :, :n].float().cpu() - case["k_cache"][layer].float()).abs().max().item() < 4e-2
        assert (dv[:, :, :n].float().cpu() - case["v_cache"][layer].float()).abs().max().item() < 4e-2
    mgr.pool.check_status()


def test_beam_search_generate_calls_the_gather_every_step():
    from pace_b200.llm.generator import Generator
    from pace_b200.llm.configs import SamplingConfig
    case = torch.load(os.path.join(G_DIR, "beam_loop_case.pt"))
    model, cfg = _golden_model(case)
    gen = Generator(model)
    nb, steps = case["num_beams"], 6
    out = gen.generate(case["prompts"], SamplingConfig(max_new_tokens=steps, num_beams=nb))
    B, P = case["prompts"].shape
    assert out.output_token_ids.shape == (B, P + steps) and torch.equal(out.output_token_ids[:, :P], case["prompts"])
    gathers = [t for t in gen.trace if t[1] == "gather"]
    assert len(gathers) == steps and all(len(g[2]) == B * nb for g in gathers)
    # every beam index names a beam of the same prompt
    for g in gathers:
        assert all(i // nb == j // nb for j, i in enumerate(g[2]))
    # the first step starts from identical beams: all survivors continue beam 0 of their prompt, as in the reference run
    assert gathers[0][2] == case["beam_idx"][0].tolist()
    assert gen.kv_cache_manager[0].seq_lens == [P + steps - 1] * (B * nb)   # the last token is never fed back
    # the re-ranking itself, against the recorded step of the reference run (CPU arithmetic on recorded logits)
    scores = torch.zeros(B, nb)
    scores[:, 1:] = -1e9
    bi, tok, _ = Generator.beam_step(case["logits"][0], scores.view(-1), nb)
    assert torch.equal(bi, case["beam_idx"][0]) and torch.equal(tok, case["tokens"][0])
