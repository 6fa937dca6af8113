"""Device-resident greedy loop (one CUDA graph per token) against the host-driven generator."""
import pytest
import torch

pytestmark = pytest.mark.gpu
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


def _prefill(model, prompts, max_new):
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    mgr = KVCacheManager(model.config, prompts.shape[1] + max_new, KVCacheType.BMC)
    with torch.inference_mode():
        logits = model(prompts.to(DEV), mgr, torch.ones_like(prompts).to(DEV)).logits
    return mgr, logits[:, -1].float().argmax(dim=-1)


def test_device_loop_reproduces_the_host_loop_token_for_token():
    from pace_b200.llm.configs import SamplingConfig
    from pace_b200.llm.device_loop import GreedyDeviceLoop
    from pace_b200.llm.generator import Generator
    cfg = _cfg(2, 256, 2, 1, 512, 97)          # head_dim 128, one KV head
    model = _model(cfg, 5)
    prompts = torch.randint(1, 97, (4, 21), generator=torch.Generator().manual_seed(3))
    N = 24
    want = Generator(model).generate(prompts, SamplingConfig(max_new_tokens=N)).output_token_ids[:, 21:]
    mgr, first = _prefill(model, prompts, N)
    assert torch.equal(first.cpu(), want[:, 0])
    loop = GreedyDeviceLoop(model, mgr, first, torch.full((4,), 21, device=DEV), max_new_tokens=N - 1)
    got = loop.run(poll_every=5)
    assert torch.equal(got.cpu(), want[:, 1:])
    # the last generated token is never fed back: prompt + first token + N - 2 more
    assert mgr[0].seq_lens == [21 + N - 1] * 4
    assert int(loop.step.item()) == N - 1


def test_device_loop_stops_on_eos_and_pads_behind_it():
    from pace_b200.llm.device_loop import GreedyDeviceLoop
    cfg = _cfg(1, 128, 1, 1, 256, 50)
    model = _model(cfg, 8)
    prompts = torch.randint(1, 50, (3, 9), generator=torch.Generator().manual_seed(4))
    N = 20
    mgr, first = _prefill(model, prompts, N + 1)
    free = GreedyDeviceLoop(model, mgr, first, torch.full((3,), 9, device=DEV), max_new_tokens=N).run().cpu()
    eos = int(free[0, 6])                       # a token sequence 0 emits at step 6 (maybe earlier too)
    mgr2, first2 = _prefill(model, prompts, N + 1)
    loop = GreedyDeviceLoop(model, mgr2, first2, torch.full((3,), 9, device=DEV), max_new_tokens=N,
                            eos_token_ids=[eos], pad_token_id=0)
    got = loop.run(poll_every=4).cpu()
    lens = loop.lengths()
    for b in range(3):
        row = free[b].tolist()
        stop = next((i + 1 for i, t in enumerate(row) if t == eos), None)
        if stop is None:
            continue
        assert lens[b] == stop
        assert got[b, :stop].tolist() == row[:stop]
        assert got[b, stop: loop.produced].eq(0).all()
    assert lens[0] <= 7


def test_device_loop_teacher_forced_against_the_reference_run(golden_dir):
    """The recorded run of the reference model on the CPU (tests/golden/llama_case.pt: its state dict, its
    token ids, its logits after the prompt and after each of three decode steps): the device-resident step
    is fed the reference's own next token before every replay, so its last-position logits stay comparable
    with the recorded ones step by step; cache lengths and capacity end as the reference's BMC cache did."""
    import os
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from pace_b200.llm.device_loop import GreedyDeviceLoop
    from pace_b200.llm.models.llama import LlamaForCausalLM
    case = torch.load(os.path.join(golden_dir, "llama_case.pt"))
    cfg = Cfg(**case["cfg"], pad_token_id=0)
    model = LlamaForCausalLM(cfg).to(torch.bfloat16)
    model.load_state_dict(case["state"], strict=True)
    model = model.to(DEV).eval()
    ids, P, steps = case["ids"].to(DEV), case["prompt_len"], case["steps"]
    B = ids.shape[0]

    def close(got, want, what):
        err = (got.float().cpu() - want).abs()
        assert err.max().item() < 2e-2 and err.mean().item() < 2e-3, (what, err.max().item(), err.mean().item())

    mgr = KVCacheManager(cfg, P + steps, KVCacheType.BMC)
    with torch.inference_mode():
        out = model(ids[:, :P], kv_cache=mgr, attention_mask=torch.ones(B, P, dtype=torch.long, device=DEV))
    close(out.logits[:, -1], case["logits"][0], "prompt")
    # the loop's warm-up step is decode step 1: it is given the reference's token, not the argmax
    loop = GreedyDeviceLoop(model, mgr, ids[:, P], torch.full((B,), P, device=DEV), max_new_tokens=steps,
                            keep_logits=True)
    close(loop.logits, case["logits"][1], "step 1")
    for t in range(2, steps + 1):
        loop.cur.copy_(ids[:, P + t - 1: P + t])            # teacher forcing: overwrite the token the step chose
        loop.graph.replay()
        torch.cuda.synchronize()
        close(loop.logits, case["logits"][t], f"step {t}")
    assert len(mgr) == case["seq_len"] and mgr[0].capacity == case["capacity"]
    assert mgr.pool.seq_len()[:, :B].tolist() == [[case["seq_len"]] * B] * cfg.num_hidden_layers
    n = case["seq_len"]
    for layer in range(2):
        dk, dv = mgr[layer].read_dense()
        assert (dk[:, :, :n].float().cpu() - case["k_cache"][layer].float()).abs().max().item() < 4e-2
        assert (dv[:, :, :n].float().cpu() - case["v_cache"][layer].float()).abs().max().item() < 4e-2
    mgr.pool.check_status()
