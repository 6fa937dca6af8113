"""The re-hosted Llama (caller of the hot path) vs the reference model's recorded run."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
G_DIR = os.path.join(os.path.dirname(__file__), "golden")
DEV = "cuda:0"


class Cfg:
    pass


def _model(case):
    from pace_b200.llm.models.llama import LlamaForCausalLM
    cfg = Cfg()
    for k, v in case["cfg"].items():
        setattr(cfg, k, v)
    cfg.pad_token_id = 0
    m = LlamaForCausalLM(cfg).to(torch.bfloat16)
    missing, unexpected = m.load_state_dict(case["state"], strict=True)
    return m.to(DEV).eval(), cfg


def test_prefill_and_decode_follow_the_reference_run():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    case = torch.load(os.path.join(G_DIR, "llama_case.pt"))
    model, cfg = _model(case)
    ids = case["ids"].to(DEV)
    P, steps = case["prompt_len"], case["steps"]
    mgr = KVCacheManager(cfg, P + steps, KVCacheType.BMC)
    mask = torch.ones(ids.shape[0], P, dtype=torch.long, device=DEV)
    with torch.inference_mode():
        for t in range(steps + 1):
            # teacher-forced: the reference's own token ids are fed, so the logits stay comparable
            out = model(ids[:, : P + t], kv_cache=mgr, attention_mask=mask)
            got = out.logits[:, -1].float().cpu()
            want = case["logits"][t]
            err = (got - want).abs()
            assert err.max().item() < 2e-2 and err.mean().item() < 2e-3, (t, err.max().item(), err.mean().item())
            mask = torch.cat([mask, mask.new_ones(mask.shape[0], 1)], dim=-1)
    # lengths / capacity as the reference's BMC cache; contents within GEMM rounding of the CPU run
    assert len(mgr) == case["seq_len"] and mgr[0].capacity == case["capacity"]
    for layer in range(2):
        dk, dv = mgr[layer].read_dense()
        n = case["seq_len"]
        assert (dk[:, :, :n].float().cpu() - case["k_cache"][layer].float()).abs().max().item() < 4e-2
        assert (dv[:, :, :n].float().cpu() - case["v_cache"][layer].float()).abs().max().item() < 4e-2
    mgr.pool.check_status()


def test_left_padded_batch_equals_per_sequence_runs():
    # reference semantics: lengths are equalised by left padding, pad positions are cached and masked
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    case = torch.load(os.path.join(G_DIR, "llama_case.pt"))
    model, cfg = _model(case)
    g = torch.Generator().manual_seed(3)
    lens = [9, 14]
    seqs = [torch.randint(1, cfg.vocab_size, (n,), generator=g) for n in lens]
    L = max(lens)
    ids = torch.zeros(2, L, dtype=torch.long)
    mask = torch.zeros(2, L, dtype=torch.long)
    for b, s in enumerate(seqs):
        ids[b, L - len(s):] = s
        mask[b, L - len(s):] = 1
    with torch.inference_mode():
        mgr = KVCacheManager(cfg, L + 4, KVCacheType.BMC)
        batched = model(ids.to(DEV), kv_cache=mgr, attention_mask=mask.to(DEV)).logits[:, -1].float().cpu()
        for b, s in enumerate(seqs):
            m1 = KVCacheManager(cfg, L + 4, KVCacheType.BMC)
            one = model(s[None].to(DEV), kv_cache=m1, attention_mask=torch.ones(1, len(s), dtype=torch.long, device=DEV))
            err = (one.logits[0, -1].float().cpu() - batched[b]).abs()
            assert err.max().item() < 2e-2


def test_ragged_forward_equals_per_sequence_runs():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    case = torch.load(os.path.join(G_DIR, "llama_case.pt"))
    model, cfg = _model(case)
    g = torch.Generator().manual_seed(4)
    first, second = [12, 5], [3, 9]
    seqs = [torch.randint(1, cfg.vocab_size, (first[b] + second[b],), generator=g) for b in range(2)]
    with torch.inference_mode():
        mgr = KVCacheManager(cfg, 64, KVCacheType.BMC)
        for counts, off in ((first, [0, 0]), (second, first)):
            n_max = max(counts)
            new = torch.zeros(2, n_max, dtype=torch.long)
            for b in range(2):
                new[b, : counts[b]] = seqs[b][off[b]: off[b] + counts[b]]
            out = model.forward_ragged(new.to(DEV), counts, mgr)
        assert mgr[0].seq_lens == [15, 14]
        for b in range(2):
            m1 = KVCacheManager(cfg, 64, KVCacheType.BMC)
            one = model(seqs[b][None].to(DEV), kv_cache=m1,
                        attention_mask=torch.ones(1, len(seqs[b]), dtype=torch.long, device=DEV))
            err = (one.logits[0, -1].float() - out.logits[b, second[b] - 1].float()).abs()
            assert err.max().item() < 2e-2
