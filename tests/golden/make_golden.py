"""Generates the golden vectors under tests/golden/ by RUNNING THE REFERENCE.

Run where the reference source tree is present (it is found through
$PACE_REF_ROOT):

    python tests/golden/make_golden.py

It imports the reference's own, unmodified Python modules (pace/llm/cache.py,
pace/ops/attention.py + the NATIVE backend, pace/llm/models/llama.py,
pace/llm/generator.py) through oracle/ref_loader.py and records what they
produce on seeded inputs:

  cache_traces.json   seq_len / capacity / mask-width traces of BMCKVCache and
                      DynamicKVCache for scripted append/remove sequences,
                      including the known-answer case of the reference's
                      tests/llm_infra/test_cache.py:53-64,76-80.
  decode_case.pt      a reduced config-1 case: ragged per-sequence caches,
                      one-token append, attention over the full cache through
                      MultiHeadAttention(NATIVE); inputs, outputs, cache contents.
  verify_case.pt      the same with S = 9 query tokens (PARD verify shape) and
                      a left-padded batch.
  beam_case.pt        update_cache_with_beam_indices on a small cache.
  pard_trace.json     append / remove lengths of the target and draft caches
                      recorded from the reference generator's own PARD loop on
                      tiny random Llama models.
  llama_case.pt       a tiny random Llama (2 layers) run through the reference
                      model: weights, token ids, logits and layer caches after
                      prefill and three decode steps.

The vectors are small (about 1.5 MB in total) and are committed; the GPU
box has no reference tree, so the tests there read only these files.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, "..", "..")))

from oracle import ref_loader  # noqa: E402


def cache_traces(ref):
    scripts = {
        "known_answer_128": dict(max_len=128, ops=[("append", 10)]),
        "decode_768": dict(max_len=768, ops=[("append", 512)] + [("append", 1)] * 60),
        "boundary_equal": dict(max_len=1024, ops=[("append", 24), ("append", 8), ("append", 1),
                                                  ("remove", 9), ("append", 40)]),
        "pard_like": dict(max_len=84, ops=[("append", 28), ("remove", 8), ("append", 9), ("remove", 3),
                                           ("append", 9), ("append", 8), ("remove", 8)]),
        "over_remove": dict(max_len=64, ops=[("append", 5), ("remove", 6), ("remove", 5), ("append", 3)]),
        "remove_on_empty": dict(max_len=64, ops=[("remove", 4), ("append", 7), ("remove", 7), ("append", 2)]),
        "chunked_prefill": dict(max_len=8192 + 64, ops=[("append", 512)] * 9 + [("append", 37)] + [("append", 1)] * 5),
    }
    out = {}
    for name, sc in scripts.items():
        for policy, cls in (("bmc", ref.BMCKVCache), ("dynamic", ref.DynamicKVCache)):
            c = cls(sc["max_len"])
            trace = []
            for kind, n in sc["ops"]:
                if kind == "append":
                    x = torch.zeros(1, 1, n, 2, dtype=torch.bfloat16)
                    k, _ = c.update_cache(x, x.clone(), concat_dim=2)
                    trace.append([int(c.seq_len), int(k.shape[2])])
                else:
                    try:
                        c.remove_cache(n)
                        cap = 0 if c.key is None else int(c.key.shape[2])
                        trace.append([int(c.seq_len), cap])
                    except ValueError as e:
                        trace.append(["error", str(e)])
            entry = dict(max_len=sc["max_len"], ops=sc["ops"], trace=trace)
            if policy == "bmc":
                entry["tokens_per_split"] = int(c.tokens_per_split)
                entry["mask_width"] = {
                    str(n): int(c.update_mask(torch.ones(2, n), n).shape[-1]) for n in (1, 10, 11, 12, 100)
                }
            out[f"{name}/{policy}"] = entry
    # the reference test's own shapes: 3-D tensors, concat_dim=1
    c = ref.BMCKVCache(128)
    k, v = c.update_cache(torch.rand(2, 10, 64), torch.rand(2, 10, 64), concat_dim=1)
    out["test_cache_py/bmc"] = dict(key_len=int(k.shape[1]), mask_w=int(c.update_mask(torch.ones(2, 10), 10).shape[-1]))
    c = ref.DynamicKVCache(128)
    k, v = c.update_cache(torch.rand(2, 10, 64), torch.rand(2, 10, 64), concat_dim=1)
    out["test_cache_py/dynamic"] = dict(key_len=int(k.shape[1]))
    return out


def _to4d(mask2d, q_len, kv_len, dtype):
    from transformers.modeling_attn_mask_utils import AttentionMaskConverter
    return AttentionMaskConverter(is_causal=True).to_4d(mask2d, q_len, key_value_length=kv_len, dtype=dtype)


def attention_case(ref, seed, B, Hq, Hkv, D, lens, S, max_len, left_pad=None):
    """Per sequence (the reference shares one length across a batch): fill a
    BMC cache with the existing tokens, append the S new ones, attend."""
    g = torch.Generator().manual_seed(seed)
    mha = ref.MultiHeadAttention(backend_impl=ref.BackendType.NATIVE, dtype=torch.bfloat16)
    rep = Hq // Hkv
    case = dict(B=B, Hq=Hq, Hkv=Hkv, D=D, S=S, max_len=max_len, lens=list(lens),
                left_pad=list(left_pad) if left_pad else [0] * B,
                k_new=[], v_new=[], q=[], out=[], k_cache=[], v_cache=[], capacity=[])
    for b in range(B):
        L = lens[b]
        k_old = torch.randn(1, Hkv, L, D, generator=g).bfloat16()
        v_old = torch.randn(1, Hkv, L, D, generator=g).bfloat16()
        k_new = torch.randn(1, Hkv, S, D, generator=g).bfloat16()
        v_new = torch.randn(1, Hkv, S, D, generator=g).bfloat16()
        q = torch.randn(1, Hq, S, D, generator=g).bfloat16()
        cache = ref.BMCKVCache(max_len)
        cache.update_cache(ref.repeat_kv(k_old, rep), ref.repeat_kv(v_old, rep), concat_dim=2)
        K, V = cache.update_cache(ref.repeat_kv(k_new, rep), ref.repeat_kv(v_new, rep), concat_dim=2)
        m2 = torch.ones(1, L + S, dtype=torch.long)
        if left_pad:
            m2[:, : left_pad[b]] = 0
        m4 = _to4d(m2, S, L + S, torch.bfloat16)
        m4 = cache.update_mask(m4, L + S)
        out = mha(q, K, V, attention_mask=m4)
        # heads 4g..4g+3 of the reference cache are copies of KV head g
        assert torch.equal(K[:, ::rep], K[:, rep - 1::rep])
        # k_old / v_old are rows [0, L) of the stored caches, so they are not stored twice
        for key, val in (("k_new", k_new), ("v_new", v_new), ("q", q),
                         ("out", out), ("k_cache", K[:, ::rep].clone()), ("v_cache", V[:, ::rep].clone())):
            case[key].append(val[0].clone())
        case["capacity"].append(int(K.shape[2]))
    return case


def beam_case(ref):
    g = torch.Generator().manual_seed(7)
    c = ref.BMCKVCache(64)
    k = torch.randn(4, 2, 13, 16, generator=g).bfloat16()
    v = torch.randn(4, 2, 13, 16, generator=g).bfloat16()
    c.update_cache(k, v, concat_dim=2)
    idx = torch.tensor([2, 2, 0, 3])
    c.update_cache_with_beam_indices(idx)
    k2 = torch.randn(4, 2, 1, 16, generator=g).bfloat16()
    v2 = torch.randn(4, 2, 1, 16, generator=g).bfloat16()
    K, V = c.update_cache(k2, v2, concat_dim=2)
    idx2 = torch.tensor([1, 0, 0, 2])
    c.update_cache_with_beam_indices(idx2)
    return dict(k=k, v=v, idx=idx, k2=k2, v2=v2, idx2=idx2, K=c.key.clone(), V=c.value.clone(),
                seq_len=int(c.seq_len), max_len=64)


def tiny_llama_config(layers, hidden, heads, kv_heads, ffn, vocab, max_pos=512):
    from transformers import PretrainedConfig

    class Cfg(PretrainedConfig):
        pass

    cfg = Cfg()
    for k, v in dict(hidden_size=hidden, intermediate_size=ffn, num_hidden_layers=layers,
                     num_attention_heads=heads, num_key_value_heads=kv_heads, vocab_size=vocab,
                     max_position_embeddings=max_pos, rope_theta=500000.0, rope_scaling=None,
                     attention_bias=False, mlp_bias=False, hidden_act="silu", rms_norm_eps=1e-5,
                     tie_word_embeddings=False, architectures=["LlamaForCausalLM"], pad_token_id=0).items():
        setattr(cfg, k, v)
    return cfg


def build_ref_llama(ref, cfg, seed):
    torch.manual_seed(seed)
    opc = ref.OperatorConfig().finalize()
    model = ref.LlamaForCausalLM(cfg, opc).to(torch.bfloat16).eval()
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() >= 2:
                p.copy_((torch.randn(p.shape, generator=g) * 0.02).to(p.dtype))
            else:
                p.copy_((1.0 + 0.1 * torch.randn(p.shape, generator=g)).to(p.dtype))
    return model


def llama_case(ref):
    cfg = tiny_llama_config(layers=2, hidden=128, heads=2, kv_heads=1, ffn=256, vocab=64)
    model = build_ref_llama(ref, cfg, seed=11)
    g = torch.Generator().manual_seed(12)
    B, P, steps = 2, 21, 3
    ids = torch.randint(1, cfg.vocab_size, (B, P + steps), generator=g)
    mask = torch.ones(B, P, dtype=torch.long)
    mgr = ref.KVCacheManager(cfg, P + steps, ref.KVCacheType.BMC)
    logits = []
    with torch.inference_mode():
        for t in range(steps + 1):
            out = model(ids[:, : P + t], kv_cache=mgr, attention_mask=mask)
            logits.append(out.logits[:, -1].float().clone())
            mask = torch.cat([mask, mask.new_ones(B, 1)], dim=-1)
    rep = cfg.num_attention_heads // cfg.num_key_value_heads
    n = int(mgr[0].seq_len)
    state = {k: v.detach().clone() for k, v in model.state_dict().items()}
    return dict(cfg={k: getattr(cfg, k) for k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                                  "num_attention_heads", "num_key_value_heads", "vocab_size",
                                                  "max_position_embeddings", "rope_theta", "rms_norm_eps")},
                state=state, ids=ids, prompt_len=P, steps=steps, logits=torch.stack(logits),
                k_cache=[mgr[i].key[:, ::rep, :n].clone() for i in range(2)],
                v_cache=[mgr[i].value[:, ::rep, :n].clone() for i in range(2)],
                seq_len=n, capacity=int(mgr[0].key.shape[2]))


def pard_trace(ref):
    """Drives the reference Generator's own speculate / verify / rollback code."""
    from pace.llm.generator import Generator
    from pace.llm.configs import PardSpecDecodeConfig
    cfg_t = tiny_llama_config(layers=2, hidden=128, heads=4, kv_heads=2, ffn=256, vocab=96)
    cfg_d = tiny_llama_config(layers=1, hidden=64, heads=4, kv_heads=2, ffn=128, vocab=96)
    events = []

    def spy(mgr, tag):
        for i, c in enumerate(mgr.cache_objects[:1]):
            up, rm = c.update_cache, c.remove_cache

            def up2(k, v, concat_dim, _up=up, _c=c):
                before = int(_c.seq_len)
                r = _up(k, v, concat_dim=concat_dim)
                events.append([tag, "append", int(k.shape[2]), before, int(_c.seq_len), int(r[0].shape[2])])
                return r

            def rm2(n, _rm=rm, _c=c):
                before = int(_c.seq_len)
                _rm(n)
                events.append([tag, "remove", int(n), before, int(_c.seq_len), int(_c.key.shape[2])])

            c.update_cache, c.remove_cache = up2, rm2

    results = {}
    for d, prompt_len, new_tokens, seed, same in ((8, 20, 12, 3, False), (4, 9, 14, 5, True), (8, 33, 24, 9, True)):
        events.clear()
        gen = object.__new__(Generator)
        gen.model = build_ref_llama(ref, cfg_t, seed)
        # an independent random draft almost never agrees with the target; a copy of
        # the target agrees on the first draft token and now and then on more
        gen.pard_model = build_ref_llama(ref, cfg_t, seed) if same else build_ref_llama(ref, cfg_d, seed + 100)
        gen.pard_config = PardSpecDecodeConfig(model_name_or_path="unused", num_speculative_tokens=d)
        gen.pard_config.pard_token = 1
        gen.kv_cache_type = ref.KVCacheType.BMC
        gen.text_streamer = None
        gen.tokenizer = None
        from pace.llm.configs import SamplingConfig
        from pace.llm.sampler import Sampler
        from pace.llm.stopping_criteria import StoppingCriteria
        g = torch.Generator().manual_seed(seed)
        prompt = torch.randint(2, cfg_t.vocab_size, (1, prompt_len), generator=g)
        sc = SamplingConfig(max_new_tokens=new_tokens, do_sample=False, pad_token_id=0, eos_token_id=[10 ** 6])
        sc.finalize()
        gen.sampling_config = sc
        gen.sampler = Sampler(sc, prompt)
        gen.attention_mask = torch.ones(1, prompt_len, dtype=torch.long)
        gen._prepare_kv_cache(gen.kv_cache_type, prompt)
        gen.stopping_criteria = StoppingCriteria(sc, prompt, None)
        gen._prepare_for_pard(prompt)
        spy(gen.kv_cache_manager, "target")
        spy(gen.pard_kv_cache_manager, "draft")
        with torch.inference_mode():
            out = gen._generate(prompt)
        results[f"d{d}_p{prompt_len}"] = dict(
            d=d, prompt_len=prompt_len, max_new_tokens=new_tokens, events=[list(e) for e in events],
            accepted=list(gen.total_speculated_tokens),
            n_out=int(out.output_token_ids.shape[-1]),
            tps=int(gen.kv_cache_manager[0].tokens_per_split))
    return results


def main():
    ref = ref_loader.load()
    torch.set_num_threads(4)
    with open(os.path.join(HERE, "cache_traces.json"), "w") as f:
        json.dump(cache_traces(ref), f, indent=1)
    torch.save(attention_case(ref, seed=1, B=4, Hq=8, Hkv=2, D=128, lens=[96, 201, 57, 130], S=1, max_len=300),
               os.path.join(HERE, "decode_case.pt"))
    torch.save(attention_case(ref, seed=2, B=3, Hq=8, Hkv=2, D=64, lens=[40, 97, 150], S=9, max_len=256,
                              left_pad=[0, 5, 17]),
               os.path.join(HERE, "verify_case.pt"))
    torch.save(beam_case(ref), os.path.join(HERE, "beam_case.pt"))
    torch.save(llama_case(ref), os.path.join(HERE, "llama_case.pt"))
    try:
        tr = pard_trace(ref)
        with open(os.path.join(HERE, "pard_trace.json"), "w") as f:
            json.dump(tr, f, indent=1)
    except Exception as e:  # keep the other vectors even when the generator cannot be driven
        print("pard_trace failed:", repr(e))
        raise
    for fn in sorted(os.listdir(HERE)):
        print(f"{os.path.getsize(os.path.join(HERE, fn)):>9d}  {fn}")


if __name__ == "__main__":
    main()
