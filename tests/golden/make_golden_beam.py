"""Regenerates tests/golden/beam_loop_case.pt by running the REFERENCE model and the REFERENCE cache
manager (needs the reference source tree, see oracle/ref_loader.py):

    python tests/golden/make_golden_beam.py

A beam-search loop in the shape of the reference's (pace/llm/generator.py:571-619: model step on the
whole history, re-rank, `inputs = inputs[beam_idx] + next token`,
`kv_cache_manager.update_cache_with_beam_indices(beam_idx)`) is driven over the unmodified
`LlamaForCausalLM` and `KVCacheManager` of the reference on the CPU, where the gather is a real
`index_select` of every layer's K and V (pace/llm/cache.py:161-167).  Re-ranking is the summed
log-probability top-k that `Generator.beam_step` of this repository restates; the reference's own
scorer class cannot be imported with the installed transformers release, which is why the loop, not
`Generator._beam_search`, is what runs here.  Recorded per step: the token ids fed, the beam indices,
the last position's logits; at the end the K/V contents of every layer.  The GPU test feeds the same
ids and beam indices to the paged cache (teacher-forced) and compares logits and contents.
"""
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from oracle import ref_loader  # noqa: E402
from make_golden import build_ref_llama, tiny_llama_config  # noqa: E402


def beam_step(logits, beam_scores, num_beams):
    n, vocab = logits.shape
    batch = n // num_beams
    logp = torch.log_softmax(logits.float(), dim=-1) + beam_scores.view(n, 1)
    top, flat = logp.view(batch, num_beams * vocab).topk(num_beams, dim=-1)
    src = torch.div(flat, vocab, rounding_mode="floor")
    beam_idx = (src + torch.arange(batch).unsqueeze(1) * num_beams).view(n)
    return beam_idx, (flat % vocab).view(n), top.reshape(n)


def main():
    ref = ref_loader.load()
    cfg = tiny_llama_config(layers=2, hidden=128, heads=2, kv_heads=1, ffn=256, vocab=64)
    model = build_ref_llama(ref, cfg, seed=21)
    g = torch.Generator().manual_seed(22)
    B, nb, P, steps = 2, 3, 70, 12            # 70-token prompts: the beams share a full 64-token page and a partial one
    prompts = torch.randint(1, cfg.vocab_size, (B, P), generator=g)
    ids = prompts.repeat_interleave(nb, dim=0)
    mask = torch.ones_like(ids)
    scores = torch.zeros(B, nb)
    scores[:, 1:] = -1e9
    scores = scores.view(-1)
    mgr = ref.KVCacheManager(cfg, P + steps, ref.KVCacheType.BMC)
    rec = dict(ids=[], beam_idx=[], tokens=[], logits=[])
    with torch.inference_mode():
        for _ in range(steps):
            logits = model(ids, kv_cache=mgr, attention_mask=mask).logits[:, -1].float()
            beam_idx, tokens, scores = beam_step(logits, scores, nb)
            rec["ids"].append(ids.clone())
            rec["logits"].append(logits.clone())
            rec["beam_idx"].append(beam_idx.clone())
            rec["tokens"].append(tokens.clone())
            ids = torch.cat([ids[beam_idx], tokens.unsqueeze(-1)], dim=-1)
            mask = torch.cat([mask, mask.new_ones(mask.shape[0], 1)], dim=-1)
            mgr.update_cache_with_beam_indices(beam_idx)
    rep = cfg.num_attention_heads // cfg.num_key_value_heads
    n = int(mgr[0].seq_len)
    out = dict(cfg={k: getattr(cfg, k) for k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                                 "num_attention_heads", "num_key_value_heads", "vocab_size",
                                                 "max_position_embeddings", "rope_theta", "rms_norm_eps")},
               state={k: v.detach().clone() for k, v in model.state_dict().items()},
               prompts=prompts, num_beams=nb, steps=steps, final_ids=ids, final_scores=scores,
               k_cache=[mgr[i].key[:, ::rep, :n].clone() for i in range(2)],
               v_cache=[mgr[i].value[:, ::rep, :n].clone() for i in range(2)], seq_len=n, **rec)
    torch.save(out, os.path.join(HERE, "beam_loop_case.pt"))
    moved = sum(int((b != torch.arange(len(b))).any()) for b in rec["beam_idx"])
    print(f"beam_loop_case.pt: {steps} steps, {moved} of them re-order the beams; final length {n}")


if __name__ == "__main__":
    main()
