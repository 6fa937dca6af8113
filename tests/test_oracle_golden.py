"""Pins the CPU oracle: restatements vs vectors recorded from the reference itself."""
import json
import os

import pytest
import torch

from oracle import attention_ref as A
from oracle import kv_cache_ref as C
from oracle import pard_ref as P
from oracle import jit_c

G = os.path.join(os.path.dirname(__file__), "golden")


def _traces():
    with open(os.path.join(G, "cache_traces.json")) as f:
        return json.load(f)


def test_known_answers_of_reference_cache_test():
    # reference tests/llm_infra/test_cache.py:53-64 (capacity 11, mask width 11) and :76-80 (length 10)
    t = _traces()
    assert t["test_cache_py/bmc"] == {"key_len": 11, "mask_w": 11}
    assert t["test_cache_py/dynamic"] == {"key_len": 10}
    c = C.SegmentedCacheRef(128)
    k, v = c.append(torch.rand(2, 10, 64), torch.rand(2, 10, 64), axis=1)
    assert k.shape[1] == 11 and c.tps == 11
    assert c.pad_mask(torch.ones(2, 10), 10).shape == (2, 11)
    d = C.GrowingCacheRef(128)
    k, v = d.append(torch.rand(2, 10, 64), torch.rand(2, 10, 64), axis=1)
    assert k.shape[1] == 10


@pytest.mark.parametrize("name", sorted(k for k in _traces() if not k.startswith("test_cache_py")))
def test_cache_traces_match_reference(name):
    e = _traces()[name]
    policy = name.split("/")[1]
    ops = [tuple(o) for o in e["ops"]]
    # integer replay
    got = C.replay_trace(ops, e["max_len"], policy)
    want = [tuple(x) if x[0] != "error" else ("error",) for x in e["trace"]]
    assert got == want
    # tensor-carrying class
    c = C.cache_class_for(policy)(e["max_len"])
    for (kind, n), w in zip(ops, e["trace"]):
        if kind == "append":
            x = torch.zeros(1, 1, n, 2)
            k, _ = c.append(x, x.clone(), axis=2)
            assert [c.seq_len, k.shape[2]] == w
        else:
            if w[0] == "error":
                with pytest.raises(ValueError, match="Cannot remove more tokens than available in cache"):
                    c.remove(n)
            else:
                c.remove(n)
                assert [c.seq_len, c.capacity] == w
    if policy == "bmc":
        assert c.tps == e["tokens_per_split"]
        for n, w in e["mask_width"].items():
            assert c.pad_mask(torch.ones(2, int(n)), int(n)).shape[-1] == w


def test_bmc_env_override(monkeypatch):
    monkeypatch.setenv("PACE_BMC_NUM_SPLITS", "4")
    assert C.bmc_tokens_per_split(1024) == 256


@pytest.mark.parametrize("fname", ["decode_case.pt", "verify_case.pt"])
def test_attention_and_cache_contents_match_reference(fname):
    case = torch.load(os.path.join(G, fname))
    for b in range(case["B"]):
        L, S = case["lens"][b], case["S"]
        kc, vc = case["k_cache"][b], case["v_cache"][b]
        # rebuild the cache with the oracle from the old rows + the new rows
        c = C.SegmentedCacheRef(case["max_len"])
        c.append(kc[None, :, :L], vc[None, :, :L], axis=2)
        K, V = c.append(case["k_new"][b][None], case["v_new"][b][None], axis=2)
        assert K.shape[2] == case["capacity"][b]
        assert torch.equal(K[0], kc) and torch.equal(V[0], vc)          # bit-exact contents incl. zero padding
        q = case["q"][b][None]
        want = case["out"][b].float()
        got = A.attend_over_cache(q, K, V, L + S, case["left_pad"][b], "native")[0].float()
        assert torch.equal(got, want)                                    # same torch op, same inputs
        jit = A.attend_over_cache(q, K, V, L + S, case["left_pad"][b], "jit")[0].float()
        assert (jit - want).abs().max() < 2e-2 and (jit - want).abs().mean() < 2e-3


def test_mask_restatement_matches_transformers():
    # semantics of the third-party converter called at reference llama.py:294-299
    try:
        from transformers.modeling_attn_mask_utils import AttentionMaskConverter
    except Exception:
        pytest.skip("converter not in this transformers release")
    import warnings
    m2 = torch.ones(3, 12, dtype=torch.long)
    m2[1, :4] = 0
    m2[2, :1] = 0
    for q in (1, 5, 12):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            want = AttentionMaskConverter(is_causal=True).to_4d(m2, q, key_value_length=12, dtype=torch.bfloat16)
        got = A.additive_mask_4d(m2, q, 12, torch.bfloat16)
        assert torch.equal(got, want)


def test_c_restatement_equals_torch_restatement():
    torch.manual_seed(3)
    q = torch.randn(2, 4, 3, 64).bfloat16()
    k = torch.randn(2, 4, 70, 64).bfloat16()
    v = torch.randn(2, 4, 70, 64).bfloat16()
    m = torch.randn(2, 1, 1, 70).bfloat16()
    a = jit_c.attention_bf16(q, k, v, m, nthreads=3).float()
    b = A.sdpa_jit_restated(q, k, v, m).float()
    assert (a - b).abs().max() <= 2 ** -7      # one bf16 ulp at |x|<2: expf vs torch.exp rounding
    n = A.sdpa_native(q, k, v, m).float()
    assert (a - n).abs().max() < 2e-2


def test_c_append_equals_narrow_copy():
    torch.manual_seed(4)
    cache = torch.zeros(2, 3, 12, 16, dtype=torch.bfloat16)
    fresh = torch.randn(2, 3, 5, 16).bfloat16()
    want = cache.clone()
    want.narrow(2, 4, 5).copy_(fresh)
    jit_c.bmc_append_bf16(cache, fresh, 4)
    assert torch.equal(cache, want)


def test_beam_gather_matches_reference():
    case = torch.load(os.path.join(G, "beam_case.pt"))
    c = C.SegmentedCacheRef(case["max_len"])
    c.append(case["k"], case["v"], axis=2)
    c.gather(case["idx"])
    c.append(case["k2"], case["v2"], axis=2)
    c.gather(case["idx2"])
    assert c.seq_len == case["seq_len"]
    assert torch.equal(c.k, case["K"]) and torch.equal(c.v, case["V"])


def test_pard_lengths_match_reference_generator():
    with open(os.path.join(G, "pard_trace.json")) as f:
        tr = json.load(f)
    for name, e in tr.items():
        d = e["d"]
        want = P.length_trace(e["prompt_len"], d, e["accepted"])
        ev = e["events"]
        assert len(ev) == 4 * len(want)
        for i, w in enumerate(want):
            da, ta, tr_, dr = ev[4 * i: 4 * i + 4]
            assert da[:3] == ["draft", "append", w["draft_append"]]
            assert ta[:3] == ["target", "append", w["target_append"]]
            # the reference skips the target removal when nothing is rejected; then two draft events follow
            assert tr_[0] == "target" and tr_[2] == w["target_remove"] and tr_[4] == w["target_len"]
            assert dr[:3] == ["draft", "remove", w["draft_remove"]] and dr[4] == w["draft_len"]
        # capacities follow the BMC rule
        for tag in ("target", "draft"):
            cap, seq = 0, 0
            for e2 in ev:
                if e2[0] != tag:
                    continue
                if e2[1] == "append":
                    cap = C.bmc_capacity_after(cap, seq, e2[2], e["tps"])
                    seq += e2[2]
                else:
                    seq -= e2[2]
                assert (seq, cap) == (e2[4], e2[5])


def test_pard_rules():
    assert P.keep_len_from_matches([True, True, False, True, True, True, True], 8) == 3
    assert P.keep_len_from_matches([True] * 7, 8) == 8
    assert P.rollback_lengths(8, 8) == (0, 7)      # nothing rejected: target keeps the unverified draft row
    assert P.rollback_lengths(8, 1) == (8, 7)
    assert P.rollback_lengths(8, 5) == (4, 7)


# ---------------------------------------------------------------------------------------------
# RoPE (the step in front of the append): oracle/rope_ref.py against the reference operator's outputs
# ---------------------------------------------------------------------------------------------
def _rope_cases():
    import torch
    return torch.load(os.path.join(os.path.dirname(__file__), "golden", "rope_cases.pt"))


def test_rope_tables_match_reference_for_every_rope_type():
    import torch
    from oracle import rope_ref
    cases = _rope_cases()
    assert set(cases) >= {"default", "linear", "dynamic", "llama3", "longrope"}
    for name, c in cases.items():
        cos, sin, rd, kind, window = rope_ref.build_tables(c["rope_scaling"], c["head_dim"],
                                                           c["max_position_embeddings"], c["rope_theta"],
                                                           c["partial_rotary_factor"], **c["kwargs"])
        assert rd == c["rotary_dim"] and cos.shape[0] == c["cache_rows"], name
        assert torch.equal(cos, c["cos_cache"]) and torch.equal(sin, c["sin_cache"]), name


def test_rope_application_is_bit_exact_against_reference():
    import torch
    from oracle import rope_ref
    for name, c in _rope_cases().items():
        cos_t, sin_t, rd, kind, window = rope_ref.build_tables(c["rope_scaling"], c["head_dim"],
                                                               c["max_position_embeddings"], c["rope_theta"],
                                                               c["partial_rotary_factor"], **c["kwargs"])
        for tag, a in c["applied"].items():
            q, k = rope_ref.rotate(c["q"], c["k"], a["position_ids"], cos_t, sin_t, rd, kind, window,
                                   neox=tag.endswith("neox"))
            assert torch.equal(q, a["q_rot"]) and torch.equal(k, a["k_rot"]), (name, tag)
