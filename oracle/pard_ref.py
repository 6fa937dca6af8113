"""CPU restatement of the PARD speculative-decoding length rules.  TEST INFRASTRUCTURE ONLY.

Follows pace/llm/generator.py of the reference:
  * draft pass appends history + (d-1) placeholder tokens        :638-667
  * target pass verifies history + d draft tokens                 :745-749
  * accept = leading matches among the first d-1 drafts, +1       :684-693
  * target rollback  d - keep + 1  iff keep < d, else nothing     :696-702
  * draft rollback   d - 1 always                                 :706

Everything here is integers; the CUDA side must reproduce it bit-exactly.
"""
from typing import List, Sequence, Tuple


def keep_len_from_matches(matches: Sequence[bool], d: int) -> int:
    """1 + number of leading True among the first d-1 entries."""
    k = 0
    for i in range(d - 1):
        if matches[i]:
            k += 1
        else:
            break
    return k + 1


def rollback_lengths(d: int, keep: int) -> Tuple[int, int]:
    """(tokens removed from the target cache, tokens removed from the draft cache)."""
    target = d - keep + 1 if d - keep > 0 else 0
    return target, d - 1


def length_trace(prompt_len: int, d: int, keeps: Sequence[int]) -> List[dict]:
    """Replay cache lengths for one sequence over len(keeps) PARD steps.

    Returns one dict per step with the append sizes and post-rollback lengths
    of both caches, exactly as the reference's generator produces them.
    """
    n = prompt_len          # tokens in the running history
    ct = cd = 0             # target / draft cached lengths
    out = []
    for keep in keeps:
        draft_app = (n + d - 1) - cd
        cd += draft_app
        target_app = (n + d) - ct
        ct += target_app
        t_rm, d_rm = rollback_lengths(d, keep)
        ct -= t_rm
        cd -= d_rm
        n += keep
        out.append(dict(draft_append=draft_app, target_append=target_app,
                        target_remove=t_rm, draft_remove=d_rm,
                        target_len=ct, draft_len=cd, history=n))
    return out
