"""Op timing behind PACE_LOG_LEVEL=profile (the reference's PROFILE_PACE_FUNCTION lines, csrc/core/logging.h:144-212).
The switch is read when the library is loaded, so the calls run in a child process."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))

CHILD = r"""
import sys, torch
sys.path.insert(0, %r)
from pace_b200 import _C
from pace_b200.llm.cache import KVCacheManager, KVCacheType
from pace_b200.ops import MultiHeadAttention
class Cfg: num_hidden_layers = 2
mgr = KVCacheManager(Cfg(), 256, KVCacheType.BMC)
mha = MultiHeadAttention()
k = torch.randn(4, 8, 70, 128, device="cuda").bfloat16()
for layer in range(2):
    K, V = mgr[layer].update_cache(k, k.clone(), concat_dim=2)
    q = torch.randn(4, 32, 1, 128, device="cuda").bfloat16()
    out = mha(q, K, V)
mgr[0].remove_cache(3)
# inside a stream capture nothing is timed (and nothing breaks)
s = torch.cuda.Stream()
s.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(s):
    mha(q, K, V)
s.synchronize()
g = torch.cuda.CUDAGraph()
with torch.cuda.graph(g, stream=s):
    mha(q, K, V)
g.replay()
torch.cuda.synchronize()
print("flushed", _C.lib.pace_profile_flush())
"""


def _run(level):
    env = dict(os.environ)
    env.pop("PACE_LOG_LEVEL", None)
    if level:
        env["PACE_LOG_LEVEL"] = level
    return subprocess.run([sys.executable, "-c", CHILD % os.path.join(ROOT, "amd-pace_b200")], env=env, capture_output=True,
                          text=True, timeout=600)


def test_profile_lines_per_call():
    out = _run("profile")
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln for ln in out.stderr.splitlines() if ln.startswith("[PACE profile] pace::")]
    ops = [re.match(r"\[PACE profile\] pace::(\w+),(.*),([0-9.]+)$", ln) for ln in lines]
    assert all(ops), lines
    names = [m.group(1) for m in ops]
    assert names.count("kv_append") == 2 and names.count("kv_truncate") == 1
    assert names.count("attn_decode") == 3                      # two eager layers + the warm-up on the side stream
    assert all(0.0 < float(m.group(3)) < 1000.0 for m in ops)   # device milliseconds
    assert "batch=4" in ops[names.index("attn_decode")].group(2)
    assert "flushed" in out.stdout


def test_profile_off_by_default():
    out = _run(None)
    assert out.returncode == 0, out.stderr[-2000:]
    assert "[PACE profile]" not in out.stderr
    assert out.stdout.strip().endswith("flushed 0")
