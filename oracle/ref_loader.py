"""Imports the reference's own Python modules, unmodified, from its source tree.

TEST INFRASTRUCTURE ONLY, and only usable where the reference tree exists: a
checkout named by $PACE_REF_ROOT, else the copy of its `pace/` package that
oracle/stage_ref.py puts under oracle/_ref/ (git-ignored).  Used by
tests/golden/make_golden.py to produce the committed golden vectors, by the CPU
tests that re-check the oracle against the live reference when it is there, and by
the timed CPU baseline of bench.py.

The reference package needs its compiled extension (`pace._C`) and a
setup-generated version module at import time (pace/__init__.py:6-15); neither
exists in a source checkout, so stand-ins are registered for the two package
objects and the submodules are then imported from the reference tree as they
lie.  generator.py:11-17 imports `BeamSearchScorer`, which newer transformers
releases dropped; a placeholder attribute is injected (beam search itself is
not exercised through this loader).
"""
import os
import sys
import types


def ref_root() -> str:
    env = os.environ.get("PACE_REF_ROOT")
    if env:
        return env
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref")


def available() -> bool:
    return os.path.isfile(os.path.join(ref_root(), "pace", "llm", "cache.py"))


def load():
    """Returns a namespace with the reference symbols the hot path touches."""
    if not available():
        raise RuntimeError(f"reference tree not found under {ref_root()}")
    import transformers
    root = ref_root()
    if "pace" not in sys.modules or not getattr(sys.modules["pace"], "_ref_stub", False):
        pace = types.ModuleType("pace")
        pace.__path__ = [os.path.join(root, "pace")]
        pace._ref_stub = True
        ext = types.ModuleType("pace._C")
        ext.pace_logger = lambda level, msg: None
        ext.thread_bind = lambda cores: None
        pace._C = pace.core = ext
        sys.modules["pace"] = pace
        sys.modules["pace._C"] = ext
        llm = types.ModuleType("pace.llm")
        llm.__path__ = [os.path.join(root, "pace", "llm")]
        sys.modules["pace.llm"] = llm
    if not hasattr(transformers, "BeamSearchScorer"):
        transformers.BeamSearchScorer = object
    ns = types.SimpleNamespace()
    from pace.llm.cache import KVCacheManager, KVCacheType, BMCKVCache, DynamicKVCache
    from pace.ops import MultiHeadAttention, BackendType
    from pace.llm.models.llama import LlamaForCausalLM, repeat_kv
    from pace.llm.configs import OperatorConfig
    ns.KVCacheManager, ns.KVCacheType = KVCacheManager, KVCacheType
    ns.BMCKVCache, ns.DynamicKVCache = BMCKVCache, DynamicKVCache
    ns.MultiHeadAttention, ns.BackendType = MultiHeadAttention, BackendType
    ns.LlamaForCausalLM, ns.repeat_kv, ns.OperatorConfig = LlamaForCausalLM, repeat_kv, OperatorConfig
    return ns
