"""The C-ABI library loads and exports every symbol the header declares (no GPU needed)."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))


def _declared():
    text = open(os.path.join(ROOT, "include", "pace_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(pace_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported():
    from pace_b200 import _C
    names = _declared()
    assert len(names) >= 20
    for n in names:
        assert hasattr(_C.lib, n), f"{n} declared in include/pace_b200.h but not exported"
    assert set(names) == set(_C.EXPORTS), "ctypes binding and header disagree"


def test_pool_sizing_and_binding_are_host_only():
    from pace_b200 import _C
    d = _C.KVPoolStruct(n_layers=2, n_kv_heads=8, head_dim=128, page_tokens=28, n_pages=10, max_seqs=4,
                        max_pages_per_seq=5)
    pb, mb = C.c_uint64(), C.c_uint64()
    assert _C.lib.pace_kv_pool_bytes(C.byref(d), C.byref(pb), C.byref(mb)) == _C.PACE_OK
    assert pb.value == 2 * 2 * 10 * 8 * 28 * 128 * 2
    assert mb.value % 256 == 0 and mb.value > 0
    # carving needs no device: any 256-byte aligned addresses
    assert _C.lib.pace_kv_pool_bind(C.byref(d), 0x10000, 0x20000) == _C.PACE_OK
    assert d.block_table == 0x20000 and d.pages == 0x10000 and d.seq_len > d.block_table
    assert _C.lib.pace_kv_pool_bind(C.byref(d), 0x10001, 0x20000) == _C.PACE_ERR_INVALID
    bad = _C.KVPoolStruct(n_layers=2, n_kv_heads=8, head_dim=96, page_tokens=28, n_pages=10, max_seqs=4,
                          max_pages_per_seq=5)
    assert _C.lib.pace_kv_pool_bytes(C.byref(bad), C.byref(pb), C.byref(mb)) == _C.PACE_ERR_INVALID


def test_invalid_arguments_are_rejected_before_any_launch():
    from pace_b200 import _C
    assert _C.lib.pace_attn_decode(None, None) == _C.PACE_ERR_INVALID
    d = _C.KVPoolStruct()
    assert _C.lib.pace_kv_pool_reset(C.byref(d), None) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_kv_append(C.byref(d), 0, None, 1, 1, None, None, None, 0, 0, 0, None) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_attn_workspace_bytes(0, 32, 8, 128, 1) == 0


def test_cpu_tensors_are_refused():
    import torch
    from pace_b200.llm.cache import BMCKVCache
    c = BMCKVCache(128)
    x = torch.zeros(2, 1, 10, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        c.update_cache(x, x, concat_dim=2)


def test_dispatcher_ops_are_registered_without_a_gpu():
    """torch.ops.pace_b200.* (what the cache and attention classes call) exist as soon as the package is
    imported, each with a CUDA kernel and a meta kernel; called with CPU tensors they raise the dispatcher's
    own "no kernel for CPU" error rather than computing anything."""
    import torch
    import pace_b200.torch_ops  # noqa: F401
    names = ["kv_reserve", "kv_append", "kv_append_layers", "kv_append_rope", "kv_truncate", "kv_gather",
             "kv_read_dense", "pard_accept", "linear_skinny", "attn_decode", "attn_decode_cuda_cores",
             "attn_verify", "attn_prefill"]
    for n in names:
        op = getattr(torch.ops.pace_b200, n)
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"pace_b200::{n}", "CUDA"), n
        assert torch._C._dispatch_has_kernel_for_dispatch_key(f"pace_b200::{n}", "Meta"), n
        assert not torch._C._dispatch_has_kernel_for_dispatch_key(f"pace_b200::{n}", "CPU"), n
        assert op.default._schema.name == f"pace_b200::{n}"
    x = torch.zeros(4, 256, dtype=torch.bfloat16)
    with pytest.raises((NotImplementedError, RuntimeError)):
        torch.ops.pace_b200.linear_skinny(x, torch.zeros(256, 256, dtype=torch.bfloat16), x.new_zeros(4), x.new_zeros(4, 256))


def test_profile_switch_follows_the_environment():
    """PACE_LOG_LEVEL=profile (the reference's switch, README "verbose" table) turns the op timer on; any
    other value leaves it off.  Read once, when the library is loaded: checked in child processes."""
    import subprocess
    import sys
    code = ("import sys; sys.path.insert(0, %r); from pace_b200 import _C; "
            "print(_C.lib.pace_profile_enabled(), _C.lib.pace_profile_flush())" % os.path.join(ROOT, "amd-pace_b200"))
    for value, want in (("profile", "1 0"), ("debug", "0 0"), (None, "0 0")):
        env = dict(os.environ)
        env.pop("PACE_LOG_LEVEL", None)
        if value is not None:
            env["PACE_LOG_LEVEL"] = value
        out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
        assert out.returncode == 0, out.stderr
        assert out.stdout.strip().splitlines()[-1] == want
