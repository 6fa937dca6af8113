"""A bounded in-kernel wait that runs out: the status bit, the time it takes, and what the pool does
afterwards.  The wait that runs out is the self-test's own (a barrier nobody arrives on, about a
millisecond): no kernel of the hot path is made to hang."""
import time

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


class Cfg:
    num_hidden_layers = 2


def _setup():
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    g = torch.Generator().manual_seed(31)
    B, Hq, Hkv, D, L = 8, 32, 8, 128, 300
    mgr = KVCacheManager(Cfg(), 400, KVCacheType.BMC)
    k = torch.randn(B, Hkv, L, D, generator=g).bfloat16().to(DEV)
    v = torch.randn(B, Hkv, L, D, generator=g).bfloat16().to(DEV)
    for l in range(2):
        mgr[l].update_cache(k, v, concat_dim=2)
    q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
    q9 = torch.randn(B, Hq, 9, D, generator=g).bfloat16().to(DEV)
    return mgr, q, q9


@pytest.mark.parametrize("kind", ["decode_mma", "decode_cuda", "verify"])
def test_wait_runs_out_then_pool_refuses_until_cleared(kind):
    from pace_b200 import _C
    from pace_b200.ops import MultiHeadAttention
    mgr, q1, q9 = _setup()
    mha = MultiHeadAttention()
    K, V = mgr[0].key, mgr[0].value
    q = q9 if kind == "verify" else q1
    sched = {"decode_mma": dict(decode_kernel="mma"), "decode_cuda": dict(decode_kernel="cuda"), "verify": {}}[kind]
    good = mha(q, K, V, **sched).clone()
    torch.cuda.synchronize()
    assert mgr.pool.query()[0] == 0

    stream = torch.cuda.current_stream().cuda_stream
    t0 = time.perf_counter()
    assert _C.lib.pace_selftest_wait_timeout(mgr.pool.ref, 1000, stream) == _C.PACE_OK
    bits, _ = mgr.pool.query()                      # synchronises
    took = time.perf_counter() - t0
    assert bits & _C.DEV_WAIT_TIMEOUT
    # one wait of about a millisecond ran out; the second warp of the self-test, whose own limit is a quarter
    # of a second, was released by the first one's abort flag
    assert took < 0.1, f"the self-test took {took:.3f} s"

    # the pool has given up: launches on it return at once and leave their output alone
    out = torch.full_like(q, 7.0)
    t0 = time.perf_counter()
    for _ in range(20):
        mha(q, K, V, out=out, **sched)
    torch.cuda.synchronize()
    took = time.perf_counter() - t0
    assert took < 0.1, f"20 launches on a pool that has given up took {took:.3f} s"
    assert torch.all(out == 7.0)
    with pytest.raises(_C.PaceError, match="wait timed out"):
        mgr.pool.check_status()

    # the host clears the word: service is back, same rows as before
    mgr.pool.clear_status()
    out2 = mha(q, K, V, **sched)
    torch.cuda.synchronize()
    assert torch.equal(out2, good)
    mgr.pool.check_status()


def test_selftest_rejects_bad_arguments():
    from pace_b200 import _C
    mgr, _, _ = _setup()
    assert _C.lib.pace_selftest_wait_timeout(None, 1000, None) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_selftest_wait_timeout(mgr.pool.ref, 0, None) == _C.PACE_ERR_INVALID
    assert _C.lib.pace_selftest_wait_timeout(mgr.pool.ref, 2000000, None) == _C.PACE_ERR_INVALID
