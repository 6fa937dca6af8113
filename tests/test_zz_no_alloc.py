"""The allocation-free decode entry point gives what the workspace-taking one gives.

Collected last on purpose (file name), so a run that stops at the first failure has already been
through every other test.  Callers that cannot allocate device memory on their decode path - an
engine that owns the whole GPU, a loop whose memory was fixed at start-up - use
pace_attn_decode_static, whose scratch is a fixed array inside the library; this test drives it
through the C ABI, twice in a row because the array keeps the previous call's contents.
"""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


class Cfg:
    num_hidden_layers = 2


def _args(mgr, layer, q, out, ws):
    from pace_b200 import _C
    pool = mgr.pool
    a = _C.AttnArgs()
    a.pool = C.pointer(pool.desc)
    a.layer, a.batch, a.n_q_heads, a.q_len = layer, q.shape[0], q.shape[1], 1
    a.seq_ids = mgr.slots_dev.data_ptr()
    a.q = q.data_ptr()
    a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(0), q.stride(1), q.stride(2)
    a.out = out.data_ptr()
    a.o_stride_b, a.o_stride_h, a.o_stride_s = out.stride(0), out.stride(1), out.stride(2)
    a.scale = 1.0 / math.sqrt(q.shape[3])
    if ws is not None:
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    return a


def test_static_scratch_decode_matches_workspace_decode():
    from pace_b200 import _C
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    g = torch.Generator().manual_seed(2024)
    B, Hq, Hkv, D = 5, 32, 8, 128
    lens = [700, 33, 512, 1, 257]
    mgr = KVCacheManager(Cfg(), 1024, KVCacheType.BMC)
    k = torch.randn(B, Hkv, max(lens), D, generator=g).bfloat16().to(DEV)
    v = torch.randn(B, Hkv, max(lens), D, generator=g).bfloat16().to(DEV)
    for layer in range(2):
        mgr[layer].update_cache(k, v, concat_dim=2, n_new_per_seq=lens)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(_C.lib.pace_attn_workspace_bytes(B, Hq, Hkv, D, 1), dtype=torch.uint8, device=DEV)
    for call in range(2):                      # second call: the array holds the first call's leftovers
        q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        a = _args(mgr, 1, q, want, ws)
        assert _C.lib.pace_attn_decode(C.byref(a), stream) == _C.PACE_OK
        b = _args(mgr, 1, q, got, None)        # no workspace: the library's own array is used
        assert _C.lib.pace_attn_decode_static(C.byref(b), stream) == _C.PACE_OK
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS, (call, err.max().item())
        # and both agree with the CPU oracle
        from oracle.attention_ref import attend_over_cache
        for bi, L in enumerate(lens):
            ref = attend_over_cache(q[bi:bi + 1].cpu(), k[bi:bi + 1, :, :L].cpu(), v[bi:bi + 1, :, :L].cpu(), L)[0].float()
            e = (got[bi].float().cpu() - ref).abs()
            assert e.max().item() < MAX_ABS and e.mean().item() < MEAN_ABS
    mgr.pool.check_status()


@pytest.mark.parametrize("Hq,Hkv,D,B", [(8, 8, 128, 6), (16, 8, 64, 6), (32, 2, 128, 4), (32, 8, 128, 1100)])
def test_static_scratch_decode_other_groups_and_batches(Hq, Hkv, D, B):
    """Groups of 1, 2 and 16 query heads per KV head (pace_attn_decode would send the first two to the
    CUDA-core kernel; this entry point always packs them into the 16-row tile), head_dim 64, and a batch
    beyond what one launch takes (several launches in a row share the array's arrival counters).  Against
    the workspace-taking entry point and, for a few sequences, the CPU oracle; two calls in a row."""
    from pace_b200 import _C
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    from oracle.attention_ref import attend_over_cache
    g = torch.Generator().manual_seed(Hq * 31 + B)
    lens = [(37 * i) % 150 + 1 for i in range(B)]
    mgr = KVCacheManager(Cfg(), 160, KVCacheType.BMC)
    k = torch.randn(B, Hkv, max(lens), D, generator=g).bfloat16().to(DEV)
    v = torch.randn(B, Hkv, max(lens), D, generator=g).bfloat16().to(DEV)
    mgr[0].update_cache(k, v, concat_dim=2, n_new_per_seq=lens)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(_C.lib.pace_attn_workspace_bytes(B, Hq, Hkv, D, 1), dtype=torch.uint8, device=DEV)
    for call in range(2):
        q = torch.randn(B, Hq, 1, D, generator=g).bfloat16().to(DEV)
        want = torch.empty_like(q)
        got = torch.full_like(q, float("nan"))
        a = _args(mgr, 0, q, want, ws)
        assert _C.lib.pace_attn_decode(C.byref(a), stream) == _C.PACE_OK
        b = _args(mgr, 0, q, got, None)
        assert _C.lib.pace_attn_decode_static(C.byref(b), stream) == _C.PACE_OK
        torch.cuda.synchronize()
        err = (got.float() - want.float()).abs()
        assert err.max().item() < MAX_ABS and err.mean().item() < MEAN_ABS, (call, err.max().item())
        for bi in list(range(0, B, max(1, B // 5)))[:6]:
            L = lens[bi]
            ref = attend_over_cache(q[bi:bi + 1].cpu(), k[bi:bi + 1, :, :L].cpu(), v[bi:bi + 1, :, :L].cpu(), L)[0].float()
            e = (got[bi].float().cpu() - ref).abs()
            assert e.max().item() < MAX_ABS and e.mean().item() < MEAN_ABS
    mgr.pool.check_status()


def test_static_scratch_decode_refuses_what_does_not_fit():
    from pace_b200 import _C
    from pace_b200.llm.cache import KVCacheManager, KVCacheType
    mgr = KVCacheManager(Cfg(), 64, KVCacheType.BMC)
    k = torch.randn(1, 1, 8, 64, device=DEV).bfloat16()
    mgr[0].update_cache(k, k.clone(), concat_dim=2)
    q = torch.randn(1, 32, 1, 64, device=DEV).bfloat16()      # 32 query heads on one KV head: beyond the 16-row tile
    out = torch.empty_like(q)
    a = _args(mgr, 0, q, out, None)
    assert _C.lib.pace_attn_decode_static(C.byref(a), torch.cuda.current_stream().cuda_stream) == _C.PACE_ERR_UNSUPPORTED
    a.q_len = 2
    assert _C.lib.pace_attn_decode_static(C.byref(a), None) == _C.PACE_ERR_INVALID
    # a layer or a batch the pool does not have is refused before the shared array is touched
    q4 = torch.randn(1, 4, 1, 64, device=DEV).bfloat16()
    b = _args(mgr, 5, q4, torch.empty_like(q4), None)
    assert _C.lib.pace_attn_decode_static(C.byref(b), None) == _C.PACE_ERR_INVALID
    c = _args(mgr, 0, q4, torch.empty_like(q4), None)
    c.batch = 9
    assert _C.lib.pace_attn_decode_static(C.byref(c), None) == _C.PACE_ERR_INVALID
