"""ctypes front end of the C restatement (jit_attention_ref.c).  TEST INFRASTRUCTURE ONLY."""
import ctypes
import os
import subprocess

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libpace_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "jit_attention_ref.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libpace_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_SO)
        _lib.pace_ref_attention_bf16.restype = ctypes.c_int
        _lib.pace_ref_attention_bf16.argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_int, ctypes.c_void_p] \
            + [ctypes.c_int] * 6
        _lib.pace_ref_bmc_append_bf16.restype = None
        _lib.pace_ref_bmc_append_bf16.argtypes = [ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_int] * 6
    return _lib


def attention_bf16(q, k, v, mask=None, nthreads: int = 1):
    """q [B,N,S,H], k/v [B,N,L,H], mask [B,1,1|S,L] or None; all bf16 CPU, contiguous."""
    assert q.dtype == torch.bfloat16 and q.device.type == "cpu"
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    B, N, S, H = q.shape
    L = k.shape[2]
    out = torch.empty_like(q)
    mptr, mrows = None, 1
    if mask is not None:
        mask = mask.to(torch.bfloat16).contiguous()
        assert mask.shape[0] == B and mask.shape[1] == 1 and mask.shape[3] == L
        mrows = mask.shape[2]
        mptr = mask.data_ptr()
    rc = lib().pace_ref_attention_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), mptr, mrows,
                                       out.data_ptr(), B, N, S, L, H, nthreads)
    if rc != 0:
        raise RuntimeError(f"pace_ref_attention_bf16 failed: {rc}")
    return out


def bmc_append_bf16(cache, fresh, seq_len: int):
    """cache [B,N,cap,H] (in place), fresh [B,N,n,H]."""
    B, N, cap, H = cache.shape
    n = fresh.shape[2]
    assert seq_len + n <= cap
    fresh = fresh.contiguous()
    lib().pace_ref_bmc_append_bf16(cache.data_ptr(), fresh.data_ptr(), B, N, cap, seq_len, n, H)
