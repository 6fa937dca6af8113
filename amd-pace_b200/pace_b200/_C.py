"""ctypes binding of libpace_b200.so (C ABI: include/pace_b200.h).

Plays the role of the reference's compiled extension module `pace._C`
(csrc/torch_extension_bindings.cpp): the Python layer above never touches CUDA
directly, it hands raw device pointers, sizes and the current stream to these
functions.
"""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libpace_b200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python amd-pace_b200/build.py` "
        "(there is no CPU or PyTorch fallback for these ops)")

lib = C.CDLL(LIB_PATH)

PACE_OK, PACE_ERR_INVALID, PACE_ERR_CUDA, PACE_ERR_UNSUPPORTED = 0, 1, 2, 3
DEV_POOL_EXHAUSTED, DEV_OVER_REMOVE, DEV_BAD_INDEX, DEV_TABLE_FULL, DEV_WAIT_TIMEOUT = 1, 2, 4, 8, 16
_DEV_NAMES = {1: "pool exhausted", 2: "over-removal", 4: "bad slot/page index", 8: "block table full",
              16: "in-kernel wait timed out"}


class KVPoolStruct(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("n_layers", "n_kv_heads", "head_dim", "page_tokens", "n_pages",
                                          "max_seqs", "max_pages_per_seq", "owns_memory")] + \
               [(n, C.c_void_p) for n in ("pages", "block_table", "seq_len", "seq_pages", "page_ref",
                                          "free_stack", "counters", "status", "table_tmp")]


ATTN_WHOLE_UNITS = 1      # PACE_ATTN_WHOLE_UNITS
ATTN_PENDING_ROW = 2      # PACE_ATTN_PENDING_ROW
ATTN_NO_EARLY_KV = 4      # PACE_ATTN_NO_EARLY_KV
ATTN_ONE_CTA_PER_SM = 8   # PACE_ATTN_ONE_CTA_PER_SM


class AttnArgs(C.Structure):
    _fields_ = [("pool", C.POINTER(KVPoolStruct)), ("layer", C.c_int32), ("batch", C.c_int32),
                ("n_q_heads", C.c_int32), ("q_len", C.c_int32), ("seq_ids", C.c_void_p),
                ("kv_start", C.c_void_p), ("q_lens", C.c_void_p), ("q", C.c_void_p),
                ("q_stride_b", C.c_int64), ("q_stride_h", C.c_int64), ("q_stride_s", C.c_int64),
                ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_h", C.c_int64),
                ("o_stride_s", C.c_int64), ("scale", C.c_float), ("workspace", C.c_void_p),
                ("workspace_bytes", C.c_uint64), ("flags", C.c_uint32),
                ("k_pending", C.c_void_p), ("v_pending", C.c_void_p),
                ("pending_stride_b", C.c_int64), ("pending_stride_h", C.c_int64), ("max_ctas", C.c_int32)]


class RopeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_t", C.c_int64), ("q_stride_h", C.c_int64),
                ("k", C.c_void_p), ("k_stride_b", C.c_int64), ("k_stride_t", C.c_int64), ("k_stride_h", C.c_int64),
                ("v", C.c_void_p), ("v_stride_b", C.c_int64), ("v_stride_t", C.c_int64), ("v_stride_h", C.c_int64),
                ("q_out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_t", C.c_int64),
                ("o_stride_h", C.c_int64), ("table_row", C.c_void_p), ("row_stride_b", C.c_int64),
                ("cos_table", C.c_void_p), ("sin_table", C.c_void_p), ("table_rows", C.c_int32),
                ("rotary_dim", C.c_int32), ("gptj_pairs", C.c_int32), ("n_q_heads", C.c_int32),
                ("k_stage", C.c_void_p), ("v_stage", C.c_void_p), ("stage_stride_b", C.c_int64),
                ("stage_stride_h", C.c_int64), ("stage_stride_t", C.c_int64)]


byref = C.byref
_P = C.POINTER(KVPoolStruct)
_SIGS = {
    "pace_last_cuda_error": (C.c_char_p, []),
    "pace_version": (C.c_char_p, []),
    "pace_kv_pool_bytes": (C.c_int, [_P, C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "pace_kv_pool_bind": (C.c_int, [_P, C.c_void_p, C.c_void_p]),
    "pace_kv_pool_create": (C.c_int, [_P]),
    "pace_kv_pool_destroy": (C.c_int, [_P]),
    "pace_kv_pool_reset": (C.c_int, [_P, C.c_void_p]),
    "pace_kv_pool_query": (C.c_int, [_P, C.POINTER(C.c_int32 * 4), C.c_void_p]),
    "pace_kv_pool_clear_status": (C.c_int, [_P, C.c_void_p]),
    "pace_selftest_wait_timeout": (C.c_int, [_P, C.c_int32, C.c_void_p]),
    "pace_kv_seq_release": (C.c_int, [_P, C.c_void_p, C.c_int32, C.c_void_p]),
    "pace_kv_reserve": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p]),
    "pace_kv_append": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p, C.c_void_p,
                                 C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_void_p]),
    "pace_kv_append_layers": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                        C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64, C.c_int64,
                                        C.c_void_p]),
    "pace_kv_append_rope": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                      C.POINTER(RopeArgs), C.c_void_p]),
    "pace_kv_truncate": (C.c_int, [_P, C.c_int32, C.c_int32, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                   C.c_void_p]),
    "pace_pard_accept": (C.c_int, [C.c_void_p] * 4 + [C.c_int32, C.c_int32] + [C.c_void_p] * 5),
    "pace_kv_gather": (C.c_int, [_P, C.c_void_p, C.c_void_p, C.c_int32, C.c_void_p]),
    "pace_kv_read_dense": (C.c_int, [_P, C.c_int32, C.c_void_p, C.c_int32, C.c_void_p, C.c_void_p, C.c_int32,
                                     C.c_void_p]),
    "pace_attn_workspace_bytes": (C.c_uint64, [C.c_int32] * 5),
    "pace_attn_decode": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "pace_attn_decode_cuda_cores": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "pace_attn_decode_static": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "pace_attn_verify": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "pace_attn_prefill": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "pace_profile_enabled": (C.c_int, []),
    "pace_profile_flush": (C.c_int, []),
    "pace_linear_workspace_bytes": (C.c_uint64, [C.c_int32]),
    "pace_linear_skinny": (C.c_int, [C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_void_p, C.c_int64, C.c_int32,
                                     C.c_int32, C.c_int32, C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]),
    "pace_attention_dense": (C.c_int, [C.c_void_p] * 4 + [C.c_int32, C.c_int32, C.c_void_p] + [C.c_int32] * 6 +
                             [C.c_void_p, C.c_uint64, C.c_void_p]),
}
EXPORTS = tuple(_SIGS)
for _name, (_res, _args) in _SIGS.items():
    _fn = getattr(lib, _name)   # AttributeError here = the library does not export what the header declares
    _fn.restype, _fn.argtypes = _res, _args


class PaceError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc == PACE_OK:
        return
    if rc == PACE_ERR_INVALID:
        raise ValueError(f"{what}: invalid argument")
    if rc == PACE_ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: shape not supported by the sm_100a kernels")
    raise PaceError(f"{what}: {lib.pace_last_cuda_error().decode()}")


def describe_status(bits: int) -> str:
    return ", ".join(v for k, v in _DEV_NAMES.items() if bits & k) or "ok"
