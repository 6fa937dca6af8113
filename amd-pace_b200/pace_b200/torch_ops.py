"""``torch.ops.pace_b200.*``: the KV-pool and paged-attention entry points as dispatcher ops.

The reference reaches its compiled kernels through ops registered with the dispatcher
(``TORCH_LIBRARY_FRAGMENT(pace, m) { m.def("attention(...)") }``, csrc/ops/attention.cpp:104-108);
this module does the same for what replaces its Python cache bookkeeping and its attention op on a
GPU.  Every op is a thin shell over one C-ABI function of libpace_b200.so: tensors go in as device
pointers and element strides, the call is stream-ordered on the current CUDA stream, nothing is
returned (results land in ``out`` / in the pool).  The Python classes of ``pace_b200.llm.cache`` and
``pace_b200.ops.backends.b200`` call these ops, so a caller that works at the dispatcher level
(tracing, ``torch.compile``, C++ through ``c10::Dispatcher``) sees the same calls they make.

A pool is named by ``pool``, the address of its ``pace_kv_pool_t`` descriptor
(``KVPool.handle``); ``pages`` / ``meta`` are the pool's two storage tensors, passed so that the
schema can say what an op writes.
"""
import ctypes as C
import math
from typing import Optional

import torch

from pace_b200 import _C

_lib = torch.library.Library("pace_b200", "DEF")

_DEFS = {
    "kv_reserve": "(int pool, Tensor(a!) meta, int layer, Tensor seq_ids, int n_new, Tensor? n_new_per_seq) -> ()",
    "kv_append": "(int pool, Tensor(a!) pages, Tensor(b!) meta, int layer, Tensor seq_ids, Tensor k_new, Tensor v_new, "
                 "Tensor? n_new_per_seq) -> ()",
    "kv_append_layers": "(int pool, Tensor(a!) pages, Tensor(b!) meta, int layer_begin, int layer_end, Tensor seq_ids, "
                        "Tensor? k_all, Tensor? v_all) -> ()",
    "kv_append_rope": "(int pool, Tensor(a!) pages, Tensor(b!) meta, int layer, Tensor seq_ids, Tensor q, Tensor k, "
                      "Tensor v, Tensor(c!) q_out, Tensor table_row, Tensor cos, Tensor sin, int rotary_dim, "
                      "bool gptj_pairs, Tensor? n_new_per_seq, Tensor(d!)? k_stage, Tensor(e!)? v_stage) -> ()",
    "kv_truncate": "(int pool, Tensor(a!) meta, int layer_begin, int layer_end, Tensor seq_ids, int remove_len, "
                   "Tensor? remove_per_seq) -> ()",
    "kv_gather": "(int pool, Tensor(a!) meta, Tensor seq_ids, Tensor beam_idx) -> ()",
    "pard_accept": "(Tensor drafts, Tensor target_next, Tensor n_target, Tensor? forced, Tensor(a!) keep, "
                   "Tensor(b!) target_remove, Tensor(c!) draft_remove, Tensor(d!) kept) -> ()",
    "kv_read_dense": "(int pool, Tensor pages, int layer, Tensor seq_ids, Tensor(a!) k_out, Tensor(b!) v_out) -> ()",
}
_DEFS["linear_skinny"] = "(Tensor x, Tensor weight, Tensor(a!) out, Tensor(b!) workspace) -> ()"
_ATTN = ("(int pool, Tensor(a!) pages, int layer, Tensor q, Tensor(b!) out, Tensor? seq_ids, Tensor? kv_start, "
         "Tensor? q_lens, Tensor(c!) workspace, float scale, int flags, Tensor? k_pending, Tensor? v_pending, "
         "int max_ctas) -> ()")
for _n in ("attn_decode", "attn_decode_cuda_cores", "attn_verify", "attn_prefill"):
    _DEFS[_n] = _ATTN
for _n, _sig in _DEFS.items():
    _lib.define(_n + _sig)


def _pool(handle: int):
    return C.byref(_C.KVPoolStruct.from_address(handle))


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


def _kv_reserve(pool, meta, layer, seq_ids, n_new, n_new_per_seq=None):
    with torch.cuda.device(meta.device):
        _C.check(_C.lib.pace_kv_reserve(_pool(pool), layer, seq_ids.data_ptr(), seq_ids.numel(), n_new,
                                        _ptr(n_new_per_seq), _stream(meta)), "pace_kv_reserve")


def _kv_append(pool, pages, meta, layer, seq_ids, k_new, v_new, n_new_per_seq=None):
    B, _, n, _ = k_new.shape
    sb, sh, st, _ = k_new.stride()
    with torch.cuda.device(pages.device):
        _C.check(_C.lib.pace_kv_append(_pool(pool), layer, seq_ids.data_ptr(), B, n, _ptr(n_new_per_seq),
                                       k_new.data_ptr(), v_new.data_ptr(), sb, sh, st, _stream(pages)), "pace_kv_append")


def _kv_append_layers(pool, pages, meta, layer_begin, layer_end, seq_ids, k_all=None, v_all=None):
    sl = sb = sh = st = 0
    if k_all is not None:
        sl, sb, sh, st, _ = k_all.stride()
    with torch.cuda.device(pages.device):
        _C.check(_C.lib.pace_kv_append_layers(_pool(pool), layer_begin, layer_end, seq_ids.data_ptr(), seq_ids.numel(), 1,
                                              None, _ptr(k_all), _ptr(v_all), sl, sb, sh, st, _stream(pages)),
                 "pace_kv_append_layers")


def _kv_append_rope(pool, pages, meta, layer, seq_ids, q, k, v, q_out, table_row, cos, sin, rotary_dim, gptj_pairs,
                    n_new_per_seq=None, k_stage=None, v_stage=None):
    B, n, Hq, _ = q.shape
    a = _C.RopeArgs()
    a.q, (a.q_stride_b, a.q_stride_t, a.q_stride_h) = q.data_ptr(), q.stride()[:3]
    a.k, (a.k_stride_b, a.k_stride_t, a.k_stride_h) = k.data_ptr(), k.stride()[:3]
    a.v, (a.v_stride_b, a.v_stride_t, a.v_stride_h) = v.data_ptr(), v.stride()[:3]
    a.q_out, (a.o_stride_b, a.o_stride_t, a.o_stride_h) = q_out.data_ptr(), q_out.stride()[:3]
    a.table_row, a.row_stride_b = table_row.data_ptr(), table_row.stride(0)
    a.cos_table, a.sin_table, a.table_rows = cos.data_ptr(), sin.data_ptr(), cos.shape[0]
    a.rotary_dim, a.gptj_pairs, a.n_q_heads = rotary_dim, int(gptj_pairs), Hq
    if k_stage is not None:      # staged rows [B, H, n, D]: the pool is left as it is
        a.k_stage, a.v_stage = k_stage.data_ptr(), v_stage.data_ptr()
        a.stage_stride_b, a.stage_stride_h, a.stage_stride_t = k_stage.stride()[:3]
    with torch.cuda.device(pages.device):
        _C.check(_C.lib.pace_kv_append_rope(_pool(pool), layer, seq_ids.data_ptr(), B, n, _ptr(n_new_per_seq),
                                            C.byref(a), _stream(pages)), "pace_kv_append_rope")


def _kv_truncate(pool, meta, layer_begin, layer_end, seq_ids, remove_len, remove_per_seq=None):
    with torch.cuda.device(meta.device):
        _C.check(_C.lib.pace_kv_truncate(_pool(pool), layer_begin, layer_end, seq_ids.data_ptr(), seq_ids.numel(),
                                         remove_len, _ptr(remove_per_seq), _stream(meta)), "pace_kv_truncate")


def _kv_gather(pool, meta, seq_ids, beam_idx):
    with torch.cuda.device(meta.device):
        _C.check(_C.lib.pace_kv_gather(_pool(pool), seq_ids.data_ptr(), beam_idx.data_ptr(), seq_ids.numel(),
                                       _stream(meta)), "pace_kv_gather")


def _pard_accept(drafts, target_next, n_target, forced, keep, target_remove, draft_remove, kept):
    B, d = drafts.shape
    with torch.cuda.device(drafts.device):
        _C.check(_C.lib.pace_pard_accept(drafts.data_ptr(), target_next.data_ptr(), n_target.data_ptr(), _ptr(forced), B, d,
                                         keep.data_ptr(), target_remove.data_ptr(), draft_remove.data_ptr(),
                                         kept.data_ptr(), _stream(drafts)), "pace_pard_accept")


def _linear_skinny(x, weight, out, workspace):
    M, K = x.shape
    N = weight.shape[0]
    with torch.cuda.device(x.device):
        _C.check(_C.lib.pace_linear_skinny(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0), out.data_ptr(),
                                           out.stride(0), M, N, K, workspace.data_ptr(), workspace.numel(), None,
                                           _stream(x)), "pace_linear_skinny")


def _kv_read_dense(pool, pages, layer, seq_ids, k_out, v_out):
    with torch.cuda.device(pages.device):
        _C.check(_C.lib.pace_kv_read_dense(_pool(pool), layer, seq_ids.data_ptr(), seq_ids.numel(), k_out.data_ptr(),
                                           v_out.data_ptr(), k_out.shape[2], _stream(pages)), "pace_kv_read_dense")


def _attn(entry: str):
    fn = getattr(_C.lib, entry)

    def impl(pool, pages, layer, q, out, seq_ids, kv_start, q_lens, workspace, scale, flags, k_pending, v_pending,
             max_ctas):
        B, Hq, S, D = q.shape
        a = _C.AttnArgs()
        a.pool = C.pointer(_C.KVPoolStruct.from_address(pool))
        a.layer, a.batch, a.n_q_heads, a.q_len = layer, B, Hq, S
        a.seq_ids, a.kv_start, a.q_lens = _ptr(seq_ids), _ptr(kv_start), _ptr(q_lens)
        a.q = q.data_ptr()
        a.q_stride_b, a.q_stride_h, a.q_stride_s = q.stride(0), q.stride(1), q.stride(2)
        a.out = out.data_ptr()
        a.o_stride_b, a.o_stride_h, a.o_stride_s = out.stride(0), out.stride(1), out.stride(2)
        a.scale = float(scale) if scale > 0 else 1.0 / math.sqrt(D)
        a.workspace, a.workspace_bytes = workspace.data_ptr(), workspace.numel()
        a.flags, a.max_ctas = int(flags), int(max_ctas)
        if k_pending is not None:
            a.k_pending, a.v_pending = k_pending.data_ptr(), v_pending.data_ptr()
            a.pending_stride_b, a.pending_stride_h = k_pending.stride(0), k_pending.stride(1)
        with torch.cuda.device(q.device):
            _C.check(fn(C.byref(a), _stream(q)), entry)
    return impl


_IMPLS = {"kv_reserve": _kv_reserve, "kv_append": _kv_append, "kv_append_layers": _kv_append_layers,
          "kv_append_rope": _kv_append_rope, "kv_truncate": _kv_truncate, "kv_gather": _kv_gather,
          "kv_read_dense": _kv_read_dense, "pard_accept": _pard_accept, "linear_skinny": _linear_skinny, "attn_decode": _attn("pace_attn_decode"),
          "attn_decode_cuda_cores": _attn("pace_attn_decode_cuda_cores"), "attn_verify": _attn("pace_attn_verify"),
          "attn_prefill": _attn("pace_attn_prefill")}
for _n, _f in _IMPLS.items():
    _lib.impl(_n, _f, "CUDA")
    # shape propagation for tracers: nothing is returned, nothing to compute
    _lib.impl(_n, (lambda *a, **k: None), "Meta")

OPS = tuple(_DEFS)
