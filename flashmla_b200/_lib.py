"""ctypes binding of libflashmla_b200.so: the structs and prototypes of include/flashmla_b200.h.

The library is loaded lazily and loading fails loudly: there is no fallback path.  If the shared
object is missing it is built in-tree with nvcc (``flashmla_b200.build``).
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_PKG = os.path.dirname(os.path.abspath(__file__))
# FLASHMLA_B200_LIB overrides the library location (e.g. an instrumented build).
LIB_PATH = os.environ.get("FLASHMLA_B200_LIB") or os.path.join(_PKG, "lib", "libflashmla_b200.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_ALIGNMENT, ERR_CUDA, ERR_ARCH, ERR_TIMEOUT = range(7)
LAYOUT_V32, LAYOUT_MXFP8, LAYOUT_MODEL1 = 0, 1, 2
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TC = 0, 1, 2
SCHED_META_INTS = 8
STATIC_SCRATCH_ROWS = 16384
OPTION_PLAIN_Q_LOADS = 1
OPTION_PLAIN_STORES = 2
STATUS_CLIPPED = 100

_i32p = C.POINTER(C.c_int32)
_f32p = C.POINTER(C.c_float)


class SchedArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("b", C.c_int), ("topk", C.c_int),
        ("block_topk", C.c_int), ("fixed_overhead_blocks", C.c_int), ("num_sm_parts", C.c_int),
        ("topk_length", C.c_void_p), ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p),
        ("extra_topk", C.c_int), ("extra_topk_length", C.c_void_p),
    ]


class DecodeArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("b", C.c_int), ("s_q", C.c_int), ("h_q", C.c_int), ("topk", C.c_int),
        ("layout", C.c_int), ("kernel", C.c_int), ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("kv", C.c_void_p), ("num_blocks", C.c_int64), ("page_block_size", C.c_int64), ("kv_stride_block", C.c_int64),
        ("indices", C.c_void_p), ("idx_stride_b", C.c_int64), ("idx_stride_s", C.c_int64),
        ("topk_length", C.c_void_p), ("attn_sink", C.c_void_p),
        ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_s", C.c_int64), ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_s", C.c_int64),
        ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p), ("num_sm_parts", C.c_int),
        ("o_accum", C.c_void_p), ("lse_accum", C.c_void_p), ("status", C.c_void_p),
        ("attn_done_event", C.c_void_p),
        ("extra_kv", C.c_void_p), ("extra_num_blocks", C.c_int64), ("extra_page_block_size", C.c_int64),
        ("extra_kv_stride_block", C.c_int64), ("extra_indices", C.c_void_p), ("extra_idx_stride_b", C.c_int64),
        ("extra_idx_stride_s", C.c_int64), ("extra_topk", C.c_int), ("extra_topk_length", C.c_void_p),
    ]


class DenseDecodeArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("b", C.c_int), ("s_q", C.c_int), ("h_q", C.c_int), ("causal", C.c_int), ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_b", C.c_int64), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("kv", C.c_void_p), ("num_blocks", C.c_int64), ("page_block_size", C.c_int64), ("kv_stride_row", C.c_int64),
        ("block_table", C.c_void_p), ("block_table_stride", C.c_int64), ("max_blocks_per_seq", C.c_int64),
        ("cache_seqlens", C.c_void_p),
        ("out", C.c_void_p), ("o_stride_b", C.c_int64), ("o_stride_s", C.c_int64), ("o_stride_h", C.c_int64),
        ("lse", C.c_void_p), ("lse_stride_b", C.c_int64), ("lse_stride_s", C.c_int64),
        ("sched_meta", C.c_void_p), ("num_splits", C.c_void_p), ("num_sm_parts", C.c_int),
        ("o_accum", C.c_void_p), ("lse_accum", C.c_void_p), ("status", C.c_void_p),
    ]


class PrefillArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("s_q", C.c_int), ("s_kv", C.c_int), ("h_q", C.c_int), ("topk", C.c_int),
        ("kernel", C.c_int), ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("kv", C.c_void_p), ("kv_stride_s", C.c_int64),
        ("indices", C.c_void_p), ("idx_stride_s", C.c_int64),
        ("attn_sink", C.c_void_p), ("topk_length", C.c_void_p),
        ("out", C.c_void_p), ("max_logits", C.c_void_p), ("lse", C.c_void_p), ("status", C.c_void_p),
        ("d_qk", C.c_int),
    ]


class PrefillBwdArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("s_q", C.c_int), ("s_kv", C.c_int), ("h_q", C.c_int), ("topk", C.c_int),
        ("kernel", C.c_int), ("sm_scale", C.c_float),
        ("q", C.c_void_p), ("q_stride_s", C.c_int64), ("q_stride_h", C.c_int64),
        ("kv", C.c_void_p), ("kv_stride_s", C.c_int64),
        ("out", C.c_void_p), ("dout", C.c_void_p), ("do_stride_s", C.c_int64), ("do_stride_h", C.c_int64),
        ("lse", C.c_void_p), ("indices", C.c_void_p), ("idx_stride_s", C.c_int64),
        ("attn_sink", C.c_void_p), ("topk_length", C.c_void_p),
        ("dq", C.c_void_p), ("dkv_accum", C.c_void_p), ("dkv", C.c_void_p),
        ("workspace", C.c_void_p), ("workspace_bytes", C.c_int64), ("status", C.c_void_p),
        ("grad_begin_event", C.c_void_p), ("grad_end_event", C.c_void_p),
    ]


class KvQuantArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("layout", C.c_int), ("n_rows", C.c_int64), ("page_block_size", C.c_int64),
        ("kv", C.c_void_p), ("kv_stride_row", C.c_int64), ("rows", C.c_void_p), ("rows_stride_block", C.c_int64),
    ]


class CacheIndexArgs(C.Structure):
    _fields_ = [
        ("device", C.c_int), ("b", C.c_int), ("page_block_size", C.c_int), ("max_pages", C.c_int),
        ("per_request", C.c_int64), ("positions", C.c_void_p), ("block_table", C.c_void_p), ("indices", C.c_void_p),
    ]


EXPORTS = {
    "fmla_version": (C.c_int, []),
    "fmla_last_error": (C.c_char_p, []),
    "fmla_set_option": (C.c_int, [C.c_int, C.c_int]),
    "fmla_tensor_map_cache_stats": (C.c_int, [C.POINTER(C.c_uint64), C.POINTER(C.c_uint64)]),
    "fmla_decode_plan": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, _i32p, _i32p, _i32p]),
    "fmla_sched_meta": (C.c_int, [C.POINTER(SchedArgs), C.c_void_p]),
    "fmla_sparse_decode": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "fmla_sparse_decode_static_scratch": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "fmla_dense_decode": (C.c_int, [C.POINTER(DenseDecodeArgs), C.c_void_p]),
    "fmla_sparse_prefill_fwd": (C.c_int, [C.POINTER(PrefillArgs), C.c_void_p]),
    "fmla_sparse_prefill_bwd": (C.c_int, [C.POINTER(PrefillBwdArgs), C.c_void_p]),
    "fmla_sparse_prefill_bwd_workspace": (C.c_int64, [C.c_int, C.c_int, C.c_int, C.c_int]),
    "fmla_kv_quantize": (C.c_int, [C.POINTER(KvQuantArgs), C.c_void_p]),
    "fmla_cache_indices": (C.c_int, [C.POINTER(CacheIndexArgs), C.c_void_p]),
}

_lib = None
_lock = threading.Lock()


def load() -> C.CDLL:
    """Returns the loaded library, building it first if the shared object is absent."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is None:
            if not os.path.exists(LIB_PATH):
                from . import build as _build
                _build.build()
            lib = C.CDLL(LIB_PATH)
            for name, (res, args) in EXPORTS.items():
                fn = getattr(lib, name)       # AttributeError if a declared symbol is missing
                fn.restype = res
                fn.argtypes = args
            _lib = lib
    return _lib


class FlashMLAError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"flashmla_b200 error {code}: {message}")
        self.code = code


def check(code: int) -> None:
    if code != OK:
        raise FlashMLAError(code, load().fmla_last_error().decode("utf-8", "replace"))
