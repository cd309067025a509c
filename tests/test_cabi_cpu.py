"""Host-side checks that need no GPU: the C-ABI library loads, exports every symbol the header
declares, and rejects bad arguments with a status code and a message before touching CUDA."""
import ctypes as C
import os
import re

import pytest

from flashmla_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_header_symbols_are_exported_and_bound():
    header = open(os.path.join(ROOT, "include", "flashmla_b200.h")).read()
    declared = set(re.findall(r"^(?:int|int64_t|const char\*)\s+(fmla_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found in the header"
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/flashmla_b200.h but not exported"
    assert declared == set(_lib.EXPORTS), "ctypes prototypes and header declarations differ"
    assert lib.fmla_version() >= 120
    # workspace query of the backward: pure host arithmetic (2 bf16 arrays of 128 heads x topk rounded up to 128 per unit)
    assert lib.fmla_sparse_prefill_bwd_workspace(4096, 128, 2048, _lib.KERNEL_AUTO) == 4096 * 2 * 128 * 2048 * 2
    assert lib.fmla_sparse_prefill_bwd_workspace(3, 256, 100, _lib.KERNEL_TC) == 3 * 2 * 2 * 128 * 128 * 2
    assert lib.fmla_sparse_prefill_bwd_workspace(3, 192, 100, _lib.KERNEL_AUTO) == 3 * 2 * 2 * 128 * 128 * 2   # 128 + 64 heads: two units
    assert lib.fmla_sparse_prefill_bwd_workspace(3, 16, 100, _lib.KERNEL_AUTO) == 0
    assert lib.fmla_sparse_prefill_bwd_workspace(3, 128, 100, _lib.KERNEL_SIMT) == 0


def test_struct_sizes_match_header_layout():
    # every struct is a sequence of naturally aligned ints, floats, pointers and int64: the ctypes
    # mirror must not be smaller than the sum of its fields and must be 8-byte aligned
    for s in (_lib.SchedArgs, _lib.DecodeArgs, _lib.DenseDecodeArgs, _lib.PrefillArgs, _lib.PrefillBwdArgs, _lib.KvQuantArgs, _lib.CacheIndexArgs):
        assert C.sizeof(s) % 8 == 0 and C.alignment(s) == 8


@pytest.mark.parametrize("fn,args", [
    ("fmla_sched_meta", _lib.SchedArgs),
    ("fmla_sparse_decode", _lib.DecodeArgs),
    ("fmla_dense_decode", _lib.DenseDecodeArgs),
    ("fmla_sparse_prefill_fwd", _lib.PrefillArgs),
    ("fmla_sparse_prefill_bwd", _lib.PrefillBwdArgs),
    ("fmla_kv_quantize", _lib.KvQuantArgs),
    ("fmla_cache_indices", _lib.CacheIndexArgs),
])
def test_null_and_zero_arguments_are_rejected(fn, args):
    lib = _lib.load()
    f = getattr(lib, fn)
    assert f(None, None) == _lib.ERR_INVALID_ARG
    assert b"null argument struct" in lib.fmla_last_error()
    assert f(C.byref(args()), None) == _lib.ERR_INVALID_ARG
    assert b"must be positive" in lib.fmla_last_error()


def test_decode_rejects_null_pointers_bad_layout_and_misalignment():
    lib = _lib.load()
    a = _lib.DecodeArgs()
    a.b, a.s_q, a.h_q, a.topk = 1, 1, 16, 64
    a.layout = 7
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_UNSUPPORTED
    a.layout = _lib.LAYOUT_V32
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_INVALID_ARG
    assert b"non-null" in lib.fmla_last_error()
    for f in ("q", "kv", "indices", "out", "lse", "sched_meta", "num_splits", "o_accum", "lse_accum"):
        setattr(a, f, 0x1000)
    a.num_sm_parts, a.num_blocks, a.page_block_size = 4, 2, 64
    a.kv_stride_block = 64 * 656 - 1
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_INVALID_ARG
    a.kv_stride_block = 64 * 656 + 8
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_ALIGNMENT
    a.kv_stride_block = 65 * 656
    a.q_stride_h = 577
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_ALIGNMENT
    a.q_stride_h = 576
    a.kernel = _lib.KERNEL_TC          # 16 heads cannot use the tensor-core kernel
    assert lib.fmla_sparse_decode(C.byref(a), None) == _lib.ERR_UNSUPPORTED


def test_dense_decode_rejects_null_pointers_bad_strides_and_head_counts():
    lib = _lib.load()
    a = _lib.DenseDecodeArgs()
    a.b, a.s_q, a.h_q, a.sm_scale = 2, 1, 128, 0.1
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_INVALID_ARG
    assert b"non-null" in lib.fmla_last_error()
    for f in ("q", "kv", "block_table", "cache_seqlens", "out", "lse", "sched_meta", "num_splits", "o_accum", "lse_accum"):
        setattr(a, f, 0x1000)
    a.num_sm_parts, a.num_blocks, a.page_block_size, a.max_blocks_per_seq, a.block_table_stride = 4, 8, 64, 4, 4
    a.q_stride_b, a.q_stride_s, a.q_stride_h = 128 * 576, 128 * 576, 576
    a.o_stride_b, a.o_stride_s, a.o_stride_h = 128 * 512, 128 * 512, 512
    a.kv_stride_row = 512
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_INVALID_ARG
    assert b"row stride" in lib.fmla_last_error()
    a.kv_stride_row = 580
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_ALIGNMENT
    a.kv_stride_row = 576
    a.block_table_stride = 3
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_INVALID_ARG
    a.block_table_stride = 4
    a.h_q = 96
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_UNSUPPORTED
    assert b"multiple of 64" in lib.fmla_last_error()
    a.h_q, a.sm_scale = 128, 0.0
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_UNSUPPORTED
    a.sm_scale = 0.1
    a.max_blocks_per_seq = a.block_table_stride = 1 << 26          # a block table row of 2^32 tokens
    assert lib.fmla_dense_decode(C.byref(a), None) == _lib.ERR_UNSUPPORTED


def test_python_interface_refuses_cpu_tensors_and_dense_mode():
    import torch
    import flash_mla
    meta, _ = flash_mla.get_mla_metadata()
    assert isinstance(meta, flash_mla.FlashMLASchedMeta) and not meta.have_initialized
    q = torch.zeros((1, 1, 16, 576), dtype=torch.bfloat16)
    kc = torch.zeros((2, 64, 1, 656), dtype=torch.uint8)
    idx = torch.zeros((1, 1, 64), dtype=torch.int32)
    with pytest.raises(AssertionError, match="num_splits must be None"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, meta, 3, None, False, True, idx)
    with pytest.raises(AssertionError, match="is_fp8_kvcache must be True"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, flash_mla.get_mla_metadata()[0], None, None, False, False, idx)
    with pytest.raises(AssertionError, match="causal must be False"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, flash_mla.get_mla_metadata()[0], None, None, True, True, idx)
    with pytest.raises(AssertionError, match="block_table and cache_seqlens must be provided when dense attention is used"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, flash_mla.get_mla_metadata()[0])
    with pytest.raises(RuntimeError, match="no CPU path"):      # the dense branch has no CPU path either
        flash_mla.flash_mla_with_kvcache(q, torch.zeros((2, 64, 1, 576), dtype=torch.bfloat16), torch.zeros((1, 2), dtype=torch.int32),
                                         torch.ones((1,), dtype=torch.int32), 512, flash_mla.get_mla_metadata()[0])
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, flash_mla.get_mla_metadata()[0], None, None, False, True, idx)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_mla.flash_mla_sparse_fwd(q[0], torch.zeros((8, 1, 576), dtype=torch.bfloat16), idx, 0.1)
    # a reused sched_meta must see the same shapes
    m = flash_mla.get_mla_metadata()[0]
    with pytest.raises(RuntimeError):
        flash_mla.flash_mla_with_kvcache(q, kc, None, None, 512, m, None, None, False, True, idx)
    q2 = torch.zeros((2, 1, 16, 576), dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="sched_meta.config.b must be equal"):
        flash_mla.flash_mla_with_kvcache(q2, kc, None, None, 512, m, None, None, False, True, idx)
