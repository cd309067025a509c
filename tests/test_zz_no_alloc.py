"""fmla_sparse_decode_static_scratch (decode with the library's built-in accumulator array) against
fmla_sparse_decode (caller-provided accumulators), both called straight through the C ABI.

The file name sorts last on purpose: the built-in array is shared per device, so this test also shows that
the entry point works after every other GPU test has used the device, as well as when run alone.
"""
import ctypes as C

import pytest
import torch

from flashmla_b200 import _lib
from flashmla_b200 import workloads as wl

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda", 0)
LAYOUT_CODE = {wl.LAYOUT_V32: _lib.LAYOUT_V32, wl.LAYOUT_MXFP8: _lib.LAYOUT_MXFP8}


class DecodeCall:
    """Device buffers and the argument struct of one decode call; scheduler output comes from fmla_sched_meta."""

    def __init__(self, w: wl.DecodeWorkload, kernel: int):
        lib = _lib.load()
        self.lib = lib
        self.stream = torch.cuda.current_stream(DEV).cuda_stream
        b, s_q, h_q, _ = w.q.shape
        topk = w.indices.shape[-1]
        self.q, self.kv, self.idx = w.q.to(DEV), w.kv_rows.to(DEV), w.indices.to(DEV)
        self.sink = None if w.attn_sink is None else w.attn_sink.to(DEV)
        self.length = None if w.topk_length is None else w.topk_length.to(DEV)
        parts, overhead, block = C.c_int32(), C.c_int32(), C.c_int32()
        _lib.check(lib.fmla_decode_plan(0, h_q, s_q, kernel, C.byref(parts), C.byref(overhead), C.byref(block)))
        self.parts = parts.value
        self.meta = torch.empty((self.parts, _lib.SCHED_META_INTS), dtype=torch.int32, device=DEV)
        self.splits = torch.empty((b + 1,), dtype=torch.int32, device=DEV)
        sa = _lib.SchedArgs(0, b, topk, block.value, overhead.value, self.parts,
                            None if self.length is None else self.length.data_ptr(),
                            self.meta.data_ptr(), self.splits.data_ptr())
        _lib.check(lib.fmla_sched_meta(C.byref(sa), self.stream))
        self.status = torch.zeros(1, dtype=torch.int32, device=DEV)
        self.rows = (b + self.parts) * s_q * h_q
        self.shape = (b, s_q, h_q)
        a = _lib.DecodeArgs()
        a.device, a.b, a.s_q, a.h_q, a.topk = 0, b, s_q, h_q, topk
        a.layout, a.kernel, a.sm_scale = LAYOUT_CODE[w.layout], kernel, float(w.sm_scale)
        a.q, a.q_stride_b, a.q_stride_s, a.q_stride_h = self.q.data_ptr(), *self.q.stride()[:3]
        a.kv, a.num_blocks, a.page_block_size, a.kv_stride_block = (
            self.kv.data_ptr(), self.kv.shape[0], self.kv.shape[1], self.kv.stride(0))
        a.indices, a.idx_stride_b, a.idx_stride_s = self.idx.data_ptr(), *self.idx.stride()[:2]
        a.topk_length = None if self.length is None else self.length.data_ptr()
        a.attn_sink = None if self.sink is None else self.sink.data_ptr()
        a.sched_meta, a.num_splits, a.num_sm_parts = self.meta.data_ptr(), self.splits.data_ptr(), self.parts
        a.status = self.status.data_ptr()
        self.args = a

    def run(self, static_scratch: bool):
        b, s_q, h_q = self.shape
        a = self.args
        out = torch.full((b, s_q, h_q, 512), float("nan"), dtype=torch.bfloat16, device=DEV)
        lse = torch.full((b, s_q, h_q), float("nan"), dtype=torch.float32, device=DEV)
        a.out, a.o_stride_b, a.o_stride_s, a.o_stride_h = out.data_ptr(), *out.stride()[:3]
        a.lse, a.lse_stride_b, a.lse_stride_s = lse.data_ptr(), *lse.stride()[:2]
        if static_scratch:
            a.o_accum = a.lse_accum = None
            code = self.lib.fmla_sparse_decode_static_scratch(C.byref(a), self.stream)
        else:
            o_acc = torch.empty((self.rows, 512), dtype=torch.float32, device=DEV)
            l_acc = torch.empty((self.rows,), dtype=torch.float32, device=DEV)
            a.o_accum, a.lse_accum = o_acc.data_ptr(), l_acc.data_ptr()
            code = self.lib.fmla_sparse_decode(C.byref(a), self.stream)
        _lib.check(code)
        torch.cuda.synchronize(DEV)
        assert int(self.status.item()) == 0, "a kernel reported a timed-out wait"
        return out, lse


CASES = {
    # name: (kernel, workload arguments); both force split requests so that the accumulators are in use
    "tc_h128": (_lib.KERNEL_TC, dict(b=6, s_q=1, h_q=128, topk=1024, lo=1500, hi=4000)),
    "simt_h16": (_lib.KERNEL_SIMT, dict(b=3, s_q=2, h_q=16, topk=512, lo=700, hi=2000)),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_static_scratch_matches_caller_scratch_twice_in_a_row(name):
    kernel, kw = CASES[name]
    first = None
    for seed in (31, 32):      # the second call finds the first call's partial results in the array
        w = wl.make_decode_workload(kw["b"], kw["s_q"], kw["h_q"], kw["topk"], kw["lo"], kw["hi"], seed=seed,
                                    invalid_frac=0.05, with_sink=True, with_topk_length=(seed == 32))
        call = DecodeCall(w, kernel)
        assert call.rows <= _lib.STATIC_SCRATCH_ROWS
        assert int(call.splits[-1].item()) > kw["b"], "the case is meant to split at least one request"
        ref_out, ref_lse = call.run(static_scratch=False)
        out, lse = call.run(static_scratch=True)
        assert not torch.isnan(out.float()).any() and not torch.isnan(lse).any()
        assert torch.equal(out.view(torch.int16), ref_out.view(torch.int16)), "out differs from fmla_sparse_decode"
        assert torch.equal(lse.view(torch.int32), ref_lse.view(torch.int32)), "lse differs from fmla_sparse_decode"
        if first is not None:
            assert not torch.equal(out.view(torch.int16), first), "the two calls were meant to differ"
        first = out.view(torch.int16).clone()


def test_static_scratch_rejects_what_does_not_fit_and_foreign_accumulators():
    w = wl.make_decode_workload(2, 1, 16, 64, 100, 200, seed=5)
    call = DecodeCall(w, _lib.KERNEL_SIMT)
    out, lse = call.run(static_scratch=True)           # fits: (2 + parts) * 16 rows
    a = call.args
    keep = a.b
    a.b = _lib.STATIC_SCRATCH_ROWS // 16 + 1            # (b + parts) * s_q * h_q is now past the limit
    assert call.lib.fmla_sparse_decode_static_scratch(C.byref(a), call.stream) == _lib.ERR_UNSUPPORTED
    assert b"exceed the built-in scratch" in call.lib.fmla_last_error()
    a.b = keep
    a.o_accum = 0x1000
    assert call.lib.fmla_sparse_decode_static_scratch(C.byref(a), call.stream) == _lib.ERR_INVALID_ARG
    assert b"must be null" in call.lib.fmla_last_error()
    torch.cuda.synchronize(DEV)
    assert int(call.status.item()) == 0


def test_static_scratch_calls_leave_the_free_device_memory_unchanged():
    """Callers of this entry point cannot allocate; neither may the entry point.  After the set-up call, further calls
    made with buffers that already exist must leave the driver's free-memory figure where it was."""
    w = wl.make_decode_workload(6, 1, 128, 1024, 1500, 4000, seed=33, invalid_frac=0.05)
    call = DecodeCall(w, _lib.KERNEL_TC)
    b, s_q, h_q = call.shape
    a = call.args
    out = torch.empty((b, s_q, h_q, 512), dtype=torch.bfloat16, device=DEV)
    lse = torch.empty((b, s_q, h_q), dtype=torch.float32, device=DEV)
    a.out, a.o_stride_b, a.o_stride_s, a.o_stride_h = out.data_ptr(), *out.stride()[:3]
    a.lse, a.lse_stride_b, a.lse_stride_s = lse.data_ptr(), *lse.stride()[:2]
    a.o_accum = a.lse_accum = None
    _lib.check(call.lib.fmla_sparse_decode_static_scratch(C.byref(a), call.stream))     # set-up call
    torch.cuda.synchronize(DEV)
    free_before, _ = torch.cuda.mem_get_info(DEV)
    for _ in range(3):
        _lib.check(call.lib.fmla_sparse_decode_static_scratch(C.byref(a), call.stream))
    torch.cuda.synchronize(DEV)
    free_after, _ = torch.cuda.mem_get_info(DEV)
    assert free_after == free_before
    assert int(call.status.item()) == 0
