"""Helpers shared by the GPU parity tests: run the public API on cuda:0, run the CPU oracle on the
same inputs, compare."""
import torch

import flash_mla
import flashmla_b200
from flashmla_b200 import workloads as wl
from oracle import attention, quant
from oracle.compare import assert_close, REF_DECODE_OUT, REF_DECODE_LSE, REF_PREFILL_OUT, REF_PREFILL_LSE, assert_north_out, NORTH_LSE

DEV = "cuda:0"


def cu(t):
    return None if t is None else t.to(DEV)


def cu_strided(t):
    """Copy of t on the GPU with t's own strides (a padded cache pool keeps its block stride; `.to` would compact it)."""
    if t is None:
        return None
    return torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=DEV).copy_(t)


def noncontig(t: torch.Tensor) -> torch.Tensor:
    """Copy of t on the GPU whose leading strides are padded (last dim stays contiguous, padded by
    128 elements so 16-byte alignment is kept), as the reference's fixtures do."""
    shape = [d + (128 if i == t.dim() - 1 else 1) for i, d in enumerate(t.shape)]
    base = torch.empty(shape, dtype=t.dtype, device=DEV)
    view = base[tuple(slice(0, d) for d in t.shape)]
    view.copy_(t)
    return view


def run_decode(w: wl.DecodeWorkload, sched=None, q=None, indices=None, kv_rows=None):
    sched = sched or flash_mla.get_mla_metadata()[0]
    out, lse = flash_mla.flash_mla_with_kvcache(
        cu(w.q) if q is None else q, cu_strided(w.kv_rows) if kv_rows is None else kv_rows, None, None, 512, sched, None,
        w.sm_scale, False, True, cu(w.indices) if indices is None else indices, cu(w.attn_sink), None, None,
        cu(w.topk_length), None, kvcache_layout=w.layout)
    assert flashmla_b200.kernel_status(DEV) == 0, "a kernel reported a timed-out wait"
    return out, lse, sched


def oracle_decode(w: wl.DecodeWorkload):
    deq = quant.dequantize_rows(w.kv_rows.contiguous(), w.layout)
    out, lse, _ = attention.sparse_decode(w.q, deq, w.indices, w.sm_scale, attn_sink=w.attn_sink, topk_length=w.topk_length)
    return out, lse


def check_decode(out, lse, ref_out, ref_lse, strict=True):
    """strict: the reference's own test tolerances; always: the acceptance gate (rel 1e-2, cos >= 0.9999, lse 1e-3)."""
    o, l = out.float().cpu(), lse.float().cpu()
    assert_north_out("out", o, ref_out.float())
    assert_close("lse", l, ref_lse.float(), **NORTH_LSE)
    if strict:
        assert_close("out", o, ref_out.float(), **REF_DECODE_OUT)
        assert_close("lse", l, ref_lse.float(), **REF_DECODE_LSE)


def run_prefill(w: wl.PrefillWorkload, q=None, kv=None, indices=None):
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(
        cu(w.q) if q is None else q, cu(w.kv) if kv is None else kv, cu(w.indices) if indices is None else indices,
        w.sm_scale, 512, cu(w.attn_sink), cu(w.topk_length))
    assert flashmla_b200.kernel_status(DEV) == 0, "a kernel reported a timed-out wait"
    return out, mx, lse


def check_prefill(out, mx, lse, ref_out, ref_mx, ref_lse, strict=True):
    o = out.float().cpu()
    assert_north_out("out", o, ref_out.float())
    assert_close("lse", lse.cpu(), ref_lse.float(), **NORTH_LSE)
    assert_close("max_logits", mx.cpu(), ref_mx.float(), **NORTH_LSE)
    if strict:
        assert_close("out", o, ref_out.float(), **REF_PREFILL_OUT)
        assert_close("lse", lse.cpu(), ref_lse.float(), **REF_PREFILL_LSE)
        assert_close("max_logits", mx.cpu(), ref_mx.float(), **REF_PREFILL_LSE)
