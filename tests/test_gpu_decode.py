"""GPU parity of sparse decode (FP8 "v32" rows and MXFP8 rows) against the reference's golden outputs
and against the CPU oracle, through the public Python API -> C ABI -> CUDA kernels."""
import ctypes as C

import numpy as np
import pytest
import torch

import flash_mla
from flashmla_b200 import _lib, workloads as wl
from oracle import sched as sched_oracle
from helpers import bf16, load_golden, t
from gpu_utils import DEV, cu, cu_strided, noncontig, run_decode, oracle_decode, check_decode
from oracle.compare import assert_north_out

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", ["decode_c1", "decode_sink_len", "decode_h128"])
def test_golden_reference_outputs(name):
    """Inputs and expected outputs come from the reference's own torch oracle (tests/golden)."""
    g = load_golden(name)
    sched = flash_mla.get_mla_metadata()[0]
    out, lse = flash_mla.flash_mla_with_kvcache(
        cu(bf16(g["q"])), cu(t(g["kv_rows"])), None, None, 512, sched, None, float(g["sm_scale"]), False, True,
        cu(t(g["indices"])), cu(t(g["attn_sink"])) if "attn_sink" in g else None, None, None,
        cu(t(g["topk_length"])) if "topk_length" in g else None)
    torch.cuda.synchronize()
    check_decode(out, lse, bf16(g["out"]), t(g["lse"]))


# Value distributions: REFD follows the reference's own decode fixtures (tests/lib.py:227-307: q ~ N(0,1)
# clamped to +-1, kv ~ N(0,1)/10, sm_scale = d^-0.55) and is held to the reference's own tolerances;
# cases without it use the benchmark's N(0,1) data and are held to the acceptance gate only, because the
# bf16 rounding of P scales with the magnitude of V.
REFD = dict(q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=576 ** -0.55)
CASES = [
    # b, s_q, h_q, topk, s_lo, s_hi, page, kwargs
    (2, 1, 16, 128, 1024, 1024, 64, dict(invalid_tail=8)),
    (4, 2, 64, 128, 100, 600, 64, dict(invalid_frac=0.05, poison_unused=True, **REFD)),
    (3, 3, 128, 576, 700, 1024, 61, dict(invalid_frac=0.02, poison_unused=True, row_pad=1, **REFD)),
    (5, 1, 128, 64, 64, 512, 2, dict(with_sink=True, **REFD)),
    (4, 3, 64, 2048, 2046, 2046, 64, dict(with_sink=True, poison_unused=True, row_pad=1, **REFD)),
    (4, 3, 128, 2048, 2046, 2046, 64, dict(with_sink=True, poison_unused=True, row_pad=1, **REFD)),
    (7, 2, 32, 192, 10, 300, 69, dict(with_topk_length=True, with_sink=True, invalid_frac=0.1, **REFD)),
    (7, 2, 128, 192, 10, 300, 69, dict(with_topk_length=True, with_sink=True, invalid_frac=0.1, **REFD)),
    (74, 1, 128, 64, 200, 512, 64, dict(invalid_frac=0.02, **REFD)),
    (321, 1, 128, 128, 64, 400, 64, dict(with_sink=True, **REFD)),
    (2, 2, 8, 320, 400, 800, 64, dict(**REFD)),
    (6, 2, 128, 512, 600, 3000, 64, dict(invalid_frac=0.02)),          # benchmark distribution
    (3, 1, 256, 256, 300, 900, 64, dict(**REFD)),                       # two head groups of 128
    (3, 2, 128, 200, 300, 700, 64, dict(invalid_frac=0.03, **REFD)),    # topk not a multiple of the 64-slot block
    (3, 2, 16, 200, 300, 700, 64, dict(invalid_frac=0.03, **REFD)),
]


@pytest.mark.parametrize("layout", [wl.LAYOUT_V32, wl.LAYOUT_MXFP8])
@pytest.mark.parametrize("case", CASES, ids=[f"b{c[0]}sq{c[1]}h{c[2]}k{c[3]}p{c[6]}" for c in CASES])
def test_against_oracle(case, layout):
    b, s_q, h_q, topk, lo, hi, page, kw = case
    w = wl.make_decode_workload(b, s_q, h_q, topk, lo, hi, page=page, layout=layout, seed=b * 131 + topk, **kw)
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse, strict="clamp" in kw or h_q % 128 != 0)


@pytest.mark.parametrize("h_q", [32, 128])
def test_all_indices_invalid_and_empty_requests(h_q):
    w = wl.make_decode_workload(4, 2, h_q, 128, 256, 256, seed=5, with_sink=True, with_topk_length=True, **REFD)
    w.indices[1] = -1                 # a request without any valid token
    w.topk_length[2] = 0              # a request of length zero
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse)
    assert torch.all(out[1] == 0) and torch.all(torch.isinf(lse[1])) and torch.all(lse[1] > 0)
    assert torch.all(out[2] == 0) and torch.all(lse[2] == float("inf"))


@pytest.mark.parametrize("h_q", [64, 128])
def test_noncontiguous_inputs_and_repeat_is_bitwise_deterministic(h_q):
    w = wl.make_decode_workload(6, 2, h_q, 256, 300, 900, seed=17, invalid_frac=0.03, row_pad=1, **REFD)
    out0, lse0, sched = run_decode(w)
    out1, lse1, _ = run_decode(w, sched=sched, q=noncontig(w.q), indices=noncontig(w.indices))
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out1, lse1, ref_out, ref_lse)


@pytest.mark.parametrize("h_q", [32, 128])
def test_batch_permutation_invariance(h_q):
    w = wl.make_decode_workload(9, 2, h_q, 192, 100, 700, seed=23, invalid_frac=0.05, **REFD)
    out0, lse0, _ = run_decode(w)
    perm = torch.randperm(9, generator=torch.Generator().manual_seed(1))
    out1, lse1, _ = run_decode(w, q=cu(w.q[perm]), indices=cu(w.indices[perm]))
    # a request may be split differently after the permutation, so compare within tolerance
    check_decode(out1, lse1.contiguous(), out0[perm.to(DEV)].cpu(), lse0[perm.to(DEV)].cpu().contiguous())


@pytest.mark.parametrize("b,s_q,h_q,topk,with_len", [(1, 1, 128, 2048, False), (3, 2, 16, 2048, True),
                                                      (128, 2, 128, 2048, False), (321, 1, 64, 576, True)])
def test_scheduler_metadata_bit_exact(b, s_q, h_q, topk, with_len):
    lib = _lib.load()
    parts, ovh, blk = C.c_int32(), C.c_int32(), C.c_int32()
    _lib.check(lib.fmla_decode_plan(0, h_q, s_q, _lib.KERNEL_AUTO, C.byref(parts), C.byref(ovh), C.byref(blk)))
    gen = torch.Generator().manual_seed(b)
    tl = torch.randint(0, topk + 1, (b,), generator=gen, dtype=torch.int32) if with_len else None
    meta = torch.full((parts.value, 8), -7, dtype=torch.int32, device=DEV)
    ns = torch.full((b + 1,), -7, dtype=torch.int32, device=DEV)
    tl_dev = cu(tl)
    a = _lib.SchedArgs(0, b, topk, blk.value, ovh.value, parts.value, None if tl is None else tl_dev.data_ptr(),
                       meta.data_ptr(), ns.data_ptr())
    _lib.check(lib.fmla_sched_meta(C.byref(a), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    want_meta, want_ns = sched_oracle.sched_meta(b, topk, None if tl is None else tl.tolist(), blk.value, ovh.value, parts.value)
    assert np.array_equal(ns.cpu().numpy(), want_ns)
    assert np.array_equal(meta.cpu().numpy(), want_meta)


def test_full_size_property_partition_of_work():
    """At the benchmark's full decode shape: the split-KV result of every query must not depend on how
    the scheduler cut the work, so decoding each half of the batch alone (a different schedule) must
    reproduce the rows of the full run."""
    w = wl.make_decode_workload(16, 2, 128, 2048, 4096, 8192, seed=3, invalid_frac=0.02, keep_bf16=False)
    out, lse, _ = run_decode(w)
    q, idx, rows = cu(w.q), cu(w.indices), cu(w.kv_rows)
    for lo, hi in ((0, 5), (5, 16)):
        o2, l2, _ = run_decode(w, q=q[lo:hi], indices=idx[lo:hi], kv_rows=rows)
        check_decode(o2, l2.contiguous(), out[lo:hi].cpu(), lse[lo:hi].cpu().contiguous(), strict=False)
    assert bool(torch.isfinite(out.float()).all())


@pytest.mark.parametrize("kernel", ["simt", "tc"])
@pytest.mark.parametrize("h_q", [64, 128, 192])
def test_both_kernel_families_agree_with_oracle(monkeypatch, kernel, h_q):
    """The CUDA-core and the tensor-core kernels on the same inputs (64 and 192 heads exercise the padded last
    head group of the tensor-core kernel), decode and prefill."""
    monkeypatch.setenv("FMLA_KERNEL", kernel)
    w = wl.make_decode_workload(5, 2, h_q, 320, 200, 1500, seed=41 + h_q, invalid_frac=0.05, with_sink=True,
                                with_topk_length=True, **REFD)
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse, strict=True)
    from oracle import attention
    from gpu_utils import run_prefill, check_prefill
    pw = wl.make_prefill_workload(11, 700, h_q, 256, seed=43 + h_q, with_sink=True, with_topk_length=True, std=0.1, sm_scale=0.5)
    o, mx, l = run_prefill(pw)
    ro, _, rm, rl = attention.sparse_prefill_fwd(pw.q, pw.kv, pw.indices, pw.sm_scale, attn_sink=pw.attn_sink,
                                                 topk_length=pw.topk_length)
    check_prefill(o, mx, l, ro, rm, rl, strict=True)


def test_plain_load_q_path():
    """Q normally reaches tensor memory through TMA tiles; the plain-load path (taken when the driver refuses q's
    strides for a tensor map) is forced here through fmla_set_option and must give the same bits."""
    lib = _lib.load()
    w = wl.make_decode_workload(4, 2, 128, 512, 600, 2500, seed=77, invalid_frac=0.05, with_sink=True, **REFD)
    from gpu_utils import run_prefill
    pw = wl.make_prefill_workload(150, 900, 128, 256, seed=78, std=0.1, sm_scale=0.5)
    out0, lse0, _ = run_decode(w)
    ref = run_prefill(pw)
    try:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_Q_LOADS, 1))
        out1, lse1, _ = run_decode(w)
        got = run_prefill(pw)
    finally:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_Q_LOADS, 0))
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    assert all(torch.equal(a, b) for a, b in zip(ref, got))


def test_plain_store_epilogue_path():
    """Results normally leave through TMA box stores; the plain-store epilogue (taken when the driver refuses out's
    strides for a tensor map) is forced here through fmla_set_option and must give the same bits, for unsplit and
    split requests and for the prefill kernel."""
    lib = _lib.load()
    w = wl.make_decode_workload(5, 2, 128, 1024, 1100, 4000, seed=79, invalid_frac=0.05, with_sink=True, **REFD)
    from gpu_utils import run_prefill
    pw = wl.make_prefill_workload(150, 900, 128, 256, seed=80, std=0.1, sm_scale=0.5)
    out0, lse0, _ = run_decode(w)
    ref = run_prefill(pw)
    try:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_STORES, 1))
        out1, lse1, _ = run_decode(w)
        got = run_prefill(pw)
    finally:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_STORES, 0))
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)
    assert all(torch.equal(a, b) for a, b in zip(ref, got))


def _raw_decode(w, kernel=None, monkeypatch=None):
    """flash_mla_with_kvcache without the helper's status assertion; returns (out, lse, status)."""
    import flashmla_b200
    if kernel is not None:
        monkeypatch.setenv("FMLA_KERNEL", kernel)
    out, lse = flash_mla.flash_mla_with_kvcache(cu(w.q), cu(w.kv_rows), None, None, 512, flash_mla.get_mla_metadata()[0], None,
                                                w.sm_scale, False, True, cu(w.indices), kvcache_layout=w.layout)
    status = flashmla_b200.kernel_status(DEV)
    if kernel is not None:
        monkeypatch.delenv("FMLA_KERNEL")
    return out, lse, status


@pytest.mark.parametrize("layout", [wl.LAYOUT_V32, wl.LAYOUT_MXFP8])
def test_cache_values_beyond_the_fp16_stage_are_reported_not_silently_clipped(layout, monkeypatch):
    """The tensor-core decode kernel stages dequantised values in fp16.  Tile scales up to 2^7 (tile maxima up to
    57344) are exact; beyond that it reports FMLA_STATUS_CLIPPED through the status word, and the CUDA-core kernel,
    which multiplies in fp32 like the reference (tests/quant.py:93-104), gives the right answer."""
    kw = dict(seed=51, invalid_frac=0.02, q_std=1e-4, layout=layout)
    # tile maxima between 2^14 and 5e4: the largest scale is exactly 2^7, nothing is clipped
    w = wl.make_decode_workload(3, 2, 128, 256, 300, 900, kv_std=2e4, clamp=5e4, **kw)
    out, lse, status = _raw_decode(w)
    assert status == 0
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse, strict=False)
    # tile maxima around 1e5: scales of 2^8, beyond the fp16 stage
    w = wl.make_decode_workload(3, 2, 128, 256, 300, 900, kv_std=4e4, **kw)
    _, _, status = _raw_decode(w)
    assert status == _lib.STATUS_CLIPPED
    out, lse, status = _raw_decode(w, "simt", monkeypatch)
    assert status == 0
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse, strict=False)


def test_queries_beyond_the_fp16_stage_are_reported():
    w = wl.make_decode_workload(2, 1, 128, 128, 200, 400, seed=52, q_std=1.0, kv_std=0.1, clamp=1.0)
    w.q[1, 0, 5, 17] = 7e4            # representable in bf16, not in fp16
    _, _, status = _raw_decode(w)
    assert status == _lib.STATUS_CLIPPED


def test_v32_scales_that_are_not_powers_of_two():
    """The V32 format stores fp32 scales; the quantiser only emits powers of two, but any scale is legal
    (tests/quant.py:101-104 multiplies by whatever is stored).  e4m3 times 1.5 * 2^k is still exact in fp16."""
    w = wl.make_decode_workload(3, 2, 128, 256, 300, 900, seed=53, invalid_frac=0.02, **REFD)
    rows = w.kv_rows.view(-1, 656)
    scales = rows[:, 512:528].contiguous().view(torch.float32)
    rows[:, 512:528] = (scales * 1.5).view(torch.uint8)
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse)


def test_unsplit_batch_is_complete_for_the_next_kernel_in_the_stream():
    """A batch in which no request is split leaves the combine kernel nothing to merge; its blocks must still wait for
    the attention kernel, or the next kernel in the stream (here a copy of `out`, launched without any host
    synchronisation) could read results that are not written yet."""
    lib = _lib.load()
    parts, ovh, blk = C.c_int32(), C.c_int32(), C.c_int32()
    _lib.check(lib.fmla_decode_plan(0, 128, 1, _lib.KERNEL_AUTO, C.byref(parts), C.byref(ovh), C.byref(blk)))
    b = parts.value                       # one whole request per partition: nothing is split
    w = wl.make_decode_workload(b, 1, 128, 2048, 2100, 2100, seed=54, **REFD)
    q, kv, idx = cu(w.q), cu(w.kv_rows), cu(w.indices)
    sched = flash_mla.get_mla_metadata()[0]
    ref, ref_lse = flash_mla.flash_mla_with_kvcache(q, kv, None, None, 512, sched, None, w.sm_scale, False, True, idx)
    torch.cuda.synchronize()
    splits = sched.num_splits.cpu()
    assert int((splits[1:] - splits[:-1]).max()) == 1, "the case is meant to have no split request"
    ref = ref.clone()
    for _ in range(20):
        out, lse = flash_mla.flash_mla_with_kvcache(q, kv, None, None, 512, sched, None, w.sm_scale, False, True, idx)
        copy = out.clone()                # the next kernel in the stream; no host synchronisation in between
        out.zero_()                       # and the one after it, so a late attention kernel would show in `out` too
        torch.cuda.synchronize()
        assert torch.equal(copy, ref)


# ---- the reference's d_qk = 512 cache format ("MODEL1": 448 e4m3 + 64 bf16 per token, 7 e8m0 scales per 64 values,
# ---- stored block-wise; tests/quant.py:55-75 of the reference) ---------------------------------------------------
@pytest.mark.parametrize("name", ["decode_model1", "decode_model1_h128"])
def test_model1_golden_reference_outputs(name):
    g = load_golden(name)
    out, lse = flash_mla.flash_mla_with_kvcache(
        cu(bf16(g["q"])), _model1_pool(t(g["kv_rows"])), None, None, 512, flash_mla.get_mla_metadata()[0], None, float(g["sm_scale"]),
        False, True, cu(t(g["indices"])), cu(t(g["attn_sink"])) if "attn_sink" in g else None, None, None,
        cu(t(g["topk_length"])) if "topk_length" in g else None)
    torch.cuda.synchronize()
    check_decode(out, lse, bf16(g["out"]), t(g["lse"]))


def _model1_pool(rows):
    """A packed (num_blocks, page, 1, 584) fixture on the GPU with blocks padded to a multiple of 576 bytes, as the
    reference allocates them (tests/quant.py:57-58): the kernels read 16-byte pieces, so blocks start 16-byte aligned."""
    nb, page = rows.shape[0], rows.shape[1]
    pool = torch.zeros((nb, (page * 584 + 575) // 576 * 576), dtype=torch.uint8, device=DEV)
    view = pool[:, :page * 584].view(nb, page, 1, 584)
    view.copy_(rows)
    return view


M1_CASES = [
    # b, s_q, h_q, topk, s_lo, s_hi, page, kwargs  (the reference's matrix: d_qk 512 x h_q {64, 128} x pages {2, 64, 69})
    (4, 1, 64, 64, 512, 512, 2, dict(with_sink=True)),
    (4, 3, 128, 576, 1024, 1024, 61, dict(invalid_frac=0.02, poison_unused=True)),
    (3, 2, 128, 2048, 2046, 2046, 64, dict(with_sink=True, with_topk_length=True)),
    (74, 1, 64, 64, 200, 512, 69, dict(invalid_frac=0.02)),
    (5, 2, 16, 200, 300, 700, 64, dict(invalid_frac=0.03)),
]


@pytest.mark.parametrize("case", M1_CASES, ids=[f"b{c[0]}sq{c[1]}h{c[2]}k{c[3]}p{c[6]}" for c in M1_CASES])
def test_model1_against_oracle(case):
    b, s_q, h_q, topk, lo, hi, page, kw = case
    w = wl.make_decode_workload(b, s_q, h_q, topk, lo, hi, page=page, layout=wl.LAYOUT_MODEL1, seed=b * 17 + topk,
                                q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=512 ** -0.55, **kw)
    out, lse, _ = run_decode(w)
    ref_out, ref_lse = oracle_decode(w)
    check_decode(out, lse, ref_out, ref_lse)


def test_model1_runs_on_the_tensor_core_kernel_and_agrees_with_the_cuda_core_kernel(monkeypatch):
    """Head counts that are multiples of 64 take the tensor-core variant for MODEL1 blocks (forced here, so that a
    silent fall-back to the CUDA-core kernel would show as an error), and both kernels give the oracle's answer."""
    w = wl.make_decode_workload(9, 2, 128, 640, 700, 3000, page=64, layout=wl.LAYOUT_MODEL1, seed=77, invalid_frac=0.02,
                                with_sink=True, with_topk_length=True, q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=512 ** -0.55)
    ref_out, ref_lse = oracle_decode(w)
    res = {}
    for kernel in ("tc", "simt"):
        monkeypatch.setenv("FMLA_KERNEL", kernel)
        out, lse, _ = run_decode(w)
        check_decode(out, lse, ref_out, ref_lse)
        res[kernel] = out.float().cpu()
    assert_north_out("tc vs simt", res["tc"], res["simt"])


def test_model1_rope_values_beyond_fp16_are_reported():
    """The tensor-core variant stages the 64 bf16 values of a MODEL1 row in fp16 like the rest of the row."""
    w = wl.make_decode_workload(2, 1, 128, 128, 200, 400, page=64, layout=wl.LAYOUT_MODEL1, seed=78, q_std=1e-4, kv_std=0.1, clamp=1.0)
    rows = w.kv_rows.contiguous().clone()
    nb, page = rows.shape[0], rows.shape[1]
    # the first bf16 value of every token (bytes 448, 449 of its 576 data bytes) becomes 0x4790 = 73728.0
    flat = rows.reshape(nb, page * 584)
    data = flat[:, :page * 576].view(nb, page, 576)
    data[:, :, 448] = 0x90
    data[:, :, 449] = 0x47
    import flashmla_b200
    flash_mla.flash_mla_with_kvcache(cu(w.q), _model1_pool(flat.view(nb, page, 1, 584)), None, None, 512, flash_mla.get_mla_metadata()[0], None,
                                     w.sm_scale, False, True, cu(w.indices))
    assert flashmla_b200.kernel_status(DEV) == _lib.STATUS_CLIPPED
