"""The case matrices of the reference's own sparse tests, ported as parameters
(tests/test_flash_mla_sparse_decoding.py:23-126 and tests/test_flash_mla_sparse_prefill.py:62-160), run against the
CPU oracle at the reference's own tolerances with inputs drawn like its fixtures (tests/lib.py:121-307).

The reference checks every case against torch on the GPU; here the checker is the CPU oracle, so the largest
combinations are sub-sampled (every shape, head count, head dimension and feature appears; the cross product of the
largest batch with the longest top-k list does not).  Cases whose answer is known in closed form (every index
invalid) are checked against that instead of the oracle, at full size.
"""
import itertools

import pytest
import torch

import flash_mla
import flashmla_b200
from flashmla_b200 import workloads as wl
from oracle import attention, quant
from gpu_utils import DEV, cu, cu_strided, check_decode, check_prefill

pytestmark = pytest.mark.gpu
PADS = (-2147483648, -123456, -1, 114514, 1919810, 2147480000, 2147483647)      # tests/lib.py:131-132


# ---- prefill (test_flash_mla_sparse_prefill.py:62-160) -----------------------------------------------------------
PREFILL_SHAPES = [(128, 128), (256, 256), (512, 512), (592, 128), (1840, 256), (1592, 384), (1521, 512),
                  (95, 128), (153, 256), (114, 384)]
PREFILL_CASES = [(d, h, s_kv, topk, s_q) for d in (512, 576) for h in (128, 64) for (s_kv, topk) in PREFILL_SHAPES
                 for s_q in (1, 62, 213)]


@pytest.mark.parametrize("d_qk,h_q,s_kv,topk,s_q", PREFILL_CASES, ids=[f"d{c[0]}h{c[1]}kv{c[2]}k{c[3]}sq{c[4]}" for c in PREFILL_CASES])
def test_prefill_regular_and_irregular_shapes(d_qk, h_q, s_kv, topk, s_q):
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=s_q + s_kv + topk, std=0.1, sm_scale=0.5, invalid_pads=PADS, d_qk=d_qk)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(cu(w.q), cu(w.kv), cu(w.indices), w.sm_scale)
    assert flashmla_b200.kernel_status(DEV) == 0
    ro, _, rm, rl = attention.sparse_prefill_fwd(w.q, w.kv, w.indices, w.sm_scale)
    check_prefill(out, mx, lse, ro, rm, rl)


FEATURE_SHAPES = [(592, 128), (1840, 256), (1592, 384), (1521, 512), (95, 128), (153, 256), (114, 384)]
FEATURE_CASES = [(d, h, s_kv, topk, s_q, sink, tl) for d in (512, 576) for h in (128, 64) for (s_kv, topk) in FEATURE_SHAPES
                 for s_q in (62, 213) for sink in (False, True) for tl in (False, True) if (sink or tl)]
FEATURE_CASES = FEATURE_CASES[::3]        # every third combination: each shape and feature still appears for both d_qk


@pytest.mark.parametrize("d_qk,h_q,s_kv,topk,s_q,sink,tl", FEATURE_CASES,
                         ids=[f"d{c[0]}h{c[1]}kv{c[2]}k{c[3]}sq{c[4]}{'S' if c[5] else ''}{'L' if c[6] else ''}" for c in FEATURE_CASES])
def test_prefill_with_sink_and_topk_length(d_qk, h_q, s_kv, topk, s_q, sink, tl):
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=3 * s_q + s_kv, std=0.1, sm_scale=0.5, invalid_pads=PADS,
                                 with_sink=sink, with_topk_length=tl, d_qk=d_qk)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(cu(w.q), cu(w.kv), cu(w.indices), w.sm_scale, 512, cu(w.attn_sink), cu(w.topk_length))
    assert flashmla_b200.kernel_status(DEV) == 0
    ro, _, rm, rl = attention.sparse_prefill_fwd(w.q, w.kv, w.indices, w.sm_scale, attn_sink=w.attn_sink, topk_length=w.topk_length)
    check_prefill(out, mx, lse, ro, rm, rl)


@pytest.mark.parametrize("d_qk", [512, 576])
@pytest.mark.parametrize("h_q", [128, 64])
@pytest.mark.parametrize("s_q,s_kv,topk", [(1, 128, 128), (1, 256, 256), (1234, 4321, 4096), (4096, 2048, 2048)])
def test_prefill_every_index_invalid(d_qk, h_q, s_q, s_kv, topk):
    """Closed form (tests/ref.py:50-52): out = 0, lse = +inf, max_logits = -inf, whatever the sink."""
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=5, device=DEV, std=0.1, sm_scale=0.5, with_sink=True,
                                 with_topk_length=True, d_qk=d_qk)
    pads = torch.tensor(PADS, dtype=torch.int32, device=DEV)
    w.indices = pads[torch.randint(0, len(PADS), w.indices.shape, device=DEV)]
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale, 512, w.attn_sink, w.topk_length)
    assert flashmla_b200.kernel_status(DEV) == 0
    assert bool((out == 0).all()) and bool((lse == float("inf")).all()) and bool((mx == float("-inf")).all())


@pytest.mark.parametrize("d_qk", [512, 576])
@pytest.mark.parametrize("h_q", [128, 64])
@pytest.mark.parametrize("s_kv,topk,s_q", [(32, 2048, 1), (64, 8192, 1), (32, 2048, 1024), (64, 8192, 1024)])
def test_prefill_blocks_without_any_valid_index(d_qk, h_q, s_kv, topk, s_q):
    """topk far above s_kv: most 64-slot blocks of a query hold no valid index at all."""
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=6, device=DEV, std=0.1, sm_scale=0.5, invalid_pads=PADS,
                                 with_sink=True, with_topk_length=True, d_qk=d_qk)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale, 512, w.attn_sink, w.topk_length)
    assert flashmla_b200.kernel_status(DEV) == 0
    toks = sorted({0, s_q // 2, s_q - 1})
    ro, _, rm, rl = attention.sparse_prefill_fwd(w.q[toks].cpu(), w.kv.cpu(), w.indices[toks].cpu(), w.sm_scale,
                                                 attn_sink=w.attn_sink.cpu(), topk_length=w.topk_length[toks].cpu())
    check_prefill(out[toks], mx[toks], lse[toks], ro, rm, rl)


@pytest.mark.parametrize("d_qk,h_q", [(576, 128), (512, 64)])
def test_prefill_more_queries_than_a_grid_dimension_holds(d_qk, h_q):
    """s_q = 70000 (test_flash_mla_sparse_prefill.py:134-141): the reference only checks that the launch works; here the
    first and last queries are compared with the oracle as well."""
    w = wl.make_prefill_workload(70000, 256, h_q, 256, seed=7, device=DEV, std=0.1, sm_scale=0.5, with_sink=True,
                                 with_topk_length=True, d_qk=d_qk)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale, 512, w.attn_sink, w.topk_length)
    assert flashmla_b200.kernel_status(DEV) == 0
    toks = [0, 1, 65535, 65536, 69999]
    ro, _, rm, rl = attention.sparse_prefill_fwd(w.q[toks].cpu(), w.kv.cpu(), w.indices[toks].cpu(), w.sm_scale,
                                                 attn_sink=w.attn_sink.cpu(), topk_length=w.topk_length[toks].cpu())
    check_prefill(out[toks], mx[toks], lse[toks], ro, rm, rl)


# ---- decode (test_flash_mla_sparse_decoding.py:23-126) -----------------------------------------------------------
def _decode_workload(d_qk, b, s_q, h_q, s_k, topk, page, seed, varlen=True, zero_len=False, all_invalid=False, sink=True,
                     with_len=False):
    """Inputs like tests/lib.py:227-307: q ~ N(0,1) clamped to +-1, kv ~ N(0,1)/10, variable sequence lengths,
    a permuted block table, unused rows poisoned with NaN, sm_scale = d_qk^-0.55."""
    layout = wl.LAYOUT_MODEL1 if d_qk == 512 else wl.LAYOUT_V32
    w = wl.make_decode_workload(b, s_q, h_q, topk, max(s_k // 2, 1) if varlen else s_k, s_k, page=page, layout=layout, seed=seed,
                                q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=d_qk ** -0.55, with_sink=sink,
                                with_topk_length=with_len, poison_unused=not (zero_len or all_invalid))
    if all_invalid:
        w.indices[:] = -1
    if zero_len:                          # requests whose sequence is empty reference nothing
        w.indices[::3] = -1
    return w


def _run_decode(w, x=None):
    args = [cu(w.q), cu_strided(w.kv_rows), None, None, 512, flash_mla.get_mla_metadata()[0], None, w.sm_scale, False, True,
            cu(w.indices), cu(w.attn_sink)]
    if x is not None:
        args += [cu_strided(x.kv_rows), cu(x.indices), cu(w.topk_length), cu(x.topk_length)]
    else:
        args += [None, None, cu(w.topk_length), None]
    out, lse = flash_mla.flash_mla_with_kvcache(*args, kvcache_layout=w.layout)
    assert flashmla_b200.kernel_status(DEV) == 0
    kw = {}
    if x is not None:
        kw = dict(extra_kv_dequant=quant.dequantize_rows(x.kv_rows.contiguous(), x.layout), extra_indices=x.indices,
                  extra_topk_length=x.topk_length)
    ref_out, ref_lse, _ = attention.sparse_decode(w.q, quant.dequantize_rows(w.kv_rows.contiguous(), w.layout), w.indices, w.sm_scale,
                                                  attn_sink=w.attn_sink, topk_length=w.topk_length, **kw)
    check_decode(out, lse, ref_out, ref_lse)


DECODE_SHAPES = [(512, 64, 2), (512, 64, 64), (512, 64, 69), (1024, 576, 2), (1024, 576, 61), (2046, 2048, 2), (2046, 2048, 64),
                 (2046, 2048, 576)]
# every (d_qk, h_q, shape, s_q) with b = 4; the larger batches with the shorter top-k lists
DECODE_CASES = [(d, h, sk, tk, pg, b, sq) for d in (576, 512) for h in (64, 128) for (sk, tk, pg) in DECODE_SHAPES
                for b in (4, 74, 321) for sq in (1, 3) if b == 4 or (b == 74 and tk <= 576 and sq == 1) or (b == 321 and tk == 64 and sq == 1)]


@pytest.mark.parametrize("d_qk,h_q,s_k,topk,page,b,s_q", DECODE_CASES,
                         ids=[f"d{c[0]}h{c[1]}sk{c[2]}k{c[3]}p{c[4]}b{c[5]}sq{c[6]}" for c in DECODE_CASES])
def test_decode_correctness_cases(d_qk, h_q, s_k, topk, page, b, s_q):
    _run_decode(_decode_workload(d_qk, b, s_q, h_q, s_k, topk, page, seed=b + topk + page, with_len=(d_qk == 512 and page % 2 == 0)))


CORNER = [(d, h, sk, tk, pg, b, inv, zl, sink) for d in (576, 512) for h in (64, 128) for (sk, tk, pg) in ((512, 64, 61), (650, 576, 53))
          for b in (4, 74) for inv in (True, False) for zl in (True, False) for sink in (True, False) if (inv or zl or sink)]
CORNER = CORNER[::2]


@pytest.mark.parametrize("d_qk,h_q,s_k,topk,page,b,all_invalid,zero_len,sink", CORNER,
                         ids=[f"d{c[0]}h{c[1]}k{c[3]}b{c[5]}{'I' if c[6] else ''}{'Z' if c[7] else ''}{'S' if c[8] else ''}" for c in CORNER])
def test_decode_corner_cases(d_qk, h_q, s_k, topk, page, b, all_invalid, zero_len, sink):
    _run_decode(_decode_workload(d_qk, b, 3, h_q, s_k, topk, page, seed=b + page, zero_len=zero_len, all_invalid=all_invalid, sink=sink))


EXTRA = [(h, sk, tk, pg, xsk, xtk, xpg, xl) for h in (64, 128)
         for (sk, tk, pg), (xsk, xtk, xpg) in itertools.product(((512, 64, 64), (1024, 576, 61), (2046, 2048, 2)),
                                                                 ((512, 64, 69), (1024, 576, 2), (2046, 2048, 64)))
         for xl in (False, True)][::2]


@pytest.mark.parametrize("h_q,s_k,topk,page,xs_k,xtopk,xpage,xlen", EXTRA,
                         ids=[f"h{c[0]}k{c[2]}p{c[3]}x{c[5]}p{c[6]}{'L' if c[7] else ''}" for c in EXTRA])
def test_decode_model1_with_an_extra_cache(h_q, s_k, topk, page, xs_k, xtopk, xpage, xlen):
    """d_qk = 512 is where the reference exercises extra_k_cache and the two topk_length arguments."""
    w = _decode_workload(512, 4, 3, h_q, s_k, topk, page, seed=topk + xtopk, with_len=xlen)
    x = _decode_workload(512, 4, 3, h_q, xs_k, xtopk, xpage, seed=topk + xtopk + 1, sink=False, with_len=xlen)
    if not xlen:
        w.topk_length = x.topk_length = None
    _run_decode(w, x)


@pytest.mark.parametrize("case", [EXTRA[0], EXTRA[7], EXTRA[-1]], ids=["first", "eighth", "last"])
def test_decode_model1_with_an_extra_cache_runs_on_the_tensor_core_kernel(case, monkeypatch):
    """Forced, so that a fall-back to the CUDA-core kernel would show as an error: the reference's MODEL1 configurations
    all come with an extra cache (test_flash_mla_sparse_decoding.py:105-112)."""
    monkeypatch.setenv("FMLA_KERNEL", "tc")
    test_decode_model1_with_an_extra_cache(*case)


def test_decode_model1_production_shape_with_an_extra_cache(monkeypatch):
    """h_q = 128, s_q = 2, topk = 128 over pages of 256 tokens + 1024 extra slots over pages of 64 with their own lengths
    (MODEL1 CONFIG2 / CONFIG4 of test_flash_mla_sparse_decoding.py:107-112), b = 74."""
    monkeypatch.setenv("FMLA_KERNEL", "tc")
    w = _decode_workload(512, 74, 2, 128, 4096, 128, 256, seed=21, with_len=True)
    x = _decode_workload(512, 74, 2, 128, 4096, 1024, 64, seed=22, sink=False, with_len=True)
    _run_decode(w, x)


@pytest.mark.parametrize("d_qk,h_q", [(576, 128), (576, 64)])
def test_decode_peak_shape_runs(d_qk, h_q):
    """b = 148, s_q = 2, topk = 16384 over 32768-token sequences (test_flash_mla_sparse_decoding.py:120-124): sampled
    requests against the oracle."""
    w = wl.make_decode_workload(148, 2, h_q, 16384, 32768, 32768, seed=9, device=DEV, q_std=1.0, kv_std=0.1, clamp=1.0,
                                sm_scale=d_qk ** -0.55, keep_bf16=False)
    out, lse = flash_mla.flash_mla_with_kvcache(w.q, w.kv_rows, None, None, 512, flash_mla.get_mla_metadata()[0], None, w.sm_scale,
                                                False, True, w.indices)
    assert flashmla_b200.kernel_status(DEV) == 0
    from test_gpu_full_size import oracle_decode_requests
    reqs = [0, 147]
    ref_out, ref_lse = oracle_decode_requests(w, w.q, w.indices, reqs)
    check_decode(out[reqs], lse[reqs].contiguous(), ref_out, ref_lse)
