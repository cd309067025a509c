"""Dense MLA decode (indices=None: bf16 paged cache, block_table, cache_seqlens, causal) through the reference's
flash_mla_with_kvcache signature (flash_mla_interface.py:161-170).  The reference has no sm_100 kernel for this branch
(csrc/api/dense_decode.h:27-29); its semantics are those of the torch reference in its own test file
(tests/test_flash_mla_dense_decoding.py:73-141), which made the fixtures."""
import random

import pytest
import torch

import flash_mla
import flashmla_b200
from oracle import attention
from oracle.compare import assert_close, assert_north_out, NORTH_LSE
from helpers import bf16, load_golden, t
from gpu_utils import DEV, cu

pytestmark = pytest.mark.gpu


def _run(q, blocked_k, block_table, cache_seqlens, causal, scale=None):
    out, lse = flash_mla.flash_mla_with_kvcache(cu(q), cu(blocked_k), cu(block_table), cu(cache_seqlens), 512,
                                                flash_mla.get_mla_metadata()[0], None, scale, causal)
    assert flashmla_b200.kernel_status(DEV) == 0
    return out.float().cpu(), lse.float().cpu()


@pytest.mark.parametrize("name", ["dense_decode", "dense_decode_h128"])
def test_golden_reference_outputs(name):
    g = load_golden(name)
    out, lse = _run(bf16(g["q"]), bf16(g["blocked_k"]), t(g["block_table"]), t(g["cache_seqlens"]), bool(g["causal"]))
    assert tuple(lse.shape) == (g["q"].shape[0], g["q"].shape[2], g["q"].shape[1])
    assert_north_out("out", out, bf16(g["out"]).float())
    assert_close("lse", lse, t(g["lse"]), **NORTH_LSE)


# b, s_q, h_q, h_kv, mean s_k, varlen, causal, zero-length requests  (the reference's matrix: b {1,2,6,64} x s_q {1,2,4} x
# s_k {20,140,4096} x h_q x h_kv {1,2,3,8} x varlen x causal, and its corner case with empty caches)
CASES = [
    (1, 1, 128, 1, 20, False, False, False),
    (2, 2, 128, 1, 140, True, True, False),
    (6, 4, 64, 1, 4096, True, True, False),
    (6, 1, 128, 2, 140, True, False, False),
    (3, 2, 9, 3, 140, False, True, False),
    (2, 4, 126, 2, 300, True, True, False),
    (64, 2, 128, 1, 500, True, True, True),
    (5, 2, 16, 8, 1000, True, False, True),
    (1, 2, 256, 1, 20000, False, True, False),      # one request split over every partition, two head groups
    (3, 1, 192, 1, 700, True, False, False),        # a last head group of 64
    (2, 4, 64, 1, 3, False, True, False),           # fewer tokens than query rows see
]


def _case_id(c):
    return f"b{c[0]}sq{c[1]}h{c[2]}hk{c[3]}sk{c[4]}{'v' if c[5] else ''}{'c' if c[6] else ''}{'z' if c[7] else ''}"


# every 47th case of the reference's own correctness matrix and every 7th of its corner cases (caches of length zero),
# tests/test_flash_mla_dense_decoding.py:203-222
_MATRIX = [(b, s_q, h_q, h_kv, s_k, varlen, causal, False)
           for b in [1, 2, 6, 64] for s_q in [1, 2, 4] for s_k in [20, 140, 4096] for h_q in [1, 3, 9, 63, 64, 126, 128]
           for h_kv in [1, 2, 3, 8] for varlen in [False, True] for causal in [False, True] if h_q % h_kv == 0]
_CORNER = [(128, 2, h_q, h_kv, 4096, True, causal, True) for h_q in [1, 3, 9, 63, 64, 126, 128] for h_kv in [1, 2, 3, 8]
           for causal in [False, True] if h_q % h_kv == 0]
REF_CASES = _MATRIX[::47] + _CORNER[::7]


@pytest.mark.parametrize("case", REF_CASES, ids=[_case_id(c) for c in REF_CASES])
def test_the_reference_s_case_matrix_sampled(case):
    _check_case(case)


@pytest.mark.parametrize("case", CASES, ids=[_case_id(c) for c in CASES])
def test_against_oracle(case):
    _check_case(case)


def _check_case(case):
    b, s_q, h_q, h_kv, s_k, varlen, causal, zeros = case
    rng = random.Random(b * 1000 + s_k)
    g = torch.Generator().manual_seed(b * 31 + s_k)
    page, d = 64, 576
    lens = [max(int(rng.normalvariate(s_k, s_k / 2)), s_q) if varlen else s_k for _ in range(b)]
    if zeros:
        for i in rng.sample(range(b), max(1, b // 4)):
            lens[i] = 0
    lens = torch.tensor(lens, dtype=torch.int32)
    max_blocks = (int(lens.max()) + page - 1) // page + 1
    block_table = torch.randperm(b * max_blocks, generator=g).to(torch.int32).view(b, max_blocks)
    q = torch.randn((b, s_q, h_q, d), generator=g).to(torch.bfloat16)
    blocked_k = (torch.randn((b * max_blocks, page, h_kv, d), generator=g) / 10).to(torch.bfloat16)
    # what lies beyond a request's length must not be read: poison it like the reference's generator does
    flat = blocked_k.view(-1, page, h_kv, d)
    for i in range(b):
        n = int(lens[i])
        for j, blk in enumerate(block_table[i].tolist()):
            lo = max(n - j * page, 0)
            if lo < page:
                flat[blk, lo:] = float("nan")
    out, lse = _run(q, blocked_k, block_table, lens, causal)
    ref_out, ref_lse = attention.dense_decode(q, torch.nan_to_num(blocked_k, nan=0.0), block_table, lens, 512, causal)
    assert_north_out("out", out, ref_out.float())
    assert_close("lse", lse, ref_lse, **NORTH_LSE)


def _random_case(b, s_q, h_q, s_k, seed, spare_blocks=3, page=64):
    g = torch.Generator().manual_seed(seed)
    d = 576
    lens = torch.randint(max(s_k // 3, s_q), s_k + 1, (b,), generator=g).to(torch.int32)
    max_blocks = (s_k + page - 1) // page + spare_blocks
    block_table = torch.randperm(b * max_blocks, generator=g).to(torch.int32).view(b, max_blocks)
    q = torch.randn((b, s_q, h_q, d), generator=g).to(torch.bfloat16)
    blocked_k = (torch.randn((b * max_blocks, page, 1, d), generator=g) / 10).to(torch.bfloat16)
    return q, blocked_k, block_table, lens


@pytest.mark.parametrize("causal", [False, True])
def test_split_kv_kernel_agrees_with_the_composition_over_index_lists(causal, monkeypatch):
    # one KV head and h_q % 64 == 0 run split-KV on the decode kernel (fmla_dense_decode); FMLA_KERNEL=simt takes the
    # other route, a sparse prefill over enumerated rows, on the CUDA-core kernel: two independent paths to one result
    q, blocked_k, block_table, lens = _random_case(9, 3, 128, 1500, seed=5)
    out, lse = _run(q, blocked_k, block_table, lens, causal)
    monkeypatch.setenv("FMLA_KERNEL", "simt")
    out2, lse2 = _run(q, blocked_k, block_table, lens, causal)
    assert_north_out("out", out, out2)
    assert_close("lse", lse, lse2, **NORTH_LSE)


@pytest.mark.parametrize("page", [16, 48, 200])
def test_split_kv_kernel_with_other_page_sizes(page):
    # the reference's dense decode takes pages of 64 tokens only (csrc/api/dense_decode.h:67); the block-table walk here
    # takes any size, also sizes that neither divide nor are multiples of the kernel's 64-token blocks
    q, blocked_k, block_table, lens = _random_case(5, 2, 128, 900, seed=page, page=page)
    block_table[1, 2] = -1                      # a hole and an entry beyond the cache: their tokens count as invalid slots
    block_table[3, 0] = blocked_k.shape[0] + 5
    out, lse = _run(q, blocked_k, block_table, lens, True)
    holes = block_table.clone()
    holes[3, 0] = -1
    ref_out, ref_lse = _dense_oracle_with_holes(q, blocked_k, holes, lens, True)
    assert_north_out("out", out, ref_out.float())
    assert_close("lse", lse, ref_lse, **NORTH_LSE)


def _dense_oracle_with_holes(q, blocked_k, block_table, lens, causal):
    """attention.dense_decode with the tokens of negative block-table entries left out: as sparse decode over the
    enumerated rows, which is what the kernel's invalid slots mean."""
    b, s_q, h_q, d = q.shape
    page = blocked_k.shape[1]
    max_len = block_table.shape[1] * page
    pos = torch.arange(max_len)
    blk = block_table[:, pos // page]
    rows = torch.where(blk >= 0, blk * page + (pos % page), torch.full_like(blk, -1))       # [b, max_len]
    idx = rows.view(b, 1, max_len).expand(b, s_q, max_len).clone()
    seen = lens.view(b, 1) - ((s_q - 1 - torch.arange(s_q)).view(1, s_q) if causal else 0)
    idx[pos.view(1, 1, max_len) >= seen.view(b, s_q, 1)] = -1
    out, lse, _ = attention.sparse_decode(q, blocked_k, idx.to(torch.int32), d ** -0.5)
    return out, lse


def test_split_kv_kernel_with_strided_tensors_and_a_reused_schedule():
    # q a slice of a wider tensor, the block table a slice of a wider table, cache rows at a pitch of 640 values; the
    # second call reuses the first call's schedule and accumulators
    q, blocked_k, block_table, lens = _random_case(4, 2, 64, 700, seed=9)
    wide_q = torch.zeros((4, 2, 64, 640), dtype=torch.bfloat16)
    wide_q[..., :576] = q
    wide_k = torch.full((blocked_k.shape[0], 64, 1, 640), float("nan"), dtype=torch.bfloat16)
    wide_k[..., :576] = blocked_k
    wide_bt = torch.full((4, block_table.shape[1] + 5), -7, dtype=torch.int32)
    wide_bt[:, :block_table.shape[1]] = block_table
    meta = flash_mla.get_mla_metadata()[0]
    ref_out, ref_lse = attention.dense_decode(q, blocked_k, block_table, lens, 512, True)
    dq, dk, dbt, dl = cu(wide_q)[..., :576], cu(wide_k)[..., :576], cu(wide_bt)[:, :block_table.shape[1]], cu(lens)
    for _ in range(2):
        out, lse = flash_mla.flash_mla_with_kvcache(dq, dk, dbt, dl, 512, meta, None, None, True)
        assert flashmla_b200.kernel_status(DEV) == 0
        assert_north_out("out", out.float().cpu(), ref_out.float())
        assert_close("lse", lse.float().cpu(), ref_lse, **NORTH_LSE)
    assert meta.tile_scheduler_metadata is not None and meta.o_accum is not None


def test_split_kv_kernel_with_plain_q_loads_and_plain_stores():
    # the paths the kernel takes when the driver refuses q's or out's strides for a tensor map, forced through
    # fmla_set_option: the same bits as with TMA tiles, for split and unsplit requests
    from flashmla_b200 import _lib
    lib = _lib.load()
    q, blocked_k, block_table, lens = _random_case(40, 2, 128, 600, seed=13)
    out0, lse0 = _run(q, blocked_k, block_table, lens, True)
    try:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_Q_LOADS, 1))
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_STORES, 1))
        out1, lse1 = _run(q, blocked_k, block_table, lens, True)
    finally:
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_Q_LOADS, 0))
        _lib.check(lib.fmla_set_option(_lib.OPTION_PLAIN_STORES, 0))
    assert torch.equal(out0, out1) and torch.equal(lse0, lse1)


def test_the_reference_s_argument_checks():
    q = torch.zeros((2, 1, 128, 576), dtype=torch.bfloat16, device=DEV)
    kc = torch.zeros((4, 64, 1, 576), dtype=torch.bfloat16, device=DEV)
    bt = torch.zeros((2, 2), dtype=torch.int32, device=DEV)
    lens = torch.ones((2,), dtype=torch.int32, device=DEV)
    with pytest.raises(AssertionError, match="block_table and cache_seqlens must be provided"):
        flash_mla.flash_mla_with_kvcache(q, kc, None, lens, 512, flash_mla.get_mla_metadata()[0])
    with pytest.raises(AssertionError, match="must be None when dense attention is used"):
        flash_mla.flash_mla_with_kvcache(q, kc, bt, lens, 512, flash_mla.get_mla_metadata()[0], attn_sink=torch.zeros(128, device=DEV))
    with pytest.raises(NotImplementedError):
        flash_mla.flash_mla_with_kvcache(q, kc, bt, lens, 512, flash_mla.get_mla_metadata()[0], is_fp8_kvcache=True)
