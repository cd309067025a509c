"""Pins the CPU oracle to the reference: every fixture under tests/golden was produced by the
reference's own tests/quant.py and tests/ref.py (see tests/golden/make_golden.py)."""
import numpy as np
import pytest
import torch

from oracle import attention, quant
from oracle.compare import assert_close
from flashmla_b200 import workloads as wl
from helpers import bf16, load_golden, t


def test_v32_rows_byte_exact():
    g = load_golden("quant_v32")
    kv = bf16(g["kv"])
    rows = quant.quantize_rows(kv, quant.LAYOUT_V32)
    assert np.array_equal(rows.numpy(), g["rows"])
    # the workload synthesiser is an independent implementation of the same format
    assert np.array_equal(wl.quantize_kv_rows(kv, wl.LAYOUT_V32).numpy(), g["rows"])
    assert np.array_equal(wl.quantize_kv_rows(kv, wl.LAYOUT_V32, row_pad=1).numpy(), g["rows"])


def test_v32_dequant_bit_exact():
    g = load_golden("quant_v32")
    deq = quant.dequantize_rows(t(g["rows"]), quant.LAYOUT_V32)
    assert np.array_equal(deq.view(torch.int16).numpy().view(np.uint16), g["dequant"])


def test_model1_rows_byte_exact_and_dequant_bit_exact():
    """The reference's d_qk = 512 cache format (tests/quant.py:55-75, :106-118)."""
    g = load_golden("quant_model1")
    kv = bf16(g["kv"])
    rows = quant.quantize_rows(kv, quant.LAYOUT_MODEL1)
    assert rows.shape == (5, 16, 1, 584) and rows.stride(0) % 576 == 0
    assert np.array_equal(rows.numpy(), g["rows"])
    assert np.array_equal(wl.quantize_kv_rows(kv, wl.LAYOUT_MODEL1).numpy(), g["rows"])
    deq = quant.dequantize_rows(t(g["rows"]), quant.LAYOUT_MODEL1)
    assert np.array_equal(deq.view(torch.int16).numpy().view(np.uint16), g["dequant"])


@pytest.mark.parametrize("name", ["decode_model1", "decode_model1_h128"])
def test_model1_decode_matches_reference(name):
    g = load_golden(name)
    deq = quant.dequantize_rows(t(g["kv_rows"]), quant.LAYOUT_MODEL1)
    sink = t(g["attn_sink"]) if "attn_sink" in g else None
    tl = t(g["topk_length"]) if "topk_length" in g else None
    out, lse, _ = attention.sparse_decode(bf16(g["q"]), deq, t(g["indices"]), float(g["sm_scale"]), attn_sink=sink, topk_length=tl)
    assert_close("out", out.float(), bf16(g["out"]).float(), abs_tol=1e-6, rel_tol=2.0 ** -7, cos_tol=1e-6)
    assert_close("lse", lse.contiguous(), t(g["lse"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-9)


def test_index_map_bit_exact():
    g = load_golden("quant_v32")
    got = quant.abs_to_cache_indices(t(g["positions"]), t(g["block_table"]), int(g["page"]))
    assert np.array_equal(got.numpy(), g["cache_rows"])
    got2 = wl.positions_to_cache_rows(t(g["positions"]), t(g["block_table"]), int(g["page"]))
    assert np.array_equal(got2.numpy(), g["cache_rows"])


@pytest.mark.parametrize("name", ["decode_c1", "decode_sink_len", "decode_h128"])
def test_decode_matches_reference(name):
    g = load_golden(name)
    rows = t(g["kv_rows"])
    deq = quant.dequantize_rows(rows, quant.LAYOUT_V32)
    sink = t(g["attn_sink"]) if "attn_sink" in g else None
    tl = t(g["topk_length"]) if "topk_length" in g else None
    out, lse, _ = attention.sparse_decode(bf16(g["q"]), deq, t(g["indices"]), float(g["sm_scale"]),
                                          attn_sink=sink, topk_length=tl)
    assert_close("out", out.float(), bf16(g["out"]).float(), abs_tol=1e-6, rel_tol=2.0 ** -7, cos_tol=1e-6)
    assert_close("lse", lse.contiguous(), t(g["lse"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-9)


def test_decode_with_extra_cache_matches_reference():
    g = load_golden("decode_extra")
    deq = quant.dequantize_rows(t(g["kv_rows"]), quant.LAYOUT_V32)
    deq2 = quant.dequantize_rows(t(g["extra_kv_rows"]), quant.LAYOUT_V32)
    out, lse, _ = attention.sparse_decode(bf16(g["q"]), deq, t(g["indices"]), float(g["sm_scale"]), attn_sink=t(g["attn_sink"]),
                                          topk_length=t(g["topk_length"]), extra_kv_dequant=deq2,
                                          extra_indices=t(g["extra_indices"]), extra_topk_length=t(g["extra_topk_length"]))
    assert_close("out", out.float(), bf16(g["out"]).float(), abs_tol=1e-6, rel_tol=2.0 ** -7, cos_tol=1e-6)
    assert_close("lse", lse.contiguous(), t(g["lse"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-9)


@pytest.mark.parametrize("name", ["prefill_small", "prefill_sink_len", "prefill_causal", "prefill_h128", "prefill_d512_h128"])
def test_prefill_matches_reference(name):
    g = load_golden(name)
    sink = t(g["attn_sink"]) if "attn_sink" in g else None
    tl = t(g["topk_length"]) if "topk_length" in g else None
    out, out_f, mx, lse = attention.sparse_prefill_fwd(bf16(g["q"]), bf16(g["kv"]), t(g["indices"]),
                                                       float(g["sm_scale"]), attn_sink=sink, topk_length=tl)
    assert_close("out_f32", out_f, t(g["out_f32"]), abs_tol=1e-5, rel_tol=1e-4, cos_tol=1e-9)
    assert_close("out", out.float(), bf16(g["out"]).float(), abs_tol=1e-6, rel_tol=2.0 ** -7, cos_tol=1e-6)
    assert_close("max_logits", mx, t(g["max_logits"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-9)
    assert_close("lse", lse, t(g["lse"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-9)


def test_mxfp8_roundtrip_and_layout():
    gen = torch.Generator().manual_seed(5)
    kv = torch.randn((3, 8, 1, 576), generator=gen).to(torch.bfloat16)
    rows = quant.quantize_rows(kv, quant.LAYOUT_MXFP8)
    assert rows.shape == (3, 8, 1, 656)
    assert np.array_equal(rows.numpy(), wl.quantize_kv_rows(kv, wl.LAYOUT_MXFP8).numpy())
    deq = quant.dequantize_rows(rows, quant.LAYOUT_MXFP8)
    # RoPE part is stored verbatim
    assert torch.equal(deq[..., 512:], kv[..., 512:])
    # e4m3 has 3 mantissa bits: per-32 scaled rounding error is at most 2^-4 of the tile maximum
    err = (deq[..., :512].float() - kv[..., :512].float()).abs().view(3, 8, 16, 32)
    amax = kv[..., :512].float().abs().view(3, 8, 16, 32).amax(-1, keepdim=True)
    assert bool((err <= amax / 16 + 1e-6).all())
    # dequantised values are representable: quantising them again reproduces the same values
    again = quant.dequantize_rows(quant.quantize_rows(deq, quant.LAYOUT_MXFP8), quant.LAYOUT_MXFP8)
    assert torch.equal(again, deq)
    # scale bytes: 2^(byte-127) is the smallest power of two >= amax/448
    sc = torch.pow(2.0, rows.view(3, 8, 656)[..., 512:528].float() - 127)
    need = (amax.squeeze(-1) / 448).clamp_min(1e-4)
    assert bool((sc >= need).all()) and bool((sc / 2 < need).all())


def test_backward_matches_autograd_and_finite_differences():
    w = wl.make_prefill_workload(5, 48, 3, 16, seed=9, std=0.5, with_sink=True, with_topk_length=True,
                                 invalid_pads=(-1, 48, 2147483647))
    w.indices[1, 0, 3] = w.indices[1, 0, 2]      # duplicate index: gradients must add up
    q = w.q.double().requires_grad_(True)
    kv = w.kv.double().requires_grad_(True)
    s_kv = kv.shape[0]
    idx = w.indices[:, 0].long().clone()
    topk = idx.shape[-1]
    idx[torch.arange(topk).unsqueeze(0) >= w.topk_length.unsqueeze(1)] = -1
    invalid = (idx < 0) | (idx >= s_kv)
    g = kv.view(s_kv, 576)[idx.masked_fill(invalid, 0)]
    s = torch.einsum("qhd,qtd->qht", q, g) * w.sm_scale
    s = s.masked_fill(invalid.unsqueeze(1), float("-inf"))
    denom = torch.exp(s).sum(-1) + torch.exp(w.attn_sink.double()).view(1, -1)
    p = torch.exp(s) / denom.unsqueeze(-1)
    p = torch.where(denom.unsqueeze(-1) > 0, p, torch.zeros_like(p))
    out = torch.einsum("qht,qtd->qhd", p, g[..., :512])
    out.backward(w.dout.double())
    dq, dkv = attention.sparse_prefill_bwd(w.q, w.kv, w.dout, w.indices, w.sm_scale, attn_sink=w.attn_sink,
                                           topk_length=w.topk_length, dtype=torch.float64)
    fin = torch.isfinite(q.grad)
    assert_close("dq", dq[fin].float(), q.grad[fin].float(), abs_tol=1e-6, rel_tol=1e-5, cos_tol=1e-10)
    assert_close("dkv", dkv.float(), kv.grad.float(), abs_tol=1e-6, rel_tol=1e-5, cos_tol=1e-10)
    # forward of the same oracle agrees with the graph used for autograd
    o_ref = attention.sparse_prefill_fwd(w.q, w.kv, w.indices, w.sm_scale, attn_sink=w.attn_sink,
                                         topk_length=w.topk_length, dtype=torch.float64)[1]
    assert_close("out", o_ref.float(), out.detach().float(), abs_tol=1e-6, rel_tol=1e-5, cos_tol=1e-10)
    # central finite difference on a handful of coordinates of kv
    eps = 1e-4
    for (r, c) in [(int(w.indices[0, 0, 0]), 5), (int(w.indices[1, 0, 2]), 530), (int(w.indices[3, 0, 1]), 100)]:
        if r < 0 or r >= s_kv:
            continue
        def f(delta):
            kv2 = w.kv.double().clone()
            kv2[r, 0, c] += delta
            o = attention.sparse_prefill_fwd(w.q, kv2, w.indices, w.sm_scale, attn_sink=w.attn_sink,
                                             topk_length=w.topk_length, dtype=torch.float64)[1]
            return float((o * w.dout.double()).sum())
        fd = (f(eps) - f(-eps)) / (2 * eps)
        assert abs(fd - float(dkv[r, 0, c])) < 1e-5 * max(1.0, abs(fd)), (r, c, fd, float(dkv[r, 0, c]))


@pytest.mark.parametrize("name", ["dense_decode", "dense_decode_h128"])
def test_dense_decode_oracle_matches_the_reference(name):
    """Dense MLA decode (bf16 paged cache, block table, causal among the s_q rows): the oracle against the torch
    reference inside the reference's own test file (tests/test_flash_mla_dense_decoding.py:73-141)."""
    g = load_golden(name)
    out, lse = attention.dense_decode(bf16(g["q"]), bf16(g["blocked_k"]), t(g["block_table"]), t(g["cache_seqlens"]), 512,
                                      bool(g["causal"]))
    assert_close("out", out.float(), bf16(g["out"]).float(), abs_tol=2e-3, rel_tol=8e-3, cos_tol=1e-5)      # both are rounded to bf16
    assert_close("lse", lse, t(g["lse"]), abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-6)


def test_dense_decode_is_sparse_decode_over_every_cached_token():
    """The product runs dense decode as a sparse prefill over index lists that enumerate the cache: the two oracles
    must agree on that construction."""
    g = load_golden("dense_decode")
    q, kc, bt, lens = bf16(g["q"]), bf16(g["blocked_k"]), t(g["block_table"]), t(g["cache_seqlens"])
    causal = bool(g["causal"])
    b, s_q, h_q, d = q.shape
    nb, page, h_kv, _ = kc.shape
    hg = h_q // h_kv
    ref_out, ref_lse = attention.dense_decode(q, kc, bt, lens, 512, causal)
    max_len = bt.shape[1] * page
    pos = torch.arange(max_len)
    rows = bt[:, pos // page].long() * page + pos % page
    flat = kc.reshape(nb * page * h_kv, 1, d)
    for i in range(b):
        for j in range(s_q):
            seen = max(int(lens[i]) - (s_q - 1 - j if causal else 0), 0)
            for k in range(h_kv):
                idx = torch.where(pos < seen, rows[i] * h_kv + k, torch.full_like(pos, -1)).to(torch.int32).view(1, 1, max_len)
                o, _, _, l = attention.sparse_prefill_fwd(q[i, j, k * hg:(k + 1) * hg].unsqueeze(0), flat, idx, d ** -0.5)
                assert_close("out", o[0].float(), ref_out[i, j, k * hg:(k + 1) * hg].float(), abs_tol=2e-3, rel_tol=8e-3, cos_tol=1e-5)
                assert_close("lse", l[0], ref_lse[i, k * hg:(k + 1) * hg, j], abs_tol=1e-5, rel_tol=1e-5, cos_tol=1e-6)
