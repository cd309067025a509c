"""The benchmark's full shapes on the GPU, checked against the CPU oracle on a sample of the requests /
query tokens (the oracle takes minutes on the whole batch), plus properties that need no oracle."""
import pytest
import torch

import flash_mla
import flashmla_b200
from flashmla_b200 import workloads as wl
from oracle import attention, quant
from gpu_utils import DEV, check_decode, check_prefill

pytestmark = pytest.mark.gpu


def oracle_decode_requests(w, q, indices, reqs):
    """Oracle on requests `reqs` only: gathers the rows they reference, dequantises those, renumbers."""
    outs, lses = [], []
    for r in reqs:
        idx = indices[r].cpu()                                   # [s_q, topk]
        rows = w.kv_rows.reshape(-1, 656)[idx.clamp_min(0).reshape(-1).long().to(w.kv_rows.device)].cpu()
        deq = quant.dequantize_rows(rows.view(-1, 1, 1, 656), w.layout)
        local = torch.arange(idx.numel(), dtype=torch.int32).view(1, *idx.shape).masked_fill(idx.unsqueeze(0) < 0, -1)
        o, l, _ = attention.sparse_decode(q[r:r + 1].cpu(), deq, local, w.sm_scale)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs), torch.cat(lses)


@pytest.mark.parametrize("layout,b,s_q,lo,hi", [(wl.LAYOUT_V32, 128, 2, 4096, 32768), (wl.LAYOUT_MXFP8, 256, 1, 8192, 8192)],
                         ids=["c2_v32", "c3_mxfp8_short_cache"])
def test_decode_full_batch_sampled_against_oracle(layout, b, s_q, lo, hi):
    """b, s_q, h_q, topk of the benchmark's decode configurations (the MXFP8 one with a shorter cache, which
    changes the pool size only: the kernel's work per request is set by topk)."""
    w = wl.make_decode_workload(b, s_q, 128, 2048, lo, hi, layout=layout, seed=17, device=DEV, invalid_frac=0.02,
                                keep_bf16=False)
    sched = flash_mla.get_mla_metadata()[0]
    out, lse = flash_mla.flash_mla_with_kvcache(w.q, w.kv_rows, None, None, 512, sched, None, w.sm_scale, False, True,
                                                w.indices, kvcache_layout=layout)
    assert flashmla_b200.kernel_status(DEV) == 0
    assert bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(lse).all())
    reqs = [0, 1, b // 2, b - 1]
    ref_out, ref_lse = oracle_decode_requests(w, w.q, w.indices, reqs)
    check_decode(out[reqs], lse[reqs].contiguous(), ref_out, ref_lse, strict=False)
    # every request is cut differently by the scheduler when decoded in another batch: same rows must come out
    half = slice(b // 2, b)
    out2, lse2 = flash_mla.flash_mla_with_kvcache(w.q[half], w.kv_rows, None, None, 512, flash_mla.get_mla_metadata()[0],
                                                  None, w.sm_scale, False, True, w.indices[half], kvcache_layout=layout)
    check_decode(out2, lse2.contiguous(), out[half].cpu(), lse[half].cpu().contiguous(), strict=False)


def test_mxfp8_decode_at_the_full_cache_size_sampled_against_oracle():
    """The MXFP8 benchmark configuration as stated: b = 256, s_q = 1, every cache sequence 65536 tokens long, i.e. a
    pool of 262144 pages (11 GB, row numbers up to 16.7 million).  The pool is written on the GPU by the cache writer
    (fmla_kv_quantize) chunk by chunk from bf16 N(0,1) data; sampled requests are checked against the oracle, which
    dequantises the very bytes the kernel reads."""
    b, s_k, page, topk, h_q = 256, 65536, 64, 2048, 128
    pages_per_seq = s_k // page
    n_pages = b * pages_per_seq
    gen = torch.Generator(device=DEV)
    gen.manual_seed(43)
    pool = torch.empty((n_pages, page, 1, 656), dtype=torch.uint8, device=DEV)
    chunk = 8192
    for lo in range(0, n_pages, chunk):
        kv = torch.randn((chunk, page, 1, 576), generator=gen, device=DEV).to(torch.bfloat16)
        flashmla_b200.quantize_k_cache(kv, wl.LAYOUT_MXFP8, out=pool[lo:lo + chunk])
    del kv
    block_table = torch.randperm(n_pages, generator=gen, device=DEV).to(torch.int32).view(b, pages_per_seq)
    positions = wl.distinct_positions(torch.full((b,), s_k, dtype=torch.int32, device=DEV), topk, gen).view(b, 1, topk)
    positions.masked_fill_(torch.rand(positions.shape, generator=gen, device=DEV) < 0.02, -1)
    indices = flashmla_b200.abs_indices2indices_in_kvcache(positions, block_table, page)
    assert int(indices.max()) > 2 ** 23, "the case is meant to reach high row numbers"
    q = torch.randn((b, 1, h_q, 576), generator=gen, device=DEV).to(torch.bfloat16)
    sm_scale = 576 ** -0.5
    out, lse = flash_mla.flash_mla_with_kvcache(q, pool, None, None, 512, flash_mla.get_mla_metadata()[0], None, sm_scale,
                                                False, True, indices, kvcache_layout=wl.LAYOUT_MXFP8)
    assert flashmla_b200.kernel_status(DEV) == 0
    assert bool(torch.isfinite(out.float()).all()) and bool(torch.isfinite(lse).all())
    w = wl.DecodeWorkload(q=q, kv_rows=pool, kv_bf16=None, block_table=block_table,
                          cache_seqlens=torch.full((b,), s_k, dtype=torch.int32), positions=positions, indices=indices,
                          sm_scale=sm_scale, layout=wl.LAYOUT_MXFP8)
    reqs = [0, 1, b // 2, b - 1]
    ref_out, ref_lse = oracle_decode_requests(w, q, indices, reqs)
    check_decode(out[reqs], lse[reqs].contiguous(), ref_out, ref_lse, strict=False)


def test_prefill_full_size_sampled_against_oracle():
    """s_q=4096, s_kv=32768, h_q=128, topk=2048, causal offset 28672: a sample of query tokens against the
    oracle, and the whole output against a second run over a permuted top-k list (softmax is order-free)."""
    w = wl.make_prefill_workload(4096, 32768, 128, 2048, seed=19, device=DEV, causal_offset=28672)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale)
    assert flashmla_b200.kernel_status(DEV) == 0
    toks = [0, 1, 2047, 4095]
    ro, _, rm, rl = attention.sparse_prefill_fwd(w.q[toks].cpu(), w.kv.cpu(), w.indices[toks].cpu(), w.sm_scale)
    check_prefill(out[toks], mx[toks], lse[toks], ro, rm, rl, strict=False)
    perm = torch.randperm(2048, device=DEV)
    out2, mx2, lse2 = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices[:, :, perm].contiguous(), w.sm_scale)
    assert torch.allclose(lse2, lse, rtol=1e-4, atol=1e-4) and torch.allclose(mx2, mx, rtol=1e-5, atol=1e-5)
    diff = (out2.float() - out.float()).abs().max().item()
    assert diff <= 1e-2 * out.float().abs().max().item(), f"permuted top-k list changed the output by {diff}"


def test_full_size_runs_are_bitwise_repeatable():
    """Races between the roles of the persistent kernel show up as rare differences between identical launches at
    full size (one query in a hundred thousand), so the same launch is repeated and compared bit for bit."""
    w = wl.make_prefill_workload(4096, 32768, 128, 2048, seed=23, device=DEV, causal_offset=28672)
    ref = [t.clone() for t in flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale)]
    for _ in range(25):
        got = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale)
        assert all(torch.equal(a, b) for a, b in zip(got, ref)), "two identical prefill launches differ"
    del w, ref, got
    wd = wl.make_decode_workload(128, 2, 128, 2048, 4096, 32768, seed=29, device=DEV, invalid_frac=0.02, keep_bf16=False)
    sched = flash_mla.get_mla_metadata()[0]

    def run():
        return flash_mla.flash_mla_with_kvcache(wd.q, wd.kv_rows, None, None, 512, sched, None, wd.sm_scale, False, True,
                                                wd.indices, kvcache_layout=wd.layout)
    ref = [t.clone() for t in run()]
    for _ in range(100):
        got = run()
        assert all(torch.equal(a, b) for a, b in zip(got, ref)), "two identical decode launches differ"
    assert flashmla_b200.kernel_status(DEV) == 0


def test_decode_and_prefill_replay_from_a_cuda_graph():
    """The calls allocate nothing and never synchronise inside the library, so a serving engine can capture them
    (after one eager call per shape, which sets kernel attributes and runs the tile scheduler) and replay."""
    wd = wl.make_decode_workload(9, 2, 128, 512, 600, 3000, seed=31, device=DEV, invalid_frac=0.03, with_sink=True)
    wp = wl.make_prefill_workload(80, 3000, 128, 384, seed=37, device=DEV)
    sched = flash_mla.get_mla_metadata()[0]

    def decode():
        return flash_mla.flash_mla_with_kvcache(wd.q, wd.kv_rows, None, None, 512, sched, None, wd.sm_scale, False, True,
                                                wd.indices, wd.attn_sink, kvcache_layout=wd.layout)

    def prefill():
        return flash_mla.flash_mla_sparse_fwd(wp.q, wp.kv, wp.indices, wp.sm_scale)
    eager = [t.clone() for t in (*decode(), *prefill())]
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side):
            captured = (*decode(), *prefill())
    for _ in range(3):
        for t in captured:
            t.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert all(torch.equal(a, b) for a, b in zip(captured, eager)), "graph replay differs from the eager call"
    assert flashmla_b200.kernel_status(DEV) == 0


def test_backward_full_size_sampled_against_oracle_and_cuda_core_kernels(monkeypatch):
    """The benchmark's backward shape (s_q=4096, s_kv=32768, h_q=128, topk=2048) on the tensor-core kernels, which
    take it in seven passes: dq is per query token, so a sample of tokens is checked against the oracle run on those
    tokens alone; dkv sums over all 4096 tokens and is checked against the CUDA-core kernels (fp32 P and dS), an
    independent implementation. Tolerance as in test_gpu_prefill_bwd_tc.py: P and dS are bf16 on the tensor cores."""
    from oracle.compare import assert_close

    def tol_for(ref):
        return dict(abs_tol=max(2e-3, 4e-3 * ref.abs().max().item()), rel_tol=2e-2, cos_tol=1e-4)
    w = wl.make_prefill_workload(4096, 32768, 128, 2048, seed=41, device=DEV, causal_offset=28672, std=0.5)
    out, _, lse = flash_mla.flash_mla_sparse_fwd(w.q, w.kv, w.indices, w.sm_scale)
    monkeypatch.setenv("FMLA_KERNEL", "tc")
    dq, dkv = flash_mla.flash_mla_sparse_bwd(w.q, w.kv, out, w.dout, w.indices, lse, w.sm_scale, return_fp32_dkv=True)
    assert flashmla_b200.kernel_status(DEV) == 0
    assert bool(torch.isfinite(dq.float()).all()) and bool(torch.isfinite(dkv).all())
    toks = [0, 1, 2047, 4095]
    ref_dq, _ = attention.sparse_prefill_bwd(w.q[toks].cpu(), w.kv.cpu(), w.dout[toks].cpu(), w.indices[toks].cpu(),
                                             w.sm_scale, out=out[toks].cpu())
    assert_close("dq", dq[toks].float().cpu(), ref_dq, **tol_for(ref_dq))
    monkeypatch.setenv("FMLA_KERNEL", "simt")
    dq2, dkv2 = flash_mla.flash_mla_sparse_bwd(w.q, w.kv, out, w.dout, w.indices, lse, w.sm_scale, return_fp32_dkv=True)
    assert_close("dkv", dkv.cpu(), dkv2.cpu(), **tol_for(dkv2.cpu()))
    assert_close("dq_all", dq.float().cpu(), dq2.float().cpu(), **tol_for(dq2.float().cpu()))
