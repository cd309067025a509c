"""GPU parity of sparse prefill forward and backward against the reference's golden outputs and the
CPU oracle, through the public Python API -> C ABI -> CUDA kernels."""
import pytest
import torch

import flash_mla
from flashmla_b200 import workloads as wl
from oracle import attention
from oracle.compare import assert_close
from helpers import bf16, load_golden, t
from gpu_utils import DEV, cu, noncontig, run_prefill, check_prefill

pytestmark = pytest.mark.gpu

PADS = (-2147483648, -123456, -1, 114514, 1919810, 2147480000, 2147483647)


@pytest.mark.parametrize("name", ["prefill_small", "prefill_sink_len", "prefill_causal", "prefill_h128", "prefill_d512_h128"])
def test_golden_reference_outputs(name):
    g = load_golden(name)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(
        cu(bf16(g["q"])), cu(bf16(g["kv"])), cu(t(g["indices"])), float(g["sm_scale"]), 512,
        cu(t(g["attn_sink"])) if "attn_sink" in g else None, cu(t(g["topk_length"])) if "topk_length" in g else None)
    torch.cuda.synchronize()
    check_prefill(out, mx, lse, bf16(g["out"]), t(g["max_logits"]), t(g["lse"]))


# REFD follows the reference's prefill fixtures (tests/lib.py:121-164: q, kv ~ N(0,1)/10, sm_scale 0.5) and is
# held to the reference's own tolerances; the other cases use the benchmark's N(0,1) data and the acceptance gate.
REFD = dict(std=0.1, sm_scale=0.5)
CASES = [
    # s_q, s_kv, h_q, topk, kwargs
    (1, 128, 128, 128, dict(**REFD)),
    (62, 1000, 128, 256, dict(invalid_pads=PADS, **REFD)),
    (13, 300, 64, 512, dict(with_sink=True, invalid_pads=PADS, **REFD)),       # topk > s_kv: padded with invalid values
    (21, 32, 128, 2048, dict(with_topk_length=True, invalid_pads=PADS, **REFD)),
    (9, 592, 16, 128, dict(with_sink=True, with_topk_length=True, invalid_pads=PADS, **REFD)),
    (213, 1840, 128, 384, dict(with_sink=True, with_topk_length=True, invalid_pads=PADS, **REFD)),
    (5, 777, 256, 200, dict(invalid_pads=PADS, **REFD)),                        # topk not a multiple of 64, two head groups
    (8, 4096, 128, 2048, dict(causal_offset=3000)),                            # benchmark distribution
]


@pytest.mark.parametrize("d_qk", [576, 512])
@pytest.mark.parametrize("case", CASES, ids=[f"sq{c[0]}kv{c[1]}h{c[2]}k{c[3]}" for c in CASES])
def test_forward_against_oracle(case, d_qk):
    """d_qk = 512 is the reference's other head dimension (csrc/api/sparse_fwd.h:213-240): q and kv rows of 512 values,
    all of them V."""
    s_q, s_kv, h_q, topk, kw = case
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=s_q + topk, d_qk=d_qk, **kw)
    out, mx, lse = run_prefill(w, q=noncontig(w.q), kv=noncontig(w.kv), indices=noncontig(w.indices))
    ref_out, _, ref_mx, ref_lse = attention.sparse_prefill_fwd(w.q, w.kv, w.indices, w.sm_scale, attn_sink=w.attn_sink,
                                                               topk_length=w.topk_length)
    check_prefill(out, mx, lse, ref_out, ref_mx, ref_lse, strict="std" in kw)


@pytest.mark.parametrize("h_q", [64, 128])
def test_rows_without_valid_index(h_q):
    w = wl.make_prefill_workload(6, 100, h_q, 128, seed=2, with_sink=True, **REFD)
    w.indices[1] = 2147483647
    w.indices[4] = -5
    out, mx, lse = run_prefill(w)
    assert torch.all(out[1] == 0) and torch.all(lse[1] == float("inf")) and torch.all(mx[1] == float("-inf"))
    ref_out, _, ref_mx, ref_lse = attention.sparse_prefill_fwd(w.q, w.kv, w.indices, w.sm_scale, attn_sink=w.attn_sink)
    check_prefill(out, mx, lse, ref_out, ref_mx, ref_lse)


def test_forward_is_bitwise_deterministic():
    w = wl.make_prefill_workload(16, 512, 128, 256, seed=8)
    a = run_prefill(w)
    b = run_prefill(w)
    assert all(torch.equal(x, y) for x, y in zip(a, b))


BWD_CASES = [
    (5, 64, 16, 64, dict(std=0.5, sm_scale=0.5)),
    (12, 200, 128, 128, dict(std=0.5, with_sink=True, with_topk_length=True, invalid_pads=PADS)),
    (7, 48, 64, 256, dict(std=1.0, invalid_pads=PADS)),
]


@pytest.mark.parametrize("case", BWD_CASES, ids=[f"sq{c[0]}kv{c[1]}h{c[2]}k{c[3]}" for c in BWD_CASES])
def test_backward_against_oracle(case, monkeypatch):
    """The CUDA-core backward (fp32 P and dS). Tolerance: dq/dkv within 2e-2 relative or 2e-3 absolute per element
    and cosine difference <= 1e-4 of the fp32 oracle (the reference has no sparse backward; parity is unpinned).
    The tensor-core backward has its own file (test_gpu_prefill_bwd_tc.py)."""
    s_q, s_kv, h_q, topk, kw = case
    monkeypatch.setenv("FMLA_KERNEL", "simt")
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=topk + h_q, **kw)
    w.indices[0, 0, 1] = w.indices[0, 0, 0]          # duplicate index inside one query
    q, kv, idx, dout = cu(w.q), cu(w.kv), cu(w.indices), cu(w.dout)
    out, mx, lse = flash_mla.flash_mla_sparse_fwd(q, kv, idx, w.sm_scale, 512, cu(w.attn_sink), cu(w.topk_length))
    dq, dkv = flash_mla.flash_mla_sparse_bwd(q, kv, out, dout, idx, lse, w.sm_scale, 512, cu(w.attn_sink), cu(w.topk_length))
    dq32, dkv32 = flash_mla.flash_mla_sparse_bwd(q, kv, out, dout, idx, lse, w.sm_scale, 512, cu(w.attn_sink),
                                                 cu(w.topk_length), return_fp32_dkv=True)
    torch.cuda.synchronize()
    ref_dq, ref_dkv = attention.sparse_prefill_bwd(w.q, w.kv, w.dout, w.indices, w.sm_scale, attn_sink=w.attn_sink,
                                                   topk_length=w.topk_length, out=out.cpu())
    tol = dict(abs_tol=2e-3, rel_tol=2e-2, cos_tol=1e-4)
    assert_close("dq", dq.float().cpu(), ref_dq, **tol)
    assert_close("dkv", dkv.float().cpu(), ref_dkv, **tol)
    assert_close("dkv_fp32", dkv32.cpu(), ref_dkv, **tol)
    assert dkv.dtype == torch.bfloat16 and dkv32.dtype == torch.float32 and tuple(dkv.shape) == (s_kv, 1, 576)
    # rows of kv that no query indexes receive exactly zero gradient
    used = torch.zeros(s_kv, dtype=torch.bool)
    vi = w.indices[(w.indices >= 0) & (w.indices < s_kv)].long()
    used[vi] = True
    assert torch.all(dkv32.cpu()[~used] == 0)


def test_autograd_function_matches_explicit_backward():
    w = wl.make_prefill_workload(4, 64, 16, 64, seed=4, std=0.5)
    q = cu(w.q).requires_grad_(True)
    kv = cu(w.kv).requires_grad_(True)
    from flashmla_b200 import flash_mla_sparse_attn
    out, mx, lse = flash_mla_sparse_attn(q, kv, cu(w.indices), w.sm_scale)
    out.backward(cu(w.dout))
    dq, dkv = flash_mla.flash_mla_sparse_bwd(q.detach(), kv.detach(), out.detach(), cu(w.dout), cu(w.indices), lse,
                                             w.sm_scale)
    assert torch.equal(q.grad, dq)
    assert_close("dkv", kv.grad.float().cpu(), dkv.float().cpu(), abs_tol=1e-2, rel_tol=2e-2, cos_tol=1e-4)
