"""Generates the golden fixtures in this directory by running the reference's own CPU code.

Run once, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's tests/quant.py and tests/ref.py (its torch oracle)
with a stub standing in for the compiled ``flash_mla`` extension, feeds them
seeded inputs made by ``flashmla_b200.workloads``, and stores inputs and the
reference's outputs as .npz files.  The fixtures are what the CPU oracle under
``oracle/`` is pinned against; the reference checkout is not needed afterwards.
bf16 tensors are stored as their uint16 bit patterns.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from flashmla_b200 import workloads as wl  # noqa: E402


def bits(t: torch.Tensor) -> np.ndarray:
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.int16).numpy().view(np.uint16)
    return t.contiguous().numpy()


def import_reference(ref_root: str):
    stub = types.ModuleType("flash_mla")
    stub.cuda = types.ModuleType("flash_mla.cuda")
    sys.modules["flash_mla"] = stub
    sys.modules["flash_mla.cuda"] = stub.cuda
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    import lib as ref_lib      # noqa
    import quant as ref_quant  # noqa
    import ref as ref_ref      # noqa
    return ref_lib, ref_quant, ref_ref


def golden_quant(ref_quant):
    gen = torch.Generator().manual_seed(11)
    kv = torch.randn((6, 16, 1, 576), generator=gen)
    kv[0, 0] *= 1e-6            # exercises the 1e-4 floor of the scale rule
    kv[1, 3, 0, :128] = 0.0     # an all-zero tile
    kv[2] *= 37.0
    kv[3, :, :, 128:256] *= 448.0
    kv = kv.to(torch.bfloat16)
    rows = ref_quant.quantize_k_cache(kv, ref_quant.FP8KVCacheLayout.V32_FP8Sparse)
    deq = ref_quant.dequantize_k_cache(rows, ref_quant.FP8KVCacheLayout.V32_FP8Sparse)
    block_table = torch.randperm(24, generator=gen).to(torch.int32).view(3, 8)
    pos = torch.randint(0, 8 * 16, (3, 2, 40), generator=gen, dtype=torch.int32)
    pos[:, :, -5:] = -1
    pos[1, 0, 3] = -1
    rows_idx = ref_quant.abs_indices2indices_in_kvcache(pos, block_table, 16)
    np.savez_compressed(
        os.path.join(HERE, "quant_v32.npz"),
        kv=bits(kv), rows=bits(rows.contiguous().view(torch.uint8)), dequant=bits(deq),
        block_table=bits(block_table), positions=bits(pos), cache_rows=bits(rows_idx), page=np.int32(16))


def golden_quant_model1(ref_quant):
    """The reference's MODEL1 quantiser (d_qk = 512, block-wise 584-byte format) on the same kind of inputs."""
    gen = torch.Generator().manual_seed(12)
    kv = torch.randn((5, 16, 1, 512), generator=gen)
    kv[0, 0] *= 1e-6            # exercises the 1e-4 floor of the scale rule
    kv[1, 3, 0, :64] = 0.0      # an all-zero tile
    kv[2] *= 37.0
    kv[3, :, :, 64:128] *= 448.0
    kv = kv.to(torch.bfloat16)
    layout = ref_quant.FP8KVCacheLayout.MODEL1_FP8Sparse
    rows = ref_quant.quantize_k_cache(kv, layout)
    deq = ref_quant.dequantize_k_cache(rows, layout)
    # the reference leaves the 8th scale byte of every token uninitialised: it is stored here as zero
    flat = rows.view(torch.uint8).reshape(5, 16 * 584).clone()
    flat[:, 16 * 576:].view(5, 16, 8)[..., 7] = 0
    np.savez_compressed(os.path.join(HERE, "quant_model1.npz"), kv=bits(kv), rows=bits(flat.view(5, 16, 1, 584)), dequant=bits(deq))


def golden_decode(ref_lib, ref_quant, ref_ref, name, *, b, s_q, h_q, topk, s_k, seed, invalid_tail=0,
                  invalid_frac=0.0, with_sink=False, with_topk_length=False, all_invalid_row=False, layout=wl.LAYOUT_V32, **dist):
    w = wl.make_decode_workload(b, s_q, h_q, topk, s_k, s_k, seed=seed, invalid_tail=invalid_tail, layout=layout,
                                invalid_frac=invalid_frac, with_sink=with_sink, with_topk_length=with_topk_length, **dist)
    if all_invalid_row:
        w.indices[0, 0, :] = -1
    rows_fp8 = w.kv_rows.view(torch.float8_e4m3fn)
    ref_layout = ref_quant.FP8KVCacheLayout.MODEL1_FP8Sparse if layout == wl.LAYOUT_MODEL1 else ref_quant.FP8KVCacheLayout.V32_FP8Sparse
    deq = ref_quant.dequantize_k_cache(rows_fp8, ref_layout)
    p = ref_lib.TestParam(s_q=s_q, s_kv=s_k, topk=topk, h_q=h_q, h_kv=1, d_qk=w.q.shape[-1], d_v=512,
                          decode=ref_lib.ExtraTestParamForDecode(b=b, is_varlen=False, have_zero_seqlen_k=False))
    scope = ref_lib.KVScope(p, w.cache_seqlens, w.block_table, deq, w.positions, w.indices, w.topk_length)
    t = ref_lib.TestcaseForDecode(p, w.q, w.attn_sink, w.sm_scale, scope, None)
    with torch.inference_mode():
        out, lse = ref_ref.ref_sparse_attn_decode(p, t)
    extra = {}
    if w.attn_sink is not None:
        extra["attn_sink"] = bits(w.attn_sink)
    if w.topk_length is not None:
        extra["topk_length"] = bits(w.topk_length)
    np.savez_compressed(
        os.path.join(HERE, f"{name}.npz"),
        q=bits(w.q), kv_rows=bits(w.kv_rows), indices=bits(w.indices), sm_scale=np.float64(w.sm_scale),
        out=bits(out), lse=bits(lse.contiguous()), **extra)


def golden_decode_extra(ref_lib, ref_quant, ref_ref, name, *, b, s_q, h_q, topk, extra_topk, s_k, seed, **dist):
    """Decode over two caches (k_cache + extra_k_cache), each with its own index list and topk_length."""
    w = wl.make_decode_workload(b, s_q, h_q, topk, s_k, s_k, seed=seed, invalid_frac=0.05, with_sink=True,
                                with_topk_length=True, **dist)
    x = wl.make_decode_workload(b, s_q, h_q, extra_topk, s_k // 2, s_k // 2, seed=seed + 1000, invalid_frac=0.1,
                                with_topk_length=True, page=32, **dist)
    x.topk_length[0] = 0                      # one request without any extra token
    scopes = []
    for z in (w, x):
        deq = ref_quant.dequantize_k_cache(z.kv_rows.view(torch.float8_e4m3fn), ref_quant.FP8KVCacheLayout.V32_FP8Sparse)
        pz = ref_lib.TestParam(s_q=s_q, s_kv=z.cache_seqlens.max().item(), topk=z.indices.shape[-1], h_q=h_q, h_kv=1, d_qk=576, d_v=512,
                               decode=ref_lib.ExtraTestParamForDecode(b=b, is_varlen=False, have_zero_seqlen_k=False))
        scopes.append(ref_lib.KVScope(pz, z.cache_seqlens, z.block_table, deq, z.positions, z.indices, z.topk_length))
    p = ref_lib.TestParam(s_q=s_q, s_kv=s_k, topk=topk, h_q=h_q, h_kv=1, d_qk=576, d_v=512,
                          decode=ref_lib.ExtraTestParamForDecode(b=b, is_varlen=False, have_zero_seqlen_k=False))
    t = ref_lib.TestcaseForDecode(p, w.q, w.attn_sink, w.sm_scale, scopes[0], scopes[1])
    with torch.inference_mode():
        out, lse = ref_ref.ref_sparse_attn_decode(p, t)
    np.savez_compressed(
        os.path.join(HERE, f"{name}.npz"),
        q=bits(w.q), kv_rows=bits(w.kv_rows), indices=bits(w.indices), topk_length=bits(w.topk_length),
        attn_sink=bits(w.attn_sink), sm_scale=np.float64(w.sm_scale),
        extra_kv_rows=bits(x.kv_rows), extra_indices=bits(x.indices), extra_topk_length=bits(x.topk_length),
        out=bits(out), lse=bits(lse.contiguous()))


def golden_prefill(ref_lib, ref_ref, name, *, s_q, s_kv, h_q, topk, seed, with_sink=False, with_topk_length=False,
                   causal_offset=None, sm_scale=None, std=1.0, dead_rows=(), d_qk=576):
    pads = (-2147483648, -123456, -1, s_kv, 114514, 1919810, 2147480000, 2147483647)
    w = wl.make_prefill_workload(s_q, s_kv, h_q, topk, seed=seed, causal_offset=causal_offset, std=std,
                                 sm_scale=sm_scale, invalid_pads=pads, with_sink=with_sink,
                                 with_topk_length=with_topk_length, d_qk=d_qk)
    for r in dead_rows:
        w.indices[r] = 2147483647
    p = ref_lib.TestParam(s_q=s_q, s_kv=s_kv, topk=topk, h_q=h_q, h_kv=1, d_qk=d_qk, d_v=512)
    t = ref_lib.Testcase(p, w.dout, w.q, w.kv, w.indices, w.sm_scale, w.attn_sink, w.topk_length)
    with torch.inference_mode():
        out, out_f32, max_logits, lse = ref_ref.ref_sparse_attn_fwd(p, t)
    extra = {}
    if w.attn_sink is not None:
        extra["attn_sink"] = bits(w.attn_sink)
    if w.topk_length is not None:
        extra["topk_length"] = bits(w.topk_length)
    np.savez_compressed(
        os.path.join(HERE, f"{name}.npz"),
        q=bits(w.q), kv=bits(w.kv), indices=bits(w.indices), dout=bits(w.dout), sm_scale=np.float64(w.sm_scale),
        out=bits(out), out_f32=bits(out_f32), max_logits=bits(max_logits), lse=bits(lse), **extra)


def golden_dense(ref_root, name, *, b, s_q, h_q, h_kv, s_k, page, causal, seed, zero_len=False):
    """Dense MLA decode: the torch reference inside the reference's own test file
    (tests/test_flash_mla_dense_decoding.py:73-141), imported with a stand-in for its helper package."""
    kk = types.ModuleType("kernelkit")
    kk.cdiv = lambda a, b: (a + b - 1) // b
    sys.modules["kernelkit"] = kk
    import test_flash_mla_dense_decoding as ref_dense   # noqa
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(max(s_q, s_k // 3), s_k + 1, (b,), generator=g, dtype=torch.int32)
    if zero_len:
        lens[1] = 0
    max_blocks = (int(lens.max()) + page - 1) // page + 1
    block_table = torch.randperm(b * max_blocks, generator=g).to(torch.int32).view(b, max_blocks)
    d = 576
    q = (torch.randn((b, s_q, h_q, d), generator=g)).to(torch.bfloat16)
    blocked_k = (torch.randn((b * max_blocks, page, h_kv, d), generator=g) / 10).to(torch.bfloat16)
    out, lse = ref_dense.reference_torch(lens, block_table, q, blocked_k, 512, causal)
    np.savez_compressed(os.path.join(HERE, name + ".npz"), q=bits(q), blocked_k=bits(blocked_k), block_table=block_table.numpy(),
                        cache_seqlens=lens.numpy(), causal=np.array(causal), out=bits(out), lse=lse.numpy())


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: python tests/golden/make_golden.py /path/to/reference")
    ref_root = sys.argv[1]
    ref_lib, ref_quant, ref_ref = import_reference(ref_root)
    golden_quant(ref_quant)
    # the CPU-runnable benchmark configuration: b=2, s_q=1, h_q=16, topk=128 (last 8 invalid), s_k=1024
    golden_decode(ref_lib, ref_quant, ref_ref, "decode_c1", b=2, s_q=1, h_q=16, topk=128, s_k=1024, seed=1,
                  invalid_tail=8)
    golden_decode(ref_lib, ref_quant, ref_ref, "decode_sink_len", b=3, s_q=2, h_q=8, topk=64, s_k=256, seed=2,
                  invalid_frac=0.1, with_sink=True, with_topk_length=True, all_invalid_row=True)
    # 128 heads (the tensor-core kernels' shape), value distributions of the reference's own fixtures
    golden_decode(ref_lib, ref_quant, ref_ref, "decode_h128", b=2, s_q=2, h_q=128, topk=192, s_k=512, seed=6,
                  invalid_frac=0.05, with_sink=True, q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=576 ** -0.55)
    golden_decode_extra(ref_lib, ref_quant, ref_ref, "decode_extra", b=3, s_q=2, h_q=16, topk=128, extra_topk=64, s_k=384,
                        seed=8, q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=576 ** -0.55)
    golden_prefill(ref_lib, ref_ref, "prefill_h128", s_q=4, s_kv=300, h_q=128, topk=256, seed=7, with_sink=True,
                   with_topk_length=True, sm_scale=0.5, std=0.1)
    golden_prefill(ref_lib, ref_ref, "prefill_small", s_q=6, s_kv=200, h_q=8, topk=128, seed=3)
    golden_prefill(ref_lib, ref_ref, "prefill_sink_len", s_q=7, s_kv=96, h_q=8, topk=128, seed=4,
                   with_sink=True, with_topk_length=True, sm_scale=0.5, std=0.1, dead_rows=(2,))
    golden_prefill(ref_lib, ref_ref, "prefill_causal", s_q=5, s_kv=64, h_q=4, topk=64, seed=5, causal_offset=20)
    # d_qk = 512: the reference's MODEL1 cache format (decode) and its 512-wide prefill
    golden_quant_model1(ref_quant)
    golden_decode(ref_lib, ref_quant, ref_ref, "decode_model1", b=3, s_q=2, h_q=16, topk=128, s_k=384, seed=9,
                  invalid_frac=0.05, with_sink=True, with_topk_length=True, layout=wl.LAYOUT_MODEL1,
                  q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=512 ** -0.55)
    golden_decode(ref_lib, ref_quant, ref_ref, "decode_model1_h128", b=2, s_q=1, h_q=128, topk=192, s_k=512, seed=10,
                  invalid_frac=0.03, layout=wl.LAYOUT_MODEL1, q_std=1.0, kv_std=0.1, clamp=1.0, sm_scale=512 ** -0.55)
    golden_prefill(ref_lib, ref_ref, "prefill_d512_h128", s_q=4, s_kv=300, h_q=128, topk=256, seed=13, with_sink=True,
                   with_topk_length=True, sm_scale=0.5, std=0.1, d_qk=512)
    # dense decode (bf16 paged cache, block table, causal among the s_q rows, two kv heads, a request of length zero)
    golden_dense(ref_root, "dense_decode", b=3, s_q=2, h_q=16, h_kv=2, s_k=200, page=64, causal=True, seed=21, zero_len=True)
    golden_dense(ref_root, "dense_decode_h128", b=2, s_q=3, h_q=128, h_kv=1, s_k=300, page=64, causal=False, seed=22)
    for f in sorted(os.listdir(HERE)):
        if f.endswith(".npz"):
            print(f, os.path.getsize(os.path.join(HERE, f)))


if __name__ == "__main__":
    main()
