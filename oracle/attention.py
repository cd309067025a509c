"""Sparse MLA attention on the CPU in fp32/fp64 (test infrastructure).

Restates the reference's torch oracle:
  prefill forward  tests/ref.py:19-52   (``sparse_prefill_fwd``)
  decode           tests/ref.py:55-103  (``sparse_decode``)
and, for the dense decode branch, the torch reference inside the reference's dense test
  dense decode     tests/test_flash_mla_dense_decoding.py:73-141  (``dense_decode``)
The backward has no counterpart in the reference (parity unpinned); it is the
analytic gradient of ``sparse_prefill_fwd`` and is checked against autograd and
finite differences in the tests.

Everything is chunked over query rows so that the gathered [rows, topk, d]
tensor stays small; rows are independent, so chunking does not change results.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

INF = float("inf")


def _chunks(n: int, step: int):
    for lo in range(0, n, step):
        yield lo, min(n, lo + step)


def _prefill_masks(indices: torch.Tensor, s_kv: int, topk_length: Optional[torch.Tensor]):
    """indices [n, topk] -> (safe int64 indices, invalid mask).  tests/ref.py:27-32."""
    idx = indices.to(torch.int64).clone()
    topk = idx.shape[-1]
    if topk_length is not None:
        beyond = torch.arange(topk).unsqueeze(0) >= topk_length.to(torch.int64).unsqueeze(1)
        idx[beyond] = -1
    invalid = (idx < 0) | (idx >= s_kv)
    idx[invalid] = 0
    return idx, invalid


def sparse_prefill_fwd(
    q: torch.Tensor,            # [s_q, h_q, d_qk] bf16
    kv: torch.Tensor,           # [s_kv, 1, d_qk] bf16
    indices: torch.Tensor,      # [s_q, 1, topk] int32
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,     # [h_q] fp32
    topk_length: Optional[torch.Tensor] = None,   # [s_q] int32
    chunk: int = 16,
    dtype: torch.dtype = torch.float32,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (out bf16, out fp, max_logits, lse) as tests/ref.py:19-52 does.

    Invalid slot = index outside [0, s_kv) or position >= topk_length[i].
    lse is the natural-log sum over valid logits; rows with no valid slot give
    out = 0, lse = +inf, max_logits = -inf.  attn_sink only rescales out.
    """
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    kvf = kv.reshape(s_kv, d_qk).to(dtype)
    out = torch.empty((s_q, h_q, d_v), dtype=dtype)
    max_logits = torch.empty((s_q, h_q), dtype=dtype)
    lse = torch.empty((s_q, h_q), dtype=dtype)
    for lo, hi in _chunks(s_q, chunk):
        idx, invalid = _prefill_masks(indices[lo:hi, 0], s_kv, None if topk_length is None else topk_length[lo:hi])
        g = kvf[idx.reshape(-1)].reshape(hi - lo, -1, d_qk)                # [n, topk, d]
        p = torch.matmul(q[lo:hi].to(dtype), g.transpose(1, 2)) * sm_scale   # [n, h, topk]
        p.masked_fill_(invalid.unsqueeze(1), -INF)
        l = torch.logsumexp(p, dim=-1)
        max_logits[lo:hi] = p.max(dim=-1).values
        l_o = l if attn_sink is None else torch.logsumexp(
            torch.stack([l, attn_sink.to(dtype).view(1, h_q).expand_as(l)]), dim=0)
        l_o = l_o.masked_fill(l_o == -INF, INF)
        out[lo:hi] = torch.matmul(torch.exp(p - l_o.unsqueeze(-1)), g[..., :d_v])
        lse[lo:hi] = l.masked_fill(l == -INF, INF)
    return out.to(torch.bfloat16), out, max_logits, lse


def sparse_decode(
    q: torch.Tensor,                 # [b, s_q, h_q, d_qk] bf16
    kv_dequant: torch.Tensor,        # [num_blocks, page, 1, d_qk] bf16 (dequantised cache)
    indices: torch.Tensor,           # [b, s_q, topk] int32 in-cache row indices, -1 invalid
    sm_scale: float,
    d_v: int = 512,
    attn_sink: Optional[torch.Tensor] = None,    # [h_q]
    topk_length: Optional[torch.Tensor] = None,  # [b]
    chunk: int = 8,
    extra_kv_dequant: Optional[torch.Tensor] = None,    # second cache, same form as kv_dequant
    extra_indices: Optional[torch.Tensor] = None,       # [b, s_q, extra_topk]
    extra_topk_length: Optional[torch.Tensor] = None,   # [b]
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Returns (out bf16 [b,s_q,h_q,d_v], lse fp32 [b,h_q,s_q], out fp32).  tests/ref.py:55-103.

    Invalid slot = index == -1 or position >= topk_length[batch].  NaNs in
    gathered rows are zeroed (the reference's fixtures poison unused rows).
    With an extra cache the query attends to the union of both index lists (tests/ref.py:77-81).
    """
    b, s_q, h_q, d_qk = q.shape

    def scope(kvd, idx, length):
        k = idx.shape[-1]
        ia = idx.reshape(b * s_q, k).to(torch.int64)
        inv = ia == -1
        if length is not None:
            tl = length.to(torch.int64).repeat_interleave(s_q)
            inv = inv | (torch.arange(k).unsqueeze(0) >= tl.unsqueeze(1))
        return kvd.reshape(-1, d_qk), ia, inv

    flat, idx_all, invalid_all = scope(kv_dequant, indices, topk_length)
    topk = indices.shape[-1]
    if extra_kv_dequant is not None:
        flat2, idx2, inv2 = scope(extra_kv_dequant, extra_indices, extra_topk_length)
        idx_all = torch.cat([idx_all, torch.where(idx2 >= 0, idx2 + flat.shape[0], idx2)], dim=1)   # rows of the second pool follow the first
        invalid_all = torch.cat([invalid_all, inv2], dim=1)
        flat = torch.cat([flat, flat2], dim=0)
        topk = idx_all.shape[1]
    qf = q.reshape(b * s_q, h_q, d_qk).float()
    out = torch.empty((b * s_q, h_q, d_v), dtype=torch.float32)
    lse = torch.empty((b * s_q, h_q), dtype=torch.float32)
    for lo, hi in _chunks(b * s_q, chunk):
        g = flat[idx_all[lo:hi].clamp_min(0).reshape(-1)].reshape(hi - lo, topk, d_qk).float()
        g = torch.nan_to_num(g, nan=0.0, posinf=INF, neginf=-INF)
        w = torch.matmul(qf[lo:hi], g.transpose(1, 2)) * sm_scale
        w.masked_fill_(invalid_all[lo:hi].unsqueeze(1), -INF)
        l = torch.logsumexp(w, dim=-1)
        o = torch.matmul(torch.exp(w - l.unsqueeze(-1)), g[..., :d_v])
        if attn_sink is not None:
            o = o * (1.0 / (1.0 + torch.exp(attn_sink.float().view(1, h_q) - l))).unsqueeze(-1)
        lonely = l == -INF
        o[lonely] = 0.0
        out[lo:hi] = o
        lse[lo:hi] = l.masked_fill(lonely, INF)
    out = out.view(b, s_q, h_q, d_v)
    return out.to(torch.bfloat16), lse.view(b, s_q, h_q).transpose(1, 2), out


def sparse_prefill_bwd(
    q: torch.Tensor, kv: torch.Tensor, dout: torch.Tensor, indices: torch.Tensor, sm_scale: float,
    d_v: int = 512, attn_sink: Optional[torch.Tensor] = None, topk_length: Optional[torch.Tensor] = None,
    chunk: int = 16, dtype: torch.dtype = torch.float32, out: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Analytic gradient of ``sparse_prefill_fwd``'s ``out`` w.r.t. q and kv.

    When ``out`` (the forward's bf16 result, an input of the backward operator) is given, delta is
    computed from it, as the kernels do; otherwise from the exact forward output.

    With P = exp(S*scale - lse_o) (lse_o includes the sink when given),
    delta = rowsum(O * dO), dP = dO V^T, dS = P * (dP - delta) * scale:
      dQ = dS K,   dK = dS^T Q (all 576 dims),   dV = P^T dO (first d_v dims).
    dKV is accumulated over duplicate indices in ``dtype`` (scatter-add).
    Returns (dq [s_q,h_q,d_qk], dkv [s_kv,1,d_qk]) in ``dtype``; invalid slots
    and rows with no valid slot contribute nothing; the sink is a constant.
    """
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    kvf = kv.reshape(s_kv, d_qk).to(dtype)
    dq = torch.zeros((s_q, h_q, d_qk), dtype=dtype)
    dkv = torch.zeros((s_kv, d_qk), dtype=dtype)
    for lo, hi in _chunks(s_q, chunk):
        n = hi - lo
        idx, invalid = _prefill_masks(indices[lo:hi, 0], s_kv, None if topk_length is None else topk_length[lo:hi])
        g = kvf[idx.reshape(-1)].reshape(n, -1, d_qk)
        qc = q[lo:hi].to(dtype)
        s = torch.matmul(qc, g.transpose(1, 2)) * sm_scale
        s.masked_fill_(invalid.unsqueeze(1), -INF)
        l = torch.logsumexp(s, dim=-1)
        l_o = l if attn_sink is None else torch.logsumexp(
            torch.stack([l, attn_sink.to(dtype).view(1, h_q).expand_as(l)]), dim=0)
        l_o = l_o.masked_fill(l_o == -INF, INF)
        p = torch.exp(s - l_o.unsqueeze(-1))                      # [n,h,topk]
        do = dout[lo:hi].to(dtype)
        o = torch.matmul(p, g[..., :d_v]) if out is None else out[lo:hi].to(dtype)
        delta = (o * do).sum(-1, keepdim=True)
        dp = torch.matmul(do, g[..., :d_v].transpose(1, 2))
        ds = p * (dp - delta) * sm_scale
        dq[lo:hi] = torch.matmul(ds, g)
        dk = torch.matmul(ds.transpose(1, 2), qc)                 # [n,topk,d_qk]
        dk[..., :d_v] += torch.matmul(p.transpose(1, 2), do)
        dk.masked_fill_(invalid.unsqueeze(-1), 0.0)
        dkv.index_add_(0, idx.reshape(-1), dk.reshape(-1, d_qk))
    return dq, dkv.view(s_kv, 1, d_qk)


def dense_decode(q: torch.Tensor, blocked_k: torch.Tensor, block_table: torch.Tensor, cache_seqlens: torch.Tensor,
                 d_v: int = 512, causal: bool = False, sm_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Dense MLA decode over a paged bf16 cache, restated from the reference's own torch reference
    (tests/test_flash_mla_dense_decoding.py:73-141).

    q [b, s_q, h_q, d] bf16, blocked_k [num_blocks, page, h_kv, d] bf16, block_table [b, max_blocks] int32,
    cache_seqlens [b] int32.  Request i attends the first cache_seqlens[i] tokens of its blocks; with ``causal`` query
    row j of its s_q rows sees only the first cache_seqlens[i] - (s_q - 1 - j).  Head h reads kv head h // (h_q / h_kv).
    Returns (out [b, s_q, h_q, d_v] in q's dtype, lse [b, h_q, s_q] fp32 natural log; a row that sees nothing gives
    out = 0 and lse = +inf).
    """
    b, s_q, h_q, d = q.shape
    page, h_kv = blocked_k.shape[1], blocked_k.shape[2]
    scale = d ** -0.5 if sm_scale is None else sm_scale
    out = torch.zeros((b, s_q, h_q, d_v), dtype=torch.float32)
    lse = torch.full((b, h_q, s_q), float("inf"), dtype=torch.float32)
    for i in range(b):
        n = int(cache_seqlens[i])
        if n == 0:
            continue
        blocks = block_table[i, : (n + page - 1) // page].long()
        kv = blocked_k[blocks].reshape(-1, h_kv, d)[:n].float()                     # [n, h_kv, d]
        kv = kv.repeat_interleave(h_q // h_kv, dim=1)                                  # [n, h_q, d]
        logits = torch.einsum("shd,nhd->hsn", q[i].float(), kv) * scale               # [h_q, s_q, n]
        if causal and s_q > 1:
            visible = torch.ones(s_q, n, dtype=torch.bool).tril(diagonal=n - s_q)
            logits = logits.masked_fill(~visible, float("-inf"))
        row_lse = torch.logsumexp(logits, dim=-1)                                      # [h_q, s_q]
        dead = row_lse == float("-inf")
        p = torch.softmax(logits, dim=-1)
        p = torch.where(dead.unsqueeze(-1), torch.zeros_like(p), p)
        out[i] = torch.einsum("hsn,nhv->shv", p, kv[..., :d_v])
        lse[i] = torch.where(dead, torch.full_like(row_lse, float("inf")), row_lse)
    return out.to(q.dtype), lse
